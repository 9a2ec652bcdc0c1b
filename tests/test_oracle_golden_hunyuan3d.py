"""Pins the Hunyuan3D-2.1 MoE oracle to outputs of the unmodified reference (tests/golden/make_golden.py)."""
import pytest
import torch

from oracle import hunyuan3d_moe_oracle as H


def _setup(g, dtype):
    m = g["meta"]
    dim, inner, e = int(m["dim"]), int(m["inner"]), int(m["n_experts"])
    n = int(m["batch"]) * int(m["seq"])
    x = H.make_input(n, dim, int(m["x_seed"])).to(dtype)
    layer = H.make_layer(dim, inner, e, int(m["w_seed"]), dtype=dtype)
    return x, layer


def _same_routing(idx, w, g_idx, g_w):
    o1, o2 = idx.argsort(dim=1), torch.from_numpy(g_idx).argsort(dim=1)
    assert torch.equal(idx.gather(1, o1), torch.from_numpy(g_idx).gather(1, o2))
    assert torch.equal(w.float().gather(1, o1), torch.from_numpy(g_w).gather(1, o2))


def _close(got, want, dtype):
    want = torch.from_numpy(want)
    if dtype == torch.bfloat16:
        assert torch.equal(got.float(), want)          # same PyTorch ops on the same data: bit for bit
    else:
        assert torch.allclose(got, want, rtol=0, atol=1e-6)


def test_state_dict_keys(golden_hunyuan3d):
    _, layer = _setup(golden_hunyuan3d, torch.float32)
    assert sorted(layer.keys()) == golden_hunyuan3d["state_dict_keys"].tolist()
    assert len(layer) == 4 * 9 + 1


@pytest.mark.parametrize("name,dtype", [("fp32", torch.float32), ("bf16", torch.bfloat16)])
def test_moe_infer_matches_reference(golden_hunyuan3d, name, dtype):
    g = golden_hunyuan3d
    x, layer = _setup(g, dtype)
    out, idx, w = H.moe_block(x, layer, gate_in_fp32=True)
    _same_routing(idx, w, g[f"{name}/idx"], g[f"{name}/w"])
    routed = H.moe_infer(x, idx.reshape(-1), w.reshape(-1, 1), layer)
    _close(routed, g[f"{name}/routed"], dtype)
    _close(H.gelu_ffn(x, layer, "shared_experts"), g[f"{name}/shared"], dtype)
    _close(out, g[f"{name}/out"], dtype)


@pytest.mark.parametrize("name,dtype", [("fp32", torch.float32), ("bf16", torch.bfloat16)])
def test_forward_as_shipped_and_training_branch(golden_hunyuan3d, name, dtype):
    """forward() as shipped gates in the activation dtype; the training-mode branch gathers with boolean masks."""
    g = golden_hunyuan3d
    x, layer = _setup(g, dtype)
    out, idx, w = H.moe_block(x, layer, gate_in_fp32=False)
    _same_routing(idx, w, g[f"{name}/idx_shipped"], g[f"{name}/w_shipped"])
    _close(out, g[f"{name}/forward"], dtype)
    masked = H.moe_forward_masked(x, idx, w, layer) + H.gelu_ffn(x, layer, "shared_experts")
    _close(masked, g[f"{name}/forward_train_branch"], dtype)
