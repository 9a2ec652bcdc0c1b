"""Pins the CPU oracle to outputs of the unmodified reference (tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

from oracle import hidream_moe_oracle as O


def _setup(golden):
    m = golden["meta"]
    dim, hidden_dim, e = int(m["dim"]), int(m["hidden_dim"]), int(m["n_experts"])
    n = int(m["batch"]) * int(m["seq"])
    x = O.make_input(n, dim, int(m["x_seed"]))
    layer = O.make_layer(dim, hidden_dim, e, int(m["w_seed"]))
    return x, layer


def test_seeded_inputs_reproduce(golden):
    """The fixtures store outputs only; inputs are regenerated from seeds, so check they are the same."""
    x, layer = _setup(golden)
    assert np.allclose([float(x.double().sum()), float(x.double().abs().sum())], golden["x_checksum"], rtol=0, atol=1e-9)
    got = [float(sum(v.double().sum() for v in layer.values())), float(sum(v.double().abs().sum() for v in layer.values()))]
    assert np.allclose(got, golden["w_checksum"], rtol=0, atol=1e-9)


def test_state_dict_keys(golden):
    """Key set of the scaled-fp8 layer = the reference module's (loaded there with strict=True)."""
    _, layer = _setup(golden)
    l8 = O.quantize_layer_fp8({k: v.bfloat16() for k, v in layer.items()}, scale_input=0.75)
    assert sorted(l8.keys()) == golden["state_dict_keys"].tolist()
    assert len(layer) == 16 and len(O.quantize_layer_fp8(layer)) == 31


def _same_routing(idx, w, g_idx, g_w):
    """topk(sorted=False) leaves the pair order open: compare as sets, weights permuted along."""
    o1, o2 = idx.argsort(dim=1), torch.from_numpy(g_idx).argsort(dim=1)
    assert torch.equal(idx.gather(1, o1), torch.from_numpy(g_idx).gather(1, o2))
    assert torch.equal(w.float().gather(1, o1), torch.from_numpy(g_w).gather(1, o2))


CASES = [
    # name,                    dtype,          gate fp32, mode,            quant kwargs
    ("fp32", torch.float32, False, O.PLAIN, None),
    ("bf16_shipped", torch.bfloat16, False, O.PLAIN, None),
    ("bf16", torch.bfloat16, True, O.PLAIN, None),
    ("fp8_dequant", torch.bfloat16, True, O.FP8_DEQUANT, {}),
    ("fp8_matmul", torch.bfloat16, True, O.FP8_MATMUL, {}),
    ("fp8_matmul_scale_input", torch.bfloat16, True, O.FP8_MATMUL, {"scale_input": 0.75}),
]


@pytest.mark.parametrize("name,dtype,gate32,mode,quant", CASES, ids=[c[0] for c in CASES])
def test_moe_infer_matches_reference(golden, name, dtype, gate32, mode, quant):
    x, layer = _setup(golden)
    x = x.to(dtype)
    layer = {k: v.to(dtype) for k, v in layer.items()}
    if quant is not None:
        layer = O.quantize_layer_fp8(layer, **quant)
    out, idx, w = O.moe_layer(x, layer, mode=mode, gate_in_fp32=gate32, branch="infer")
    _same_routing(idx, w, golden[f"{name}/idx"], golden[f"{name}/w"])
    ref = torch.from_numpy(golden[f"{name}/out"])
    if dtype == torch.float32:
        torch.testing.assert_close(out, ref, rtol=1e-6, atol=1e-7)
    elif mode == O.FP8_MATMUL:
        # the oracle emulates torch._scaled_mm with float math: allow a bf16 ulp on a handful of elements
        diff = (out.float() - ref).abs()
        assert float(diff.max()) <= 2 ** -7 * float(ref.abs().max())
        assert float((diff > 0).float().mean()) < 0.02
    else:
        assert torch.equal(out.float(), ref)


@pytest.mark.parametrize("name,dtype", [("fp32", torch.float32), ("bf16_shipped", torch.bfloat16)])
def test_forward_branch_matches_reference(golden, name, dtype):
    """The masked branch forward() really takes equals moe_infer + shared bit for bit."""
    assert golden["meta"][f"{name}_forward_equals_infer"] == "True"
    x, layer = _setup(golden)
    x = x.to(dtype)
    layer = {k: v.to(dtype) for k, v in layer.items()}
    out, _, _ = O.moe_layer(x, layer, gate_in_fp32=False, branch="masked")
    ref = torch.from_numpy(golden[f"{name}/forward"])
    if dtype == torch.float32:
        torch.testing.assert_close(out, ref, rtol=1e-6, atol=1e-7)
    else:
        assert torch.equal(out.float(), ref)


def test_real_scaled_mm_agrees_with_emulation(golden):
    """torch._scaled_mm on the CPU against the float emulation the oracle uses at full size."""
    x, layer = _setup(golden)
    x = x.bfloat16()
    l8 = O.quantize_layer_fp8({k: v.bfloat16() for k, v in layer.items()})
    a = O.linear(x, l8, "shared_experts.w1", O.FP8_MATMUL, use_real_scaled_mm=True)
    b = O.linear(x, l8, "shared_experts.w1", O.FP8_MATMUL, use_real_scaled_mm=False)
    diff = (a.float() - b.float()).abs()
    assert float((diff > 0).float().mean()) < 0.01
    assert float(diff.max()) <= 2 ** -7 * float(a.float().abs().max())


def test_gate_has_no_renormalisation():
    x = O.make_input(512, 256, 3)
    layer = O.make_layer(256, 1024, 4, 0)
    _, w = O.gate(x, layer["gate.weight"])
    s = w.sum(1)
    assert float(s.max()) < 1.0 and 0.5 < float(s.mean()) < 1.0


def test_empty_and_single_expert_routing():
    """Edge cases of moe_infer: trailing experts without tokens, all tokens to one pair."""
    x = O.make_input(8, 256, 5)
    layer = O.make_layer(256, 1024, 4, 0)
    idx = torch.tensor([[0, 1]] * 8)
    w = torch.full((8, 2), 0.25)
    out = O.moe_infer(x, idx.reshape(-1), w.reshape(-1, 1), layer)
    ref = 0.25 * (O.swiglu_ffn(x, layer, "experts.0") + O.swiglu_ffn(x, layer, "experts.1"))
    torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-6)
    masked = O.moe_forward_masked(x, idx, w, layer)
    torch.testing.assert_close(masked, ref, rtol=1e-5, atol=1e-6)


def test_block_ffn_matches_reference(golden):
    """LayerNorm + modulation + MoE + gate/residual as the single-stream block spells it (model.py:429-433)."""
    m = golden["meta"]
    b, s, dim = int(m["batch"]), int(m["seq"]), int(m["dim"])
    x, layer = _setup(golden)
    x = x.bfloat16().view(b, s, dim)
    layer = {k: v.bfloat16() for k, v in layer.items()}
    shift, scale, gate = O.make_modulation(b, dim)
    out = O.block_ffn(x, layer, shift, scale, gate, gate_in_fp32=False, branch="masked")
    assert torch.equal(out.reshape(-1, dim).float(), torch.from_numpy(golden["block_bf16/out"]))
    dense = O.block_ffn(x, layer, shift, scale, gate, dense_prefix="shared_experts")
    assert torch.equal(dense.reshape(-1, dim).float(), torch.from_numpy(golden["block_bf16/dense_out"]))
