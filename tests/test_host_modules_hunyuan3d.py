"""Host-side mirror of the Hunyuan3D-2.1 MoE block on the CPU: interface, state-dict keys, and its stock
composition held to the reference's golden outputs (no GPU, no kernels)."""
import inspect

import pytest
import torch

from comfyui_b200 import ops
from comfyui_b200.ldm.hunyuan3dv2_1 import hunyuandit as M
from oracle import hunyuan3d_moe_oracle as H


def _module(g, dtype):
    m = g["meta"]
    dim, inner, e = int(m["dim"]), int(m["inner"]), int(m["n_experts"])
    mod = M.MoEBlock(dim, num_experts=e, moe_top_k=2, ff_inner_dim=inner, operations=ops.disable_weight_init,
                     device="cpu", dtype=dtype)
    layer = H.make_layer(dim, inner, e, int(m["w_seed"]), dtype=dtype)
    res = mod.load_state_dict(layer, strict=True)
    assert not res.missing_keys and not res.unexpected_keys
    n = int(m["batch"]) * int(m["seq"])
    x = H.make_input(n, dim, int(m["x_seed"])).to(dtype).view(int(m["batch"]), int(m["seq"]), dim)
    return mod, x, layer


def test_constructor_signatures_match_reference():
    assert list(inspect.signature(M.MoEBlock.__init__).parameters) == [
        "self", "dim", "num_experts", "moe_top_k", "dropout", "ff_inner_dim", "operations", "device", "dtype"]
    assert list(inspect.signature(M.MoEGate.__init__).parameters) == [
        "self", "embed_dim", "num_experts", "num_experts_per_tok", "aux_loss_alpha", "device", "dtype"]
    assert list(inspect.signature(M.FeedForward.__init__).parameters) == [
        "self", "dim", "dim_out", "mult", "dropout", "inner_dim", "operations", "device", "dtype"]
    assert list(inspect.signature(M.MoEBlock.moe_infer).parameters) == [
        "self", "x", "flat_expert_indices", "flat_expert_weights"]


def test_state_dict_keys(golden_hunyuan3d):
    mod, _, layer = _module(golden_hunyuan3d, torch.float32)
    assert sorted(mod.state_dict().keys()) == golden_hunyuan3d["state_dict_keys"].tolist()


@pytest.mark.parametrize("name,dtype", [("fp32", torch.float32), ("bf16", torch.bfloat16)])
def test_stock_composition_reproduces_reference(golden_hunyuan3d, name, dtype):
    g = golden_hunyuan3d
    mod, x, _ = _module(g, dtype)
    n, d = x.shape[0] * x.shape[1], x.shape[2]
    with torch.no_grad():
        mod.eval()
        got = mod(x.clone()).view(n, d).float()
        want = torch.from_numpy(g[f"{name}/forward"])
        assert torch.equal(got, want) if dtype == torch.bfloat16 else torch.allclose(got, want, rtol=0, atol=1e-6)
        idx, w, aux = mod.gate(x)
        assert aux is None and idx.shape == (n, 2) and w.dtype == dtype
        mod.train()
        got = mod(x.clone()).view(n, d).float()
        want = torch.from_numpy(g[f"{name}/forward_train_branch"])
        assert torch.equal(got, want) if dtype == torch.bfloat16 else torch.allclose(got, want, rtol=0, atol=1e-6)


def test_cpu_call_is_not_eligible_for_the_kernels(golden_hunyuan3d):
    mod, x, _ = _module(golden_hunyuan3d, torch.bfloat16)
    mod.eval()
    assert ops.hunyuan3d_moe_forward(mod, x) is None
    assert ops.gelu_ffn_forward(mod.shared_experts, x) is None
