"""Host-side mirror of the reference's module and comfy.ops interface, checked on the CPU against
outputs of the unmodified reference (golden fixtures)."""
import pytest
import torch

from comfyui_b200 import model_management, ops
from comfyui_b200.ldm.hidream.model import FeedForwardSwiGLU, MOEFeedForwardSwiGLU, MoEGate
from oracle import hidream_moe_oracle as O


def _case(golden, dtype, operations, quant=None):
    m = golden["meta"]
    dim, hidden_dim, e = int(m["dim"]), int(m["hidden_dim"]), int(m["n_experts"])
    b, s = int(m["batch"]), int(m["seq"])
    layer = {k: v.to(dtype) for k, v in O.make_layer(dim, hidden_dim, e, int(m["w_seed"])).items()}
    if quant is not None:
        layer = O.quantize_layer_fp8(layer, **quant)
    x = O.make_input(b * s, dim, int(m["x_seed"])).to(dtype).view(b, s, dim)
    mod = MOEFeedForwardSwiGLU(dim, hidden_dim, e, 2, dtype=dtype, device="cpu", operations=operations).eval()
    res = mod.load_state_dict(layer, strict=True)
    assert not res.missing_keys and not res.unexpected_keys
    return mod, x, layer


def test_state_dict_keys_and_shapes():
    mod = MOEFeedForwardSwiGLU(2560, 4 * 2560, 4, 2, dtype=torch.bfloat16, device="meta",
                               operations=ops.disable_weight_init)
    sd = mod.state_dict()
    assert len(sd) == 16
    assert sd["experts.3.w1.weight"].shape == (6912, 2560)
    assert sd["experts.0.w2.weight"].shape == (2560, 6912)
    assert sd["shared_experts.w3.weight"].shape == (3584, 2560)
    assert sd["gate.weight"].shape == (4, 2560)
    scaled = ops.scaled_fp8_ops(fp8_matrix_mult=True, scale_input=True, override_dtype=torch.float8_e4m3fn)
    mod8 = MOEFeedForwardSwiGLU(256, 1024, 4, 2, dtype=torch.bfloat16, device="cpu", operations=scaled)
    sd8 = mod8.state_dict()
    assert len(sd8) == 16 + 15 * 2
    assert sd8["experts.1.w2.weight"].dtype == torch.float8_e4m3fn
    assert sd8["experts.1.w2.scale_weight"].shape == () and sd8["experts.1.w2.scale_input"].dtype == torch.float32
    assert sd8["gate.weight"].dtype == torch.bfloat16   # the gate is a bare Parameter, not an operations.Linear


@pytest.mark.parametrize("name,dtype", [("fp32", torch.float32), ("bf16_shipped", torch.bfloat16)])
def test_forward_matches_reference(golden, name, dtype):
    mod, x, _ = _case(golden, dtype, ops.disable_weight_init)
    with torch.no_grad():
        out = mod(x).view(-1, x.shape[-1])
        idx, w, aux = mod.gate(x)
    assert aux is None and idx.dtype == torch.int64 and w.dtype == dtype
    ref = torch.from_numpy(golden[f"{name}/forward"])
    if dtype == torch.float32:
        torch.testing.assert_close(out, ref, rtol=1e-6, atol=1e-7)
    else:
        assert torch.equal(out.float(), ref)
    g_idx = torch.from_numpy(golden[f"{name}/idx"])
    assert torch.equal(idx.sort(dim=1).values, g_idx.sort(dim=1).values)


@pytest.mark.parametrize("name,fp8_mm,quant", [
    ("fp8_dequant", False, {}),
    ("fp8_matmul", True, {}),
    ("fp8_matmul_scale_input", True, {"scale_input": 0.75}),
])
def test_scaled_fp8_namespaces_match_reference(golden, name, fp8_mm, quant):
    operations = ops.scaled_fp8_ops(fp8_matrix_mult=fp8_mm, scale_input="scale_input" in quant,
                                    override_dtype=torch.float8_e4m3fn)
    mod, x, _ = _case(golden, torch.bfloat16, operations, quant)
    x2 = x.view(-1, x.shape[-1])
    idx = torch.from_numpy(golden[f"{name}/idx"])
    w = torch.from_numpy(golden[f"{name}/w"]).bfloat16()
    with torch.no_grad():
        out = mod.moe_infer(x2, idx.view(-1), w.view(-1, 1)) + mod.shared_experts(x2)
    assert torch.equal(out.float(), torch.from_numpy(golden[f"{name}/out"]))


def test_pick_operations_rules(monkeypatch):
    bf16, fp32, e4m3 = torch.bfloat16, torch.float32, torch.float8_e4m3fn
    monkeypatch.setattr(model_management, "FORCE_FP8_COMPUTE", False)
    assert ops.pick_operations(bf16, bf16) is ops.disable_weight_init
    assert ops.pick_operations(bf16, None) is ops.disable_weight_init
    assert ops.pick_operations(fp32, bf16) is ops.manual_cast
    scaled = ops.pick_operations(None, bf16, scaled_fp8=e4m3, fp8_optimizations=True)
    lin = scaled.Linear(8, 8, bias=False)
    assert lin.weight.dtype == e4m3 and lin.fp8_matrix_mult is False     # no fp8 compute on this CPU-only host
    monkeypatch.setattr(model_management, "FORCE_FP8_COMPUTE", True)
    scaled = ops.pick_operations(None, bf16, scaled_fp8=e4m3, fp8_optimizations=True)
    lin = scaled.Linear(8, 8, bias=False)
    assert lin.fp8_matrix_mult is True and lin.scale_input is not None
    assert ops.pick_operations(e4m3, bf16, fp8_optimizations=True) is ops.fp8_ops
    assert ops.pick_operations(e4m3, bf16, fp8_optimizations=True, disable_fast_fp8=True) is ops.manual_cast


def test_cast_bias_weight_and_weight_function():
    lin = ops.manual_cast.Linear(16, 8, bias=True, dtype=torch.float32)
    with torch.no_grad():
        lin.weight.normal_()
        lin.bias.normal_()
    x = torch.randn(4, 16).bfloat16()
    w, b = ops.cast_bias_weight(lin, x)
    assert w.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    torch.testing.assert_close(lin(x), torch.nn.functional.linear(x, w, b))
    # a LoRA-style closure: applied on a copy, the stored weight stays untouched
    before = lin.weight.clone()
    lin.weight_function = [lambda t: t + 1]
    w2, _ = ops.cast_bias_weight(lin, x)
    torch.testing.assert_close(w2, w + 1)
    assert torch.equal(lin.weight, before)
    plain = ops.disable_weight_init.Linear(16, 8, bias=False, dtype=torch.float32)
    plain.weight_function = [lambda t: t * 0]
    with torch.no_grad():
        plain.weight.normal_()
    assert float(plain(torch.randn(2, 16)).abs().max()) == 0.0     # forward switches to the cast path


def test_cast_to_semantics():
    w = torch.randn(4, 4)
    assert model_management.cast_to(w, torch.float32, w.device) is w
    c = model_management.cast_to(w, torch.float32, w.device, copy=True)
    assert c is not w and torch.equal(c, w)
    assert model_management.cast_to(w, torch.bfloat16).dtype == torch.bfloat16


def test_shim_declines_ineligible_calls(golden):
    """CPU tensors, fp32 activations, LoRA closures: the shim returns None and the stock composition runs."""
    mod, x, _ = _case(golden, torch.bfloat16, ops.disable_weight_init)
    assert ops.hidream_moe_forward(mod, x) is None
    assert ops.hidream_gate(mod.gate, x) is None
    assert ops.swiglu_ffn_forward(mod.shared_experts, x) is None
    assert ops.hidream_moe_infer(mod, x.view(-1, x.shape[-1]), torch.zeros(256, dtype=torch.int64),
                                 torch.zeros(256, 1)) is None
    assert ops._linear_state(mod.experts[0].w1, x.device) is not None
    mod.experts[0].w1.weight_function = [lambda t: t]
    ops.BAKE_PATCHED_WEIGHTS = False            # patched Linears left to the stock composition
    try:
        assert ops._linear_state(mod.experts[0].w1, x.device) is None
    finally:
        ops.BAKE_PATCHED_WEIGHTS = True
    assert ops._linear_state(mod.experts[0].w1, x.device) is not None     # default: evaluated once for the kernels


def test_stochastic_rounding_is_unbiased_and_exact_on_grid():
    grid = torch.tensor([0.0, 0.5, 1.0, 1.125, -3.5, 448.0, 2.0 ** -9])
    assert torch.equal(ops.stochastic_rounding(grid, torch.float8_e4m3fn, seed=1).float(), grid)
    v = torch.full((20000,), 1.03125)     # a quarter of the way from 1.0 to 1.125
    q = ops.stochastic_rounding(v, torch.float8_e4m3fn, seed=3).float()
    assert set(q.unique().tolist()) == {1.0, 1.125}
    assert abs(float(q.mean()) - 1.03125) < 2e-3
    assert torch.equal(ops.stochastic_rounding(v, torch.float8_e4m3fn, seed=3).float(), q)


def test_ffn_hidden_rounding():
    ffn = FeedForwardSwiGLU(2560, 4 * 2560, dtype=torch.bfloat16, device="meta", operations=ops.disable_weight_init)
    assert ffn.w1.weight.shape == (6912, 2560)
    ffn = FeedForwardSwiGLU(2560, 2 * 2560, dtype=torch.bfloat16, device="meta", operations=ops.disable_weight_init)
    assert ffn.w1.weight.shape == (3584, 2560)
    g = MoEGate(64, 4, 2, dtype=torch.float32, device="cpu")
    assert g.weight.shape == (4, 64) and g.norm_topk_prob is False and g.top_k == 2


def test_block_feed_forward_stock_path_matches_reference(golden):
    """block_feed_forward with CPU tensors runs the stock composition: the reference block's lines, bit for bit."""
    from comfyui_b200.ldm.hidream.model import block_feed_forward

    mod, x, _ = _case(golden, torch.bfloat16, ops.disable_weight_init)
    b, s, dim = x.shape
    norm = ops.disable_weight_init.LayerNorm(dim, eps=1e-06, elementwise_affine=False)
    shift, scale, gate = O.make_modulation(b, dim)
    assert ops.hidream_block_ffn(norm, mod, x, shift, scale, gate) is None
    with torch.no_grad():
        out = block_feed_forward(norm, mod, x, shift, scale, gate)
        dense = block_feed_forward(norm, mod.shared_experts, x, shift, scale, gate)
    assert torch.equal(out.reshape(-1, dim).float(), torch.from_numpy(golden["block_bf16/out"]))
    assert torch.equal(dense.reshape(-1, dim).float(), torch.from_numpy(golden["block_bf16/dense_out"]))


def test_registered_torch_ops_trace_without_a_gpu():
    """The kernels are registered with torch.library; their fake implementations give shapes and dtypes on the
    meta device, so tracing a model that contains the layer needs no GPU."""
    from comfyui_b200 import torch_ops  # noqa: F401

    meta = dict(dtype=torch.bfloat16, device="meta")
    x, gate = torch.empty(64, 256, **meta), torch.empty(4, 256, **meta)
    w13, w2 = [torch.empty(768, 256, **meta)] * 5, [torch.empty(256, 768, **meta)] * 5
    out = torch.ops.comfyui_b200.hidream_moe(x, gate, w13, w13, w2, [], [], [], [], [])
    assert out.shape == x.shape and out.dtype == torch.bfloat16
    idx, w = torch.ops.comfyui_b200.hidream_gate(x, gate)
    assert idx.shape == (64, 2) and idx.dtype == torch.int64 and w.dtype == torch.float32
    mod = torch.empty(2, 256, **meta)
    blk = torch.ops.comfyui_b200.hidream_moe_block(x, mod, mod, mod, 32, 1e-6, gate, w13, w13, w2, [], [], [], [], [])
    assert blk.shape == x.shape
    schema = str(torch.ops.comfyui_b200.hidream_moe.default._schema)
    assert "Tensor[] w1" in schema and "-> Tensor" in schema


def test_patched_weights_are_evaluated_once_for_the_kernels():
    """A Linear with weight_function closures (a LoRA attached, not baked): the shim hands the kernels the patched weight
    evaluated once, re-evaluates when the closures or the weight change, and forgets it when the closures go away."""
    from comfyui_b200 import ops

    lin = ops.disable_weight_init.Linear(16, 8, bias=False, dtype=torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(8, 16))
    calls = []
    delta = torch.randn(8, 16).bfloat16()

    def lora(w):
        calls.append(1)
        return w + delta

    cpu = torch.device("cpu")
    assert ops._linear_state(lin, cpu)[0] is lin.weight or torch.equal(ops._linear_state(lin, cpu)[0], lin.weight)
    lin.weight_function = [lora]
    w1 = ops._linear_state(lin, cpu)[0]
    w2 = ops._linear_state(lin, cpu)[0]
    assert len(calls) == 1 and w1 is w2 and torch.equal(w1, lin.weight + delta)
    assert torch.equal(lin(torch.eye(16).bfloat16()), torch.nn.functional.linear(torch.eye(16).bfloat16(), w1))
    seen = len(calls)                                       # (the stock forward above evaluated the closure itself)
    lin.weight_function = [lambda w: lora(w)]               # new closures: evaluated again
    ops._linear_state(lin, cpu)
    assert len(calls) == seen + 1
    with torch.no_grad():
        lin.weight.add_(1.0)                                # the weight changed in place: evaluated again
    w3 = ops._linear_state(lin, cpu)[0]
    assert len(calls) == seen + 2 and torch.equal(w3, lin.weight + delta)
    lin.weight_function = []
    assert ops._linear_state(lin, cpu)[0] is lin.weight and "_b200_baked" not in lin.__dict__
    lin.weight_function = [lora]
    ops.BAKE_PATCHED_WEIGHTS = False
    try:
        assert ops._linear_state(lin, cpu) is None
    finally:
        ops.BAKE_PATCHED_WEIGHTS = True


def test_cache_keys_accept_inference_tensors():
    """ComfyUI runs under torch.inference_mode(): weights loaded or patched there are inference tensors, which keep no
    version counter; the shim's cache keys must not ask for one."""
    from comfyui_b200 import ops, torch_ops

    with torch.inference_mode():
        lin = ops.disable_weight_init.Linear(16, 8, bias=False, dtype=torch.bfloat16)
        lin.weight = torch.nn.Parameter(torch.randn(8, 16).bfloat16(), requires_grad=False)
        assert lin.weight.is_inference()
        state = ops._linear_state(lin, torch.device("cpu"))
        lin.weight_function = [lambda w: w * 2]
        baked = ops._linear_state(lin, torch.device("cpu"))
    assert state is not None and baked is not None and torch.equal(baked[0], lin.weight * 2)
    assert ops._tensor_key(baked[0])[1] == 0 and torch_ops._key([baked[0]])[0][1] == 0
