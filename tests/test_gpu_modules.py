"""The drop-in modules on a B200: the call a HiDream block makes, routed to the kernels by the shim."""
import pytest
import torch

from oracle import hidream_moe_oracle as O

pytestmark = pytest.mark.gpu


def _module(dev, dim, hidden_dim, operations, layer):
    from comfyui_b200.ldm.hidream.model import MOEFeedForwardSwiGLU

    mod = MOEFeedForwardSwiGLU(dim, hidden_dim, 4, 2, dtype=torch.bfloat16, device=dev, operations=operations).eval()
    mod.load_state_dict({k: v.to(dev) for k, v in layer.items()}, strict=True)
    return mod


def test_module_forward_uses_kernels_and_matches_oracle(cuda_device):
    from comfyui_b200 import _native, ops

    dev = cuda_device
    dim, hidden_dim, b, s = 512, 2048, 2, 224 + 3
    layer = {k: v.bfloat16() for k, v in O.make_layer(dim, hidden_dim, 4, seed=0).items()}
    x = O.make_input(b * s, dim, seed=1).bfloat16()
    mod = _module(dev, dim, hidden_dim, ops.disable_weight_init, layer)
    xd = x.to(dev).view(b, s, dim)
    assert _native._lib is not None or _native.load() is not None
    with torch.inference_mode():
        assert ops._layer_pack(mod, xd) is not None
        out = mod(xd)
        idx, w, aux = mod.gate(xd)
    assert out.shape == xd.shape and out.dtype == torch.bfloat16 and aux is None
    assert idx.dtype == torch.int64 and w.dtype == torch.bfloat16 and idx.shape == (b * s, 2)
    ref, ridx, rw = O.moe_layer(x, layer, gate_in_fp32=True)
    assert torch.equal(idx.cpu().sort(dim=1).values, ridx.sort(dim=1).values)
    torch.testing.assert_close(out.view(-1, dim).cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)

    # moe_infer with caller-supplied routing (routed part only), and the dense shared expert alone
    with torch.inference_mode():
        routed = mod.moe_infer(xd.view(-1, dim), ridx.to(dev).view(-1), rw.to(dev).view(-1, 1))
        shared = mod.shared_experts(xd)
    ref_routed = O.moe_infer(x, ridx.reshape(-1), rw.reshape(-1, 1), layer)
    torch.testing.assert_close(routed.cpu().float(), ref_routed.float(), rtol=2e-2, atol=2e-2)
    ref_shared = O.swiglu_ffn(x, layer, "shared_experts")
    torch.testing.assert_close(shared.view(-1, dim).cpu().float(), ref_shared.float(), rtol=2e-2, atol=2e-2)


def test_weight_replacement_is_picked_up(cuda_device):
    """A model patcher may replace a Parameter object or update it in place; the cached pack must follow."""
    from comfyui_b200 import ops

    dev = cuda_device
    dim, hidden_dim, n = 256, 1024, 200
    layer = {k: v.bfloat16() for k, v in O.make_layer(dim, hidden_dim, 4, seed=0).items()}
    x = O.make_input(n, dim, seed=1).bfloat16()
    mod = _module(dev, dim, hidden_dim, ops.disable_weight_init, layer)
    xd = x.to(dev).view(1, n, dim)
    with torch.inference_mode():
        first = mod(xd).clone()
    # replace one Parameter object (set_attr_param style) and update another in place (copy_to_param style)
    layer2 = dict(layer)
    layer2["experts.1.w2.weight"] = layer["experts.1.w2.weight"] * 2
    layer2["shared_experts.w1.weight"] = layer["shared_experts.w1.weight"] * 0.5
    mod.experts[1].w2.weight = torch.nn.Parameter(layer2["experts.1.w2.weight"].to(dev), requires_grad=False)
    with torch.no_grad():
        mod.shared_experts.w1.weight.data.copy_(layer2["shared_experts.w1.weight"].to(dev))
    with torch.inference_mode():
        second = mod(xd)
    assert not torch.equal(first, second)
    ref, _, _ = O.moe_layer(x, layer2, gate_in_fp32=True)
    torch.testing.assert_close(second.view(-1, dim).cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)


def test_ineligible_calls_run_the_stock_composition(cuda_device, monkeypatch):
    """A bias closure on a Linear, patched weights with baking switched off, or fp32 activations: the module still
    answers, through PyTorch, like the reference."""
    from comfyui_b200 import ops

    dev = cuda_device
    dim, hidden_dim, n = 256, 1024, 64
    layer = {k: v.bfloat16() for k, v in O.make_layer(dim, hidden_dim, 4, seed=0).items()}
    x = O.make_input(n, dim, seed=1).bfloat16()
    mod = _module(dev, dim, hidden_dim, ops.disable_weight_init, layer)
    xd = x.to(dev).view(1, n, dim)
    mod.experts[0].w1.weight_function = [lambda w: w * 1.0]
    assert ops._layer_pack(mod, xd) is not None             # patched weights are evaluated once for the kernels ...
    monkeypatch.setattr(ops, "BAKE_PATCHED_WEIGHTS", False)
    assert ops._layer_pack(mod, xd) is None                 # ... unless that is switched off
    assert ops._layer_pack(mod, xd.float()) is None
    with torch.inference_mode():
        out = mod(xd)
    ref, _, _ = O.moe_layer(x, layer, gate_in_fp32=True)
    assert out.shape == xd.shape
    assert float((out.view(-1, dim).cpu().float() - ref.float()).abs().mean()) < 2e-2


def test_scaled_fp8_module(cuda_device):
    from comfyui_b200 import ops

    dev = cuda_device
    dim, hidden_dim, n = 512, 2048, 300
    layer = O.quantize_layer_fp8({k: v.bfloat16() for k, v in O.make_layer(dim, hidden_dim, 4, seed=0).items()})
    x = O.make_input(n, dim, seed=1).bfloat16()
    operations = ops.scaled_fp8_ops(fp8_matrix_mult=True, scale_input=False, override_dtype=torch.float8_e4m3fn)
    mod = _module(dev, dim, hidden_dim, operations, layer)
    xd = x.to(dev).view(1, n, dim)
    with torch.inference_mode():
        assert ops._layer_pack(mod, xd) is not None and ops._layer_pack(mod, xd).fp8
        out = mod(xd).view(-1, dim).cpu()
        idx, w, _ = mod.gate(xd)
    ref, _, _ = O.moe_layer(x, layer, mode=O.FP8_MATMUL, routing=(idx.cpu(), w.cpu()))
    rel = float((out.float() - ref.float()).norm() / ref.float().norm())
    assert rel < 1e-2, rel
    # the dequantising flavour (fp8_matrix_mult=False) is not what the kernels compute: stock path
    operations = ops.scaled_fp8_ops(fp8_matrix_mult=False, scale_input=False, override_dtype=torch.float8_e4m3fn)
    mod2 = _module(dev, dim, hidden_dim, operations, layer)
    assert ops._layer_pack(mod2, xd) is None


@pytest.mark.parametrize("scale_input", [None, 0.75])
def test_scaled_fp8_dense_ffn(cuda_device, scale_input):
    """The shared expert of a scaled-fp8 module called on its own (what a block's text feed-forward is): the input is
    quantised by the stand-alone quantiser, then one group of the fp8 GEMM."""
    from comfyui_b200 import ops

    dev = cuda_device
    dim, hidden_dim, n = 512, 2048, 300
    layer = O.quantize_layer_fp8({k: v.bfloat16() for k, v in O.make_layer(dim, hidden_dim, 4, seed=0).items()},
                                 scale_input=scale_input)
    x = O.make_input(n, dim, seed=1).bfloat16()
    operations = ops.scaled_fp8_ops(fp8_matrix_mult=True, scale_input=scale_input is not None,
                                    override_dtype=torch.float8_e4m3fn)
    mod = _module(dev, dim, hidden_dim, operations, layer)
    xd = x.to(dev).view(1, n, dim)
    with torch.inference_mode():
        fast = ops.swiglu_ffn_forward(mod.shared_experts, xd)
        assert fast is not None
        out = mod.shared_experts(xd).view(-1, dim).cpu()
    ref = O.swiglu_ffn(x.clone(), layer, "shared_experts", O.FP8_MATMUL)
    rel = float((out.float() - ref.float()).norm() / ref.float().norm())
    assert rel < 1e-2, rel


def test_device_status_word_is_reported(cuda_device):
    """Failure reporting without provoking a failure: the kernels write a code to the status word when a bounded
    wait gives up; here the word is set from the host and the host-side plumbing must turn it into an error."""
    from comfyui_b200 import _native as N
    from comfyui_b200 import moe_ops as M

    status = torch.zeros((2,), dtype=torch.int32, device=cuda_device)
    M.read_status(status)                                   # clean word: no error
    status[0] = 2                                           # the code the MMA role would leave
    with pytest.raises(N.MoeError) as err:
        M.read_status(status)
    assert err.value.code == N.ETIMEOUT and "status word = 2" in str(err.value)


@pytest.mark.parametrize("b,s,dim", [(2, 64, 256), (1, 333, 512), (2, 4096, 2560), (3, 7, 2560)])
def test_ln_modulate_and_gate_residual(cuda_device, b, s, dim):
    """The element-wise passes around the feed-forward against the PyTorch composition of the reference block."""
    from comfyui_b200 import moe_ops as M

    dev = cuda_device
    x = O.make_input(b * s, dim, seed=b + s).bfloat16().view(b, s, dim)
    shift, scale, gate = O.make_modulation(b, dim, seed=5)
    ref = torch.nn.functional.layer_norm(x, (dim,), None, None, 1e-6) * (1 + scale) + shift
    got = M.ln_modulate(x.view(-1, dim).to(dev), shift.to(dev)[:, 0], scale.to(dev)[:, 0], s).cpu().view(b, s, dim)
    diff = (got.float() - ref.float()).abs()
    # fp32 statistics in a different summation order: at most one bf16 ulp, on a small fraction of the elements
    assert float((diff > 0).float().mean()) < 0.02
    # (a one-ulp step of the product can be large relative to a sum that nearly cancels: absolute bound)
    torch.testing.assert_close(got.float(), ref.float(), rtol=2e-2, atol=2e-2)
    y = O.make_input(b * s, dim, seed=77).bfloat16().view(b, s, dim)
    ref2 = gate * y + x
    got2 = M.gate_residual(y.view(-1, dim).to(dev), gate.to(dev)[:, 0], x.view(-1, dim).to(dev), s).cpu().view(b, s, dim)
    assert torch.equal(got2, ref2)


@pytest.mark.parametrize("b,s,dim,e,w32", [(2, 4096, 2560, 4, False), (1, 4480, 2560, 4, False), (2, 300, 512, 4, True),
                                          (3, 33, 256, 8, False), (1, 1, 256, 2, False), (2, 129, 1024, 4, False)])
def test_gate_fused_into_the_layernorm_pass(cuda_device, b, s, dim, e, w32):
    """LayerNorm + modulation + gate in one pass: every output is bit-identical to the two separate kernels."""
    from comfyui_b200 import moe_ops as M

    dev = cuda_device
    x = O.make_input(b * s, dim, seed=b + s + 3).bfloat16().to(dev)
    shift, scale, _ = O.make_modulation(b, dim, seed=6)
    shift, scale = shift.to(dev)[:, 0], scale.to(dev)[:, 0]
    g = torch.Generator().manual_seed(e)
    w_gate = (torch.randn((e, dim), generator=g) * 0.02).to(torch.float32 if w32 else torch.bfloat16).to(dev)
    x_mod = M.ln_modulate(x, shift, scale, s)
    idx, w, counts, ties, flags = M.gate_topk(x_mod, w_gate, want_flags=True)
    f_mod, f_idx, f_w, f_counts, f_ties, f_flags = M.ln_modulate_gate(x, shift, scale, s, w_gate, want_flags=True)
    assert torch.equal(f_mod, x_mod)
    assert torch.equal(f_idx, idx) and torch.equal(f_w, w)
    assert torch.equal(f_counts, counts) and int(f_ties) == int(ties) and torch.equal(f_flags, flags)
    assert int(f_counts.sum()) == 2 * b * s


def test_gate_and_layernorm_timings_are_reported(cuda_device):
    """Device time of the gate, the LayerNorm + modulation pass, the two in a row and the fused pass at the bench size,
    printed for the record (run with -s) and not asserted: the GPU is shared, a timing is not a pass criterion.  Cold:
    a 512 MB buffer is zeroed in front of every launch; hot: 50 launches queued behind a long kernel, so that the
    events see device time and not the host's launch rate."""
    from comfyui_b200 import moe_ops as M

    dev = cuda_device
    n, d, e = 8192, 2560, 4
    x = O.make_input(n, d, seed=1).bfloat16().to(dev)
    g = torch.Generator().manual_seed(e)
    w_gate = (torch.randn((e, d), generator=g) * 0.02).bfloat16().to(dev)
    shift, scale, _ = O.make_modulation(2, d, seed=6)
    shift, scale = shift.to(dev)[:, 0], scale.to(dev)[:, 0]
    out = torch.empty_like(x)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    big = torch.randn((8192, 8192), device=dev, dtype=torch.bfloat16)

    def cold(fn, reps=20):
        for _ in range(3):
            fn()
        total = 0.0
        for _ in range(reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / reps * 1e3

    def hot(fn, reps=50):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        for _ in range(6):
            big @ big
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3

    cases = {
        "gate": lambda: M.gate_topk(x, w_gate),
        "layernorm + modulation": lambda: M.ln_modulate(x, shift, scale, n // 2, out=out),
        "the two in a row": lambda: (M.ln_modulate(x, shift, scale, n // 2, out=out), M.gate_topk(out, w_gate)),
        "fused pass": lambda: M.ln_modulate_gate(x, shift, scale, n // 2, w_gate),
    }
    for name, fn in cases.items():
        print(f"{name:24s} cold {cold(fn):6.1f} us   hot {hot(fn):6.1f} us")


def test_block_feed_forward_on_kernels(cuda_device, golden):
    """block_feed_forward on the GPU: fused LayerNorm/modulation, MoE, gate/residual epilogue in the combine."""
    from comfyui_b200 import ops
    from comfyui_b200.ldm.hidream.model import block_feed_forward

    dev = cuda_device
    dim, hidden_dim, b, s = 512, 2048, 2, 300
    layer = {k: v.bfloat16() for k, v in O.make_layer(dim, hidden_dim, 4, seed=0).items()}
    x = O.make_input(b * s, dim, seed=1).bfloat16().view(b, s, dim)
    shift, scale, gate = O.make_modulation(b, dim, seed=9)
    mod = _module(dev, dim, hidden_dim, ops.disable_weight_init, layer)
    norm = ops.disable_weight_init.LayerNorm(dim, eps=1e-06, elementwise_affine=False)
    ada = torch.cat([shift, scale, gate], dim=-1).to(dev)             # one tensor, chunked like the block does
    shift_d, scale_d, gate_d = ada.chunk(3, dim=-1)
    xd = x.to(dev)
    with torch.inference_mode():
        assert ops.hidream_block_ffn(norm, mod, xd, shift_d, scale_d, gate_d) is not None
        out = block_feed_forward(norm, mod, xd, shift_d, scale_d, gate_d).cpu()
        dense = block_feed_forward(norm, mod.shared_experts, xd, shift_d, scale_d, gate_d).cpu()
    ref = O.block_ffn(x, layer, shift, scale, gate, gate_in_fp32=True)
    close = (out.float() - ref.float()).abs() <= 2e-2 + 2e-2 * ref.float().abs()
    # a token whose LayerNorm output differs by one bf16 ulp can be re-routed; allow a handful of such rows
    bad_rows = (~close).any(dim=-1).sum()
    assert int(bad_rows) <= 3, int(bad_rows)
    ref_dense = O.block_ffn(x, layer, shift, scale, gate, dense_prefix="shared_experts")
    torch.testing.assert_close(dense.float(), ref_dense.float(), rtol=2e-2, atol=2e-2)

    # the golden fixture of the reference block lines (as-shipped bf16 gate there, fp32 gate here: compare rows
    # that are not re-routed)
    m = golden["meta"]
    gdim, gb, gs = int(m["dim"]), int(m["batch"]), int(m["seq"])
    glayer = {k: v.bfloat16() for k, v in O.make_layer(gdim, int(m["hidden_dim"]), 4, int(m["w_seed"])).items()}
    gx = O.make_input(gb * gs, gdim, int(m["x_seed"])).bfloat16().view(gb, gs, gdim)
    gshift, gscale, ggate = O.make_modulation(gb, gdim)
    gmod = _module(dev, gdim, int(m["hidden_dim"]), ops.disable_weight_init, glayer)
    gnorm = ops.disable_weight_init.LayerNorm(gdim, eps=1e-06, elementwise_affine=False)
    gada = torch.cat([gshift, gscale, ggate], dim=-1).to(dev)
    with torch.inference_mode():
        gout = block_feed_forward(gnorm, gmod, gx.to(dev), *gada.chunk(3, dim=-1)).cpu().view(-1, gdim)
    gref = torch.from_numpy(golden["block_bf16/out"])
    close = (gout.float() - gref).abs() <= 2e-2 + 2e-2 * gref.abs()
    assert int((~close).any(dim=-1).sum()) <= 3


def test_layer_call_replays_from_a_cuda_graph(cuda_device):
    """The layer makes no host synchronisation and, once its workspace exists, no allocation of its own, so a
    sampler can record the call into a CUDA graph and replay it with new inputs."""
    from comfyui_b200 import ops

    dev = cuda_device
    dim, hidden_dim, n = 512, 2048, 640
    layer = {k: v.bfloat16() for k, v in O.make_layer(dim, hidden_dim, 4, seed=0).items()}
    mod = _module(dev, dim, hidden_dim, ops.disable_weight_init, layer)
    x_static = O.make_input(n, dim, seed=1).bfloat16().to(dev).view(1, n, dim)
    side = torch.cuda.Stream(device=dev)
    with torch.inference_mode():
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):          # warm-up on the capture stream: workspace, function attributes
            for _ in range(2):
                mod(x_static)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            y_static = mod(x_static)
        for seed in (7, 8):
            x_new = O.make_input(n, dim, seed=seed).bfloat16().to(dev).view(1, n, dim)
            x_static.copy_(x_new)
            graph.replay()
            torch.cuda.synchronize()
            eager = mod(x_new)
            assert torch.equal(y_static, eager)
    ops.release_workspaces()


def test_unscaled_fp8_ops_module(cuda_device):
    """comfy.ops.fp8_ops: e4m3 weights without scales (scale_weight = scale_input = None), fp8 matmul."""
    from comfyui_b200 import ops

    dev = cuda_device
    dim, hidden_dim, n = 256, 1024, 200
    layer = {k: v.bfloat16() for k, v in O.make_layer(dim, hidden_dim, 4, seed=0, std=0.5).items()}
    layer = {k: (v.to(torch.float8_e4m3fn) if k != "gate.weight" else v) for k, v in layer.items()}
    x = (O.make_input(n, dim, seed=1) * 0.1).bfloat16()
    from comfyui_b200.ldm.hidream.model import MOEFeedForwardSwiGLU

    mod = MOEFeedForwardSwiGLU(dim, hidden_dim, 4, 2, dtype=torch.float8_e4m3fn, device=dev, operations=ops.fp8_ops).eval()
    mod.gate.weight = torch.nn.Parameter(layer["gate.weight"].to(dev), requires_grad=False)
    mod.load_state_dict({k: v.to(dev) for k, v in layer.items()}, strict=True)
    xd = x.to(dev).view(1, n, dim)
    with torch.inference_mode():
        pack = ops._layer_pack(mod, xd)
        assert pack is not None and pack.fp8 and pack.experts[0].scale_w1 is None
        out = mod(xd).view(-1, dim).cpu()
        idx, w, _ = mod.gate(xd)
    ref, _, _ = O.moe_layer(x, layer, mode=O.FP8_MATMUL, routing=(idx.cpu(), w.cpu()))
    rel = float((out.float() - ref.float()).norm() / ref.float().norm())
    assert rel < 1e-2, rel


def test_quantize_e4m3_matches_reference_cast(cuda_device):
    """The stand-alone activation quantiser: clamp + cast of comfy/ops.py:338-340, and the scale_input form of :342-343."""
    from comfyui_b200 import moe_ops as M

    g = torch.Generator().manual_seed(5)
    x = (torch.randn((257, 512), generator=g) * 40).bfloat16()
    x[0, :8] = torch.tensor([448., 449., 464., 1000., -1000., 2.0 ** -10, 0.001, -0.0]).bfloat16()
    got = M.quantize_e4m3(x.to(cuda_device)).cpu()
    want = torch.clamp(x, min=-448, max=448).to(torch.float8_e4m3fn)
    assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
    scale = torch.tensor(0.75, dtype=torch.float32)
    got = M.quantize_e4m3(x.to(cuda_device), scale.to(cuda_device)).cpu()
    inv = (1.0 / scale).to(torch.bfloat16)
    want = (x * inv).to(torch.float8_e4m3fn)        # no clamp in this branch of the reference: overflow becomes NaN
    assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
    assert int((want.view(torch.uint8) & 0x7f == 0x7f).sum()) >= 4


def test_lora_closures_reach_the_kernels(cuda_device):
    """Experts whose Linears carry weight_function closures (a LoRA attached by a patcher) still take the kernels: the
    patched weights are evaluated once; the result matches the stock composition, which evaluates them on every call."""
    from comfyui_b200 import ops

    dev = cuda_device
    dim, hidden_dim = 512, 2048
    layer = {k: v.bfloat16() for k, v in O.make_layer(dim, hidden_dim, 4, seed=0).items()}
    mod = _module(dev, dim, hidden_dim, ops.disable_weight_init, layer)
    g = torch.Generator().manual_seed(3)
    count = [0]
    for ffn in list(mod.experts) + [mod.shared_experts]:
        for lin in (ffn.w1, ffn.w2, ffn.w3):
            a = (torch.randn((lin.weight.shape[0], 8), generator=g) * 0.05).bfloat16().to(dev)
            b = (torch.randn((8, lin.weight.shape[1]), generator=g) * 0.05).bfloat16().to(dev)

            def patch(w, a=a, b=b):
                count[0] += 1
                return w + (a @ b)

            lin.weight_function = [patch]
    x = O.make_input(300, dim, seed=1).bfloat16().to(dev).view(1, 300, dim)
    with torch.inference_mode():
        assert ops._layer_pack(mod, x) is not None, "patched experts must stay eligible"
        evaluated = count[0]
        assert evaluated == 15
        fast = mod(x)
        fast2 = mod(x)
        assert count[0] == evaluated and torch.equal(fast, fast2)          # no re-evaluation on later calls
        ops.ENABLE_SM100_KERNELS = False
        try:
            stock = mod(x)
        finally:
            ops.ENABLE_SM100_KERNELS = True
    assert count[0] > evaluated                                              # the stock path evaluates per call
    idx_fast = ops.hidream_gate(mod.gate, x)[0]
    same = torch.ones(300, dtype=torch.bool)
    with torch.inference_mode():
        ops.ENABLE_SM100_KERNELS = False
        try:
            idx_stock = mod.gate(x)[0]
        finally:
            ops.ENABLE_SM100_KERNELS = True
    same = (idx_fast.sort(dim=1).values == idx_stock.view(-1, 2).sort(dim=1).values).all(dim=1).cpu()
    torch.testing.assert_close(fast.view(-1, dim)[same].float().cpu(), stock.view(-1, dim)[same].float().cpu(),
                               rtol=2e-2, atol=2e-2)
