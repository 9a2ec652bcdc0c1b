"""Parity of the q / k / v glue kernel (RMSNorm + concatenation + rotary embedding) with the attention oracle.
Needs a B200."""
import pytest
import torch

from oracle import hidream_attention_oracle as A
from tests.test_oracle_golden_attention import setup_case

pytestmark = pytest.mark.gpu

BF16_RTOL = BF16_ATOL = 2e-2


def _module(layer, dim, heads, single, dev):
    from comfyui_b200 import ops
    from comfyui_b200.ldm.hidream import model as M

    mod = M.HiDreamAttention(query_dim=dim, heads=heads, dim_head=dim // heads,
                             processor=M.HiDreamAttnProcessor_flashattn(), single=single, dtype=torch.bfloat16,
                             device=dev, operations=ops.disable_weight_init).eval()
    mod.load_state_dict({k: v.to(dev) for k, v in layer.items()}, strict=True)
    return mod


def _close(got, want, what, same_inputs=False):
    got, want = got.float().cpu(), want.float()
    torch.testing.assert_close(got, want, rtol=BF16_RTOL, atol=BF16_ATOL, msg=lambda m: f"{what}: {m}")
    if same_inputs:
        # fed the same projected tensors the kernel follows the reference's rounding points: all but a few elements are
        # identical, the rest differ by one bf16 ulp where the fp32 sum of squares was accumulated in another order
        assert (got != want).float().mean() < 0.01, what


@pytest.mark.parametrize("single", [False, True], ids=["double", "single"])
def test_golden_fixture_on_gpu(cuda_device, golden_attention, single):
    """q, k, v where the unmodified reference hands them to its attention call, and the processor's outputs."""
    from comfyui_b200 import ops

    g = golden_attention
    layer, img, txt, freqs, heads = setup_case(g, torch.bfloat16, single)
    dev = cuda_device
    mod = _module(layer, img.shape[-1], heads, single, dev)
    tag = f"bf16/{'single' if single else 'double'}"
    with torch.no_grad():
        if single:
            seq = torch.cat([img, txt], dim=1).to(dev)
            fast = ops.hidream_qkv(mod, seq, None, freqs.to(dev))
            out = mod(seq, None, None, rope=freqs.to(dev))
            _close(out, torch.from_numpy(g[f"{tag}/out"]), "out")
        else:
            fast = ops.hidream_qkv(mod, img.to(dev), txt.to(dev), freqs.to(dev))
            out_i, out_t = mod(img.to(dev), None, txt.to(dev), rope=freqs.to(dev))
            _close(out_i, torch.from_numpy(g[f"{tag}/out_i"]), "out_i")
            _close(out_t, torch.from_numpy(g[f"{tag}/out_t"]), "out_t")
    assert fast is not None, "the call must be eligible for the kernels"
    for got, key in zip(fast, ("q", "k", "v")):
        _close(got, torch.from_numpy(g[f"{tag}/{key}"]), key)


@pytest.mark.parametrize("heads,head_dim,axes,s_img,s_txt,half,b", [
    (20, 128, [64, 32, 32], 4096, 384, False, 2),   # HiDream-I1: 2 x (4096 image + 384 text) tokens
    (4, 64, [32, 16, 16], 31, 5, False, 2),
    (4, 64, [16, 8, 8], 48, 16, True, 2),            # rotary embedding on the first half of every head only
    (4, 64, [32, 16, 16], 31, 5, False, 3),          # three batch elements: the value projections no longer fit the
                                                     # launch that writes them into place, and are copied instead
    (4, 64, [32, 16, 16], 64, 8, False, 1),
])
def test_kernel_against_oracle(cuda_device, heads, head_dim, axes, s_img, s_txt, half, b):
    from comfyui_b200 import ops

    dev, dim = cuda_device, heads * head_dim
    side = int(s_img ** 0.5)
    hh, ww = (side, s_img // side) if side * (s_img // side) == s_img else (1, s_img)
    layer = A.make_layer(dim, heads, head_dim, False, seed=3, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(4)
    img = torch.randn((b, s_img, dim), generator=g).bfloat16()
    txt = torch.randn((b, s_txt, dim), generator=g).bfloat16()
    freqs = A.rope_table(A.make_ids(b, hh, ww, s_txt), axes)
    assert freqs.shape[-3] * 2 == (head_dim // 2 if half else head_dim)
    mod = _module(layer, dim, heads, False, dev)
    with torch.no_grad():
        fast = ops.hidream_qkv(mod, img.to(dev), txt.to(dev), freqs.to(dev))
        # the projections as the shim itself computes them (one launch of the grouped GEMM), so that only the glue is
        # under test
        pairs = [(mod.to_q, img.to(dev)), (mod.to_k, img.to(dev)), (mod.to_v, img.to(dev)),
                 (mod.to_q_t, txt.to(dev)), (mod.to_k_t, txt.to(dev)), (mod.to_v_t, txt.to(dev))]
        outs = ops.grouped_projections(pairs)
        if outs is None:                                   # widths the grouped GEMM does not take: library GEMMs
            outs = [lin(t) for lin, t in pairs]
        proj = dict(zip(("q", "k", "v", "q_t", "k_t", "v_t"), outs))
    assert fast is not None
    want = A.norm_cat_rope({k: v.cpu() for k, v in proj.items()}, layer, freqs, heads)
    for got, ref, key in zip(fast, want, ("q", "k", "v")):
        assert got.shape == ref.shape
        _close(got, ref, key, same_inputs=True)
    # and end to end against the CPU oracle (projections included), within the bf16 tolerance
    for got, ref, key in zip(fast, A.qkv(layer, img, txt, freqs, heads), ("q", "k", "v")):
        _close(got, ref, key)


def test_fused_glue_timing_is_reported(cuda_device):
    """Timing at the model's size, printed for the record and not asserted (the GPU is shared; a timing is not a
    parity property): the six projections are common to both paths."""
    from comfyui_b200 import ops

    dev, heads, head_dim, b, s_img, s_txt = cuda_device, 20, 128, 2, 4096, 384
    dim = heads * head_dim
    layer = A.make_layer(dim, heads, head_dim, False, seed=5, dtype=torch.bfloat16)
    mod = _module(layer, dim, heads, False, dev)
    g = torch.Generator().manual_seed(6)
    img = torch.randn((b, s_img, dim), generator=g).bfloat16().to(dev)
    txt = torch.randn((b, s_txt, dim), generator=g).bfloat16().to(dev)
    freqs = A.rope_table(A.make_ids(b, 64, 64, s_txt), [64, 32, 32]).to(dev)

    def timed(fn, reps=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    with torch.no_grad():
        fast = timed(lambda: mod(img, None, txt, rope=freqs))
        ops.ENABLE_SM100_KERNELS = False
        try:
            stock = timed(lambda: mod(img, None, txt, rope=freqs))
        finally:
            ops.ENABLE_SM100_KERNELS = True
    print(f"HiDreamAttention forward, 2 x (4096 + 384) tokens: {fast:.3f} ms with the fused q/k/v glue, "
          f"{stock:.3f} ms as PyTorch composes it")


@pytest.mark.parametrize("rows,k,n,bias", [(8192, 2560, 2560, True), (768, 2560, 2560, True), (300, 512, 768, False),
                                           (1, 64, 256, True)])
def test_grouped_linear_against_torch(cuda_device, rows, k, n, bias):
    """Several Linears in one launch of the grouped GEMM: each output equals F.linear within the bf16 tolerance (fp32
    accumulation in another order, one rounding), ragged row counts and strided inputs included."""
    from comfyui_b200 import moe_ops as M

    dev = cuda_device
    g = torch.Generator().manual_seed(rows + n)
    xs = [torch.randn((r, k), generator=g).bfloat16().to(dev) for r in (rows, max(rows // 3, 1), rows)]
    xs[2] = torch.randn((rows, k + 64), generator=g).bfloat16().to(dev)[:, :k]          # leading dimension > width
    ws = [(torch.randn((n, k), generator=g) * 0.02).bfloat16().to(dev) for _ in xs]
    bs = [(torch.randn((n,), generator=g) * 0.1).bfloat16().to(dev) if bias else None for _ in xs]
    outs = M.grouped_linear(list(zip(xs, ws, bs)))
    M.read_status(M.device_status(dev))
    for x, w, b, out in zip(xs, ws, bs, outs):
        ref = torch.nn.functional.linear(x.float(), w.float(), None if b is None else b.float())
        torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
        assert float((out.float() - ref).norm() / ref.norm()) < 3e-3


def test_grouped_linear_shares_maps_and_refuses_too_many(cuda_device):
    """Nine groups over one x need 19 tensor maps and run; nine groups with nothing in common would need 27 (the
    parameter block holds 22) and are refused before anything is launched."""
    from comfyui_b200 import _native as N, moe_ops as M

    dev = cuda_device
    g = torch.Generator().manual_seed(9)
    x = torch.randn((200, 128), generator=g).bfloat16().to(dev)
    ws = [(torch.randn((256, 128), generator=g) * 0.05).bfloat16().to(dev) for _ in range(9)]
    outs = M.grouped_linear([(x, w, None) for w in ws])
    M.read_status(M.device_status(dev))
    for w, out in zip(ws, outs):
        torch.testing.assert_close(out.float(), torch.nn.functional.linear(x.float(), w.float()), rtol=2e-2, atol=2e-2)
    xs = [torch.randn((200, 128), generator=g).bfloat16().to(dev) for _ in range(9)]
    with pytest.raises(N.MoeError) as err:
        M.grouped_linear([(xi, w, None) for xi, w in zip(xs, ws)])
    assert err.value.code == N.EUNSUPPORTED
    torch.cuda.synchronize()


def test_attention_projections_take_the_grouped_gemm(cuda_device, monkeypatch):
    """On an eligible call the six q / k / v projections and the two output projections run as two grouped launches."""
    from comfyui_b200 import moe_ops as M

    dev, heads, head_dim, b, s_img, s_txt = cuda_device, 4, 128, 2, 256, 32
    dim = heads * head_dim
    layer = A.make_layer(dim, heads, head_dim, False, seed=5, dtype=torch.bfloat16)
    mod = _module(layer, dim, heads, False, dev)
    g = torch.Generator().manual_seed(6)
    img = torch.randn((b, s_img, dim), generator=g).bfloat16()
    txt = torch.randn((b, s_txt, dim), generator=g).bfloat16()
    freqs = A.rope_table(A.make_ids(b, 16, 16, s_txt), [64, 32, 32])
    calls = []
    stock = M.grouped_linear
    monkeypatch.setattr(M, "grouped_linear", lambda groups, outs=None, status=None: calls.append(len(groups)) or stock(groups, outs, status))
    with torch.no_grad():
        got_i, got_t = mod(img.to(dev), None, txt.to(dev), rope=freqs.to(dev))
    # q and k of image and text tokens, their v per batch element (written straight into the joint v buffer's rows);
    # out projections per batch element
    assert calls == [8, 4]
    want_i, want_t = A.processor(layer, img, txt, freqs, heads)
    torch.testing.assert_close(got_i.float().cpu(), want_i.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(got_t.float().cpu(), want_t.float(), rtol=2e-2, atol=2e-2)


ATTN_SHAPES = [(1, 128, 128, 1), (1, 128, 256, 1), (2, 300, 333, 3), (1, 1000, 77, 2), (1, 1024, 1024, 4),
               (2, 4480, 4480, 20), (1, 4864, 4864, 20)]


@pytest.mark.parametrize("b,sq,skv,h", ATTN_SHAPES)
def test_attention_kernel_against_fp32_softmax(cuda_device, b, sq, skv, h):
    """softmax(q k^T / sqrt(d)) v on the tcgen05 kernel against the same in fp32: bf16 tolerance, and no further from
    the fp32 result than PyTorch's own bf16 attention on this GPU is (plus a margin of one bf16 ulp of the output)."""
    from comfyui_b200 import moe_ops as M

    dev = cuda_device
    g = torch.Generator().manual_seed(b + sq + skv + h)
    q = torch.randn((b, sq, h, 128), generator=g).bfloat16().to(dev)
    k = torch.randn((b, skv, h, 128), generator=g).bfloat16().to(dev)
    v = torch.randn((b, skv, h, 128), generator=g).bfloat16().to(dev)
    out = M.attention_forward(q, k, v)
    M.read_status(M.device_status(dev))

    def sdpa(q, k, v):
        o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        return o.transpose(1, 2).reshape(q.shape[0], q.shape[1], -1)

    want = sdpa(q.float(), k.float(), v.float())
    lib = sdpa(q, k, v).float()
    assert out.shape == (b, sq, h * 128) and not torch.isnan(out.float()).any()
    torch.testing.assert_close(out.float(), want, rtol=BF16_RTOL, atol=BF16_ATOL)
    err, err_lib = (out.float() - want).abs().max(), (lib - want).abs().max()
    rel = (out.float() - want).norm() / want.norm()
    assert rel < 4e-3 and float(err) <= 2 * float(err_lib) + 4e-3, (float(err), float(err_lib), float(rel))


def test_attention_kernel_with_peaked_scores(cuda_device):
    """Scores far apart (one key dominates a row, and the dominant key arrives late in the sequence): the reference
    maximum has to be raised and the accumulator rescaled on a late step."""
    from comfyui_b200 import moe_ops as M

    dev = cuda_device
    g = torch.Generator().manual_seed(3)
    b, s, h = 1, 640, 2
    q = torch.randn((b, s, h, 128), generator=g).bfloat16()
    k = torch.randn((b, s, h, 128), generator=g).bfloat16()
    v = torch.randn((b, s, h, 128), generator=g).bfloat16()
    k[:, 600] = q[:, 5] * 3.0                       # query 5 matches key 600 very strongly (score ~ 3 * |q|^2 / sqrt(d))
    k[:, 300] = q[:, 9] * 1.5
    q, k, v = q.to(dev), k.to(dev), v.to(dev)
    out = M.attention_forward(q, k, v).float()
    M.read_status(M.device_status(dev))
    o = torch.nn.functional.scaled_dot_product_attention(q.float().transpose(1, 2), k.float().transpose(1, 2),
                                                         v.float().transpose(1, 2))
    want = o.transpose(1, 2).reshape(b, s, -1)
    torch.testing.assert_close(out, want, rtol=BF16_RTOL, atol=BF16_ATOL)
    torch.testing.assert_close(out[:, 5, :128], v[:, 600, 0].float(), rtol=BF16_RTOL, atol=BF16_ATOL)


def test_blocks_use_the_attention_kernel(cuda_device, monkeypatch):
    """The attention call of a HiDream block goes through the kernel on an eligible call and through PyTorch's attention
    when switched to the library; both agree within the bf16 tolerance."""
    from comfyui_b200 import moe_ops as M, ops

    dev, heads, head_dim, b, s_img, s_txt = cuda_device, 4, 128, 2, 256, 32
    dim = heads * head_dim
    layer = A.make_layer(dim, heads, head_dim, False, seed=5, dtype=torch.bfloat16)
    mod = _module(layer, dim, heads, False, dev)
    g = torch.Generator().manual_seed(6)
    img = torch.randn((b, s_img, dim), generator=g).bfloat16().to(dev)
    txt = torch.randn((b, s_txt, dim), generator=g).bfloat16().to(dev)
    freqs = A.rope_table(A.make_ids(b, 16, 16, s_txt), [64, 32, 32]).to(dev)
    calls = []
    stock = M.attention_forward
    monkeypatch.setattr(M, "attention_forward", lambda *a, **k: calls.append(1) or stock(*a, **k))
    with torch.no_grad():
        fast_i, fast_t = mod(img, None, txt, rope=freqs)
        assert calls == [1]
        monkeypatch.setattr(ops, "ATTENTION_BACKEND", "library")
        lib_i, lib_t = mod(img, None, txt, rope=freqs)
        assert calls == [1]
    torch.testing.assert_close(fast_i.float(), lib_i.float(), rtol=BF16_RTOL, atol=BF16_ATOL)
    torch.testing.assert_close(fast_t.float(), lib_t.float(), rtol=BF16_RTOL, atol=BF16_ATOL)
