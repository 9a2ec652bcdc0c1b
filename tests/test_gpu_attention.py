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


@pytest.mark.parametrize("heads,head_dim,axes,s_img,s_txt,half", [
    (20, 128, [64, 32, 32], 4096, 384, False),      # HiDream-I1: 2 x (4096 image + 384 text) tokens
    (4, 64, [32, 16, 16], 31, 5, False),
    (4, 64, [16, 8, 8], 48, 16, True),               # rotary embedding on the first half of every head only
])
def test_kernel_against_oracle(cuda_device, heads, head_dim, axes, s_img, s_txt, half):
    from comfyui_b200 import ops

    dev, dim, b = cuda_device, heads * head_dim, 2
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
        # the projections as this GPU's library GEMM computes them, so that only the glue is under test
        proj = {"q": mod.to_q(img.to(dev)), "k": mod.to_k(img.to(dev)), "v": mod.to_v(img.to(dev)),
                "q_t": mod.to_q_t(txt.to(dev)), "k_t": mod.to_k_t(txt.to(dev)), "v_t": mod.to_v_t(txt.to(dev))}
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
