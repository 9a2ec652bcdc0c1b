"""One denoising step of the reduced HiDream-I1 transformer on the kernels against the unmodified reference's output
(tests/golden/hidream_model_small.npz, the case whose MoE gates run on the fp32 copy of their input).  Needs a B200."""
import pytest
import torch

from oracle import hidream_model_recipe as R
from tests.test_model_cpu import build, gate_on_fp32_copy, golden_model  # noqa: F401

pytestmark = pytest.mark.gpu


def _stats(got, want):
    err = (got - want).abs()
    return (float((got - want).norm() / want.norm()), float((err > 2e-2 + 2e-2 * want.abs()).float().mean()),
            float(err.max()))


def test_step_on_kernels_matches_reference(cuda_device, golden_model, monkeypatch):  # noqa: F811
    """A step is 4 blocks deep, every one a chain of a dozen bf16 operations, and a token the fp32 gate sends to other
    experts on the GPU than on the CPU (a near-tie met with a one-ulp different LayerNorm output) changes that token by
    O(1) and, through the later blocks' attention, every other token a little.  So the bar for the whole step is
    statistical and is stated next to what PyTorch's own CUDA composition of the same modules reaches against the same
    golden output: rel-RMS below 1e-2, and not worse than 1.5 x the stock composition's + 2e-3."""
    from comfyui_b200 import ops

    dev = cuda_device
    m, _ = build(torch.bfloat16, dev)
    inputs = [t.to(dev) for t in R.make_inputs(torch.bfloat16)]
    want = torch.from_numpy(golden_model["bf16_fp32gate/out"])
    taken = []
    stock_ffn = ops.hidream_block_ffn
    monkeypatch.setattr(ops, "hidream_block_ffn", lambda *a, **k: taken.append(stock_ffn(*a, **k)) or taken[-1])
    with torch.no_grad():
        got = m(*inputs).float().cpu()
    assert len(taken) == 6 and all(t is not None for t in taken)        # 2 x (image + text) + 2 single-stream blocks
    ops.ENABLE_SM100_KERNELS = False
    gate_on_fp32_copy(monkeypatch)
    try:
        with torch.no_grad():
            stock = m(*inputs).float().cpu()
    finally:
        ops.ENABLE_SM100_KERNELS = True
    rel, frac, worst = _stats(got, want)
    rel_s, frac_s, worst_s = _stats(stock, want)
    print(f"denoising step vs the reference's output: kernels rel-RMS {rel:.3e}, {frac:.2e} of the elements outside "
          f"2e-2, worst {worst:.3f}; stock CUDA composition {rel_s:.3e}, {frac_s:.2e}, {worst_s:.3f}; "
          f"kernels vs stock {_stats(got, stock)[0]:.3e}")
    assert got.shape == want.shape and not torch.isnan(got).any()
    assert rel < 1e-2 and rel < 1.5 * rel_s + 2e-3
    assert frac < 5e-3 + 2 * frac_s


def test_step_replays_from_a_cuda_graph(cuda_device):
    """The whole model call makes no host synchronisation and allocates only through the caching allocator, so it can be
    captured once and replayed: the replay gives the bytes of the eager call, and a second replay on other inputs
    (copied into the captured tensors) the bytes of an eager call on those."""
    dev = cuda_device
    m, _ = build(torch.bfloat16, dev)
    inputs = [t.to(dev) for t in R.make_inputs(torch.bfloat16)]
    with torch.inference_mode():
        eager = m(*inputs).clone()
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            m(*inputs)                                  # workspaces and packs exist before the capture
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=side):
                captured = m(*inputs)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(captured, eager)
        inputs[0].copy_(inputs[0].flip(0))              # other latents in the same tensors
        graph.replay()
        torch.cuda.synchronize()
        again = captured.clone()
        assert torch.equal(again, m(*inputs))
    from comfyui_b200 import ops

    ops.check_device_status()
