"""The stochastic-rounding kernel against the reference's chain of fp16 tensor operations run on the same GPU with the
same generator: the bytes must be identical.  Needs a B200."""
import pytest
import torch

from tests.golden.make_golden import rounding_input

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("seed", [0, 7])
def test_kernel_equals_the_composition(cuda_device, dtype, seed):
    from comfyui_b200 import ops

    v = rounding_input(torch.float32).to(dtype).to(cuda_device)
    fast = ops.stochastic_rounding(v, torch.float8_e4m3fn, seed=seed)
    ops.ENABLE_SM100_KERNELS = False
    try:
        stock = ops.stochastic_rounding(v, torch.float8_e4m3fn, seed=seed)
    finally:
        ops.ENABLE_SM100_KERNELS = True
    assert torch.equal(fast.view(torch.uint8), stock.view(torch.uint8))


def test_values_next_to_powers_of_two_and_every_fp16_exponent(cuda_device):
    """The reference takes floor(log2 |x|) of an fp16-rounded logarithm, which picks the exponent one too high just
    below a power of two; the kernel has to make the same choice.  All fp16 bit patterns are run through both."""
    from comfyui_b200 import moe_ops as M, ops

    bits = torch.arange(0, 65536, dtype=torch.int32).to(torch.int16)
    x = bits.view(torch.float16).to(cuda_device)
    x = x[~torch.isnan(x)].contiguous()
    g = torch.Generator(device=cuda_device)
    for seed in (1, 2):
        g.manual_seed(seed)
        rand = torch.rand(x.size(), dtype=torch.float16, device=cuda_device, generator=g)
        fast = M.stochastic_round_e4m3(x, rand)
        g.manual_seed(seed)
        stock = ops._stochastic_round_fp8_slice(x, torch.float8_e4m3fn, g).to(torch.float8_e4m3fn)
        same = fast.view(torch.uint8) == stock.view(torch.uint8)
        assert bool(same.all()), f"{int((~same).sum())} of {same.numel()} fp16 values round differently"


def test_set_weight_on_the_device(cuda_device):
    """A weight as large as one expert matrix: sliced like the reference (about 4096 x 4096 elements per slice), unbiased."""
    from comfyui_b200 import ops

    operations = ops.scaled_fp8_ops(fp8_matrix_mult=True, scale_input=False, override_dtype=torch.float8_e4m3fn)
    lin = operations.Linear(2560, 6912, bias=False, dtype=torch.bfloat16, device=cuda_device)
    w = torch.randn((6912, 2560), device=cuda_device) * 0.02
    lin.scale_weight.data.fill_(float(w.abs().max() / 448))
    lin.set_weight(w, seed=5)
    back = lin.convert_weight(lin.weight.data.float())
    assert abs(float((back - w).mean())) < 2e-6                 # stochastic rounding has no bias
    assert float((back - w).abs().max()) <= float(w.abs().max()) / 8
    first = lin.weight.data.clone()
    lin.set_weight(w, seed=5)
    assert torch.equal(first.view(torch.uint8), lin.weight.data.view(torch.uint8))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(6912, 2560), (2560, 3584), (3, 5), (1,)])
def test_scaled_e4m3_weight_quantiser(cuda_device, dtype, shape):
    """s = max|w| / 448, wq = (w / s).to(e4m3): the kernel against the three torch operations, byte for byte."""
    from comfyui_b200 import moe_ops as M

    g = torch.Generator().manual_seed(sum(shape))
    w = (torch.randn(shape, generator=g) * 0.02).to(dtype)
    wq, scale = M.quantize_weight_e4m3(w.to(cuda_device))
    # the three operations on the CPU, where `tensor / 448.0` is a true fp32 division (PyTorch's CUDA kernel multiplies by
    # the reciprocal of a Python scalar instead, which can differ in the last bit)
    ref_s = w.float().abs().max() / 448.0
    ref_q = (w.float() / ref_s).to(torch.float8_e4m3fn)
    assert scale.dtype == torch.float32 and scale.shape == () and torch.equal(scale.cpu(), ref_s)
    assert torch.equal(wq.cpu().view(torch.uint8), ref_q.view(torch.uint8))
    assert int(wq.view(torch.uint8).bitwise_and(0x7f).max()) == 0x7e        # the largest element lands on +-448
