"""comfy.float.stochastic_rounding and scaled_fp8_ops.Linear.set_weight as restated in comfyui_b200.ops, on the CPU,
against bytes produced by the unmodified reference (tests/golden/weight_rounding.npz)."""
import os

import numpy as np
import pytest
import torch

from comfyui_b200 import ops
from tests.golden.make_golden import rounding_input

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "weight_rounding.npz")


@pytest.fixture(scope="module")
def golden():
    with np.load(GOLDEN) as z:
        return {k: z[k] for k in z.files}


@pytest.mark.parametrize("name,dtype", [("fp32", torch.float32), ("bf16", torch.bfloat16)])
@pytest.mark.parametrize("tname,target", [("e4m3", torch.float8_e4m3fn), ("e5m2", torch.float8_e5m2)])
@pytest.mark.parametrize("seed", [0, 7])
def test_stochastic_rounding_matches_reference(golden, name, dtype, tname, target, seed):
    q = ops.stochastic_rounding(rounding_input(dtype), target, seed=seed)
    assert q.dtype == target
    assert np.array_equal(q.view(torch.uint8).numpy(), golden[f"{name}/{tname}/seed{seed}"])


def test_set_weight_matches_reference(golden):
    operations = ops.scaled_fp8_ops(fp8_matrix_mult=True, scale_input=False, override_dtype=torch.float8_e4m3fn)
    lin = operations.Linear(160, 96, bias=False, dtype=torch.bfloat16, device="cpu")
    lin.scale_weight.data.fill_(0.0123)
    lin.set_weight(rounding_input(torch.float32), seed=3)
    assert np.array_equal(lin.weight.data.view(torch.uint8).numpy(), golden["set_weight/seed3"])
    # round trip through convert_weight: the dequantised weight is within one e4m3 step of the input
    back = lin.convert_weight(lin.weight.data.float())
    x = rounding_input(torch.float32).clamp(-448 * 0.0123, 448 * 0.0123)
    assert float((back - x)[1:].abs().max()) <= float(x[1:].abs().max()) / 8 + 1e-3


def test_other_dtypes_are_plain_casts():
    v = rounding_input(torch.float32)
    assert torch.equal(ops.stochastic_rounding(v, torch.bfloat16, seed=1), v.bfloat16())
    assert ops.stochastic_rounding(v, torch.float16, seed=1).dtype == torch.float16
