"""The drop-in HiDreamImageTransformer2DModel on the CPU (stock PyTorch composition, no kernels) against the output of
the unmodified reference model stored in tests/golden/hidream_model_small.npz: same state-dict keys in the same order,
same step output."""
import os

import numpy as np
import pytest
import torch

from oracle import hidream_model_recipe as R

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hidream_model_small.npz")


@pytest.fixture(scope="module")
def golden_model():
    return np.load(GOLDEN)


def build(dtype, device="cpu"):
    from comfyui_b200 import ops
    from comfyui_b200.ldm.hidream.model import HiDreamImageTransformer2DModel

    m = HiDreamImageTransformer2DModel(**R.CONFIG, dtype=dtype, device=device, operations=ops.disable_weight_init).eval()
    shapes = {k: v.shape for k, v in m.state_dict().items()}
    m.load_state_dict({k: v.to(device) for k, v in R.make_state(shapes, dtype).items()}, strict=True)
    return m, shapes


def gate_on_fp32_copy(monkeypatch):
    """The routing convention of the kernels for the stock composition: MoEGate.forward on x.float(), weights cast back."""
    from comfyui_b200.ldm.hidream import model as M

    stock = M.MoEGate.forward

    def forward(self, hidden_states):
        idx, w, aux = stock(self, hidden_states.float())
        return idx, w.to(hidden_states.dtype), aux

    monkeypatch.setattr(M.MoEGate, "forward", forward)


def test_state_dict_keys_and_shapes(golden_model):
    _, shapes = build(torch.bfloat16)
    assert list(shapes.keys()) == [str(k) for k in golden_model["keys"]]
    assert [",".join(str(d) for d in s) for s in shapes.values()] == [str(s) for s in golden_model["shapes"]]


@pytest.mark.parametrize("name,dtype,fp32_gate", [("fp32", torch.float32, False), ("bf16", torch.bfloat16, False),
                                                  ("bf16_fp32gate", torch.bfloat16, True)])
def test_step_output_matches_reference(golden_model, monkeypatch, name, dtype, fp32_gate):
    m, _ = build(dtype)
    if fp32_gate:
        gate_on_fp32_copy(monkeypatch)
    with torch.no_grad():
        out = m(*R.make_inputs(dtype)).float()
    want = torch.from_numpy(golden_model[f"{name}/out"])
    assert out.shape == want.shape == (R.BATCH, R.CONFIG["out_channels"], R.HEIGHT, R.WIDTH)
    if dtype == torch.bfloat16:
        assert torch.equal(out, want)
    else:
        torch.testing.assert_close(out, want, rtol=1e-5, atol=1e-6)
