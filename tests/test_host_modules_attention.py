"""Host-side mirror of HiDream's attention module on the CPU: interface, state-dict keys, and its stock composition
held to the reference's golden outputs (no GPU, no kernels)."""
import inspect

import pytest
import torch

from comfyui_b200 import ops
from comfyui_b200.ldm.hidream import model as M
from tests.test_oracle_golden_attention import setup_case


def test_constructor_signature_matches_reference():
    assert list(inspect.signature(M.HiDreamAttention.__init__).parameters) == [
        "self", "query_dim", "heads", "dim_head", "upcast_attention", "upcast_softmax", "scale_qk", "eps", "processor",
        "out_dim", "single", "dtype", "device", "operations"]
    assert list(inspect.signature(M.HiDreamAttention.forward).parameters) == [
        "self", "norm_image_tokens", "image_tokens_masks", "norm_text_tokens", "rope", "transformer_options"]


@pytest.mark.parametrize("name,dtype", [("fp32", torch.float32), ("bf16", torch.bfloat16)])
@pytest.mark.parametrize("single", [False, True], ids=["double", "single"])
def test_stock_composition_reproduces_reference(golden_attention, name, dtype, single):
    g = golden_attention
    layer, img, txt, freqs, heads = setup_case(g, dtype, single)
    dim = img.shape[-1]
    mod = M.HiDreamAttention(query_dim=dim, heads=heads, dim_head=dim // heads,
                             processor=M.HiDreamAttnProcessor_flashattn(), single=single, dtype=dtype, device="cpu",
                             operations=ops.disable_weight_init)
    res = mod.load_state_dict(layer, strict=True)
    assert not res.missing_keys and not res.unexpected_keys
    tag = f"{name}/{'single' if single else 'double'}"
    assert sorted(mod.state_dict().keys()) == g[f"{tag}/keys"].tolist()

    def same(got, want):
        want = torch.from_numpy(want)
        assert torch.equal(got.float(), want) if dtype == torch.bfloat16 else torch.allclose(got, want, rtol=0, atol=2e-6)

    with torch.no_grad():
        if single:
            same(mod(torch.cat([img, txt], dim=1), None, None, rope=freqs), g[f"{tag}/out"])
        else:
            out_i, out_t = mod(img, None, txt, rope=freqs)
            same(out_i, g[f"{tag}/out_i"])
            same(out_t, g[f"{tag}/out_t"])
        assert ops.hidream_qkv(mod, img, None if single else txt, freqs) is None      # CPU call: not eligible
