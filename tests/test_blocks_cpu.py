"""The two HiDream transformer blocks on the CPU: the block oracle and the drop-in block modules (stock composition)
against outputs of the unmodified reference blocks."""
import ast

import pytest
import torch

from comfyui_b200 import ops
from comfyui_b200.ldm.hidream import model as M
from oracle import hidream_attention_oracle as A
from oracle import hidream_block_oracle as B


def block_case(g, dtype, single):
    m = g["meta"]
    heads, head_dim, n_exp = int(m["heads"]), int(m["head_dim"]), int(m["n_experts"])
    dim = heads * head_dim
    batch, hh, ww, n_text = int(m["batch"]), int(m["height"]), int(m["width"]), int(m["n_text"])
    gen = torch.Generator().manual_seed(int(m["x_seed"]))
    img = torch.randn((batch, hh * ww, dim), generator=gen).to(dtype)
    txt = torch.randn((batch, n_text, dim), generator=gen).to(dtype)
    ada = torch.randn((batch, dim), generator=gen).to(dtype)
    layer = B.make_layer(dim, heads, head_dim, n_exp, single, seed=int(m["w_seed"]), dtype=dtype)
    freqs = A.rope_table(A.make_ids(batch, hh, ww, n_text), ast.literal_eval(m["axes"]))
    return layer, img, txt, ada, freqs, heads, head_dim, n_exp


def _same(got, want, dtype):
    want = torch.from_numpy(want)
    if dtype == torch.bfloat16:
        assert torch.equal(got.float(), want)
    else:
        assert torch.allclose(got, want, rtol=0, atol=5e-6)


CASES = [("fp32", torch.float32, False), ("fp32", torch.float32, True), ("bf16", torch.bfloat16, False),
         ("bf16", torch.bfloat16, True)]


@pytest.mark.parametrize("name,dtype,single", CASES)
def test_block_oracle_matches_reference(golden_block, name, dtype, single):
    g = golden_block
    layer, img, txt, ada, freqs, heads, _, _ = block_case(g, dtype, single)
    tag = f"{name}/{'single' if single else 'double'}"
    assert sorted(layer.keys()) == g[f"{tag}/keys"].tolist()
    if single:
        _same(B.single_block(layer, torch.cat([img, txt], dim=1), ada, freqs, heads), g[f"{tag}/out"], dtype)
    else:
        out_i, out_t = B.double_block(layer, img, txt, ada, freqs, heads)
        _same(out_i, g[f"{tag}/out_i"], dtype)
        _same(out_t, g[f"{tag}/out_t"], dtype)


@pytest.mark.parametrize("name,dtype,single", CASES)
def test_block_modules_reproduce_reference(golden_block, name, dtype, single):
    g = golden_block
    layer, img, txt, ada, freqs, heads, head_dim, n_exp = block_case(g, dtype, single)
    cls = M.HiDreamImageSingleTransformerBlock if single else M.HiDreamImageTransformerBlock
    mod = cls(heads * head_dim, heads, head_dim, n_exp, 2, dtype=dtype, device="cpu", operations=ops.disable_weight_init)
    res = mod.load_state_dict(layer, strict=True)
    assert not res.missing_keys and not res.unexpected_keys
    tag = f"{name}/{'single' if single else 'double'}"
    assert sorted(mod.state_dict().keys()) == g[f"{tag}/keys"].tolist()
    with torch.no_grad():
        if single:
            _same(mod(torch.cat([img, txt], dim=1), None, None, ada, freqs), g[f"{tag}/out"], dtype)
        else:
            out_i, out_t = mod(img, None, txt, ada, freqs)
            _same(out_i, g[f"{tag}/out_i"], dtype)
            _same(out_t, g[f"{tag}/out_t"], dtype)


def test_block_wrapper():
    blk = M.HiDreamImageBlock(256, 4, 64, 4, 2, block_type=M.BlockType.SingleTransformerBlock, dtype=torch.float32,
                              device="cpu", operations=ops.disable_weight_init)
    assert isinstance(blk.block, M.HiDreamImageSingleTransformerBlock)
