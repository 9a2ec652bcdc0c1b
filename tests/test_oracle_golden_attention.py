"""Pins the attention oracle (q / k / v glue, rope table, joint attention) to outputs of the unmodified reference."""
import ast

import pytest
import torch

from oracle import hidream_attention_oracle as A


def setup_case(g, dtype, single):
    m = g["meta"]
    heads, head_dim = int(m["heads"]), int(m["head_dim"])
    dim = heads * head_dim
    batch, hh, ww, n_text = int(m["batch"]), int(m["height"]), int(m["width"]), int(m["n_text"])
    gen = torch.Generator().manual_seed(int(m["x_seed"]))
    img = torch.randn((batch, hh * ww, dim), generator=gen).to(dtype)
    txt = torch.randn((batch, n_text, dim), generator=gen).to(dtype)
    layer = A.make_layer(dim, heads, head_dim, single, seed=int(m["w_seed"]), dtype=dtype)
    freqs = A.rope_table(A.make_ids(batch, hh, ww, n_text), ast.literal_eval(m["axes"]))
    return layer, img, txt, freqs, heads


def _same(got, want, dtype):
    want = torch.from_numpy(want)
    if dtype == torch.bfloat16:
        assert torch.equal(got.float(), want)
    else:
        assert torch.allclose(got, want, rtol=0, atol=2e-6)


def test_rope_table(golden_attention):
    _, _, _, freqs, _ = setup_case(golden_attention, torch.float32, False)
    assert torch.equal(freqs, torch.from_numpy(golden_attention["rope"]))


@pytest.mark.parametrize("name,dtype", [("fp32", torch.float32), ("bf16", torch.bfloat16)])
@pytest.mark.parametrize("single", [False, True], ids=["double", "single"])
def test_processor_matches_reference(golden_attention, name, dtype, single):
    g = golden_attention
    layer, img, txt, freqs, heads = setup_case(g, dtype, single)
    tag = f"{name}/{'single' if single else 'double'}"
    assert sorted(layer.keys()) == g[f"{tag}/keys"].tolist()
    if single:
        seq = torch.cat([img, txt], dim=1)
        q, k, v = A.qkv(layer, seq, None, freqs, heads)
        out = A.processor(layer, seq, None, freqs, heads)
        _same(out, g[f"{tag}/out"], dtype)
    else:
        q, k, v = A.qkv(layer, img, txt, freqs, heads)
        out_i, out_t = A.processor(layer, img, txt, freqs, heads)
        _same(out_i, g[f"{tag}/out_i"], dtype)
        _same(out_t, g[f"{tag}/out_t"], dtype)
    for got, key in ((q, "q"), (k, "k"), (v, "v")):
        _same(got, g[f"{tag}/{key}"], dtype)
