"""CPU oracle for the q / k / v glue and the joint attention of a HiDream block.  TEST INFRASTRUCTURE ONLY.

Restates in functional PyTorch: ``EmbedND`` (``comfy/ldm/hidream/model.py:21-33``) over ``rope`` of
``comfy/ldm/flux/math.py:25-36``; ``apply_rope`` (``math.py:38-47``); the RMSNorm the block's ``operations.RMSNorm``
resolves to (``comfy/rmsnorm.py:14-20``: ``torch.nn.functional.rms_norm``); and ``HiDreamAttnProcessor_flashattn``
(``model.py:79-146``): projections, q / k RMSNorm over the whole projected row, concatenation of image and text
tokens, rotary embedding, scaled-dot-product attention, output projections.

Nothing in the product path imports it.  Parity pin: ``tests/golden/make_golden.py`` runs the unmodified reference
modules on seeded inputs (``hidream_attention_small.npz``); ``tests/test_oracle_golden_attention.py`` holds this file
to those outputs.

A "layer" is a dict with the reference's state-dict keys: ``to_q/to_k/to_v/to_out.{weight,bias}``,
``q_rms_norm/k_rms_norm.weight`` and, for a double-stream block, the same with the suffix ``_t``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

Layer = Dict[str, torch.Tensor]


def rope(pos: torch.Tensor, dim: int, theta: int) -> torch.Tensor:
    """math.py:25-36: [..., n] positions -> [..., n, dim/2, 2, 2] rotation matrices (fp32)."""
    scale = torch.linspace(0, (dim - 2) / dim, steps=dim // 2, dtype=torch.float64)
    omega = 1.0 / (theta ** scale)
    out = torch.einsum("...n,d->...nd", pos.to(dtype=torch.float32), omega)
    out = torch.stack([torch.cos(out), -torch.sin(out), torch.sin(out), torch.cos(out)], dim=-1)
    return out.reshape(*out.shape[:-1], 2, 2).to(dtype=torch.float32)


def rope_table(ids: torch.Tensor, axes_dim: List[int], theta: int = 10000) -> torch.Tensor:
    """EmbedND.forward (model.py:27-33): ids [B, S, n_axes] -> [B, S, 1, sum(axes_dim)/2, 2, 2]."""
    emb = torch.cat([rope(ids[..., i], axes_dim[i], theta) for i in range(ids.shape[-1])], dim=-3)
    return emb.unsqueeze(2)


def apply_rope1(x: torch.Tensor, freqs_cis: torch.Tensor) -> torch.Tensor:
    """math.py:38-44."""
    x_ = x.to(dtype=freqs_cis.dtype).reshape(*x.shape[:-1], -1, 1, 2)
    x_out = freqs_cis[..., 0] * x_[..., 0]
    x_out.addcmul_(freqs_cis[..., 1], x_[..., 1])
    return x_out.reshape(*x.shape).type_as(x)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """rmsnorm.py:14-20 with a weight."""
    return F.rms_norm(x, weight.shape, weight=weight.to(x.dtype), eps=eps)


def _lin(x, layer, name):
    return F.linear(x, layer[name + ".weight"], layer.get(name + ".bias"))


def project(layer: Layer, image_tokens: torch.Tensor, text_tokens: Optional[torch.Tensor]) -> Dict[str, torch.Tensor]:
    """The six (three for a single-stream block) Linear projections of model.py:97-111, before any norm."""
    proj = {n: _lin(image_tokens, layer, "to_" + n) for n in ("q", "k", "v")}
    if text_tokens is not None:
        proj.update({n + "_t": _lin(text_tokens, layer, f"to_{n}_t") for n in ("q", "k", "v")})
    return proj


def norm_cat_rope(proj: Dict[str, torch.Tensor], layer: Layer, freqs: torch.Tensor, heads: int, eps: float = 1e-5
                  ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """model.py:97-137 from the projected tensors on: q / k RMSNorm, split into heads, concatenation of image and text
    tokens, rotary embedding.  Returns (query, key, value) [B, S_img (+ S_txt), heads, head_dim]."""
    dtype, b = proj["q"].dtype, proj["q"].shape[0]
    q = rms_norm(proj["q"], layer["q_rms_norm.weight"], eps).to(dtype)
    k = rms_norm(proj["k"], layer["k_rms_norm.weight"], eps).to(dtype)
    v = proj["v"]
    head_dim = k.shape[-1] // heads
    q, k, v = (t.view(b, -1, heads, head_dim) for t in (q, k, v))
    if "q_t" in proj:
        qt = rms_norm(proj["q_t"], layer["q_rms_norm_t.weight"], eps).to(dtype)
        kt = rms_norm(proj["k_t"], layer["k_rms_norm_t.weight"], eps).to(dtype)
        vt = proj["v_t"]
        qt, kt, vt = (t.view(b, -1, heads, head_dim) for t in (qt, kt, vt))
        q, k, v = torch.cat([q, qt], dim=1), torch.cat([k, kt], dim=1), torch.cat([v, vt], dim=1)
    if q.shape[-1] == freqs.shape[-3] * 2:
        q, k = apply_rope1(q, freqs), apply_rope1(k, freqs)
    else:
        q1, q2 = q.chunk(2, dim=-1)
        k1, k2 = k.chunk(2, dim=-1)
        q, k = torch.cat([apply_rope1(q1, freqs), q2], dim=-1), torch.cat([apply_rope1(k1, freqs), k2], dim=-1)
    return q, k, v


def qkv(layer: Layer, image_tokens: torch.Tensor, text_tokens: Optional[torch.Tensor], freqs: torch.Tensor, heads: int,
        eps: float = 1e-5) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """model.py:97-137: (query, key, value) as handed to the attention call."""
    return norm_cat_rope(project(layer, image_tokens, text_tokens), layer, freqs, heads, eps)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """model.py:75-76 through attention_pytorch (comfy/ldm/modules/attention.py): [B, S, H, D] -> [B, S, H*D]."""
    b, s, h, d = q.shape
    out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=None,
                                         dropout_p=0.0, is_causal=False)
    return out.transpose(1, 2).reshape(b, s, h * d)


def processor(layer: Layer, image_tokens: torch.Tensor, text_tokens: Optional[torch.Tensor], freqs: torch.Tensor,
              heads: int, eps: float = 1e-5):
    """The whole processor call: (image out, text out) for a double-stream block, image out for a single-stream one."""
    q, k, v = qkv(layer, image_tokens, text_tokens, freqs, heads, eps)
    hidden = attention(q, k, v)
    if text_tokens is None:
        return _lin(hidden, layer, "to_out")
    n_img = image_tokens.shape[1]
    return _lin(hidden[:, :n_img], layer, "to_out"), _lin(hidden[:, n_img:], layer, "to_out_t")


def make_layer(dim: int, heads: int, head_dim: int, single: bool, seed: int = 0, dtype: torch.dtype = torch.float32,
               std: float = 0.02) -> Layer:
    """Seeded synthetic weights in the order of the reference module's named_parameters(); norm weights around 1."""
    g = torch.Generator().manual_seed(seed)
    inner = heads * head_dim
    layer: Layer = {}

    def draw(name, shape, scale=std, shift=0.0):
        layer[name] = (torch.randn(shape, generator=g, dtype=torch.float32) * scale + shift).to(dtype)

    def block(sfx):
        draw(f"to_q{sfx}.weight", (inner, dim)); draw(f"to_q{sfx}.bias", (inner,), 0.1)
        draw(f"to_k{sfx}.weight", (inner, inner)); draw(f"to_k{sfx}.bias", (inner,), 0.1)
        draw(f"to_v{sfx}.weight", (inner, inner)); draw(f"to_v{sfx}.bias", (inner,), 0.1)
        draw(f"to_out{sfx}.weight", (dim, inner)); draw(f"to_out{sfx}.bias", (dim,), 0.1)
        draw(f"q_rms_norm{sfx}.weight", (inner,), 0.2, 1.0); draw(f"k_rms_norm{sfx}.weight", (inner,), 0.2, 1.0)

    block("")
    if not single:
        block("_t")
    return layer


def make_ids(batch: int, height: int, width: int, n_text: int) -> torch.Tensor:
    """Position ids like the model's: image tokens carry (0, row, column), text tokens zeros; [B, S, 3]."""
    img = torch.zeros(height, width, 3)
    img[..., 1] = torch.arange(height)[:, None]
    img[..., 2] = torch.arange(width)[None, :]
    ids = torch.cat([img.reshape(-1, 3), torch.zeros(n_text, 3)], dim=0)
    return ids.unsqueeze(0).repeat(batch, 1, 1)
