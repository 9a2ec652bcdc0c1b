"""CPU oracle for the two HiDream transformer blocks.  TEST INFRASTRUCTURE ONLY.

Restates ``HiDreamImageSingleTransformerBlock.forward`` (``comfy/ldm/hidream/model.py:408-434``) and
``HiDreamImageTransformerBlock.forward`` (``:485-524``) on top of the attention oracle and the MoE oracle: adaLN
modulation (SiLU + Linear, chunked into 6 or 12 vectors), LayerNorm without affine, ``* (1 + scale) + shift``, the
attention module, ``gate * (.) + residual``, and the same around the feed-forwards (MoE for image tokens, dense SwiGLU
for text tokens).  As shipped the MoE gate runs in the activation dtype; ``gate_in_fp32`` selects the fp32 gate the
kernels use.

Pinned by ``tests/golden/hidream_block_small.npz`` (outputs of the unmodified reference blocks); nothing in the product
path imports this file.

A "layer" is a dict with the block's state-dict keys: ``adaLN_modulation.1.{weight,bias}``, ``attn1.*`` (attention
oracle keys), ``ff_i.*`` (MoE oracle keys) and, for the double-stream block, ``ff_t.w{1,2,3}.weight``.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.nn.functional as F

from . import hidream_attention_oracle as A
from . import hidream_moe_oracle as O

Layer = Dict[str, torch.Tensor]


def _sub(layer: Layer, prefix: str) -> Layer:
    return {k[len(prefix):]: v for k, v in layer.items() if k.startswith(prefix)}


def _modulation(layer: Layer, adaln_input: torch.Tensor, n: int):
    ada = F.linear(F.silu(adaln_input), layer["adaLN_modulation.1.weight"], layer["adaLN_modulation.1.bias"])
    return ada[:, None].chunk(n, dim=-1)


def _norm_mod(x, shift, scale):
    wtype = x.dtype
    n = F.layer_norm(x, (x.shape[-1],), None, None, 1e-6).to(dtype=wtype)
    return n * (1 + scale) + shift


def single_block(layer: Layer, tokens: torch.Tensor, adaln_input: torch.Tensor, freqs: torch.Tensor, heads: int,
                 gate_in_fp32: bool = False, routing_out=None) -> torch.Tensor:
    shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = _modulation(layer, adaln_input, 6)
    attn = A.processor(_sub(layer, "attn1."), _norm_mod(tokens, shift_msa, scale_msa), None, freqs, heads)
    tokens = gate_msa * attn + tokens
    return O.block_ffn(tokens, _sub(layer, "ff_i."), shift_mlp, scale_mlp, gate_mlp, gate_in_fp32=gate_in_fp32,
                       routing_out=routing_out)


def double_block(layer: Layer, image_tokens: torch.Tensor, text_tokens: torch.Tensor, adaln_input: torch.Tensor,
                 freqs: torch.Tensor, heads: int, gate_in_fp32: bool = False,
                 routing_out=None) -> Tuple[torch.Tensor, torch.Tensor]:
    (shift_msa_i, scale_msa_i, gate_msa_i, shift_mlp_i, scale_mlp_i, gate_mlp_i,
     shift_msa_t, scale_msa_t, gate_msa_t, shift_mlp_t, scale_mlp_t, gate_mlp_t) = _modulation(layer, adaln_input, 12)
    attn_i, attn_t = A.processor(_sub(layer, "attn1."), _norm_mod(image_tokens, shift_msa_i, scale_msa_i),
                                 _norm_mod(text_tokens, shift_msa_t, scale_msa_t), freqs, heads)
    image_tokens = gate_msa_i * attn_i + image_tokens
    text_tokens = gate_msa_t * attn_t + text_tokens
    image_tokens = O.block_ffn(image_tokens, _sub(layer, "ff_i."), shift_mlp_i, scale_mlp_i, gate_mlp_i,
                               gate_in_fp32=gate_in_fp32, routing_out=routing_out)
    text_tokens = O.block_ffn(text_tokens, layer, shift_mlp_t, scale_mlp_t, gate_mlp_t, dense_prefix="ff_t")
    return image_tokens, text_tokens


def make_layer(dim: int, heads: int, head_dim: int, n_experts: int, single: bool, seed: int = 0,
               dtype: torch.dtype = torch.float32) -> Layer:
    """Seeded synthetic block: adaLN Linear, attention, MoE feed-forward, text feed-forward (double-stream only)."""
    g = torch.Generator().manual_seed(seed + 1000)
    n_mod = 6 if single else 12
    layer: Layer = {
        "adaLN_modulation.1.weight": (torch.randn((n_mod * dim, dim), generator=g) * 0.02).to(dtype),
        "adaLN_modulation.1.bias": (torch.randn((n_mod * dim,), generator=g) * 0.3).to(dtype),
    }
    layer.update({"attn1." + k: v for k, v in A.make_layer(dim, heads, head_dim, single, seed, dtype).items()})
    layer.update({"ff_i." + k: v for k, v in O.make_layer(dim, 4 * dim, n_experts, seed, dtype).items()})
    if not single:
        h = O.ffn_hidden(4 * dim)
        for name, shape in (("w1", (h, dim)), ("w2", (dim, h)), ("w3", (h, dim))):
            layer[f"ff_t.{name}.weight"] = (torch.randn(shape, generator=g) * 0.02).to(dtype)
    return layer
