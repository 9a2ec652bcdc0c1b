"""CPU oracle for the Hunyuan3D-2.1 mixture-of-experts block.  TEST INFRASTRUCTURE ONLY.

Restates, in plain functional PyTorch on the CPU, ``comfy/ldm/hunyuan3dv2_1/hunyuandit.py:8-185`` of ComfyUI:
``GELU`` (Linear with bias followed by the exact, erf-based GELU, ``:8-26``), ``FeedForward`` (that, a dropout
that is a no-op in eval, and a second Linear with bias, ``:28-50``), ``MoEGate.forward`` (``:86-112``, the same
softmax / top-2 gate as HiDream's) and ``MoEBlock`` with both its branches: the masked one taken in training
mode (``:140-152``) and ``moe_infer`` (``:157-185``: sort by expert, per-expert feed-forward, ``mul_`` by the
routing weight, ``index_add_`` into a zeroed cache), plus the always-on shared expert (``:154``).

It is the checker the CUDA kernels are compared with; nothing in the product path imports it.

Parity pin: the reference has no vectors for this path; ``tests/golden/make_golden.py`` runs the unmodified
reference module on seeded inputs and ``tests/test_oracle_golden.py`` holds this file to those outputs.

A "layer" is a dict with the reference's state-dict keys:
    gate.weight [E, D]; experts.{e}.net.0.proj.{weight,bias}; experts.{e}.net.2.{weight,bias};
    shared_experts.net.0.proj.{weight,bias}; shared_experts.net.2.{weight,bias}.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.nn.functional as F

from .hidream_moe_oracle import gate, gate_scores_fp64, make_input  # noqa: F401  (same gate, same input recipe)

Layer = Dict[str, torch.Tensor]


def gelu_ffn(x: torch.Tensor, layer: Layer, prefix: str) -> torch.Tensor:
    """FeedForward.forward (hunyuandit.py:47-50): net.0 = GELU(proj), net.1 = Dropout (identity), net.2 = Linear."""
    h = F.linear(x, layer[f"{prefix}.net.0.proj.weight"], layer.get(f"{prefix}.net.0.proj.bias"))
    h = F.gelu(h)
    return F.linear(h, layer[f"{prefix}.net.2.weight"], layer.get(f"{prefix}.net.2.bias"))


def n_experts(layer: Layer) -> int:
    return layer["gate.weight"].shape[0]


def moe_infer(x: torch.Tensor, flat_idx: torch.Tensor, flat_w: torch.Tensor, layer: Layer, top_k: int = 2) -> torch.Tensor:
    """MoEBlock.moe_infer (hunyuandit.py:157-185).  x [N, D]; flat_idx [N*k]; flat_w [N*k, 1]."""
    cache = torch.zeros_like(x)
    order = flat_idx.argsort()
    ends = flat_idx.bincount().cumsum(0).tolist()
    token_of = order // top_k
    start = 0
    for e, end in enumerate(ends):
        if start == end:
            continue
        tok = token_of[start:end]
        out = gelu_ffn(x[tok], layer, f"experts.{e}")
        out.mul_(flat_w[order[start:end]])
        cache.index_add_(0, tok, out)
        start = end
    return cache


def moe_forward_masked(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, layer: Layer, top_k: int = 2) -> torch.Tensor:
    """The training-mode branch (hunyuandit.py:140-150) without its auxiliary loss: boolean-mask gathers."""
    flat = idx.reshape(-1)
    xr = x.repeat_interleave(top_k, dim=0)
    y = torch.empty_like(xr)
    for e in range(n_experts(layer)):
        m = flat == e
        y[m] = gelu_ffn(xr[m], layer, f"experts.{e}").to(xr.dtype)
    return (y.view(*w.shape, -1) * w.unsqueeze(-1)).sum(dim=1)


def moe_block(x: torch.Tensor, layer: Layer, gate_in_fp32: bool = True, top_k: int = 2
              ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """MoEBlock.forward in eval mode on x [N, D]: (out, topk_idx, topk_weight as used)."""
    if gate_in_fp32:
        idx, w = gate(x.float(), layer["gate.weight"].float(), top_k)
        w = w.to(x.dtype)
    else:
        idx, w = gate(x, layer["gate.weight"], top_k)
    routed = moe_infer(x, idx.reshape(-1), w.reshape(-1, 1), layer, top_k)
    return routed + gelu_ffn(x, layer, "shared_experts"), idx, w


def make_layer(dim: int, inner: int, num_experts: int = 8, seed: int = 0, dtype: torch.dtype = torch.float32,
               std: float = 0.02) -> Layer:
    """Seeded synthetic weights drawn in fp32 in the order of the reference module's named_parameters()
    (experts.e.net.0.proj.weight, .bias, net.2.weight, .bias; gate.weight; shared_experts likewise), then cast."""
    g = torch.Generator().manual_seed(seed)
    layer: Layer = {}

    def draw(name, shape, scale=1.0):
        layer[name] = (torch.randn(shape, generator=g, dtype=torch.float32) * (std * scale)).to(dtype)

    def ffn(prefix):
        # biases five times the weight scale, so that a dropped or misplaced bias cannot hide in the tolerance
        draw(prefix + ".net.0.proj.weight", (inner, dim))
        draw(prefix + ".net.0.proj.bias", (inner,), 5.0)
        draw(prefix + ".net.2.weight", (dim, inner))
        draw(prefix + ".net.2.bias", (dim,), 5.0)

    for e in range(num_experts):
        ffn(f"experts.{e}")
    draw("gate.weight", (num_experts, dim))
    ffn("shared_experts")
    return layer
