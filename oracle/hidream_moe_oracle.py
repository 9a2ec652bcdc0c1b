"""CPU oracle for the HiDream mixture-of-experts feed-forward.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain functional PyTorch on the CPU, the algorithm of ComfyUI's
``comfy/ldm/hidream/model.py:215-346`` (FeedForwardSwiGLU, MoEGate, MOEFeedForwardSwiGLU with both its
``forward`` branch and ``moe_infer``) and of the ``comfy.ops`` Linear variants that store its weights
(``comfy/ops.py:103-115`` plain, ``:314-358`` fp8 matmul, ``:379-410`` scaled fp8).  It is the checker
the CUDA kernels are compared with; nothing in the product path imports it.  Only the tests, the
smoke check and the CPU-baseline leg of the benchmark may call it.

Parity pin: the reference ships no golden vectors or known-answer tests for this path, so the pin is
the reference itself: ``tests/golden/make_golden.py`` imports the unmodified reference modules, runs
them on seeded inputs and stores the outputs; ``tests/test_oracle_golden.py`` checks every function
below against those files.

A "layer" is a dict with the reference's state-dict keys:
    gate.weight [E, D]; experts.{e}.w{1,2,3}.weight; shared_experts.w{1,2,3}.weight;
    optional ``.scale_weight`` / ``.scale_input`` fp32 scalars next to a weight (scaled fp8).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

Layer = Dict[str, torch.Tensor]

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0

# How a Linear's weight is applied; mirrors which comfy.ops namespace built the module.
PLAIN = "plain"              # disable_weight_init / manual_cast: F.linear on the stored weight
FP8_DEQUANT = "fp8_dequant"  # scaled_fp8_ops with fp8_matrix_mult=False   (comfy/ops.py:405-410)
FP8_MATMUL = "fp8_matmul"    # scaled_fp8_ops with fp8_matrix_mult=True    (comfy/ops.py:314-358)


def ffn_hidden(hidden_dim: int, multiple_of: int = 256) -> int:
    """Hidden width FeedForwardSwiGLU derives from its argument (model.py:225-231)."""
    h = int(2 * hidden_dim / 3)
    return multiple_of * ((h + multiple_of - 1) // multiple_of)


# ------------------------------------------------------------------------------------------- Linear
def scaled_mm_emulated(xq: torch.Tensor, wq: torch.Tensor, scale_a: torch.Tensor, scale_b: torch.Tensor,
                       out_dtype: torch.dtype) -> torch.Tensor:
    """Arithmetic of torch._scaled_mm with per-tensor scales: fp32 accumulation of the e4m3 values,
    times both scales, one rounding to out_dtype.  Used because the CPU implementation of
    torch._scaled_mm is far too slow at layer size; the golden test checks the two agree."""
    acc = xq.float() @ wq.float().t()
    return (acc * (scale_a.float() * scale_b.float())).to(out_dtype)


def linear(x: torch.Tensor, layer: Layer, name: str, mode: str = PLAIN, use_real_scaled_mm: bool = False) -> torch.Tensor:
    """One bias-free operations.Linear call on a 2-D input [M, in] -> [M, out]."""
    w = layer[name + ".weight"]
    if mode == PLAIN:
        # ops.py:111-115 -> torch.nn.Linear.forward; a weight stored in another dtype is cast on use (:61-95)
        return F.linear(x, w.to(x.dtype))
    scale_w = layer.get(name + ".scale_weight")
    scale_in = layer.get(name + ".scale_input")
    if mode == FP8_DEQUANT:
        # ops.py:405-410: cast the fp8 weight to the activation dtype, fold the scale into the smaller operand
        wd = w.to(x.dtype)
        s = scale_w.to(x.dtype)
        if wd.numel() < x.numel():
            return F.linear(x, wd * s)
        return F.linear(x * s, wd)
    if mode == FP8_MATMUL:
        # ops.py:314-358 (2-D input is unsqueezed to [M, 1, in] there; values are unaffected)
        if w.dtype != FP8:
            raise ValueError("fp8 matmul needs an e4m3 weight (ops.py:316-317 returns None otherwise)")
        one = torch.ones((), dtype=torch.float32)
        sw = one if scale_w is None else scale_w
        if scale_in is None:
            si = one
            xq = torch.clamp(x, min=-FP8_MAX, max=FP8_MAX).to(FP8)           # :338-340
        else:
            si = scale_in
            xq = (x * (1.0 / si).to(x.dtype)).to(FP8)                        # :342-343, no clamp
        if use_real_scaled_mm:
            return torch._scaled_mm(xq.contiguous(), w.t(), out_dtype=x.dtype, scale_a=si, scale_b=sw)
        return scaled_mm_emulated(xq, w, si, sw, x.dtype)
    raise ValueError(mode)


# ------------------------------------------------------------------------------------------- modules
def swiglu_ffn(x: torch.Tensor, layer: Layer, prefix: str, mode: str = PLAIN, **kw) -> torch.Tensor:
    """FeedForwardSwiGLU.forward (model.py:237-238): w2(silu(w1 x) * w3 x)."""
    a = linear(x, layer, prefix + ".w1", mode, **kw)
    b = linear(x, layer, prefix + ".w3", mode, **kw)
    return linear(F.silu(a) * b, layer, prefix + ".w2", mode, **kw)


def gate(x: torch.Tensor, w_gate: torch.Tensor, top_k: int = 2) -> Tuple[torch.Tensor, torch.Tensor]:
    """MoEGate.forward (model.py:263-283): logits in x.dtype, softmax, top-k (unsorted), no renormalisation
    (norm_topk_prob is False, :253).  x is [N, D]; returns (idx int64 [N, k], weight [N, k] in x.dtype).
    Feed ``x.float()`` for the fp32 gate the parity contract is stated on."""
    logits = F.linear(x, w_gate.to(x.dtype))
    scores = logits.softmax(dim=-1)
    topk_weight, topk_idx = torch.topk(scores, k=top_k, dim=-1, sorted=False)
    return topk_idx, topk_weight


def gate_scores_fp64(x: torch.Tensor, w_gate: torch.Tensor) -> torch.Tensor:
    """fp64 arbiter for near-ties: the scores of the same bf16/fp32 data without fp32 summation noise."""
    return F.linear(x.double(), w_gate.double()).softmax(dim=-1)


def n_experts(layer: Layer) -> int:
    return layer["gate.weight"].shape[0]


def moe_infer(x: torch.Tensor, flat_idx: torch.Tensor, flat_w: torch.Tensor, layer: Layer, mode: str = PLAIN,
              top_k: int = 2, **kw) -> torch.Tensor:
    """MOEFeedForwardSwiGLU.moe_infer (model.py:327-346).  x [N, D]; flat_idx [N*k]; flat_w [N*k, 1]."""
    cache = torch.zeros_like(x)
    order = flat_idx.argsort()
    ends = flat_idx.bincount().cumsum(0).tolist()       # no minlength: trailing empty experts drop out
    token_of = order // top_k
    start = 0
    for e, end in enumerate(ends):
        if start == end:
            continue
        tok = token_of[start:end]
        out = swiglu_ffn(x[tok], layer, f"experts.{e}", mode, **kw)
        out.mul_(flat_w[order[start:end]])              # rounds into out.dtype
        cache = cache.to(out.dtype)
        cache.scatter_reduce_(0, tok.view(-1, 1).repeat(1, x.shape[-1]), out, reduce="sum")
        start = end
    return cache


def moe_forward_masked(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, layer: Layer, mode: str = PLAIN,
                       **kw) -> torch.Tensor:
    """The branch MOEFeedForwardSwiGLU.forward really takes (model.py:314-320): repeat_interleave,
    one boolean-mask pass per expert, weight-multiply and sum over k.  Routed part only."""
    top_k = idx.shape[1]
    flat = idx.reshape(-1)
    xr = x.repeat_interleave(top_k, dim=0)
    y = torch.empty_like(xr)
    for e in range(n_experts(layer)):
        m = flat == e
        y[m] = swiglu_ffn(xr[m], layer, f"experts.{e}", mode, **kw).to(x.dtype)
    y = (y.view(*w.shape, -1) * w.unsqueeze(-1)).sum(dim=1)
    return y.to(x.dtype)


def moe_layer(x: torch.Tensor, layer: Layer, mode: str = PLAIN, gate_in_fp32: bool = True, branch: str = "infer",
              routing: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, **kw):
    """Whole layer on x [N, D]: routed experts + always-on shared expert (model.py:307-325).

    gate_in_fp32=True is the parity contract: indices from the fp32 gate on the same data, weights then
    cast to x.dtype (what the as-shipped gate would hand to moe_infer).  False = the as-shipped gate in
    x.dtype.  Returns (out [N, D], idx int64 [N, 2], weight [N, 2] in x.dtype).
    """
    if routing is None:
        gx = x.float() if gate_in_fp32 else x
        idx, w = gate(gx, layer["gate.weight"])
        w = w.to(x.dtype)
    else:
        idx, w = routing
    if branch == "infer":
        routed = moe_infer(x, idx.reshape(-1), w.reshape(-1, 1), layer, mode, top_k=idx.shape[1], **kw)
    else:
        routed = moe_forward_masked(x, idx, w, layer, mode, **kw)
    out = routed + swiglu_ffn(x, layer, "shared_experts", mode, **kw)
    return out, idx, w


def block_ffn(x: torch.Tensor, layer: Layer, shift: torch.Tensor, scale: torch.Tensor, gate_mlp: torch.Tensor,
              eps: float = 1e-6, mode: str = PLAIN, dense_prefix: Optional[str] = None,
              routing_out: Optional[list] = None, **moe_kw) -> torch.Tensor:
    """Feed-forward half of a HiDream block (model.py:429-433; :515-523 for the double-stream block):
    LayerNorm without affine -> * (1 + scale) + shift -> feed-forward -> gate * (.) + x.
    x [B, S, D]; shift / scale / gate_mlp [B, 1, D].  ``dense_prefix`` selects a plain FeedForwardSwiGLU (the text
    side, ``ff_t``) instead of the MoE; ``moe_kw`` goes to moe_layer (routing, gate_in_fp32, branch); ``routing_out``,
    a list, receives the (idx, weight) pair the MoE used."""
    wtype = x.dtype
    b, s, d = x.shape
    normed = F.layer_norm(x, (d,), None, None, eps).to(dtype=wtype)
    normed = normed * (1 + scale) + shift
    flat = normed.to(dtype=wtype).reshape(-1, d)
    if dense_prefix is not None:
        ff = swiglu_ffn(flat, layer, dense_prefix, mode)
    else:
        ff, idx, w = moe_layer(flat, layer, mode=mode, **moe_kw)
        if routing_out is not None:
            routing_out.append((idx, w))
    return gate_mlp * ff.view(b, s, d) + x


def make_modulation(batch: int, dim: int, seed: int = 2, dtype: torch.dtype = torch.bfloat16):
    """Seeded stand-in for one adaLN output: a [B, 6*dim] tensor chunked into six [B, 1, dim] views like the
    blocks do (model.py:419-420); returns (shift_mlp, scale_mlp, gate_mlp), i.e. chunks 3, 4, 5."""
    g = torch.Generator().manual_seed(seed)
    ada = (torch.randn((batch, 6 * dim), generator=g, dtype=torch.float32) * 0.5).to(dtype)
    chunks = ada[:, None].chunk(6, dim=-1)
    return chunks[3], chunks[4], chunks[5]


# ------------------------------------------------------------------------------------------- synthetic layers
def make_layer(dim: int, hidden_dim: int, num_experts: int = 4, seed: int = 0, dtype: torch.dtype = torch.float32,
               std: float = 0.02) -> Layer:
    """Seeded synthetic weights, drawn in fp32 in the order of the reference module's named_parameters()
    (shared_experts.w1, w2, w3; experts.e.w1, w2, w3; gate.weight) and then cast."""
    g = torch.Generator().manual_seed(seed)
    h, hs = ffn_hidden(hidden_dim), ffn_hidden(hidden_dim // 2)
    layer: Layer = {}

    def draw(name, shape):
        layer[name] = (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(dtype)

    for p, hh in [("shared_experts", hs)] + [(f"experts.{e}", h) for e in range(num_experts)]:
        draw(p + ".w1.weight", (hh, dim))
        draw(p + ".w2.weight", (dim, hh))
        draw(p + ".w3.weight", (hh, dim))
    draw("gate.weight", (num_experts, dim))
    return layer


def make_input(n_tokens: int, dim: int, seed: int = 1, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn((n_tokens, dim), generator=g, dtype=torch.float32).to(dtype)


def quantize_layer_fp8(layer: Layer, scale_input: Optional[float] = None) -> Layer:
    """Per-tensor scaled fp8 of every expert Linear: s = max|w| / 448, wq = (w / s).to(e4m3); the gate keeps
    its dtype (it is a bare Parameter, not an operations.Linear)."""
    out: Layer = {}
    for k, v in layer.items():
        if k == "gate.weight":
            out[k] = v
            continue
        w = v.float()
        s = (w.abs().max() / FP8_MAX).reshape(())
        out[k] = (w / s).to(FP8)
        base = k[: -len(".weight")]
        out[base + ".scale_weight"] = s.to(torch.float32)
        if scale_input is not None:
            out[base + ".scale_input"] = torch.tensor(scale_input, dtype=torch.float32)
    return out


def skew_router(layer: Layer, x: torch.Tensor, bias: float = 1.16) -> None:
    """In-place skew: constant feature x[:, 0] = 1 and gate.weight[:, 0] = (bias, 0, ...), so expert 0 wins
    about 60 % of the top-1 picks without changing the module interface (the gate has no bias term)."""
    x[:, 0] = 1
    layer["gate.weight"][:, 0] = 0
    layer["gate.weight"][0, 0] = bias
