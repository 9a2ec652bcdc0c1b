"""HiDream's mixture-of-experts feed-forward: drop-in modules backed by the sm_100a kernels.

Same constructors, forward signatures, attribute names and state-dict keys as
``comfy/ldm/hidream/model.py:215-346`` (``FeedForwardSwiGLU``, ``MoEGate``, ``MOEFeedForwardSwiGLU``), so a
HiDream transformer block can build these instead and load the same checkpoint:

    shared_experts.{w1,w2,w3}.weight, experts.{i}.{w1,w2,w3}.weight, gate.weight
    (+ .scale_weight / .scale_input per Linear under scaled-fp8 operations)

Every ``forward`` first offers the call to the dispatch shim in ``comfyui_b200.ops``; when the call is
eligible (B200, bf16 activations, bf16 or scaled-e4m3 weights resident on the device, no LoRA closures)
the whole layer runs as five kernel launches.  Otherwise the module's own PyTorch composition below runs,
which is what the reference executes everywhere.

One deliberate numerical difference on the kernel path: the gate is evaluated in fp32 on the bf16
activations (the reference's gate runs in the activation dtype, ``model.py:268``), routing weights are
then rounded to the activation dtype as the reference's are.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import model_management
from ... import ops as b200_ops


class FeedForwardSwiGLU(nn.Module):
    """w2(silu(w1 x) * w3 x) with three bias-free Linears (``model.py:215-238``)."""

    def __init__(self, dim: int, hidden_dim: int, multiple_of: int = 256, ffn_dim_multiplier: Optional[float] = None,
                 dtype=None, device=None, operations=None):
        super().__init__()
        hidden_dim = int(2 * hidden_dim / 3)
        if ffn_dim_multiplier is not None:
            hidden_dim = int(ffn_dim_multiplier * hidden_dim)
        hidden_dim = -(-hidden_dim // multiple_of) * multiple_of   # round up to a multiple

        make = dict(bias=False, dtype=dtype, device=device)
        self.w1 = operations.Linear(dim, hidden_dim, **make)
        self.w2 = operations.Linear(hidden_dim, dim, **make)
        self.w3 = operations.Linear(dim, hidden_dim, **make)

    def forward(self, x):
        fast = b200_ops.swiglu_ffn_forward(self, x)
        if fast is not None:
            return fast
        return self.w2(F.silu(self.w1(x)) * self.w3(x))


class MoEGate(nn.Module):
    """Softmax router: top-k of ``num_routed_experts`` scores, no renormalisation, no auxiliary loss
    (``model.py:242-283``).  ``weight`` is a bare Parameter [E, D], left uninitialised until a checkpoint is
    loaded, exactly like the reference."""

    def __init__(self, embed_dim, num_routed_experts=4, num_activated_experts=2, aux_loss_alpha=0.01, dtype=None,
                 device=None, operations=None):
        super().__init__()
        self.top_k = num_activated_experts
        self.n_routed_experts = num_routed_experts
        self.scoring_func = "softmax"
        self.alpha = aux_loss_alpha
        self.seq_aux = False
        self.norm_topk_prob = False
        self.gating_dim = embed_dim
        self.weight = nn.Parameter(torch.empty((num_routed_experts, embed_dim), dtype=dtype, device=device))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        pass

    def forward(self, hidden_states):
        bsz, seq_len, h = hidden_states.shape
        if self.scoring_func != "softmax":
            raise NotImplementedError(f"insupportable scoring function for MoE gating: {self.scoring_func}")
        if not self.norm_topk_prob:
            fast = b200_ops.hidream_gate(self, hidden_states)
            if fast is not None:
                return fast[0], fast[1], None

        flat = hidden_states.view(-1, h)
        w = model_management.cast_to(self.weight, dtype=flat.dtype, device=flat.device)
        scores = F.linear(flat, w, None).softmax(dim=-1)
        topk_weight, topk_idx = torch.topk(scores, k=self.top_k, dim=-1, sorted=False)
        if self.top_k > 1 and self.norm_topk_prob:
            topk_weight = topk_weight / (topk_weight.sum(dim=-1, keepdim=True) + 1e-20)
        return topk_idx, topk_weight, None


class MOEFeedForwardSwiGLU(nn.Module):
    """Routed SwiGLU experts plus an always-on shared expert (``model.py:287-346``)."""

    def __init__(self, dim: int, hidden_dim: int, num_routed_experts: int, num_activated_experts: int, dtype=None,
                 device=None, operations=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device, operations=operations)
        self.shared_experts = FeedForwardSwiGLU(dim, hidden_dim // 2, **kw)
        self.experts = nn.ModuleList([FeedForwardSwiGLU(dim, hidden_dim, **kw) for _ in range(num_routed_experts)])
        self.gate = MoEGate(embed_dim=dim, num_routed_experts=num_routed_experts,
                            num_activated_experts=num_activated_experts, **kw)
        self.num_activated_experts = num_activated_experts

    def forward(self, x):
        fast = b200_ops.hidream_moe_forward(self, x)
        if fast is not None:
            return fast

        # stock composition: gate, one masked pass per expert, weighted sum over k, shared expert
        out_dtype, shape, k = x.dtype, x.shape, self.num_activated_experts
        topk_idx, topk_weight, _ = self.gate(x)
        tokens = x.view(-1, shape[-1])
        slot_expert = topk_idx.view(-1)
        slot_x = tokens.repeat_interleave(k, dim=0)
        slot_y = torch.empty_like(slot_x, dtype=out_dtype)
        for i, expert in enumerate(self.experts):
            mask = slot_expert == i
            slot_y[mask] = expert(slot_x[mask]).to(dtype=out_dtype)
        y = (slot_y.view(*topk_weight.shape, -1) * topk_weight.unsqueeze(-1)).sum(dim=1)
        y = y.view(*shape).to(dtype=out_dtype)
        return y + self.shared_experts(x)

    @torch.no_grad()
    def moe_infer(self, x, flat_expert_indices, flat_expert_weights):
        fast = b200_ops.hidream_moe_infer(self, x, flat_expert_indices, flat_expert_weights)
        if fast is not None:
            return fast

        # stock composition: sort slots by expert, run each expert on its slice, scatter-add back
        k = self.num_activated_experts
        acc = torch.zeros_like(x)
        order = flat_expert_indices.argsort()
        ends = flat_expert_indices.bincount().cpu().numpy().cumsum(0)
        token_of = order // k
        begin = 0
        for i, end in enumerate(ends):
            if end > begin:
                tok = token_of[begin:end]
                y = self.experts[i](x[tok])
                y.mul_(flat_expert_weights[order[begin:end]])
                acc = acc.to(y.dtype)
                acc.scatter_reduce_(0, tok.view(-1, 1).repeat(1, x.shape[-1]), y, reduce="sum")
            begin = end
        return acc


def block_feed_forward(norm, ff, tokens, shift, scale, gate):
    """Feed-forward half of a HiDream transformer block (``model.py:429-433`` for the single-stream block,
    ``:515-523`` for the image and the text side of the double-stream block):

        tokens + gate * ff(norm(tokens) * (1 + scale) + shift)

    ``norm`` is the block's ``operations.LayerNorm(dim, eps=1e-6, elementwise_affine=False)``, ``ff`` its
    ``MOEFeedForwardSwiGLU`` or ``FeedForwardSwiGLU``; shift / scale / gate are the ``[B, 1, dim]`` chunks of the adaLN
    output.  A block's forward calls this instead of spelling the four lines out, so that the kernels can fuse the
    element-wise passes with the feed-forward."""
    fast = b200_ops.hidream_block_ffn(norm, ff, tokens, shift, scale, gate)
    if fast is not None:
        return fast
    wtype = tokens.dtype
    normed = norm(tokens).to(dtype=wtype)
    normed = normed * (1 + scale) + shift
    return gate * ff(normed.to(dtype=wtype)) + tokens
