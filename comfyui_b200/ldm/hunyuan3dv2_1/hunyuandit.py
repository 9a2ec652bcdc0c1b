"""Hunyuan3D-2.1's mixture-of-experts block: drop-in modules backed by the sm_100a kernels.

Same constructors, forward signatures, attribute names and state-dict keys as
``comfy/ldm/hunyuan3dv2_1/hunyuandit.py:8-185`` (``GELU``, ``FeedForward``, ``MoEGate``, ``MoEBlock``):

    experts.{i}.net.0.proj.{weight,bias}, experts.{i}.net.2.{weight,bias}, gate.weight,
    shared_experts.net.0.proj.{weight,bias}, shared_experts.net.2.{weight,bias}

The routing (softmax gate, top-2, stable permutation) and the weighted combine are the HiDream kernels; only the
expert feed-forward differs: Linear + bias, exact GELU, Linear + bias, run as two passes of the grouped
tcgen05 GEMM with the bias / GELU epilogue.  In eval mode an eligible call (B200, bf16 activations and weights on
the device, no LoRA closures) runs as five launches; everything else, and training mode, runs the module's own
PyTorch composition below, which is what the reference executes everywhere.  As for HiDream, the kernel path
evaluates the gate in fp32 on the bf16 activations.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import model_management
from ... import ops as b200_ops


class GELU(nn.Module):
    """Linear with bias followed by the exact GELU (``hunyuandit.py:8-26``)."""

    def __init__(self, dim_in: int, dim_out: int, operations, device, dtype):
        super().__init__()
        self.proj = operations.Linear(dim_in, dim_out, device=device, dtype=dtype)

    def gelu(self, gate: torch.Tensor) -> torch.Tensor:
        if gate.device.type == "mps":
            return F.gelu(gate.to(dtype=torch.float32)).to(dtype=gate.dtype)
        return F.gelu(gate)

    def forward(self, hidden_states):
        return self.gelu(self.proj(hidden_states))


class FeedForward(nn.Module):
    """``net`` = [GELU(dim -> inner), Dropout, Linear(inner -> dim_out)] (``hunyuandit.py:28-50``)."""

    def __init__(self, dim: int, dim_out=None, mult: int = 4, dropout: float = 0.0, inner_dim=None, operations=None,
                 device=None, dtype=None):
        super().__init__()
        if inner_dim is None:
            inner_dim = int(dim * mult)
        dim_out = dim_out if dim_out is not None else dim
        self.net = nn.ModuleList([
            GELU(dim, inner_dim, operations=operations, device=device, dtype=dtype),
            nn.Dropout(dropout),
            operations.Linear(inner_dim, dim_out, device=device, dtype=dtype),
        ])

    def _apply(self, fn, *args, **kwargs):
        b200_ops.drop_packs(self)       # .to() / .cuda() / .cpu() replace the weights the packs point into
        return super()._apply(fn, *args, **kwargs)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        if not (self.training and self.net[1].p > 0):
            fast = b200_ops.gelu_ffn_forward(self, hidden_states)
            if fast is not None:
                return fast
        for module in self.net:
            hidden_states = module(hidden_states)
        return hidden_states


class MoEGate(nn.Module):
    """Softmax router, top-k of ``num_experts`` scores (``hunyuandit.py:73-112``).  The auxiliary load-balancing
    loss exists in training mode only."""

    def __init__(self, embed_dim, num_experts=16, num_experts_per_tok=2, aux_loss_alpha=0.01, device=None, dtype=None):
        super().__init__()
        self.top_k = num_experts_per_tok
        self.n_routed_experts = num_experts
        self.alpha = aux_loss_alpha
        self.gating_dim = embed_dim
        self.weight = nn.Parameter(torch.empty((num_experts, embed_dim), device=device, dtype=dtype))

    def forward(self, hidden_states: torch.Tensor):
        if not self.training:
            fast = b200_ops.hidream_gate(self, hidden_states)
            if fast is not None:
                return fast[0], fast[1], None
        flat = hidden_states.view(-1, hidden_states.size(-1))
        w = model_management.cast_to(self.weight, dtype=flat.dtype, device=flat.device)
        scores = F.linear(flat, w, bias=None).softmax(dim=-1)
        topk_weight, topk_idx = torch.topk(scores, k=self.top_k, dim=-1, sorted=False)
        aux_loss = None
        if self.training and self.alpha > 0.0:
            counts = torch.bincount(topk_idx.view(-1), minlength=self.n_routed_experts).float()
            usage = counts / topk_idx.numel()
            aux_loss = (scores.mean(0) * usage * self.n_routed_experts).sum() * self.alpha
        return topk_idx, topk_weight, aux_loss


class _AddAuxLoss(torch.autograd.Function):
    """Identity in the forward pass; lets the auxiliary loss receive a gradient (``hunyuandit.py:52-71``)."""

    @staticmethod
    def forward(ctx, x, loss):
        ctx.requires_aux_loss = loss.requires_grad
        ctx.dtype = loss.dtype
        return x

    @staticmethod
    def backward(ctx, grad_output):
        grad_loss = None
        if ctx.requires_aux_loss:
            grad_loss = torch.ones(1, dtype=ctx.dtype, device=grad_output.device)
        return grad_output, grad_loss


class MoEBlock(nn.Module):
    """Routed GELU feed-forwards plus an always-on shared one (``hunyuandit.py:114-185``)."""

    def __init__(self, dim, num_experts: int = 6, moe_top_k: int = 2, dropout: float = 0.0, ff_inner_dim: int = None,
                 operations=None, device=None, dtype=None):
        super().__init__()
        self.moe_top_k = moe_top_k
        self.num_experts = num_experts
        kw = dict(dropout=dropout, inner_dim=ff_inner_dim, operations=operations, device=device, dtype=dtype)
        self.experts = nn.ModuleList([FeedForward(dim, **kw) for _ in range(num_experts)])
        self.gate = MoEGate(dim, num_experts=num_experts, num_experts_per_tok=moe_top_k, device=device, dtype=dtype)
        self.shared_experts = FeedForward(dim, **kw)

    def _apply(self, fn, *args, **kwargs):
        b200_ops.drop_packs(self)       # .to() / .cuda() / .cpu() replace the weights the packs point into
        return super()._apply(fn, *args, **kwargs)

    def forward(self, hidden_states) -> torch.Tensor:
        fast = b200_ops.hunyuan3d_moe_forward(self, hidden_states)
        if fast is not None:
            return fast

        identity, shape = hidden_states, hidden_states.shape
        topk_idx, topk_weight, aux_loss = self.gate(hidden_states)
        tokens = hidden_states.view(-1, shape[-1])
        slot_expert = topk_idx.view(-1)
        if self.training:
            slot_x = tokens.repeat_interleave(self.moe_top_k, dim=0)
            slot_y = torch.empty_like(slot_x, dtype=slot_x.dtype)
            for i, expert in enumerate(self.experts):
                mask = slot_expert == i
                slot_y[mask] = expert(slot_x[mask]).to(slot_x.dtype)
            y = (slot_y.view(*topk_weight.shape, -1) * topk_weight.unsqueeze(-1)).sum(dim=1).view(*shape)
            y = _AddAuxLoss.apply(y, aux_loss)
        else:
            y = self.moe_infer(tokens, flat_expert_indices=slot_expert,
                               flat_expert_weights=topk_weight.view(-1, 1)).view(*shape)
        return y + self.shared_experts(identity)

    @torch.no_grad()
    def moe_infer(self, x, flat_expert_indices, flat_expert_weights):
        fast = b200_ops.hunyuan3d_moe_infer(self, x, flat_expert_indices, flat_expert_weights)
        if fast is not None:
            return fast

        # stock composition: sort slots by expert, run each expert on its slice, index_add_ back
        acc = torch.zeros_like(x)
        order = flat_expert_indices.argsort()
        ends = flat_expert_indices.bincount().cumsum(0)
        token_of = order // self.moe_top_k
        for i, end in enumerate(ends):
            begin = 0 if i == 0 else ends[i - 1]
            if begin == end:
                continue
            tok = token_of[begin:end]
            out = self.experts[i](x[tok])
            out.mul_(flat_expert_weights[order[begin:end]])
            acc.index_add_(0, tok, out)
        return acc
