"""HiDream's mixture-of-experts feed-forward: drop-in modules backed by the sm_100a kernels.

Same constructors, forward signatures, attribute names and state-dict keys as
``comfy/ldm/hidream/model.py:215-346`` (``FeedForwardSwiGLU``, ``MoEGate``, ``MOEFeedForwardSwiGLU``), so a
HiDream transformer block can build these instead and load the same checkpoint:

    shared_experts.{w1,w2,w3}.weight, experts.{i}.{w1,w2,w3}.weight, gate.weight
    (+ .scale_weight / .scale_input per Linear under scaled-fp8 operations)

Every ``forward`` first offers the call to the dispatch shim in ``comfyui_b200.ops``; when the call is
eligible (B200, bf16 activations, bf16 or scaled-e4m3 weights resident on the device; LoRA closures are baked once)
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

    def _apply(self, fn, *args, **kwargs):
        b200_ops.drop_packs(self)       # .to() / .cuda() / .cpu() replace the weights the packs point into
        return super()._apply(fn, *args, **kwargs)

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

    def _apply(self, fn, *args, **kwargs):
        b200_ops.drop_packs(self)
        return super()._apply(fn, *args, **kwargs)

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


# ---------------------------------------------------------------------------------------------------------------
# Joint attention of the block (``comfy/ldm/hidream/model.py:75-213``).  The six projections and the output
# projections stay ``operations.Linear`` calls and the attention itself stays PyTorch's scaled-dot-product attention,
# as in the reference on a CUDA device; what the kernels take over is everything in between.
# ---------------------------------------------------------------------------------------------------------------
def _apply_rope1(x, freqs_cis):
    """``comfy/ldm/flux/math.py:38-44``: fp32 2x2 rotation of neighbouring pairs, rounded back to x's dtype."""
    x_ = x.to(dtype=freqs_cis.dtype).reshape(*x.shape[:-1], -1, 1, 2)
    x_out = freqs_cis[..., 0] * x_[..., 0]
    x_out.addcmul_(freqs_cis[..., 1], x_[..., 1])
    return x_out.reshape(*x.shape).type_as(x)


def attention(query, key, value, transformer_options={}):
    """[B, S, H, D] x 3 -> [B, S, H * D] (``model.py:75-76`` over ``attention_pytorch``)."""
    fast = b200_ops.hidream_attention(query, key, value)
    if fast is not None:
        return fast
    b, s, h, d = query.shape
    out = F.scaled_dot_product_attention(query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2),
                                         attn_mask=None, dropout_p=0.0, is_causal=False)
    return out.transpose(1, 2).reshape(b, s, h * d)


class HiDreamAttnProcessor_flashattn:
    """Processor of ``HiDreamAttention`` (``model.py:79-146``)."""

    def __call__(self, attn, image_tokens, image_tokens_masks=None, text_tokens=None, rope=None, transformer_options={},
                 *args, **kwargs):
        dtype, b = image_tokens.dtype, image_tokens.shape[0]
        n_img = image_tokens.shape[1]
        fast = b200_ops.hidream_qkv(attn, image_tokens, text_tokens, rope, image_tokens_masks)
        if fast is not None:
            query, key, value = fast
        else:
            query = attn.q_rms_norm(attn.to_q(image_tokens)).to(dtype=dtype)
            key = attn.k_rms_norm(attn.to_k(image_tokens)).to(dtype=dtype)
            value = attn.to_v(image_tokens)
            head_dim = key.shape[-1] // attn.heads
            query, key, value = (t.view(b, -1, attn.heads, head_dim) for t in (query, key, value))
            if image_tokens_masks is not None:
                key = key * image_tokens_masks.view(b, -1, 1, 1)
            if not attn.single:
                query_t = attn.q_rms_norm_t(attn.to_q_t(text_tokens)).to(dtype=dtype)
                key_t = attn.k_rms_norm_t(attn.to_k_t(text_tokens)).to(dtype=dtype)
                value_t = attn.to_v_t(text_tokens)
                query_t, key_t, value_t = (t.view(b, -1, attn.heads, head_dim) for t in (query_t, key_t, value_t))
                query = torch.cat([query, query_t], dim=1)
                key = torch.cat([key, key_t], dim=1)
                value = torch.cat([value, value_t], dim=1)
            if query.shape[-1] == rope.shape[-3] * 2:
                query, key = _apply_rope1(query, rope), _apply_rope1(key, rope)
            else:
                q1, q2 = query.chunk(2, dim=-1)
                k1, k2 = key.chunk(2, dim=-1)
                query = torch.cat([_apply_rope1(q1, rope), q2], dim=-1)
                key = torch.cat([_apply_rope1(k1, rope), k2], dim=-1)

        hidden = attention(query, key, value, transformer_options=transformer_options)
        if attn.single:
            fast = b200_ops.grouped_projections([(attn.to_out, hidden)])
            return fast[0] if fast is not None else attn.to_out(hidden)
        hidden_i, hidden_t = torch.split(hidden, [n_img, hidden.shape[1] - n_img], dim=1)
        fast = b200_ops.grouped_projections([(attn.to_out, hidden_i), (attn.to_out_t, hidden_t)])
        if fast is not None:
            return fast[0], fast[1]
        return attn.to_out(hidden_i), attn.to_out_t(hidden_t)


class HiDreamAttention(nn.Module):
    """Projections and norms of the block's attention (``model.py:148-213``); same constructor and state-dict keys:
    ``to_q/to_k/to_v/to_out.{weight,bias}``, ``q_rms_norm/k_rms_norm.weight`` and the ``_t`` set unless ``single``."""

    def __init__(self, query_dim: int, heads: int = 8, dim_head: int = 64, upcast_attention: bool = False,
                 upcast_softmax: bool = False, scale_qk: bool = True, eps: float = 1e-5, processor=None,
                 out_dim: int = None, single: bool = False, dtype=None, device=None, operations=None):
        super().__init__()
        self.inner_dim = out_dim if out_dim is not None else dim_head * heads
        self.query_dim = query_dim
        self.upcast_attention = upcast_attention
        self.upcast_softmax = upcast_softmax
        self.out_dim = out_dim if out_dim is not None else query_dim
        self.scale_qk = scale_qk
        self.scale = dim_head ** -0.5 if self.scale_qk else 1.0
        self.heads = out_dim // dim_head if out_dim is not None else heads
        self.sliceable_head_dim = heads
        self.single = single
        self.linear_cls = operations.Linear
        kw = dict(dtype=dtype, device=device)
        for sfx in ([""] if single else ["", "_t"]):
            setattr(self, "to_q" + sfx, operations.Linear(query_dim, self.inner_dim, **kw))
            setattr(self, "to_k" + sfx, operations.Linear(self.inner_dim, self.inner_dim, **kw))
            setattr(self, "to_v" + sfx, operations.Linear(self.inner_dim, self.inner_dim, **kw))
            setattr(self, "to_out" + sfx, operations.Linear(self.inner_dim, self.out_dim, **kw))
            setattr(self, "q_rms_norm" + sfx, operations.RMSNorm(self.inner_dim, eps, **kw))
            setattr(self, "k_rms_norm" + sfx, operations.RMSNorm(self.inner_dim, eps, **kw))
        self.processor = processor

    def forward(self, norm_image_tokens, image_tokens_masks=None, norm_text_tokens=None, rope=None,
                transformer_options={}):
        return self.processor(self, image_tokens=norm_image_tokens, image_tokens_masks=image_tokens_masks,
                              text_tokens=norm_text_tokens, rope=rope, transformer_options=transformer_options)


# ---------------------------------------------------------------------------------------------------------------
# The two transformer blocks (``comfy/ldm/hidream/model.py:363-575``): same constructors, attribute names and
# state-dict keys; their forwards are the reference's lines with the element-wise passes handed to the kernels where
# a call is eligible (each helper falls back to the PyTorch composition on its own).
# ---------------------------------------------------------------------------------------------------------------
def _modulated_norm(norm, tokens, shift, scale):
    fast = b200_ops.hidream_modulated_norm(norm, tokens, shift, scale)
    if fast is not None:
        return fast
    wtype = tokens.dtype
    return norm(tokens).to(dtype=wtype) * (1 + scale) + shift


def _gated_residual(y, gate, tokens):
    fast = b200_ops.hidream_gated_residual(y, gate, tokens)
    if fast is not None:
        return fast
    return gate * y + tokens


class BlockType:
    TransformerBlock = 1
    SingleTransformerBlock = 2


def _block_ffn(dim, num_routed_experts, num_activated_experts, kw):
    if num_routed_experts > 0:
        return MOEFeedForwardSwiGLU(dim=dim, hidden_dim=4 * dim, num_routed_experts=num_routed_experts,
                                    num_activated_experts=num_activated_experts, **kw)
    return FeedForwardSwiGLU(dim=dim, hidden_dim=4 * dim, **kw)


class HiDreamImageSingleTransformerBlock(nn.Module):
    """Single-stream block (``model.py:363-434``): one modulated attention and one modulated MoE feed-forward over the
    concatenated image + text sequence."""

    def __init__(self, dim: int, num_attention_heads: int, attention_head_dim: int, num_routed_experts: int = 4,
                 num_activated_experts: int = 2, dtype=None, device=None, operations=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device, operations=operations)
        self.num_attention_heads = num_attention_heads
        self.adaLN_modulation = nn.Sequential(nn.SiLU(), operations.Linear(dim, 6 * dim, bias=True, dtype=dtype,
                                                                           device=device))
        self.norm1_i = operations.LayerNorm(dim, eps=1e-06, elementwise_affine=False, dtype=dtype, device=device)
        self.attn1 = HiDreamAttention(query_dim=dim, heads=num_attention_heads, dim_head=attention_head_dim,
                                      processor=HiDreamAttnProcessor_flashattn(), single=True, **kw)
        self.norm3_i = operations.LayerNorm(dim, eps=1e-06, elementwise_affine=False, dtype=dtype, device=device)
        self.ff_i = _block_ffn(dim, num_routed_experts, num_activated_experts, kw)

    def forward(self, image_tokens, image_tokens_masks=None, text_tokens=None, adaln_input=None, rope=None,
                transformer_options={}):
        shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = \
            self.adaLN_modulation(adaln_input)[:, None].chunk(6, dim=-1)
        normed = _modulated_norm(self.norm1_i, image_tokens, shift_msa, scale_msa)
        attn_out = self.attn1(normed, image_tokens_masks, rope=rope, transformer_options=transformer_options)
        image_tokens = _gated_residual(attn_out, gate_msa, image_tokens)
        return block_feed_forward(self.norm3_i, self.ff_i, image_tokens, shift_mlp, scale_mlp, gate_mlp)


class HiDreamImageTransformerBlock(nn.Module):
    """Double-stream block (``model.py:437-524``): joint attention over image and text tokens with separate
    projections, a MoE feed-forward for the image tokens and a dense SwiGLU feed-forward for the text tokens."""

    def __init__(self, dim: int, num_attention_heads: int, attention_head_dim: int, num_routed_experts: int = 4,
                 num_activated_experts: int = 2, dtype=None, device=None, operations=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device, operations=operations)
        self.num_attention_heads = num_attention_heads
        self.adaLN_modulation = nn.Sequential(nn.SiLU(), operations.Linear(dim, 12 * dim, bias=True, dtype=dtype,
                                                                           device=device))
        ln = dict(eps=1e-06, elementwise_affine=False)
        self.norm1_i = operations.LayerNorm(dim, dtype=dtype, device=device, **ln)
        self.norm1_t = operations.LayerNorm(dim, dtype=dtype, device=device, **ln)
        self.attn1 = HiDreamAttention(query_dim=dim, heads=num_attention_heads, dim_head=attention_head_dim,
                                      processor=HiDreamAttnProcessor_flashattn(), single=False, **kw)
        self.norm3_i = operations.LayerNorm(dim, dtype=dtype, device=device, **ln)
        self.ff_i = _block_ffn(dim, num_routed_experts, num_activated_experts, kw)
        self.norm3_t = operations.LayerNorm(dim, **ln)
        self.ff_t = FeedForwardSwiGLU(dim=dim, hidden_dim=4 * dim, **kw)

    def forward(self, image_tokens, image_tokens_masks=None, text_tokens=None, adaln_input=None, rope=None,
                transformer_options={}):
        (shift_msa_i, scale_msa_i, gate_msa_i, shift_mlp_i, scale_mlp_i, gate_mlp_i,
         shift_msa_t, scale_msa_t, gate_msa_t, shift_mlp_t, scale_mlp_t, gate_mlp_t) = \
            self.adaLN_modulation(adaln_input)[:, None].chunk(12, dim=-1)
        normed_i = _modulated_norm(self.norm1_i, image_tokens, shift_msa_i, scale_msa_i)
        normed_t = _modulated_norm(self.norm1_t, text_tokens, shift_msa_t, scale_msa_t)
        attn_i, attn_t = self.attn1(normed_i, image_tokens_masks, normed_t, rope=rope,
                                    transformer_options=transformer_options)
        image_tokens = _gated_residual(attn_i, gate_msa_i, image_tokens)
        text_tokens = _gated_residual(attn_t, gate_msa_t, text_tokens)
        image_tokens = block_feed_forward(self.norm3_i, self.ff_i, image_tokens, shift_mlp_i, scale_mlp_i, gate_mlp_i)
        text_tokens = block_feed_forward(self.norm3_t, self.ff_t, text_tokens, shift_mlp_t, scale_mlp_t, gate_mlp_t)
        return image_tokens, text_tokens


class HiDreamImageBlock(nn.Module):
    """Wrapper the model stacks (``model.py:527-575``): ``.block`` is one of the two classes above."""

    def __init__(self, dim: int, num_attention_heads: int, attention_head_dim: int, num_routed_experts: int = 4,
                 num_activated_experts: int = 2, block_type=BlockType.TransformerBlock, dtype=None, device=None,
                 operations=None):
        super().__init__()
        cls = {BlockType.TransformerBlock: HiDreamImageTransformerBlock,
               BlockType.SingleTransformerBlock: HiDreamImageSingleTransformerBlock}[block_type]
        self.block = cls(dim, num_attention_heads, attention_head_dim, num_routed_experts, num_activated_experts,
                         dtype=dtype, device=device, operations=operations)

    def forward(self, image_tokens, image_tokens_masks=None, text_tokens=None, adaln_input=None, rope=None,
                transformer_options={}):
        return self.block(image_tokens, image_tokens_masks, text_tokens, adaln_input, rope,
                          transformer_options=transformer_options)


# ---------------------------------------------------------------------------------------------------------------
# The model around the blocks (``comfy/ldm/hidream/model.py:21-72, 349-357, 571-829``): embedders, per-layer text
# projections, the block loop with its Llama-state concatenations, final layer.  Same constructor, attribute names and
# state-dict keys as the reference, so a HiDream-I1 checkpoint loads with ``load_state_dict(strict=True)``; the
# forward is the reference's sequence of steps, and every block inside it takes the kernels where it is eligible.
# ---------------------------------------------------------------------------------------------------------------
import math  # noqa: E402
from typing import List, Tuple  # noqa: E402


def rope(pos: torch.Tensor, dim: int, theta: int) -> torch.Tensor:
    """Rotation matrices of one position axis (``comfy/ldm/flux/math.py:23-36``): [..., n] positions ->
    [..., n, dim / 2, 2, 2] fp32 with rows (cos, -sin), (sin, cos); the angles are formed in fp64 frequencies times fp32
    positions, as there."""
    if dim % 2:
        raise ValueError("rope: dim must be even")
    exponent = torch.linspace(0, (dim - 2) / dim, steps=dim // 2, dtype=torch.float64, device=pos.device)
    omega = 1.0 / (theta ** exponent)
    angle = torch.einsum("...n,d->...nd", pos.to(dtype=torch.float32), omega)
    mat = torch.stack([torch.cos(angle), -torch.sin(angle), torch.sin(angle), torch.cos(angle)], dim=-1)
    return mat.reshape(*mat.shape[:-1], 2, 2).to(dtype=torch.float32)


class EmbedND(nn.Module):
    """Rotary table of multi-axis position ids (``model.py:21-33``): ids [B, S, axes] -> [B, S, 1, sum(axes_dim) / 2, 2, 2]."""

    def __init__(self, theta: int, axes_dim: List[int]):
        super().__init__()
        self.theta = theta
        self.axes_dim = axes_dim

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        parts = [rope(ids[..., i], self.axes_dim[i], self.theta) for i in range(ids.shape[-1])]
        return torch.cat(parts, dim=-3).unsqueeze(2)


def _sinusoidal_embedding(timesteps: torch.Tensor, channels: int, flip_sin_to_cos: bool, downscale_freq_shift: float,
                          scale: float = 1, max_period: int = 10000) -> torch.Tensor:
    """``comfy/ldm/lightricks/model.py:13-64``: [N] timesteps -> [N, channels] sinusoidal features in fp32."""
    if timesteps.dim() != 1:
        raise ValueError("timesteps must be one-dimensional")
    half = channels // 2
    exponent = -math.log(max_period) * torch.arange(start=0, end=half, dtype=torch.float32, device=timesteps.device)
    exponent = exponent / (half - downscale_freq_shift)
    emb = scale * (timesteps[:, None].float() * torch.exp(exponent)[None, :])
    emb = torch.cat([torch.sin(emb), torch.cos(emb)], dim=-1)
    if flip_sin_to_cos:
        emb = torch.cat([emb[:, half:], emb[:, :half]], dim=-1)
    if channels % 2 == 1:
        emb = F.pad(emb, (0, 1, 0, 0))
    return emb


class Timesteps(nn.Module):
    """``comfy/ldm/lightricks/model.py:116-132``."""

    def __init__(self, num_channels: int, flip_sin_to_cos: bool, downscale_freq_shift: float, scale: int = 1):
        super().__init__()
        self.num_channels = num_channels
        self.flip_sin_to_cos = flip_sin_to_cos
        self.downscale_freq_shift = downscale_freq_shift
        self.scale = scale

    def forward(self, timesteps):
        return _sinusoidal_embedding(timesteps, self.num_channels, self.flip_sin_to_cos, self.downscale_freq_shift,
                                     self.scale)


class TimestepEmbedding(nn.Module):
    """Linear, SiLU, Linear (``comfy/ldm/lightricks/model.py:67-113``); keys ``linear_1``, ``linear_2`` (``cond_proj``)."""

    def __init__(self, in_channels: int, time_embed_dim: int, act_fn: str = "silu", out_dim: int = None,
                 post_act_fn: Optional[str] = None, cond_proj_dim=None, sample_proj_bias=True, dtype=None, device=None,
                 operations=None):
        super().__init__()
        self.linear_1 = operations.Linear(in_channels, time_embed_dim, sample_proj_bias, dtype=dtype, device=device)
        self.cond_proj = None
        if cond_proj_dim is not None:
            self.cond_proj = operations.Linear(cond_proj_dim, in_channels, bias=False, dtype=dtype, device=device)
        self.act = nn.SiLU()
        self.linear_2 = operations.Linear(time_embed_dim, out_dim if out_dim is not None else time_embed_dim,
                                          sample_proj_bias, dtype=dtype, device=device)
        self.post_act = None

    def forward(self, sample, condition=None):
        if condition is not None:
            sample = sample + self.cond_proj(condition)
        return self.linear_2(self.act(self.linear_1(sample)))


class PatchEmbed(nn.Module):
    """``model.py:36-51``: one Linear over flattened patches; key ``proj``."""

    def __init__(self, patch_size=2, in_channels=4, out_channels=1024, dtype=None, device=None, operations=None):
        super().__init__()
        self.patch_size = patch_size
        self.out_channels = out_channels
        self.proj = operations.Linear(in_channels * patch_size * patch_size, out_channels, bias=True, dtype=dtype,
                                      device=device)

    def forward(self, latent):
        return self.proj(latent)


class PooledEmbed(nn.Module):
    """``model.py:54-60``; key ``pooled_embedder``."""

    def __init__(self, text_emb_dim, hidden_size, dtype=None, device=None, operations=None):
        super().__init__()
        self.pooled_embedder = TimestepEmbedding(in_channels=text_emb_dim, time_embed_dim=hidden_size, dtype=dtype,
                                                 device=device, operations=operations)

    def forward(self, pooled_embed):
        return self.pooled_embedder(pooled_embed)


class TimestepEmbed(nn.Module):
    """``model.py:63-72``; keys ``timestep_embedder.*`` (``time_proj`` has no parameters)."""

    def __init__(self, hidden_size, frequency_embedding_size=256, dtype=None, device=None, operations=None):
        super().__init__()
        self.time_proj = Timesteps(num_channels=frequency_embedding_size, flip_sin_to_cos=True, downscale_freq_shift=0)
        self.timestep_embedder = TimestepEmbedding(in_channels=frequency_embedding_size, time_embed_dim=hidden_size,
                                                   dtype=dtype, device=device, operations=operations)

    def forward(self, timesteps, wdtype):
        return self.timestep_embedder(self.time_proj(timesteps).to(dtype=wdtype))


class TextProjection(nn.Module):
    """``model.py:349-357``: bias-free Linear; key ``linear``."""

    def __init__(self, in_features, hidden_size, dtype=None, device=None, operations=None):
        super().__init__()
        self.linear = operations.Linear(in_features=in_features, out_features=hidden_size, bias=False, dtype=dtype,
                                        device=device)

    def forward(self, caption):
        return self.linear(caption)


class LastLayer(nn.Module):
    """``comfy/ldm/flux/layers.py:264-278``: modulated LayerNorm (``addcmul(shift, norm(x), 1 + scale)``) and the output
    Linear; keys ``linear``, ``adaLN_modulation.1`` (``norm_final`` has no parameters)."""

    def __init__(self, hidden_size: int, patch_size: int, out_channels: int, dtype=None, device=None, operations=None):
        super().__init__()
        self.norm_final = operations.LayerNorm(hidden_size, elementwise_affine=False, eps=1e-6, dtype=dtype, device=device)
        self.linear = operations.Linear(hidden_size, patch_size * patch_size * out_channels, bias=True, dtype=dtype,
                                        device=device)
        self.adaLN_modulation = nn.Sequential(nn.SiLU(), operations.Linear(hidden_size, 2 * hidden_size, bias=True,
                                                                           dtype=dtype, device=device))

    def forward(self, x, vec, modulation_dims=None):
        if vec.ndim == 2:
            vec = vec[:, None, :]
        shift, scale = self.adaLN_modulation(vec).chunk(2, dim=-1)
        if modulation_dims is not None:
            raise NotImplementedError("per-range modulation is not used by HiDream")
        return self.linear(torch.addcmul(shift, self.norm_final(x), 1 + scale))


def pad_to_patch_size(img, patch_size=(2, 2), padding_mode="circular"):
    """``comfy/ldm/common_dit.py:5-13``: pad the trailing spatial dimensions up to multiples of the patch size."""
    pad = ()
    for i in range(img.ndim - 2):
        pad = (0, (patch_size[i] - img.shape[i + 2] % patch_size[i]) % patch_size[i]) + pad
    return F.pad(img, pad, mode=padding_mode)


class HiDreamImageTransformer2DModel(nn.Module):
    """The HiDream-I1 diffusion transformer (``model.py:571-829``): one call = one denoising step.

    forward(x [B, C, H, W] latent, t [B] timesteps, y [B, text_emb_dim] pooled embedding, context [B, S_t5, C_t5],
    encoder_hidden_states_llama3 [B, L, S_llama, C_llama]) -> [B, C_out, H, W]."""

    def __init__(self, patch_size: Optional[int] = None, in_channels: int = 64, out_channels: Optional[int] = None,
                 num_layers: int = 16, num_single_layers: int = 32, attention_head_dim: int = 128,
                 num_attention_heads: int = 20, caption_channels: List[int] = None, text_emb_dim: int = 2048,
                 num_routed_experts: int = 4, num_activated_experts: int = 2, axes_dims_rope: Tuple[int, int] = (32, 32),
                 max_resolution: Tuple[int, int] = (128, 128), llama_layers: List[int] = None, image_model=None,
                 dtype=None, device=None, operations=None):
        super().__init__()
        self.patch_size = patch_size
        self.num_attention_heads = num_attention_heads
        self.attention_head_dim = attention_head_dim
        self.num_layers = num_layers
        self.num_single_layers = num_single_layers
        self.gradient_checkpointing = False
        self.dtype = dtype
        self.out_channels = out_channels or in_channels
        self.inner_dim = num_attention_heads * attention_head_dim
        self.llama_layers = llama_layers
        kw = dict(dtype=dtype, device=device, operations=operations)

        self.t_embedder = TimestepEmbed(self.inner_dim, **kw)
        self.p_embedder = PooledEmbed(text_emb_dim, self.inner_dim, **kw)
        self.x_embedder = PatchEmbed(patch_size=patch_size, in_channels=in_channels, out_channels=self.inner_dim, **kw)
        self.pe_embedder = EmbedND(theta=10000, axes_dim=axes_dims_rope)

        def blocks(count, block_type):
            return nn.ModuleList([
                HiDreamImageBlock(dim=self.inner_dim, num_attention_heads=num_attention_heads,
                                  attention_head_dim=attention_head_dim, num_routed_experts=num_routed_experts,
                                  num_activated_experts=num_activated_experts, block_type=block_type, **kw)
                for _ in range(count)])

        self.double_stream_blocks = blocks(num_layers, BlockType.TransformerBlock)
        self.single_stream_blocks = blocks(num_single_layers, BlockType.SingleTransformerBlock)
        self.final_layer = LastLayer(self.inner_dim, patch_size, self.out_channels, **kw)
        # one projection per block for that block's Llama layer, and a last one for the T5 states
        widths = [caption_channels[1]] * (num_layers + num_single_layers) + [caption_channels[0]]
        self.caption_projection = nn.ModuleList([TextProjection(in_features=w, hidden_size=self.inner_dim, **kw)
                                                 for w in widths])
        self.max_seq = max_resolution[0] * max_resolution[1] // (patch_size * patch_size)

    def expand_timesteps(self, timesteps, batch_size, device):
        if not torch.is_tensor(timesteps):
            dtype = torch.float64 if isinstance(timesteps, float) else torch.int64
            timesteps = torch.tensor([timesteps], dtype=dtype, device=device)
        elif timesteps.dim() == 0:
            timesteps = timesteps[None].to(device)
        return timesteps.expand(batch_size)

    def patchify(self, x, max_seq, img_sizes=None):
        """[B, C, H, W] -> [B, (H / p)(W / p), p p C] (patch pixels outermost, channels innermost), as ``:682-705``."""
        if not isinstance(x, torch.Tensor) or img_sizes is not None:
            raise NotImplementedError("only same-size batches given as one tensor are supported")
        p = self.patch_size
        b, c, h, w = x.shape
        ph, pw = h // p, w // p
        x = x.reshape(b, c, ph, p, pw, p).permute(0, 2, 4, 3, 5, 1).reshape(b, ph * pw, p * p * c)
        return x, None, [[ph, pw]] * b

    def unpatchify(self, x: torch.Tensor, img_sizes) -> torch.Tensor:
        p = self.patch_size
        out = []
        for i, (ph, pw) in enumerate(img_sizes):
            tile = x[i, :ph * pw].reshape(1, ph, pw, p, p, -1)
            out.append(tile.permute(0, 5, 1, 3, 2, 4).reshape(1, -1, ph * p, pw * p))
        return torch.cat(out, dim=0)

    def forward(self, x, t, y=None, context=None, encoder_hidden_states_llama3=None, image_cond=None, control=None,
                transformer_options={}):
        return self._forward(x, t, y, context, encoder_hidden_states_llama3, image_cond, control, transformer_options)

    def _forward(self, x, t, y=None, context=None, encoder_hidden_states_llama3=None, image_cond=None, control=None,
                 transformer_options={}):
        bs, c, h, w = x.shape
        if image_cond is not None:
            x = torch.cat([x, image_cond], dim=-1)
        latent = pad_to_patch_size(x, (self.patch_size, self.patch_size))
        batch, wdtype, dev = latent.shape[0], latent.dtype, latent.device

        # conditioning vector of every block's adaLN: timestep embedding + pooled text embedding
        adaln_input = self.t_embedder(self.expand_timesteps(t, batch, dev), wdtype) + self.p_embedder(y)

        tokens, masks, img_sizes = self.patchify(latent, self.max_seq)
        ph, pw = img_sizes[0]
        img_ids = torch.zeros(ph, pw, 3, device=dev)
        img_ids[..., 1] += torch.arange(ph, device=dev)[:, None]
        img_ids[..., 2] += torch.arange(pw, device=dev)[None, :]
        img_ids = img_ids.reshape(1, ph * pw, 3).expand(batch, -1, -1)
        tokens = self.x_embedder(tokens)

        # text states: one Llama layer per block (projected by that block's own Linear), then T5 last
        llama = encoder_hidden_states_llama3.movedim(1, 0)
        text = [self.caption_projection[i](llama[k]).view(batch, -1, tokens.shape[-1])
                for i, k in enumerate(self.llama_layers)]
        text.append(self.caption_projection[-1](context).view(batch, -1, tokens.shape[-1]))

        n_text = text[-1].shape[1] + text[-2].shape[1] + text[0].shape[1]
        txt_ids = torch.zeros(batch, n_text, 3, device=dev, dtype=img_ids.dtype)
        rope_table = self.pe_embedder(torch.cat((img_ids, txt_ids), dim=1))

        block_id = 0
        carried = torch.cat([text[-1], text[-2]], dim=1)          # T5 and the last Llama layer travel through the blocks
        carried_len = carried.shape[1]
        for block in self.double_stream_blocks:
            cur = torch.cat([carried, text[block_id]], dim=1)
            tokens, carried = block(image_tokens=tokens, image_tokens_masks=masks, text_tokens=cur,
                                    adaln_input=adaln_input, rope=rope_table, transformer_options=transformer_options)
            carried = carried[:, :carried_len]
            block_id += 1

        n_image = tokens.shape[1]
        tokens = torch.cat([tokens, carried], dim=1)
        joint_len = tokens.shape[1]
        for block in self.single_stream_blocks:
            tokens = torch.cat([tokens, text[block_id]], dim=1)
            tokens = block(image_tokens=tokens, image_tokens_masks=masks, text_tokens=None, adaln_input=adaln_input,
                           rope=rope_table, transformer_options=transformer_options)
            tokens = tokens[:, :joint_len]
            block_id += 1

        out = self.final_layer(tokens[:, :n_image, ...], adaln_input)
        return -self.unpatchify(out, img_sizes)[:, :, :h, :w]
