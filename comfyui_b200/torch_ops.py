"""torch.library registration of the C-ABI kernels (namespace ``comfyui_b200``).

The dispatch shim in ``comfyui_b200.ops`` calls these ops, so the layer shows up in PyTorch's dispatcher like any
other operator: it can be traced (fake / meta implementations give shapes and dtypes without touching a GPU), and
profilers attribute its time to one named op.  The real implementations only marshal pointers into the shared
library; there is no PyTorch arithmetic behind them.

Weights travel as lists with one entry per routed expert followed by the shared expert (E + 1 entries):
``w1``, ``w3``, ``w2`` and, for scaled fp8, ``scale_w1``, ``scale_w3``, ``scale_w2`` (fp32 scalars; empty lists for bf16)
plus ``scale_in13`` / ``scale_in2`` (either empty, or E + 1 entries).
"""
from __future__ import annotations

import weakref
from collections import OrderedDict
from typing import List, Optional, Sequence

import torch

from . import moe_ops

# Packs (ctypes structs + the tensors they point into) by the identity and version of every tensor.  The packs the
# dispatch shim builds belong to their module (cached on it, dropped with it, or when its weights move); this table
# only finds them again from the operator's tensor arguments and must not keep them, or their weights, alive: after a
# model has been unloaded its expert weights (23 GB for a HiDream-I1) would otherwise stay on the GPU.  Packs made for
# direct calls of the operators (no module behind them) are kept in a two-entry table of their own.
_packs = weakref.WeakValueDictionary()
_direct_packs = OrderedDict()
_DIRECT_SLOTS = 2


def _remember(table: OrderedDict, key, value) -> None:
    while len(table) >= _DIRECT_SLOTS:
        table.popitem(last=False)
    table[key] = value


def _key(tensors: Sequence[torch.Tensor]):
    return tuple((t.data_ptr(), 0 if t.is_inference() else t._version, t.dtype, tuple(t.shape),
                  t.stride(0) if t.dim() else 0) for t in tensors)


def _opt(lst: List[torch.Tensor], i: int) -> Optional[torch.Tensor]:
    return lst[i] if lst else None


def _layer(gate, w1, w3, w2, scale_w1, scale_w3, scale_w2, scale_in13, scale_in2) -> moe_ops.LayerPack:
    """LayerPack for these tensors, cached on their identity and version."""
    all_t = [gate, *w1, *w3, *w2, *scale_w1, *scale_w3, *scale_w2, *scale_in13, *scale_in2]
    key = _key(all_t)
    hit = _packs.get(key)
    if hit is not None:
        return hit
    ffns = [moe_ops.FfnPack(w1[i], w3[i], w2[i], scale_w1=_opt(scale_w1, i), scale_w3=_opt(scale_w3, i),
                            scale_w2=_opt(scale_w2, i), scale_in13=_opt(scale_in13, i), scale_in2=_opt(scale_in2, i))
            for i in range(len(w1))]
    layer = moe_ops.LayerPack(gate, ffns[:-1], ffns[-1], top_k=2)
    _packs[key] = layer
    _remember(_direct_packs, key, layer)
    return layer


def register(layer) -> tuple:
    """Makes a pack the dispatch shim built findable from the operator's arguments (without keeping it alive) and
    returns those list arguments."""
    if isinstance(layer, moe_ops.MlpLayerPack):
        args = mlp_layer_args(layer)
        _mlp_packs[_key([layer.gate, *args[0], *args[1], *args[2], *args[3]])] = layer
    else:
        args = layer_args(layer)
        _packs[_key([layer.gate] + [t for lst in args for t in lst])] = layer
    return args


_workspaces = {}


def _workspace(layer: moe_ops.LayerPack, n_tokens: int) -> moe_ops.Workspace:
    key = (n_tokens, layer.dim, layer.n_experts, layer.experts[0].hidden, layer.shared.hidden, layer.fp8,
           layer.gate.device, torch.cuda.current_stream().cuda_stream)
    ws = _workspaces.get(key)
    if ws is None:
        while len(_workspaces) >= 4:
            _workspaces.pop(next(iter(_workspaces)))
        ws = moe_ops.Workspace.for_layer(layer, n_tokens)
        _workspaces[key] = ws
    return ws


def release_workspaces() -> None:
    """Drops the device workspaces (0.5 GB at 8192 tokens, shared by all layers) and every pack this module holds."""
    _workspaces.clear()
    _packs.clear()
    _direct_packs.clear()
    _mlp_packs.clear()
    _direct_mlp_packs.clear()


@torch.library.custom_op("comfyui_b200::hidream_moe", mutates_args=())
def hidream_moe(x: torch.Tensor, gate: torch.Tensor, w1: List[torch.Tensor], w3: List[torch.Tensor],
                w2: List[torch.Tensor], scale_w1: List[torch.Tensor], scale_w3: List[torch.Tensor],
                scale_w2: List[torch.Tensor], scale_in13: List[torch.Tensor],
                scale_in2: List[torch.Tensor]) -> torch.Tensor:
    """MOEFeedForwardSwiGLU.forward on x [N, D] (bf16, contiguous, CUDA)."""
    layer = _layer(gate, w1, w3, w2, scale_w1, scale_w3, scale_w2, scale_in13, scale_in2)
    return moe_ops.moe_forward(layer, x, _workspace(layer, x.shape[0]))


@hidream_moe.register_fake
def _(x, gate, w1, w3, w2, scale_w1, scale_w3, scale_w2, scale_in13, scale_in2):
    return torch.empty_like(x)


@torch.library.custom_op("comfyui_b200::hidream_moe_block", mutates_args=())
def hidream_moe_block(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor, gate_mlp: torch.Tensor,
                      tokens_per_batch: int, eps: float, gate: torch.Tensor, w1: List[torch.Tensor],
                      w3: List[torch.Tensor], w2: List[torch.Tensor], scale_w1: List[torch.Tensor],
                      scale_w3: List[torch.Tensor], scale_w2: List[torch.Tensor], scale_in13: List[torch.Tensor],
                      scale_in2: List[torch.Tensor]) -> torch.Tensor:
    """gate_mlp * MoE(LayerNorm(x) * (1 + scale) + shift) + x on x [N, D]."""
    layer = _layer(gate, w1, w3, w2, scale_w1, scale_w3, scale_w2, scale_in13, scale_in2)
    return moe_ops.moe_ffn_block(layer, x, shift, scale, gate_mlp, tokens_per_batch, eps, _workspace(layer, x.shape[0]))


@hidream_moe_block.register_fake
def _(x, shift, scale, gate_mlp, tokens_per_batch, eps, gate, w1, w3, w2, scale_w1, scale_w3, scale_w2, scale_in13,
      scale_in2):
    return torch.empty_like(x)


@torch.library.custom_op("comfyui_b200::hidream_gate", mutates_args=())
def hidream_gate(x: torch.Tensor, gate: torch.Tensor) -> List[torch.Tensor]:
    """MoEGate.forward on x [N, D]: [topk_idx int64 [N, 2], topk_weight fp32 [N, 2]]."""
    idx, weight, _, _, _ = moe_ops.gate_topk(x, gate)
    return [idx.to(torch.int64), weight]


@hidream_gate.register_fake
def _(x, gate):
    n = x.shape[0]
    return [x.new_empty((n, 2), dtype=torch.int64), x.new_empty((n, 2), dtype=torch.float32)]


_mlp_packs = weakref.WeakValueDictionary()
_direct_mlp_packs = OrderedDict()


def _mlp_layer(gate, w1, b1, w2, b2) -> moe_ops.MlpLayerPack:
    """MlpLayerPack for these tensors, cached on their identity and version."""
    key = _key([gate, *w1, *b1, *w2, *b2])
    hit = _mlp_packs.get(key)
    if hit is not None:
        return hit
    ffns = [moe_ops.MlpPack(w1[i], _opt(b1, i), w2[i], _opt(b2, i)) for i in range(len(w1))]
    layer = moe_ops.MlpLayerPack(gate, ffns[:-1], ffns[-1], top_k=2)
    _mlp_packs[key] = layer
    _remember(_direct_mlp_packs, key, layer)
    return layer


@torch.library.custom_op("comfyui_b200::hunyuan3d_moe", mutates_args=())
def hunyuan3d_moe(x: torch.Tensor, gate: torch.Tensor, w1: List[torch.Tensor], b1: List[torch.Tensor],
                  w2: List[torch.Tensor], b2: List[torch.Tensor]) -> torch.Tensor:
    """MoEBlock.forward (eval) of Hunyuan3D-2.1 on x [N, D] (bf16, contiguous, CUDA).  Weight lists hold the routed
    experts followed by the shared expert; the bias lists are either empty or of the same length."""
    layer = _mlp_layer(gate, w1, b1, w2, b2)
    return moe_ops.moe_mlp_forward(layer, x, _workspace(layer, x.shape[0]))


@hunyuan3d_moe.register_fake
def _(x, gate, w1, b1, w2, b2):
    return torch.empty_like(x)


def mlp_layer_args(layer: moe_ops.MlpLayerPack):
    """The list arguments of hunyuan3d_moe for an MlpLayerPack (routed experts first, shared expert last)."""
    ffns = list(layer.experts) + [layer.shared]

    def col(name):
        vals = [getattr(f, name) for f in ffns]
        return [] if any(v is None for v in vals) else vals

    return [f.w1 for f in ffns], col("b1"), [f.w2 for f in ffns], col("b2")


def layer_args(layer: moe_ops.LayerPack):
    """The list arguments of the ops above for a LayerPack (routed experts first, shared expert last)."""
    ffns = list(layer.experts) + [layer.shared]

    def col(name):
        vals = [getattr(f, name) for f in ffns]
        if all(v is None for v in vals):
            return []
        if any(v is None for v in vals):
            raise ValueError(f"{name} is set on some feed-forwards of the layer and missing on others: the operator's "
                             "list arguments cannot express that")
        return vals

    return ([f.w1 for f in ffns], [f.w3 for f in ffns], [f.w2 for f in ffns], col("scale_w1"), col("scale_w3"),
            col("scale_w2"), col("scale_in13"), col("scale_in2"))
