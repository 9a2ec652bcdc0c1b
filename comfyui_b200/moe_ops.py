"""Tensor-level wrappers around the C ABI (include/comfy_b200_moe.h).

PyTorch is used for device memory and streams only: every function here passes raw device pointers
of tensors it was given (or of workspaces it allocated through torch's caching allocator) to the
shared library and launches on ``torch.cuda.current_stream()``.  None of them has a PyTorch or CPU
implementation behind it.
"""
from __future__ import annotations

import ctypes
import weakref
from dataclasses import dataclass, field
from typing import Optional, Sequence, Tuple

import torch

from . import _native as N

_FP8 = torch.float8_e4m3fn


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return N.BF16
    if dt == torch.float32:
        return N.FP32
    if dt == _FP8:
        return N.FP8_E4M3
    raise ValueError(f"unsupported dtype {dt}")


def _need_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("the sm_100a kernels need CUDA tensors; there is no CPU path")


# Status words (int32 [2]: [0] the sticky device status word, [1] a near-tie counter) that calls of this module
# have used and nobody has dropped yet; check_all_status() reads them all.
_status_words = weakref.WeakSet()
_device_status = {}


def device_status(device) -> torch.Tensor:
    """The status word shared by every call on `device` that brings no workspace of its own (dense feed-forwards)."""
    key = str(device)
    st = _device_status.get(key)
    if st is None:
        st = torch.zeros((N.STATUS_WORDS,), dtype=torch.int32, device=device)
        _device_status[key] = st
        _status_words.add(st)
    return st


def check_all_status() -> None:
    """Reads every live status word (one stream synchronisation each) and raises for the first code found.  Status
    words are sticky, so calling this once after a model forward covers every layer of it."""
    for st in list(_status_words):
        read_status(st)


def plan_sizes(n_tokens: int, n_experts: int, top_k: int = 2) -> Tuple[int, int]:
    """(rows_cap, n_blocks) for the permuted buffers and the per-block count scratch."""
    rows = ctypes.c_int64()
    blocks = ctypes.c_int()
    N.check("comfy_moe_plan_sizes", N.load().comfy_moe_plan_sizes(n_tokens, n_experts, top_k, rows, blocks))
    return rows.value, blocks.value


# --------------------------------------------------------------------------------------- weights
@dataclass
class FfnPack:
    """Device pointers of one FeedForwardSwiGLU; keeps the tensors alive."""

    w1: torch.Tensor
    w3: torch.Tensor
    w2: torch.Tensor
    scale_w1: Optional[torch.Tensor] = None
    scale_w3: Optional[torch.Tensor] = None
    scale_w2: Optional[torch.Tensor] = None
    scale_in13: Optional[torch.Tensor] = None
    scale_in2: Optional[torch.Tensor] = None
    max_sms: int = 0        # 0 = all; see ComfyMoeFfnWeights.max_sms

    def __post_init__(self):
        _need_cuda(self.w1, self.w2, self.w3)
        for w in (self.w1, self.w2, self.w3):
            if w.dim() != 2 or w.stride(1) != 1:
                raise ValueError("expert weights must be 2-D with a contiguous last dimension")
        if self.w1.shape != self.w3.shape or self.w1.stride(0) != self.w3.stride(0):
            raise ValueError("w1 and w3 must share shape and leading dimension")
        if self.w2.shape != (self.w1.shape[1], self.w1.shape[0]):
            raise ValueError("w2 must be [dim, hidden]")
        for s in (self.scale_w1, self.scale_w3, self.scale_w2, self.scale_in13, self.scale_in2):
            if s is not None and (s.dtype != torch.float32 or s.numel() != 1 or not s.is_cuda):
                raise ValueError("scales must be fp32 scalars on the device")

    @property
    def hidden(self) -> int:
        return self.w1.shape[0]

    @property
    def dim(self) -> int:
        return self.w1.shape[1]

    def fill(self, s: N.FfnWeights) -> None:
        s.w1, s.w3, s.w2 = self.w1.data_ptr(), self.w3.data_ptr(), self.w2.data_ptr()
        s.ld13, s.ld2 = self.w1.stride(0), self.w2.stride(0)
        s.hidden = self.hidden
        s.max_sms = self.max_sms
        for name in ("scale_w1", "scale_w3", "scale_w2", "scale_in13", "scale_in2"):
            t = getattr(self, name)
            setattr(s, name, None if t is None else t.data_ptr())

    def struct(self) -> N.FfnWeights:
        s = N.FfnWeights()
        self.fill(s)
        return s


@dataclass
class LayerPack:
    """Everything comfy_moe_forward needs to know about one MOEFeedForwardSwiGLU."""

    gate: torch.Tensor
    experts: Sequence[FfnPack]
    shared: FfnPack
    top_k: int = 2
    c_layer: N.Layer = field(init=False)

    def __post_init__(self):
        _need_cuda(self.gate)
        if not self.gate.is_contiguous():
            raise ValueError("gate weight must be contiguous")
        L = N.Layer()
        L.dim = self.gate.shape[1]
        L.n_experts = len(self.experts)
        L.top_k = self.top_k
        L.w_dtype = _dtype_code(self.experts[0].w1.dtype)
        L.gate_dtype = _dtype_code(self.gate.dtype)
        L.w_gate = self.gate.data_ptr()
        for i, e in enumerate(self.experts):
            e.fill(L.experts[i])
        self.shared.fill(L.shared)
        self.c_layer = L

    @property
    def dim(self) -> int:
        return self.gate.shape[1]

    @property
    def n_experts(self) -> int:
        return len(self.experts)

    @property
    def fp8(self) -> bool:
        return self.experts[0].w1.dtype == _FP8


# --------------------------------------------------------------------------------------- workspace
class Workspace:
    """Device buffers for one call of the layer at a given token count.  Owned by the caller."""

    def __init__(self, n_tokens: int, dim: int, n_experts: int, hidden: int, hidden_shared: int, fp8: bool,
                 device: torch.device, top_k: int = 2):
        self.n_tokens, self.dim, self.n_experts = n_tokens, dim, n_experts
        self.hidden, self.hidden_shared, self.fp8 = hidden, hidden_shared, fp8
        rows_cap, n_blocks = plan_sizes(n_tokens, n_experts, top_k)
        self.rows_cap, self.n_blocks = rows_cap, n_blocks
        act = _FP8 if fp8 else torch.bfloat16
        i32 = dict(dtype=torch.int32, device=device)
        self.topk_idx = torch.empty((n_tokens, top_k), **i32)
        self.topk_weight = torch.empty((n_tokens, top_k), dtype=torch.float32, device=device)
        self.block_counts = torch.empty((max(n_blocks, 1), n_experts), **i32)
        self.block_offsets = torch.empty((max(n_blocks, 1), n_experts), **i32)
        self.expert_counts = torch.zeros((n_experts,), **i32)
        self.expert_offsets = torch.zeros((n_experts + 1,), **i32)
        self.row_map = torch.empty((n_tokens, top_k), **i32)
        self.status = torch.zeros((N.STATUS_WORDS,), **i32)
        _status_words.add(self.status)
        self.x_perm = torch.empty((rows_cap, dim), dtype=act, device=device)
        self.x_q = torch.empty((n_tokens, dim), dtype=act, device=device) if fp8 else None
        self.h_perm = torch.empty((rows_cap, hidden), dtype=act, device=device)
        self.y_perm = torch.empty((rows_cap, dim), dtype=torch.bfloat16, device=device)
        self.h_shared = torch.empty((max(n_tokens, 1), hidden_shared), dtype=act, device=device)
        self.y_shared = torch.empty((max(n_tokens, 1), dim), dtype=torch.bfloat16, device=device)
        self.x_mod = None          # allocated on first use by moe_ffn_block
        ws = N.Workspace()
        for name in ("topk_idx", "topk_weight", "block_counts", "block_offsets", "expert_counts", "expert_offsets",
                     "row_map", "status", "x_perm", "x_q", "h_perm", "y_perm", "h_shared", "y_shared"):
            t = getattr(self, name)
            setattr(ws, name, None if t is None else t.data_ptr())
        ws.rows_cap = rows_cap
        ws.x_mod = None
        self.c_ws = ws

    def need_x_mod(self) -> None:
        if self.x_mod is None:
            self.x_mod = torch.empty((max(self.n_tokens, 1), self.dim), dtype=torch.bfloat16, device=self.x_perm.device)
            self.c_ws.x_mod = self.x_mod.data_ptr()

    @classmethod
    def for_layer(cls, layer: LayerPack, n_tokens: int) -> "Workspace":
        return cls(n_tokens, layer.dim, layer.n_experts, layer.experts[0].hidden, layer.shared.hidden, layer.fp8,
                   layer.gate.device, layer.top_k)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in vars(self).values() if isinstance(t, torch.Tensor))


# --------------------------------------------------------------------------------------- kernels
def gate_topk(x: torch.Tensor, w_gate: torch.Tensor, *, neartie_eps: float = 1e-6, want_flags: bool = False,
              topk_idx: Optional[torch.Tensor] = None, topk_weight: Optional[torch.Tensor] = None,
              block_counts: Optional[torch.Tensor] = None):
    """Fused MoEGate.forward.  x: bf16 [N, D] contiguous; w_gate: bf16 or fp32 [E, D].

    Returns (topk_idx int32 [N,2], topk_weight fp32 [N,2], block_counts int32 [n_blocks,E],
    neartie_count int32 [1], neartie_flags uint8 [N] or None).
    """
    _need_cuda(x, w_gate)
    if x.dtype != torch.bfloat16 or x.dim() != 2 or not x.is_contiguous():
        raise ValueError("x must be a contiguous bf16 [N, D] tensor")
    n, d = x.shape
    e = w_gate.shape[0]
    w_gate = w_gate.contiguous()
    _, n_blocks = plan_sizes(n, e)
    dev = x.device
    if topk_idx is None:
        topk_idx = torch.empty((n, 2), dtype=torch.int32, device=dev)
    if topk_weight is None:
        topk_weight = torch.empty((n, 2), dtype=torch.float32, device=dev)
    if block_counts is None:
        block_counts = torch.empty((max(n_blocks, 1), e), dtype=torch.int32, device=dev)
    count = torch.zeros((1,), dtype=torch.int32, device=dev)
    flags = torch.zeros((n,), dtype=torch.uint8, device=dev) if want_flags else None
    rc = N.load().comfy_moe_gate_topk(_ptr(x), _ptr(w_gate), _dtype_code(w_gate.dtype), n, d, e, 2, _ptr(topk_idx),
                                      _ptr(topk_weight), _ptr(block_counts), _ptr(count), _ptr(flags),
                                      float(neartie_eps), _stream())
    N.check("comfy_moe_gate_topk", rc)
    return topk_idx, topk_weight, block_counts, count, flags


def route_count(topk_idx: torch.Tensor, n_experts: int) -> torch.Tensor:
    """Per-block expert counts of caller-supplied int32 routing [N, 2] (what the gate kernel emits itself)."""
    _need_cuda(topk_idx)
    if topk_idx.dtype != torch.int32 or not topk_idx.is_contiguous():
        raise ValueError("topk_idx must be a contiguous int32 tensor")
    n = topk_idx.numel() // 2
    _, n_blocks = plan_sizes(n, n_experts)
    block_counts = torch.empty((max(n_blocks, 1), n_experts), dtype=torch.int32, device=topk_idx.device)
    rc = N.load().comfy_moe_route_count(_ptr(topk_idx), n, n_experts, _ptr(block_counts), _stream())
    N.check("comfy_moe_route_count", rc)
    return block_counts


def route_plan(block_counts: torch.Tensor, n_tokens: int, n_experts: int):
    """Per-expert scan of the block counts.  Returns (block_offsets, expert_counts, expert_offsets)."""
    _need_cuda(block_counts)
    dev = block_counts.device
    block_offsets = torch.empty_like(block_counts)
    expert_counts = torch.empty((n_experts,), dtype=torch.int32, device=dev)
    expert_offsets = torch.empty((n_experts + 1,), dtype=torch.int32, device=dev)
    rc = N.load().comfy_moe_route_plan(_ptr(block_counts), n_tokens, n_experts, _ptr(block_offsets),
                                       _ptr(expert_counts), _ptr(expert_offsets), _stream())
    N.check("comfy_moe_route_plan", rc)
    return block_offsets, expert_counts, expert_offsets


def permute(x: torch.Tensor, topk_idx: torch.Tensor, block_offsets: torch.Tensor, expert_offsets: torch.Tensor,
            n_experts: int, *, fp8: bool = False, act_scale: Optional[torch.Tensor] = None,
            xq_scale: Optional[torch.Tensor] = None, want_xq: bool = False, zero_fill: bool = False,
            overflow_count: Optional[torch.Tensor] = None):
    """Row permutation into per-expert blocks.  Returns (x_perm, row_map, x_q or None).  ``overflow_count`` (int32 [1],
    fp8 with a scale only) grows by the number of elements the reference's unclamped cast turns into NaN."""
    _need_cuda(x, topk_idx)
    n, d = x.shape
    rows_cap, _ = plan_sizes(n, n_experts)
    act = _FP8 if fp8 else torch.bfloat16
    alloc = torch.zeros if zero_fill else torch.empty
    x_perm = alloc((rows_cap, d), dtype=act, device=x.device) if not fp8 else \
        alloc((rows_cap, d), dtype=torch.uint8, device=x.device).view(_FP8)
    row_map = torch.empty((n, 2), dtype=torch.int32, device=x.device)
    x_q = torch.empty((n, d), dtype=_FP8, device=x.device) if (fp8 and want_xq) else None
    rc = N.load().comfy_moe_permute(_ptr(x), _ptr(topk_idx), _ptr(block_offsets), _ptr(expert_offsets), n, d,
                                    n_experts, N.FP8_E4M3 if fp8 else N.BF16, _ptr(act_scale), _ptr(x_perm),
                                    _ptr(x_q), _ptr(xq_scale), _ptr(row_map), _ptr(overflow_count), _stream())
    N.check("comfy_moe_permute", rc)
    return x_perm, row_map, x_q


def plan_permute(x: torch.Tensor, topk_idx: torch.Tensor, block_counts: torch.Tensor, n_experts: int, *,
                 fp8: bool = False, zero_fill: bool = False):
    """route_plan + permute in one launch.  Returns (x_perm, row_map, expert_counts, expert_offsets)."""
    _need_cuda(x, topk_idx, block_counts)
    n, d = x.shape
    dev = x.device
    rows_cap, _ = plan_sizes(n, n_experts)
    alloc = torch.zeros if zero_fill else torch.empty
    x_perm = alloc((rows_cap, d), dtype=torch.uint8, device=dev).view(_FP8) if fp8 else \
        alloc((rows_cap, d), dtype=torch.bfloat16, device=dev)
    row_map = torch.empty((n, 2), dtype=torch.int32, device=dev)
    scratch = torch.empty_like(block_counts)
    counts = torch.empty((n_experts,), dtype=torch.int32, device=dev)
    offsets = torch.empty((n_experts + 1,), dtype=torch.int32, device=dev)
    rc = N.load().comfy_moe_plan_permute(_ptr(x), _ptr(topk_idx), _ptr(block_counts), n, d, n_experts,
                                         N.FP8_E4M3 if fp8 else N.BF16, None, _ptr(scratch), _ptr(counts),
                                         _ptr(offsets), _ptr(x_perm), None, None, _ptr(row_map), None, _stream())
    N.check("comfy_moe_plan_permute", rc)
    return x_perm, row_map, counts, offsets


def grouped_swiglu(experts: Sequence[FfnPack], shared: Optional[FfnPack], row_start: Optional[torch.Tensor],
                   row_count: Optional[torch.Tensor], x_perm: Optional[torch.Tensor],
                   x_shared: Optional[torch.Tensor], *, status: Optional[torch.Tensor] = None,
                   check_status: bool = True, h_perm: Optional[torch.Tensor] = None,
                   y_perm: Optional[torch.Tensor] = None, h_shared: Optional[torch.Tensor] = None,
                   y_shared: Optional[torch.Tensor] = None):
    """Both passes of the grouped expert GEMM.  Group g = rows [row_start[g], row_start[g] + row_count[g]) of
    x_perm with the weights experts[g] (int32 device tensors; the routing plan's expert_offsets and
    expert_counts on one GPU).  ``h_perm`` / ``y_perm`` may be given (buffers of x_perm's row count, e.g. a result
    buffer that peers read), and so may ``h_shared`` / ``y_shared`` ([n_tokens, hidden_s] / [n_tokens, dim]);
    otherwise they are allocated.  Returns (y_perm or None, y_shared or None, h_perm, h_shared)."""
    ref = experts[0] if experts else shared
    dim, fp8 = ref.dim, ref.w1.dtype == _FP8
    dev = ref.w1.device
    act = _FP8 if fp8 else torch.bfloat16
    n_e = len(experts)
    arr = (N.FfnWeights * max(n_e, 1))()
    for i, e in enumerate(experts):
        e.fill(arr[i])
    rows_cap = 0 if x_perm is None else x_perm.shape[0]
    if n_e:
        if h_perm is None:
            h_perm = torch.empty((rows_cap, experts[0].hidden), dtype=act, device=dev)
        if y_perm is None:
            y_perm = torch.empty((rows_cap, dim), dtype=torch.bfloat16, device=dev)
        if h_perm.shape != (rows_cap, experts[0].hidden) or y_perm.shape != (rows_cap, dim) or \
                not h_perm.is_contiguous() or not y_perm.is_contiguous():
            raise ValueError("h_perm / y_perm must be contiguous buffers with x_perm's row count")
    else:
        h_perm = y_perm = None
    n_tokens = 0 if x_shared is None else x_shared.shape[0]
    sh = h_sh = y_sh = None
    if shared is not None and n_tokens > 0:
        sh = shared.struct()
        h_sh = h_shared if h_shared is not None else torch.empty((n_tokens, shared.hidden), dtype=act, device=dev)
        y_sh = y_shared if y_shared is not None else torch.empty((n_tokens, dim), dtype=torch.bfloat16, device=dev)
        if h_sh.shape != (n_tokens, shared.hidden) or y_sh.shape != (n_tokens, dim) or not h_sh.is_contiguous() or \
                not y_sh.is_contiguous():
            raise ValueError("h_shared / y_shared must be contiguous [n_tokens, hidden] / [n_tokens, dim] buffers")
    if status is None:
        status = device_status(dev)
    rc = N.load().comfy_moe_grouped_swiglu(
        N.FP8_E4M3 if fp8 else N.BF16, n_e, arr, ctypes.byref(sh) if sh is not None else None,
        _ptr(row_start), _ptr(row_count), rows_cap, n_tokens, dim, _ptr(x_perm), _ptr(h_perm), _ptr(y_perm), _ptr(x_shared),
        _ptr(h_sh), _ptr(y_sh), _ptr(status), _stream())
    N.check("comfy_moe_grouped_swiglu", rc)
    if check_status:
        read_status(status)
    return y_perm, y_sh, h_perm, h_sh


def grouped_swiglu_scatter(groups: Sequence[FfnPack], row_start: torch.Tensor, row_count: torch.Tensor,
                           x_perm: torch.Tensor, h_perm: torch.Tensor, y_out_ptrs: Sequence[int],
                           y_row_shift: torch.Tensor, y_rows_cap: int, status: torch.Tensor) -> None:
    """Both passes of the grouped expert GEMM over routed groups, group i's results written to the buffer at address
    ``y_out_ptrs[i]`` (bf16 [y_rows_cap, dim], possibly another GPU's memory) at row + y_row_shift[i]."""
    n_g = len(groups)
    if len(y_out_ptrs) != n_g:
        raise ValueError("one output buffer per group")
    fp8 = groups[0].w1.dtype == _FP8
    arr = (N.FfnWeights * n_g)()
    for i, e in enumerate(groups):
        e.fill(arr[i])
    outs = (ctypes.c_void_p * n_g)(*[int(p) for p in y_out_ptrs])
    rc = N.load().comfy_moe_grouped_swiglu_scatter(
        N.FP8_E4M3 if fp8 else N.BF16, n_g, arr, _ptr(row_start), _ptr(row_count), x_perm.shape[0], groups[0].dim,
        _ptr(x_perm), _ptr(h_perm), outs, _ptr(y_row_shift), y_rows_cap, _ptr(status), _stream())
    N.check("comfy_moe_grouped_swiglu_scatter", rc)


def combine(y_perm: torch.Tensor, row_map: torch.Tensor, topk_weight: torch.Tensor,
            y_shared: Optional[torch.Tensor], out: Optional[torch.Tensor] = None,
            y_perm_b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = bf16(bf16(bf16(w0*y[r0]) + bf16(w1*y[r1])) + y_shared[t]); with y_perm_b every y is the bf16 sum of
    two partial results (hidden-split experts)."""
    _need_cuda(y_perm, row_map, topk_weight, y_shared, y_perm_b)
    n = row_map.shape[0]
    d = y_perm.shape[1]
    if out is None:
        out = torch.empty((n, d), dtype=torch.bfloat16, device=y_perm.device)
    lib = N.load()
    if y_perm_b is None:
        rc = lib.comfy_moe_combine(_ptr(y_perm), _ptr(row_map), _ptr(topk_weight), _ptr(y_shared), n, d, _ptr(out),
                                   _stream())
    else:
        rc = lib.comfy_moe_combine_partials(_ptr(y_perm), _ptr(y_perm_b), _ptr(row_map), _ptr(topk_weight),
                                            _ptr(y_shared), n, d, _ptr(out), _stream())
    N.check("comfy_moe_combine", rc)
    return out


def quantize_e4m3(x: torch.Tensor, scale: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                  overflow_count: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 -> e4m3 as the reference's fp8 Linear quantises its input: clamp and round without a scale; multiply by
    bf16(1 / scale) and cast without a clamp (overflow -> NaN, counted in ``overflow_count`` int32 [1]) with one."""
    _need_cuda(x, scale)
    if x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("x must be a contiguous bf16 tensor")
    if out is None:
        out = torch.empty(x.shape, dtype=_FP8, device=x.device)
    if overflow_count is None:
        overflow_count = device_status(x.device)[2:3]
    N.check("comfy_moe_quantize_e4m3", N.load().comfy_moe_quantize_e4m3(_ptr(x), _ptr(scale), x.numel(), _ptr(out),
                                                                        _ptr(overflow_count), _stream()))
    return out


def read_status(status: torch.Tensor) -> None:
    """Synchronises the current stream and raises if a device-side wait gave up."""
    h = ctypes.c_int32(0)
    rc = N.load().comfy_moe_read_status(_ptr(status), _stream(), h)
    if rc != N.OK:
        raise N.MoeError("comfy_moe_read_status", rc, f"device status word = {h.value}")


def validate_routing(ws: "Workspace") -> None:
    """Debug aid: checks the routing the last layer call left in ``ws`` on the device (ids, rows, offsets, counts) and
    raises if it is inconsistent.  One stream synchronisation."""
    rc = N.load().comfy_moe_validate_routing(_ptr(ws.topk_idx), _ptr(ws.row_map), _ptr(ws.expert_counts),
                                             _ptr(ws.expert_offsets), ws.n_tokens, ws.n_experts, ws.rows_cap,
                                             _ptr(ws.status), _stream())
    N.check("comfy_moe_validate_routing", rc)
    read_status(ws.status)


def moe_forward(layer: LayerPack, x: torch.Tensor, ws: Optional[Workspace] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The whole layer through comfy_moe_forward.  x: bf16 [N, D] contiguous on the device."""
    _need_cuda(x)
    if x.dtype != torch.bfloat16 or x.dim() != 2 or not x.is_contiguous():
        raise ValueError("x must be a contiguous bf16 [N, D] tensor")
    n = x.shape[0]
    if ws is None or ws.n_tokens != n:
        ws = Workspace.for_layer(layer, n)
    if out is None:
        out = torch.empty_like(x)
    rc = N.load().comfy_moe_forward(ctypes.byref(layer.c_layer), ctypes.byref(ws.c_ws), _ptr(x), n, _ptr(out),
                                    _stream())
    N.check("comfy_moe_forward", rc)
    return out


# --------------------------------------------------------------------------------------- block glue
def _modulation(*vectors: torch.Tensor) -> int:
    """Common batch stride (elements) of bf16 [B, D] / [B, 1, D] modulation vectors that are views of one tensor."""
    strides = set()
    for v in vectors:
        _need_cuda(v)
        if v.dtype != torch.bfloat16 or v.stride(-1) != 1:
            raise ValueError("modulation vectors must be bf16 with a contiguous last dimension")
        strides.add(v.stride(0) if v.shape[0] > 1 else 0)
    if len(strides) != 1:
        raise ValueError("modulation vectors must share one batch stride")
    return strides.pop()


def ln_modulate(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor, tokens_per_batch: int, eps: float = 1e-6,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """LayerNorm(x) * (1 + scale) + shift in one pass.  x: bf16 [N, D]; shift, scale: bf16 [B, D] views."""
    _need_cuda(x)
    n, d = x.shape
    stride = _modulation(shift, scale)
    if out is None:
        out = torch.empty_like(x)
    rc = N.load().comfy_moe_ln_modulate(_ptr(x), _ptr(shift), _ptr(scale), stride, n, tokens_per_batch, d, float(eps),
                                        _ptr(out), _stream())
    N.check("comfy_moe_ln_modulate", rc)
    return out


def ln_modulate_gate(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor, tokens_per_batch: int,
                     w_gate: torch.Tensor, eps: float = 1e-6, *, neartie_eps: float = 1e-6, want_flags: bool = False):
    """ln_modulate and gate_topk of its output in one pass.  Returns (out, topk_idx, topk_weight, block_counts,
    neartie_count, neartie_flags or None), each bit-identical to what the two separate calls give."""
    _need_cuda(x, w_gate)
    n, d = x.shape
    e = w_gate.shape[0]
    stride = _modulation(shift, scale)
    _, n_blocks = plan_sizes(n, e)
    dev = x.device
    out = torch.empty_like(x)
    topk_idx = torch.empty((n, 2), dtype=torch.int32, device=dev)
    topk_weight = torch.empty((n, 2), dtype=torch.float32, device=dev)
    block_counts = torch.empty((max(n_blocks, 1), e), dtype=torch.int32, device=dev)
    count = torch.zeros((1,), dtype=torch.int32, device=dev)
    flags = torch.zeros((n,), dtype=torch.uint8, device=dev) if want_flags else None
    w_gate = w_gate.contiguous()
    rc = N.load().comfy_moe_ln_modulate_gate(_ptr(x), _ptr(shift), _ptr(scale), stride, n, tokens_per_batch, d, float(eps),
                                             _ptr(out), _ptr(w_gate), _dtype_code(w_gate.dtype), e, 2, _ptr(topk_idx),
                                             _ptr(topk_weight), _ptr(block_counts), _ptr(count), _ptr(flags),
                                             float(neartie_eps), _stream())
    N.check("comfy_moe_ln_modulate_gate", rc)
    return out, topk_idx, topk_weight, block_counts, count, flags


def gate_residual(y: torch.Tensor, gate: torch.Tensor, residual: torch.Tensor, tokens_per_batch: int) -> torch.Tensor:
    """gate * y + residual with PyTorch's bf16 rounding points.  y, residual: bf16 [N, D]; gate: bf16 [B, D] view."""
    _need_cuda(y, residual)
    n, d = y.shape
    out = torch.empty_like(y)
    rc = N.load().comfy_moe_gate_residual(_ptr(y), _ptr(gate), _modulation(gate), _ptr(residual), n, tokens_per_batch, d,
                                          _ptr(out), _stream())
    N.check("comfy_moe_gate_residual", rc)
    return out


def moe_ffn_block(layer: LayerPack, x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor, gate: torch.Tensor,
                  tokens_per_batch: int, eps: float = 1e-6, ws: Optional[Workspace] = None) -> torch.Tensor:
    """gate * MoE(LayerNorm(x) * (1 + scale) + shift) + x through comfy_moe_ffn_block.  x: bf16 [N, D]."""
    _need_cuda(x)
    n = x.shape[0]
    if ws is None or ws.n_tokens != n:
        ws = Workspace.for_layer(layer, n)
    ws.need_x_mod()
    out = torch.empty_like(x)
    rc = N.load().comfy_moe_ffn_block(ctypes.byref(layer.c_layer), ctypes.byref(ws.c_ws), _ptr(x), _ptr(shift),
                                      _ptr(scale), _ptr(gate), _modulation(shift, scale, gate), n, tokens_per_batch,
                                      float(eps), _ptr(out), _stream())
    N.check("comfy_moe_ffn_block", rc)
    return out


# --------------------------------------------------------------------------------------- GELU-MLP experts
@dataclass
class MlpPack:
    """Device pointers of one GELU feed-forward (Linear + bias, GELU, Linear + bias); keeps the tensors alive."""

    w1: torch.Tensor
    b1: Optional[torch.Tensor]
    w2: torch.Tensor
    b2: Optional[torch.Tensor]

    def __post_init__(self):
        _need_cuda(self.w1, self.w2, self.b1, self.b2)
        for w in (self.w1, self.w2):
            if w.dtype != torch.bfloat16 or w.dim() != 2 or w.stride(1) != 1:
                raise ValueError("expert weights must be 2-D bf16 with a contiguous last dimension")
        if self.w2.shape != (self.w1.shape[1], self.w1.shape[0]):
            raise ValueError("w2 must be [dim, hidden]")
        for b, n in ((self.b1, self.w1.shape[0]), (self.b2, self.w2.shape[0])):
            if b is not None and (b.dtype != torch.bfloat16 or b.shape != (n,) or not b.is_contiguous()):
                raise ValueError("biases must be contiguous bf16 vectors over the output features")

    @property
    def hidden(self) -> int:
        return self.w1.shape[0]

    @property
    def dim(self) -> int:
        return self.w1.shape[1]

    def fill(self, s: N.MlpWeights) -> None:
        s.w1, s.w2 = self.w1.data_ptr(), self.w2.data_ptr()
        s.b1 = None if self.b1 is None else self.b1.data_ptr()
        s.b2 = None if self.b2 is None else self.b2.data_ptr()
        s.ld1, s.ld2 = self.w1.stride(0), self.w2.stride(0)
        s.hidden = self.hidden
        s.reserved = 0

    def struct(self) -> N.MlpWeights:
        s = N.MlpWeights()
        self.fill(s)
        return s


@dataclass
class MlpLayerPack:
    """Everything comfy_moe_forward_gelu_mlp needs to know about one MoEBlock."""

    gate: torch.Tensor
    experts: Sequence[MlpPack]
    shared: MlpPack
    top_k: int = 2
    c_layer: N.MlpLayer = field(init=False)
    fp8 = False

    def __post_init__(self):
        _need_cuda(self.gate)
        if not self.gate.is_contiguous():
            raise ValueError("gate weight must be contiguous")
        L = N.MlpLayer()
        L.dim = self.gate.shape[1]
        L.n_experts = len(self.experts)
        L.top_k = self.top_k
        L.gate_dtype = _dtype_code(self.gate.dtype)
        L.w_gate = self.gate.data_ptr()
        for i, e in enumerate(self.experts):
            e.fill(L.experts[i])
        self.shared.fill(L.shared)
        self.c_layer = L

    @property
    def dim(self) -> int:
        return self.gate.shape[1]

    @property
    def n_experts(self) -> int:
        return len(self.experts)


def grouped_gelu_mlp(experts: Sequence[MlpPack], shared: Optional[MlpPack], row_start: Optional[torch.Tensor],
                     row_count: Optional[torch.Tensor], x_perm: Optional[torch.Tensor],
                     x_shared: Optional[torch.Tensor], *, check_status: bool = True):
    """Both passes of the grouped GELU-MLP expert GEMM; arguments as grouped_swiglu.
    Returns (y_perm or None, y_shared or None, h_perm, h_shared)."""
    ref = experts[0] if experts else shared
    dim, dev = ref.dim, ref.w1.device
    n_e = len(experts)
    arr = (N.MlpWeights * max(n_e, 1))()
    for i, e in enumerate(experts):
        e.fill(arr[i])
    rows_cap = 0 if x_perm is None else x_perm.shape[0]
    h_perm = y_perm = None
    if n_e:
        h_perm = torch.empty((rows_cap, experts[0].hidden), dtype=torch.bfloat16, device=dev)
        y_perm = torch.empty((rows_cap, dim), dtype=torch.bfloat16, device=dev)
    n_tokens = 0 if x_shared is None else x_shared.shape[0]
    sh = h_sh = y_sh = None
    if shared is not None and n_tokens > 0:
        sh = shared.struct()
        h_sh = torch.empty((n_tokens, shared.hidden), dtype=torch.bfloat16, device=dev)
        y_sh = torch.empty((n_tokens, dim), dtype=torch.bfloat16, device=dev)
    status = device_status(dev)
    rc = N.load().comfy_moe_grouped_gelu_mlp(
        n_e, arr, ctypes.byref(sh) if sh is not None else None, _ptr(row_start), _ptr(row_count), rows_cap, n_tokens,
        dim, _ptr(x_perm), _ptr(h_perm), _ptr(y_perm), _ptr(x_shared), _ptr(h_sh), _ptr(y_sh), _ptr(status), _stream())
    N.check("comfy_moe_grouped_gelu_mlp", rc)
    if check_status:
        read_status(status)
    return y_perm, y_sh, h_perm, h_sh


def moe_mlp_forward(layer: MlpLayerPack, x: torch.Tensor, ws: Optional[Workspace] = None,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """MoEBlock.forward (eval) through comfy_moe_forward_gelu_mlp.  x: bf16 [N, D] contiguous on the device."""
    _need_cuda(x)
    if x.dtype != torch.bfloat16 or x.dim() != 2 or not x.is_contiguous():
        raise ValueError("x must be a contiguous bf16 [N, D] tensor")
    n = x.shape[0]
    if ws is None or ws.n_tokens != n:
        ws = Workspace.for_layer(layer, n)
    if out is None:
        out = torch.empty_like(x)
    rc = N.load().comfy_moe_forward_gelu_mlp(ctypes.byref(layer.c_layer), ctypes.byref(ws.c_ws), _ptr(x), n,
                                             _ptr(out), _stream())
    N.check("comfy_moe_forward_gelu_mlp", rc)
    return out


# --------------------------------------------------------------------------------------- attention glue
def rmsnorm_rope(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, rope: Optional[torch.Tensor],
                 heads: int, out: torch.Tensor, out_row_offset: int = 0, rope_row_offset: int = 0) -> torch.Tensor:
    """RMSNorm (optional) + rotary embedding (optional) of one projected tensor, written into rows
    [out_row_offset, out_row_offset + S) of every batch element of ``out`` [B, S_total, heads, head_dim].

    x: bf16 [B, S, heads * head_dim] (last dim contiguous, rows evenly strided); weight: bf16 [heads * head_dim] or
    None; rope: fp32 [B or 1, S_rope, 1, pairs, 2, 2] or None, rotated rows start at ``rope_row_offset``."""
    _need_cuda(x, weight, rope, out)
    b, s, inner = x.shape
    head_dim = inner // heads
    if x.dtype != torch.bfloat16 or x.stride(2) != 1 or x.stride(0) != s * x.stride(1):
        raise ValueError("x must be bf16 [B, S, inner] with evenly strided rows")
    if out.dtype != torch.bfloat16 or out.shape[0] != b or out.shape[2:] != (heads, head_dim) or \
            not out[0].is_contiguous() or out_row_offset + s > out.shape[1]:
        raise ValueError("out must be bf16 [B, S_total, heads, head_dim] with room for the rows")
    rope_stride = pairs = 0
    if rope is not None:
        if rope.dtype != torch.float32 or rope.dim() != 6 or rope.shape[2] != 1 or rope.shape[4:] != (2, 2) or \
                not rope[0].is_contiguous() or rope_row_offset + s > rope.shape[1]:
            raise ValueError("rope must be fp32 [B or 1, S_rope, 1, pairs, 2, 2]")
        pairs = rope.shape[3]
        rope_stride = rope.stride(0) if rope.shape[0] > 1 else 0
    rc = N.load().comfy_attn_rmsnorm_rope(_ptr(x), x.stride(1), _ptr(weight), eps, _ptr(rope), rope_stride,
                                          rope_row_offset, pairs, b * s, s, heads, head_dim, _ptr(out), out.stride(0),
                                          out_row_offset, _stream())
    N.check("comfy_attn_rmsnorm_rope", rc)
    return out


# --------------------------------------------------------------------------------------- weight ingest
def stochastic_round_e4m3(x: torch.Tensor, rand: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One slice of the reference's stochastic rounding to e4m3: x fp32 / bf16 / fp16 (contiguous), rand the fp16
    uniforms the reference would draw for it.  Returns the e4m3 tensor (``out`` if given)."""
    _need_cuda(x, rand, out)
    codes = {torch.float32: N.FP32, torch.bfloat16: N.BF16, torch.float16: N.FP16}
    if x.dtype not in codes or not x.is_contiguous() or rand.dtype != torch.float16 or rand.shape != x.shape or \
            not rand.is_contiguous():
        raise ValueError("x must be contiguous fp32 / bf16 / fp16 and rand fp16 of the same shape")
    if out is None:
        out = torch.empty(x.shape, dtype=_FP8, device=x.device)
    N.check("comfy_moe_stochastic_round_e4m3",
            N.load().comfy_moe_stochastic_round_e4m3(_ptr(x), codes[x.dtype], _ptr(rand), x.numel(), _ptr(out), _stream()))
    return out


def quantize_weight_e4m3(w: torch.Tensor):
    """Per-tensor scaled e4m3 of a weight: returns (wq e4m3 like w, scale fp32 scalar on the device) with
    scale = max|w| / 448 and wq = (w / scale) rounded to nearest even, the layout scaled-fp8 Linears load."""
    _need_cuda(w)
    codes = {torch.float32: N.FP32, torch.bfloat16: N.BF16, torch.float16: N.FP16}
    if w.dtype not in codes or not w.is_contiguous():
        raise ValueError("w must be a contiguous fp32 / bf16 / fp16 tensor")
    out = torch.empty(w.shape, dtype=_FP8, device=w.device)
    scale = torch.empty((), dtype=torch.float32, device=w.device)
    N.check("comfy_moe_quantize_weight_e4m3",
            N.load().comfy_moe_quantize_weight_e4m3(_ptr(w), codes[w.dtype], w.numel(), _ptr(scale), _ptr(out), _stream()))
    return out, scale


def grouped_linear(groups: Sequence[Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]],
                   outs: Optional[Sequence[torch.Tensor]] = None, status: Optional[torch.Tensor] = None):
    """Several ``F.linear(x, w, b)`` in one launch.  groups: (x [rows, in] bf16 with a contiguous last dimension,
    w [out, in] bf16, bias [out] bf16 or None); returns the list of outputs [rows, out] (``outs`` if given)."""
    if not groups:
        return []
    arr = (N.LinearGroup * len(groups))()
    res = []
    dev = groups[0][0].device
    for i, (x, w, b) in enumerate(groups):
        _need_cuda(x, w, b)
        if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 2 or \
                x.stride(1) != 1 or w.stride(1) != 1 or x.shape[1] != w.shape[1]:
            raise ValueError("grouped_linear: x [rows, in] and w [out, in] must be bf16 with contiguous last dimensions")
        if b is not None and (b.dtype != torch.bfloat16 or b.shape != (w.shape[0],) or not b.is_contiguous()):
            raise ValueError("grouped_linear: bias must be a contiguous bf16 vector over the output features")
        out = outs[i] if outs is not None else torch.empty((x.shape[0], w.shape[0]), dtype=torch.bfloat16, device=dev)
        if out.shape != (x.shape[0], w.shape[0]) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
            raise ValueError("grouped_linear: out must be bf16 [rows, out] with a contiguous last dimension")
        g = arr[i]
        g.x, g.w, g.out = x.data_ptr(), w.data_ptr(), out.data_ptr()
        g.bias = None if b is None else b.data_ptr()
        g.ld_x, g.ld_w, g.ld_out = x.stride(0), w.stride(0), out.stride(0)
        g.rows, g.in_features, g.out_features = x.shape[0], x.shape[1], w.shape[0]
        res.append(out)
    if status is None:
        status = device_status(dev)
    N.check("comfy_moe_grouped_linear", N.load().comfy_moe_grouped_linear(len(groups), arr, _ptr(status), _stream()))
    return res


def attention_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None,
                      status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """softmax(q k^T * scale) v per head.  q [B, Sq, H, 128], k / v [B, Skv, H, 128] bf16 contiguous ->
    [B, Sq, H * 128]; scale defaults to 1 / sqrt(128)."""
    _need_cuda(q, k, v)
    b, sq, h, d = q.shape
    if k.shape != v.shape or k.shape[0] != b or k.shape[2:] != (h, d):
        raise ValueError("attention_forward: k and v must be [B, Skv, H, D] matching q's batch, heads and head_dim")
    for t in (q, k, v):
        if t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise ValueError("attention_forward: q, k, v must be contiguous bf16 tensors")
    out = torch.empty((b, sq, h * d), dtype=torch.bfloat16, device=q.device)
    if status is None:
        status = device_status(q.device)
    rc = N.load().comfy_attn_forward(_ptr(q), _ptr(k), _ptr(v), b, sq, k.shape[1], h, d,
                                     float(scale if scale is not None else d ** -0.5), _ptr(out), _ptr(status), _stream())
    N.check("comfy_attn_forward", rc)
    return out
