"""Operator namespaces for the HiDream MoE feed-forward, interface-compatible with ``comfy/ops.py``.

What is mirrored (same names, arguments and behaviour, Linear only — the MoE path builds nothing else):

* ``CastWeightBiasOp`` attributes ``comfy_cast_weights`` / ``weight_function`` / ``bias_function``
  (``comfy/ops.py:97-100``) and ``cast_bias_weight`` (``:61-95``);
* ``disable_weight_init.Linear`` (``:103-115``), ``manual_cast.Linear`` (``:283-284``);
* ``fp8_linear`` (``:314-358``), ``fp8_ops.Linear`` (``:360-377``), ``scaled_fp8_ops(...)`` (``:379-428``);
* ``pick_operations`` (``:449-473``).

What is new: the dispatch shim at the bottom.  ``hidream_moe_forward`` / ``hidream_moe_infer`` /
``hidream_gate`` / ``swiglu_ffn_forward`` check, on every call, whether the module's current weights
can be handed to the sm_100a kernels (bf16, or e4m3 with per-tensor scales; resident on the input's
device; LoRA closures on a weight are evaluated once and the patched weight kept) and if so run the whole
layer there.  They return ``None`` when the call is not eligible, and the module then runs its stock PyTorch
composition, exactly as the reference would.
"""
from __future__ import annotations

import contextlib
import logging
import os
from typing import Optional

import torch
import torch.nn.functional as F

from . import model_management

FP8 = torch.float8_e4m3fn


# =========================================================================== reference-compatible part
def cast_to_input(weight, input, non_blocking=False, copy=True):
    return model_management.cast_to(weight, input.dtype, input.device, non_blocking=non_blocking, copy=copy)


def cast_bias_weight(s, input=None, dtype=None, device=None, bias_dtype=None):
    """Weight (and bias) of module ``s`` cast for use with ``input``, then passed through the module's
    ``weight_function`` / ``bias_function`` lists (LoRA closures attached by a model patcher)."""
    if input is not None:
        dtype = input.dtype if dtype is None else dtype
        bias_dtype = dtype if bias_dtype is None else bias_dtype
        device = input.device if device is None else device

    side = model_management.get_offload_stream(device)
    in_side = side if side is not None else contextlib.nullcontext()
    non_blocking = model_management.device_supports_non_blocking(device)

    def prepared(tensor, fns, to_dtype):
        if tensor is None:
            return None
        out = model_management.cast_to(tensor, to_dtype, device, non_blocking=non_blocking, copy=len(fns) > 0,
                                       stream=side)
        if fns:
            with in_side:
                for fn in fns:
                    out = fn(out)
        return out

    bias = prepared(s.bias, s.bias_function, bias_dtype)
    weight = prepared(s.weight, s.weight_function, dtype)
    model_management.sync_stream(device, side)
    return weight, bias


class CastWeightBiasOp:
    comfy_cast_weights = False
    weight_function = []
    bias_function = []


class disable_weight_init:
    """Layers that skip parameter initialisation (weights always come from a checkpoint)."""

    class Linear(torch.nn.Linear, CastWeightBiasOp):
        def reset_parameters(self):
            return None

        def forward_comfy_cast_weights(self, input):
            weight, bias = cast_bias_weight(self, input)
            return F.linear(input, weight, bias)

        def forward(self, *args, **kwargs):
            if self.comfy_cast_weights or self.weight_function or self.bias_function:
                return self.forward_comfy_cast_weights(*args, **kwargs)
            return super().forward(*args, **kwargs)


class _LayerNorm(torch.nn.LayerNorm, CastWeightBiasOp):
    """operations.LayerNorm (``comfy/ops.py:173-189``): the HiDream blocks build their norms through it."""

    def reset_parameters(self):
        return None

    def forward_comfy_cast_weights(self, input):
        if self.weight is not None:
            weight, bias = cast_bias_weight(self, input)
        else:
            weight, bias = None, None
        return F.layer_norm(input, self.normalized_shape, weight, bias, self.eps)

    def forward(self, *args, **kwargs):
        if self.comfy_cast_weights or self.weight_function or self.bias_function:
            return self.forward_comfy_cast_weights(*args, **kwargs)
        return super().forward(*args, **kwargs)


disable_weight_init.LayerNorm = _LayerNorm


class _RMSNorm(torch.nn.RMSNorm, CastWeightBiasOp):
    """operations.RMSNorm (``comfy/ops.py``, over ``comfy/rmsnorm.py:14-20``): ``torch.nn.functional.rms_norm`` with the
    weight cast to the activation's dtype and device; HiDream's attention builds its q / k norms through it."""

    def reset_parameters(self):
        self.bias = None
        return None

    def forward_comfy_cast_weights(self, input):
        weight = None
        if self.weight is not None:
            weight, _ = cast_bias_weight(self, input)
        return F.rms_norm(input, self.normalized_shape, weight, self.eps)

    def forward(self, input):
        if self.comfy_cast_weights or self.weight_function or self.bias_function:
            return self.forward_comfy_cast_weights(input)
        weight = None if self.weight is None else model_management.cast_to(self.weight, dtype=input.dtype,
                                                                          device=input.device)
        return F.rms_norm(input, self.normalized_shape, weight, self.eps)


disable_weight_init.RMSNorm = _RMSNorm


class manual_cast(disable_weight_init):
    """Weights stored in one dtype and cast to the activation dtype on every call."""

    class Linear(disable_weight_init.Linear):
        comfy_cast_weights = True

    class LayerNorm(disable_weight_init.LayerNorm):
        comfy_cast_weights = True

    class RMSNorm(disable_weight_init.RMSNorm):
        comfy_cast_weights = True


def fp8_linear(self, input):
    """fp8 x fp8 matmul of an e4m3 Linear: quantise the activation, ``torch._scaled_mm`` with per-tensor
    scales, output in the activation dtype.  Returns None when the weight is not e4m3 (caller falls back)."""
    w_dtype = self.weight.dtype
    if w_dtype != FP8:
        return None
    was_2d = input.dim() == 2
    if was_2d:
        input = input.unsqueeze(1)
    if input.dim() != 3:
        return None
    shape, act_dtype = input.shape, input.dtype
    w, bias = cast_bias_weight(self, input, dtype=w_dtype, bias_dtype=act_dtype)

    def on_device(scale):
        if scale is None:
            return torch.ones((), device=input.device, dtype=torch.float32)
        return scale.to(input.device)

    scale_weight = on_device(self.scale_weight)
    if self.scale_input is None:
        scale_input = on_device(None)
        input = torch.clamp(input, min=-448, max=448, out=input)   # in place, like the reference
        xq = input.reshape(-1, shape[2]).to(w_dtype).contiguous()
    else:
        scale_input = on_device(self.scale_input)
        xq = (input * (1.0 / scale_input).to(act_dtype)).reshape(-1, shape[2]).to(w_dtype).contiguous()

    kwargs = dict(out_dtype=act_dtype, scale_a=scale_input, scale_b=scale_weight)
    if bias is not None:
        kwargs["bias"] = bias
    o = torch._scaled_mm(xq, w.t(), **kwargs)
    if isinstance(o, tuple):
        o = o[0]
    if was_2d:
        return o.reshape(shape[0], -1)
    return o.reshape((-1, shape[1], self.weight.shape[0]))


class fp8_ops(manual_cast):
    """Unscaled fp8 weights multiplied in fp8 when possible."""

    class Linear(manual_cast.Linear):
        fp8_matrix_mult = True

        def reset_parameters(self):
            self.scale_weight = None
            self.scale_input = None
            return None

        def forward_comfy_cast_weights(self, input):
            if not self.training:
                try:
                    out = fp8_linear(self, input)
                    if out is not None:
                        return out
                except Exception as e:  # same policy as the reference: log and use the cast path
                    logging.info("Exception during fp8 op: {}".format(e))
            weight, bias = cast_bias_weight(self, input)
            return F.linear(input, weight, bias)


def scaled_fp8_ops(fp8_matrix_mult=False, scale_input=False, override_dtype=None):
    """Namespace factory for per-tensor scaled fp8 weights: ``weight`` e4m3 plus a ``scale_weight`` fp32
    scalar (and ``scale_input`` when requested) per Linear."""
    logging.info("Using scaled fp8: fp8 matrix mult: {}, scale input: {}".format(fp8_matrix_mult, scale_input))
    use_fp8_mm, with_scale_input = fp8_matrix_mult, scale_input

    class scaled_fp8_op(manual_cast):
        class Linear(manual_cast.Linear):
            fp8_matrix_mult = use_fp8_mm

            def __init__(self, *args, **kwargs):
                if override_dtype is not None:
                    kwargs["dtype"] = override_dtype
                super().__init__(*args, **kwargs)

            def reset_parameters(self):
                def unit():
                    return torch.nn.parameter.Parameter(
                        data=torch.ones((), device=self.weight.device, dtype=torch.float32), requires_grad=False)

                if not hasattr(self, "scale_weight"):
                    self.scale_weight = unit()
                if not with_scale_input:
                    self.scale_input = None
                if not hasattr(self, "scale_input"):
                    self.scale_input = unit()
                return None

            def forward_comfy_cast_weights(self, input):
                if use_fp8_mm:
                    out = fp8_linear(self, input)
                    if out is not None:
                        return out
                weight, bias = cast_bias_weight(self, input)
                scale = self.scale_weight.to(device=weight.device, dtype=weight.dtype)
                if weight.numel() < input.numel():
                    return F.linear(input, weight * scale, bias)
                return F.linear(input * scale, weight, bias)

            def convert_weight(self, weight, inplace=False, **kwargs):
                scale = self.scale_weight.to(device=weight.device, dtype=weight.dtype)
                if inplace:
                    weight *= scale
                    return weight
                return weight * scale

            def set_weight(self, weight, inplace_update=False, seed=None, return_weight=False, **kwargs):
                scaled = weight / self.scale_weight.to(device=weight.device, dtype=weight.dtype)
                q = stochastic_rounding(scaled, self.weight.dtype, seed=seed)
                if return_weight:
                    return q
                if inplace_update:
                    self.weight.data.copy_(q)
                else:
                    self.weight = torch.nn.Parameter(q, requires_grad=False)

    return scaled_fp8_op


_FP8_FORMATS = {torch.float8_e4m3fn: (4, 3, 7), torch.float8_e5m2: (5, 2, 15)}     # exponent bits, mantissa bits, bias


def _stochastic_round_fp8_slice(x: torch.Tensor, dtype: torch.dtype, generator) -> torch.Tensor:
    """One slice of ``comfy/float.py:14-46``: every step is an fp16 tensor operation, as in the reference (so each
    result is rounded to fp16 before the next step), the random offsets are fp16 uniforms drawn from ``generator``."""
    e_bits, m_bits, bias = _FP8_FORMATS[dtype]
    x = x.half()
    sign = torch.sign(x)
    mag = x.abs()
    sign = torch.where(mag == 0, 0, sign)
    exponent = torch.clamp(torch.floor(torch.log2(mag)) + bias, 0, 2 ** e_bits - 1)
    normal = ~(exponent == 0)
    scaled = torch.where(normal,
                         (mag / (2.0 ** (exponent - bias)) - 1.0) * (2 ** m_bits),
                         mag / (2.0 ** (-bias + 1 - m_bits)))
    scaled += torch.rand(scaled.size(), dtype=scaled.dtype, layout=scaled.layout, device=scaled.device,
                         generator=generator)
    frac = scaled.floor() / (2 ** m_bits)
    sign *= torch.where(normal, (2.0 ** (exponent - bias)) * (1.0 + frac), (2.0 ** (-bias + 1)) * frac)
    info = torch.finfo(dtype)
    torch.clamp(sign, min=info.min, max=info.max, out=sign)
    return sign


def stochastic_rounding(value: torch.Tensor, dtype: torch.dtype, seed=0) -> torch.Tensor:
    """``comfy/float.py:50-67``: fp8 targets are rounded stochastically (each element to one of its two neighbouring
    representable values, the upper one with probability equal to its fractional position), in row slices of about
    4096 x 4096 elements that draw from one generator seeded with ``seed``; every other dtype is a plain cast.
    On a B200 the e4m3 case runs as one fused kernel per slice, fed the same random numbers."""
    if dtype not in _FP8_FORMATS:
        return value.to(dtype=dtype)
    generator = torch.Generator(device=value.device)
    generator.manual_seed(0 if seed is None else int(seed))
    output = torch.empty_like(value, dtype=dtype)
    num_slices = max(1, (value.numel() / (4096 * 4096)))
    slice_size = max(1, round(value.shape[0] / num_slices))
    for i in range(0, value.shape[0], slice_size):
        part = value[i:i + slice_size]
        fast = _stochastic_round_kernel(part, dtype, generator, output[i:i + slice_size])
        if fast is None:
            output[i:i + slice_size].copy_(_stochastic_round_fp8_slice(part, dtype, generator))
    return output


def _stochastic_round_kernel(part: torch.Tensor, dtype: torch.dtype, generator, out: torch.Tensor):
    """The fused kernel for one slice, or None when the slice is not eligible (then the composition above runs)."""
    if not ENABLE_SM100_KERNELS or dtype != FP8 or not part.is_cuda or not model_management.is_sm100(part.device):
        return None
    if part.dtype not in (torch.float32, torch.bfloat16, torch.float16) or not part.is_contiguous() or \
            not out.is_contiguous() or part.numel() == 0:
        return None
    from . import moe_ops

    rand = torch.rand(part.size(), dtype=torch.float16, device=part.device, generator=generator)
    return moe_ops.stochastic_round_e4m3(part, rand, out)


def pick_operations(weight_dtype, compute_dtype, load_device=None, disable_fast_fp8=False, fp8_optimizations=False,
                    scaled_fp8=None):
    """Choose the operator namespace for a model, by the same rules as the reference."""
    fp8_compute = model_management.supports_fp8_compute(load_device)
    if scaled_fp8 is not None:
        return scaled_fp8_ops(fp8_matrix_mult=fp8_compute and fp8_optimizations, scale_input=fp8_optimizations,
                              override_dtype=scaled_fp8)
    if fp8_compute and fp8_optimizations and not disable_fast_fp8:
        return fp8_ops
    if compute_dtype is None or weight_dtype == compute_dtype:
        return disable_weight_init
    return manual_cast


# =========================================================================== dispatch shim (new)
# Switches an embedding application can flip.
ENABLE_SM100_KERNELS = True
# Read the device status word (one stream synchronisation) after every fused call; for debugging.
CHECK_STATUS_EVERY_CALL = False
# Debug runs (COMFY_B200_DEBUG=1): after every fused layer call, check the routing it produced on the device (expert
# ids, rows, offsets, counts) and read the status word.  Stands in for a memory checker at the level of the data
# structures the kernels index with.
DEBUG_VALIDATE = os.environ.get("COMFY_B200_DEBUG", "0") not in ("", "0")
# NVTX ranges around the fused calls (COMFY_B200_NVTX=1), so that a timeline shows the layer as one named span.
NVTX_RANGES = os.environ.get("COMFY_B200_NVTX", "0") not in ("", "0")


class _Range:
    """``with _Range("name"):`` pushes an NVTX range when NVTX_RANGES is set, and does nothing otherwise."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if NVTX_RANGES:
            torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        if NVTX_RANGES:
            torch.cuda.nvtx.range_pop()


def _after_layer_call(layer, n_tokens: int) -> None:
    from . import moe_ops

    if DEBUG_VALIDATE:
        moe_ops.validate_routing(_workspace(layer, n_tokens))
    elif CHECK_STATUS_EVERY_CALL:
        moe_ops.read_status(_workspace(layer, n_tokens).status)



def _version_of(t: torch.Tensor) -> int:
    """In-place update counter of a tensor; tensors created under torch.inference_mode() keep none (and cannot be
    updated in place outside it), so their identity is their storage."""
    return 0 if t.is_inference() else t._version


def _tensor_key(t: Optional[torch.Tensor]):
    if t is None:
        return None
    return (t.data_ptr(), _version_of(t), t.dtype, t.device, tuple(t.shape), t.stride(0) if t.dim() else 0)


# A Linear that carries weight_function closures (what a model patcher attaches instead of baking a LoRA into the
# weights, comfy/model_patcher.py:125-149, 670-676) normally evaluates them on every forward.  They are deterministic
# (a LoRA delta; for fp8 targets a stochastic rounding seeded by the weight's key), so the kernels take the patched
# weight evaluated ONCE and kept beside the module until the closures or the weight change: the result the stock path
# computes on every call, at the price of a second copy of the patched weights on the device (which is what the
# reference itself holds after a full load, comfy/model_patcher.py:594-619).  Set to False to leave patched Linears to
# the stock composition.
BAKE_PATCHED_WEIGHTS = True


def _patched_weight(lin, device):
    """``lin.weight`` after its ``weight_function`` closures, evaluated once per (weight, closures) and cached on the
    module; None when the weight is not on ``device`` or the closures change its dtype or shape."""
    fns = list(lin.weight_function)
    w = lin.weight
    key = (_tensor_key(w), tuple(id(f) for f in fns))
    cached = lin.__dict__.get("_b200_baked")
    if cached is not None and cached[0] == key:
        return cached[2]
    if w.device != device:
        return None
    out = w.detach().clone()              # the closures may work in place; the reference hands them a copy too
    for fn in fns:
        out = fn(out)
    if out.dtype != w.dtype or out.shape != w.shape or out.device != w.device:
        return None
    out = out.detach().contiguous()
    lin.__dict__["_b200_baked"] = (key, fns, out)      # holding the closures keeps their ids from being reused
    return out


def _linear_state(lin, device):
    """(weight, scale_weight, scale_input) if this Linear can feed the kernels as it is now, else None."""
    if lin.bias_function or lin.bias is not None:
        return None
    w = lin.weight
    if lin.weight_function:
        if not BAKE_PATCHED_WEIGHTS:
            return None
        w = _patched_weight(lin, device)
        if w is None:
            return None
    else:
        lin.__dict__.pop("_b200_baked", None)
    if w.device != device or w.dim() != 2 or w.stride(1) != 1:
        return None
    if w.dtype == torch.bfloat16:
        return (w, None, None)
    if w.dtype == FP8 and getattr(lin, "fp8_matrix_mult", False) and not lin.training:
        sw = getattr(lin, "scale_weight", None)
        si = getattr(lin, "scale_input", None)
        for s in (sw, si):
            if s is not None and (s.device != device or s.dtype != torch.float32 or s.numel() != 1):
                return None
        return (w, sw, si)
    return None


def _ffn_pack(ffn, device, moe_ops):
    """FfnPack for a FeedForwardSwiGLU, or None.  Cached on the module, keyed on the identity and version
    of every tensor, so a patched, re-loaded or moved weight is picked up on the next call."""
    states = [_linear_state(l, device) for l in (ffn.w1, ffn.w3, ffn.w2)]
    if any(s is None for s in states):
        return None
    key = tuple(_tensor_key(t) for s in states for t in s)
    cached = getattr(ffn, "_b200_pack", None)
    if cached is not None and cached[0] == key:
        return cached[1]
    (w1, s1, i1), (w3, s3, i3), (w2, s2, i2) = states
    if w1.dtype != w3.dtype or w1.dtype != w2.dtype or w1.shape != w3.shape or w1.stride(0) != w3.stride(0):
        return None
    if (i1 is None) != (i3 is None):
        return None
    if i1 is not None and float(i1) != float(i3):   # w1 and w3 must quantise their common input alike
        return None
    try:
        pack = moe_ops.FfnPack(w1.detach(), w3.detach(), w2.detach(), scale_w1=s1, scale_w3=s3, scale_w2=s2,
                               scale_in13=i1, scale_in2=i2)
    except ValueError:
        return None
    object.__setattr__(ffn, "_b200_pack", (key, pack))
    return pack


def _input_ok(x: torch.Tensor, dim: int) -> bool:
    return (ENABLE_SM100_KERNELS and x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
            and x.shape[-1] == dim and dim % 256 == 0 and x.numel() > 0
            and model_management.is_sm100(x.device))


def _layer_pack(moe, x):
    """LayerPack for a MOEFeedForwardSwiGLU under the current weights, or None when not eligible."""
    from . import moe_ops

    gate_w = moe.gate.weight
    dim = gate_w.shape[1]
    if not _input_ok(x, dim):
        return None
    if moe.num_activated_experts != 2 or not (2 <= len(moe.experts) <= 8):
        return None
    if gate_w.device != x.device or gate_w.dtype not in (torch.bfloat16, torch.float32) or not gate_w.is_contiguous():
        return None
    packs = [_ffn_pack(e, x.device, moe_ops) for e in moe.experts]
    shared = _ffn_pack(moe.shared_experts, x.device, moe_ops)
    if shared is None or any(p is None for p in packs):
        return None
    if any(p.w1.dtype != packs[0].w1.dtype or p.hidden != packs[0].hidden for p in packs) or \
            shared.w1.dtype != packs[0].w1.dtype:
        return None
    if packs[0].hidden % 128 or shared.hidden % 128:
        return None
    key = (_tensor_key(gate_w),) + tuple(id(p) for p in packs) + (id(shared),)
    cached = getattr(moe, "_b200_layer", None)
    if cached is not None and cached[0] == key:
        return cached[1]
    layer = None
    ins = {None if p.scale_in13 is None else float(p.scale_in13) for p in packs}   # host reads: cache misses only
    if len(ins) == 1:    # the permuted activations are quantised once for all routed experts
        layer = moe_ops.LayerPack(gate_w.detach(), packs, shared, top_k=2)
    object.__setattr__(moe, "_b200_layer", (key, layer))
    return layer


def _workspace(layer, n_tokens: int):
    from . import torch_ops

    return torch_ops._workspace(layer, n_tokens)


def check_device_status() -> None:
    """Synchronises and raises ``MoeError`` if any kernel call since the last check left a code in a device status
    word (a bounded wait that ran out, routed rows that did not fit a peer buffer).  The words are sticky, so one call
    at a natural synchronisation point, e.g. after a model forward, covers every layer that ran."""
    from . import moe_ops

    moe_ops.check_all_status()


def release_workspaces() -> None:
    """Drop the cached device workspaces (they are shared by every MoE layer of a model)."""
    from . import torch_ops

    torch_ops.release_workspaces()


def _op_args(layer):
    """List arguments of the registered torch ops for this layer, cached on the pack."""
    from . import torch_ops

    args = getattr(layer, "_op_args", None)
    if args is None:
        args = torch_ops.register(layer)
        layer._op_args = args
    return args


def drop_packs(module) -> None:
    """Forgets the pointer packs cached on a module tree (they hold views of the weights they were built from, i.e.
    keep that device memory alive).  The drop-in modules call this from ``_apply``, so ``model.to(offload_device)``,
    which is how a model patcher unloads a model, frees the expert weights at once; after replacing Parameters by
    hand, call it (or just call the module again: stale packs are replaced on the next call)."""
    for m in module.modules():
        m.__dict__.pop("_b200_pack", None)
        m.__dict__.pop("_b200_layer", None)
        m.__dict__.pop("_b200_baked", None)


def hidream_moe_forward(moe, x: torch.Tensor) -> Optional[torch.Tensor]:
    """MOEFeedForwardSwiGLU.forward on the sm_100a kernels, or None when this call is not eligible.
    Goes through the registered operator ``torch.ops.comfyui_b200.hidream_moe``."""
    layer = _layer_pack(moe, x)
    if layer is None:
        return None
    from . import moe_ops, torch_ops  # noqa: F401  (importing torch_ops registers the operators)

    x2 = x.view(-1, x.shape[-1])
    with _Range("comfyui_b200::hidream_moe"):
        out = torch.ops.comfyui_b200.hidream_moe(x2, layer.gate, *_op_args(layer))
    _after_layer_call(layer, x2.shape[0])
    return out.view(x.shape)


def hidream_gate(gate, x: torch.Tensor):
    """MoEGate.forward on the fused gate kernel: (idx int64 [N,2], weight [N,2] in x.dtype) or None."""
    w = gate.weight
    if not _input_ok(x, w.shape[1]) or gate.top_k != 2 or w.shape[0] not in (2, 4, 8):
        return None
    if w.device != x.device or w.dtype not in (torch.bfloat16, torch.float32):
        return None
    from . import torch_ops  # noqa: F401  (registers the operators)

    idx, weight = torch.ops.comfyui_b200.hidream_gate(x.view(-1, x.shape[-1]), w.detach())
    return idx, weight.to(x.dtype)


def hidream_moe_infer(moe, x: torch.Tensor, flat_expert_indices: torch.Tensor,
                      flat_expert_weights: torch.Tensor) -> Optional[torch.Tensor]:
    """moe_infer (routed experts only, caller-supplied routing) on the kernels, or None."""
    if x.dim() != 2:
        return None
    layer = _layer_pack(moe, x)
    if layer is None or not flat_expert_indices.is_cuda:
        return None
    from . import moe_ops

    n = x.shape[0]
    e = layer.n_experts
    idx = flat_expert_indices.reshape(n, 2).to(torch.int32).contiguous()
    w = flat_expert_weights.reshape(n, 2).to(torch.float32).contiguous()
    counts = moe_ops.route_count(idx, e)
    block_offsets, expert_counts, expert_offsets = moe_ops.route_plan(counts, n, e)
    in13 = layer.experts[0].scale_in13
    x_perm, row_map, _ = moe_ops.permute(x, idx, block_offsets, expert_offsets, e, fp8=layer.fp8, act_scale=in13)
    y_perm, _, _, _ = moe_ops.grouped_swiglu(layer.experts, None, expert_offsets, expert_counts, x_perm, None,
                                              check_status=CHECK_STATUS_EVERY_CALL)
    return moe_ops.combine(y_perm, row_map, w, None)


def swiglu_ffn_forward(ffn, x: torch.Tensor) -> Optional[torch.Tensor]:
    """A dense FeedForwardSwiGLU (the shared expert alone, or a block's text FFN) as a one-group call."""
    from . import moe_ops

    dim = ffn.w1.weight.shape[1]
    if not _input_ok(x, dim):
        return None
    pack = _ffn_pack(ffn, x.device, moe_ops)
    if pack is None or pack.hidden % 128:
        return None
    x2 = x.view(-1, dim)
    if pack.w1.dtype == FP8:
        x2 = moe_ops.quantize_e4m3(x2, pack.scale_in13)     # the activation quantiser of comfy/ops.py:338-343
    _, y, _, _ = moe_ops.grouped_swiglu([], pack, None, None, None, x2, check_status=CHECK_STATUS_EVERY_CALL)
    return y.view(x.shape)


# ---- q / k / v glue of the HiDream attention processor ----------------------------------------------------------
def _bias_linear_state(lin, device, in_features):
    """(weight, bias or None) if this bf16 Linear can feed the grouped GEMM as it is now, else None."""
    if lin.weight_function or lin.bias_function:
        return None
    w, b = lin.weight, lin.bias
    if w.device != device or w.dtype != torch.bfloat16 or w.dim() != 2 or w.stride(1) != 1 or w.shape[1] != in_features:
        return None
    if w.shape[0] % 256 or w.shape[1] % 64 or w.stride(0) % 8 or w.data_ptr() % 16:
        return None
    if b is not None and (b.device != device or b.dtype != torch.bfloat16 or not b.is_contiguous() or b.data_ptr() % 16):
        return None
    return (w.detach(), None if b is None else b.detach())


def grouped_projections(pairs, dests=None):
    """``[lin(x) for lin, x in pairs]`` for bias Linears that share a launch: every (Linear, tokens [.., in]) pair becomes
    one group of one call of the grouped tcgen05 GEMM (a [B, S, in] slice of a longer sequence, whose batch elements
    are not adjacent in memory, becomes one group per batch element).  ``dests`` may name, per pair, a [B, S, out] view
    to write into (rows contiguous; batch elements anywhere), e.g. the rows of a longer joint sequence.  Returns the list
    of outputs, or None when any pair is not eligible (bf16 weights on the tokens' device, no patch closures,
    out_features % 256 == 0, in_features % 64 == 0, at most nine groups)."""
    if not ENABLE_SM100_KERNELS or not pairs:
        return None
    from . import moe_ops

    groups, outs, results = [], [], []
    for i, (lin, x) in enumerate(pairs):
        if not (x.is_cuda and x.dtype == torch.bfloat16 and x.stride(-1) == 1 and model_management.is_sm100(x.device)):
            return None
        state = _bias_linear_state(lin, x.device, x.shape[-1])
        if state is None or x.data_ptr() % 16:
            return None
        w, bias = state
        out = dests[i] if dests is not None and dests[i] is not None else None
        if out is None:
            out = torch.empty(x.shape[:-1] + (w.shape[0],), dtype=x.dtype, device=x.device)
        elif not (out.shape == x.shape[:-1] + (w.shape[0],) and out.dtype == x.dtype and out.device == x.device and
                  out.dim() == 3 and out.stride(2) == 1 and out.stride(1) == out.shape[2] and
                  out.data_ptr() % 16 == 0 and (out.stride(0) * 2) % 16 == 0):
            return None
        if x.is_contiguous() and out.is_contiguous():
            parts = [(x.reshape(-1, x.shape[-1]), out.view(-1, w.shape[0]))]
        elif x.dim() == 3 and x.stride(1) == x.shape[2] and (x.stride(0) * 2) % 16 == 0:
            parts = [(x[j], out[j]) for j in range(x.shape[0])]
        else:
            return None
        for xi, oi in parts:
            groups.append((xi, w, bias))
            outs.append(oi)
        results.append(out)
    operands = {(t.data_ptr(), tuple(t.shape), t.stride(0)) for xi, wi, _ in groups for t in (xi, wi)}
    operands |= {(o.data_ptr(), tuple(o.shape), o.stride(0)) for o in outs}
    if len(groups) > 9 or len(operands) > moe_ops.N.LINEAR_MAX_MAPS:     # one tensor map per distinct operand
        return None
    moe_ops.grouped_linear(groups, outs)
    return results


def _norm_weight(norm, device):
    """bf16 weight of an RMSNorm that can feed the kernel as it is now, else None."""
    if getattr(norm, "weight_function", None) or getattr(norm, "bias_function", None) or norm.weight is None:
        return None
    w = norm.weight
    if w.device != device or w.dtype != torch.bfloat16 or not w.is_contiguous():
        return None
    return w.detach()


def hidream_qkv(attn, image_tokens: torch.Tensor, text_tokens: Optional[torch.Tensor], rope: torch.Tensor,
                image_tokens_masks=None):
    """What ``HiDreamAttnProcessor_flashattn`` does between the six projections and the attention call
    (``comfy/ldm/hidream/model.py:97-137``): q / k RMSNorm, concatenation of image and text tokens, rotary embedding.
    Returns (query, key, value) as [B, S_img + S_txt, heads, head_dim], or None when the call is not eligible.  The
    projections run as one launch of the grouped GEMM when their Linears are eligible, else through the modules' own
    ``forward`` (library GEMMs, as in the reference)."""
    x = image_tokens
    if image_tokens_masks is not None or not ENABLE_SM100_KERNELS or rope is None:
        return None
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 3 and model_management.is_sm100(x.device)):
        return None
    if rope.dtype != torch.float32 or rope.device != x.device or rope.dim() != 6 or not rope.is_contiguous():
        return None
    heads = attn.heads
    inner = attn.inner_dim
    head_dim = inner // heads
    pairs = rope.shape[-3]
    if inner > 4096 or head_dim % 8 or pairs * 2 > head_dim or rope.shape[0] not in (1, x.shape[0]):
        return None
    joint = not attn.single
    if joint and (text_tokens is None or text_tokens.dtype != x.dtype or text_tokens.device != x.device):
        return None
    norms = [attn.q_rms_norm, attn.k_rms_norm] + ([attn.q_rms_norm_t, attn.k_rms_norm_t] if joint else [])
    weights = [_norm_weight(n, x.device) for n in norms]
    if any(w is None for w in weights) or any(abs(n.eps - norms[0].eps) > 0 for n in norms):
        return None
    from . import moe_ops

    b, s_img = x.shape[0], x.shape[1]
    s_txt = text_tokens.shape[1] if joint else 0
    if rope.shape[1] < s_img + s_txt:
        return None
    eps = norms[0].eps if norms[0].eps is not None else torch.finfo(x.dtype).eps
    q, k, v = (torch.empty((b, s_img + s_txt, heads, head_dim), dtype=x.dtype, device=x.device) for _ in range(3))
    # the three (six) projections: one launch of the grouped GEMM when the Linears are plain bf16, else one library
    # GEMM each, as in the reference
    pairs = [(attn.to_q, x), (attn.to_k, x), (attn.to_v, x)]
    if joint:
        pairs += [(attn.to_q_t, text_tokens), (attn.to_k_t, text_tokens), (attn.to_v_t, text_tokens)]
    # the value projections need nothing but the concatenation: the GEMM writes them straight into their rows of v
    v_rows = v.view(b, s_img + s_txt, inner)
    dests = [None, None, v_rows[:, :s_img]] + ([None, None, v_rows[:, s_img:]] if joint else [])
    proj = grouped_projections(pairs, dests)
    v_done = proj is not None
    if proj is None:
        proj = grouped_projections(pairs)
    if proj is None:
        proj = [lin(t) for lin, t in pairs]
    moe_ops.rmsnorm_rope(proj[0], weights[0], eps, rope, heads, q)
    moe_ops.rmsnorm_rope(proj[1], weights[1], eps, rope, heads, k)
    if not v_done:
        moe_ops.rmsnorm_rope(proj[2], None, eps, None, heads, v)
    if joint:
        moe_ops.rmsnorm_rope(proj[3], weights[2], eps, rope, heads, q, s_img, s_img)
        moe_ops.rmsnorm_rope(proj[4], weights[3], eps, rope, heads, k, s_img, s_img)
        if not v_done:
            moe_ops.rmsnorm_rope(proj[5], None, eps, None, heads, v, s_img, 0)
    return q, k, v


# Which kernel runs softmax(q k^T) v on the block path: "kernel" = this library's tcgen05 attention, "library" = PyTorch's
# scaled_dot_product_attention (what the reference calls).  COMFY_B200_ATTENTION overrides.
ATTENTION_BACKEND = os.environ.get("COMFY_B200_ATTENTION", "kernel")


def hidream_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor) -> Optional[torch.Tensor]:
    """``attention(query, key, value)`` of ``comfy/ldm/hidream/model.py:75-76`` on the tcgen05 attention kernel:
    [B, S, H, 128] x 3 (bf16, contiguous) -> [B, S, H * 128], or None when the call is not eligible."""
    if not ENABLE_SM100_KERNELS or ATTENTION_BACKEND != "kernel":
        return None
    q = query
    if not (q.is_cuda and q.dtype == torch.bfloat16 and q.dim() == 4 and q.shape[-1] == 128 and
            model_management.is_sm100(q.device)):
        return None
    for t in (key, value):
        if t.dtype != q.dtype or t.device != q.device or t.dim() != 4 or t.shape[0] != q.shape[0] or \
                t.shape[2:] != q.shape[2:] or not t.is_contiguous():
            return None
    if key.shape != value.shape or not q.is_contiguous() or q.shape[1] == 0 or key.shape[1] == 0:
        return None
    from . import moe_ops

    with _Range("comfyui_b200::attention"):
        return moe_ops.attention_forward(query, key, value)


# ---- Hunyuan3D-2.1 MoE block (GELU feed-forwards with biases) ------------------------------------------------
def _biased_linear_state(lin, device):
    """(weight, bias or None) if this Linear can feed the GELU-MLP kernels as it is now, else None."""
    if lin.weight_function or lin.bias_function:
        return None
    w, b = lin.weight, lin.bias
    if w.device != device or w.dtype != torch.bfloat16 or w.dim() != 2 or w.stride(1) != 1:
        return None
    if b is not None and (b.device != device or b.dtype != torch.bfloat16 or not b.is_contiguous()):
        return None
    return (w, b)


def _mlp_pack(ffn, device, moe_ops):
    """MlpPack for a FeedForward (net.0.proj, net.2), or None; cached on the module like _ffn_pack."""
    states = [_biased_linear_state(l, device) for l in (ffn.net[0].proj, ffn.net[2])]
    if any(s is None for s in states):
        return None
    key = tuple(_tensor_key(t) for s in states for t in s)
    cached = getattr(ffn, "_b200_pack", None)
    if cached is not None and cached[0] == key:
        return cached[1]
    (w1, b1), (w2, b2) = states
    try:
        pack = moe_ops.MlpPack(w1.detach(), None if b1 is None else b1.detach(), w2.detach(),
                               None if b2 is None else b2.detach())
    except ValueError:
        return None
    object.__setattr__(ffn, "_b200_pack", (key, pack))
    return pack


def _mlp_layer_pack(moe, x):
    """MlpLayerPack for a MoEBlock under the current weights, or None when not eligible."""
    from . import moe_ops

    gate_w = moe.gate.weight
    dim = gate_w.shape[1]
    if not _input_ok(x, dim) or moe.training:
        return None
    if moe.moe_top_k != 2 or len(moe.experts) not in (2, 4, 8):
        return None
    if gate_w.device != x.device or gate_w.dtype not in (torch.bfloat16, torch.float32) or not gate_w.is_contiguous():
        return None
    packs = [_mlp_pack(e, x.device, moe_ops) for e in moe.experts]
    shared = _mlp_pack(moe.shared_experts, x.device, moe_ops)
    if shared is None or any(p is None for p in packs):
        return None
    if any(p.hidden != packs[0].hidden or (p.b1 is None) != (packs[0].b1 is None) or
           (p.b2 is None) != (packs[0].b2 is None) for p in packs + [shared]):
        return None
    if packs[0].hidden % 256:
        return None
    key = (_tensor_key(gate_w),) + tuple(id(p) for p in packs) + (id(shared),)
    cached = getattr(moe, "_b200_layer", None)
    if cached is not None and cached[0] == key:
        return cached[1]
    layer = moe_ops.MlpLayerPack(gate_w.detach(), packs, shared, top_k=2)
    object.__setattr__(moe, "_b200_layer", (key, layer))
    return layer


def hunyuan3d_moe_forward(moe, x: torch.Tensor) -> Optional[torch.Tensor]:
    """MoEBlock.forward (eval mode) on the sm_100a kernels, or None when this call is not eligible.
    Goes through the registered operator ``torch.ops.comfyui_b200.hunyuan3d_moe``."""
    layer = _mlp_layer_pack(moe, x)
    if layer is None:
        return None
    from . import moe_ops, torch_ops

    args = getattr(layer, "_op_args", None)
    if args is None:
        args = torch_ops.register(layer)
        layer._op_args = args
    x2 = x.view(-1, x.shape[-1])
    with _Range("comfyui_b200::hunyuan3d_moe"):
        out = torch.ops.comfyui_b200.hunyuan3d_moe(x2, layer.gate, *args)
    _after_layer_call(layer, x2.shape[0])
    return out.view(x.shape)


def hunyuan3d_moe_infer(moe, x: torch.Tensor, flat_expert_indices: torch.Tensor,
                        flat_expert_weights: torch.Tensor) -> Optional[torch.Tensor]:
    """MoEBlock.moe_infer (routed experts only, caller-supplied routing) on the kernels, or None."""
    if x.dim() != 2:
        return None
    layer = _mlp_layer_pack(moe, x)
    if layer is None or not flat_expert_indices.is_cuda:
        return None
    from . import moe_ops

    n, e = x.shape[0], layer.n_experts
    idx = flat_expert_indices.reshape(n, 2).to(torch.int32).contiguous()
    w = flat_expert_weights.reshape(n, 2).to(torch.float32).contiguous()
    counts = moe_ops.route_count(idx, e)
    block_offsets, expert_counts, expert_offsets = moe_ops.route_plan(counts, n, e)
    x_perm, row_map, _ = moe_ops.permute(x, idx, block_offsets, expert_offsets, e)
    y_perm, _, _, _ = moe_ops.grouped_gelu_mlp(layer.experts, None, expert_offsets, expert_counts, x_perm, None,
                                                check_status=CHECK_STATUS_EVERY_CALL)
    return moe_ops.combine(y_perm, row_map, w, None)


def gelu_ffn_forward(ffn, x: torch.Tensor) -> Optional[torch.Tensor]:
    """A dense GELU FeedForward (the shared expert alone) as a one-group call."""
    from . import moe_ops

    dim = ffn.net[0].proj.weight.shape[1]
    if not _input_ok(x, dim):
        return None
    pack = _mlp_pack(ffn, x.device, moe_ops)
    if pack is None or pack.hidden % 256:
        return None
    _, y, _, _ = moe_ops.grouped_gelu_mlp([], pack, None, None, None, x.view(-1, dim),
                                          check_status=CHECK_STATUS_EVERY_CALL)
    return y.view(x.shape)


def _modulation_ok(x: torch.Tensor, *vectors: torch.Tensor) -> bool:
    """shift / scale / gate as the blocks produce them: bf16 chunks [B, 1, D] of one adaLN output on x's device."""
    b, d = x.shape[0], x.shape[-1]
    strides = set()
    for v in vectors:
        if v is None or v.device != x.device or v.dtype != torch.bfloat16 or v.shape[-1] != d or v.stride(-1) != 1:
            return False
        if v.numel() != b * d or v.shape[0] != b or v.data_ptr() % 16 or v.stride(0) % 8:
            return False
        strides.add(v.stride(0))
    return len(strides) == 1


def hidream_block_ffn(norm, ff, x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor,
                      gate: torch.Tensor) -> Optional[torch.Tensor]:
    """Feed-forward half of a HiDream block, ``gate * ff(norm(x) * (1 + scale) + shift) + x``, on the kernels:
    LayerNorm + modulation in one pass, the MoE (or dense SwiGLU) feed-forward, and the gate / residual epilogue
    folded into the combine.  ``norm`` is the block's LayerNorm module (no affine).  None when not eligible."""
    if x.dim() != 3 or getattr(norm, "weight", None) is not None or getattr(norm, "bias", None) is not None:
        return None
    if not _modulation_ok(x, shift, scale, gate):
        return None
    from . import moe_ops

    b, s, d = x.shape
    x2 = x.view(-1, d)
    if hasattr(ff, "experts"):
        layer = _layer_pack(ff, x)
        if layer is None:
            return None
        from . import torch_ops  # noqa: F401  (registers the operators)

        with _Range("comfyui_b200::hidream_moe_block"):
            out = torch.ops.comfyui_b200.hidream_moe_block(x2, shift, scale, gate, s, float(norm.eps), layer.gate,
                                                           *_op_args(layer))
        _after_layer_call(layer, x2.shape[0])
        return out.view(x.shape)
    if not _input_ok(x, ff.w1.weight.shape[1]):
        return None
    pack = _ffn_pack(ff, x.device, moe_ops)
    if pack is None or pack.hidden % 128:
        return None
    x_mod = moe_ops.ln_modulate(x2, shift, scale, s, norm.eps)
    if pack.w1.dtype == FP8:
        x_mod = moe_ops.quantize_e4m3(x_mod, pack.scale_in13)
    _, y, _, _ = moe_ops.grouped_swiglu([], pack, None, None, None, x_mod, check_status=CHECK_STATUS_EVERY_CALL)
    return moe_ops.gate_residual(y, gate, x2, s).view(x.shape)


def hidream_modulated_norm(norm, x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor) -> Optional[torch.Tensor]:
    """``norm(x) * (1 + scale) + shift`` (``comfy/ldm/hidream/model.py:415-416``, ``:497-500``) in one pass, or None."""
    if x.dim() != 3 or getattr(norm, "weight", None) is not None or getattr(norm, "bias", None) is not None:
        return None
    if not _input_ok(x, x.shape[-1]) or not _modulation_ok(x, shift, scale):
        return None
    from . import moe_ops

    b, s, d = x.shape
    return moe_ops.ln_modulate(x.view(-1, d), shift, scale, s, norm.eps).view(x.shape)


def hidream_gated_residual(y: torch.Tensor, gate: torch.Tensor, residual: torch.Tensor) -> Optional[torch.Tensor]:
    """``gate * y + residual`` (``model.py:424``, ``:512-513``) in one pass, or None."""
    x = residual
    if x.dim() != 3 or y.shape != x.shape or y.dtype != x.dtype or not y.is_contiguous():
        return None
    if not _input_ok(x, x.shape[-1]) or not _modulation_ok(x, gate):
        return None
    from . import moe_ops

    b, s, d = x.shape
    return moe_ops.gate_residual(y.view(-1, d), gate, x.view(-1, d), s).view(x.shape)
