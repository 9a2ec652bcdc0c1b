"""ctypes binding of libcomfy_b200_moe.so (declared in include/comfy_b200_moe.h).

There is no CPU or PyTorch fallback here: if the shared library is missing the import of the
kernels fails with an error that tells how to build it.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_uint32, c_void_p

from . import build as _build

ABI_VERSION = 9

OK, EINVAL, EUNSUPPORTED, ECUDA, ETIMEOUT, EDEVICE, ETOOLARGE = range(7)
BF16, FP32, FP8_E4M3, FP16 = 0, 1, 2, 3
ROW_ALIGN = 128
TOKENS_PER_BLOCK = 32
MAX_EXPERTS = 8
STATIC_MAX_TOKENS = 131072
STATUS_WORDS = 4         # [0] sticky device status, [1] near-ties of the last gate call, [2] e4m3 overflows, [3] reserved
LINEAR_MAX_MAPS = 22     # COMFY_MOE_LINEAR_MAX_MAPS: distinct operands of one comfy_moe_grouped_linear call
MAX_RANKS = 8
EP_ARRIVED, EP_DONE = 0, 1

EXPORTS = (
    "comfy_moe_abi_version",
    "comfy_moe_error_string",
    "comfy_moe_plan_sizes",
    "comfy_moe_gate_topk",
    "comfy_moe_route_count",
    "comfy_moe_route_plan",
    "comfy_moe_permute",
    "comfy_moe_plan_permute",
    "comfy_moe_route_static",
    "comfy_moe_validate_routing",
    "comfy_moe_grouped_swiglu",
    "comfy_moe_grouped_gelu_mlp",
    "comfy_moe_grouped_swiglu_scatter",
    "comfy_moe_grouped_swiglu_ex",
    "comfy_moe_combine",
    "comfy_moe_combine_partials",
    "comfy_moe_forward",
    "comfy_moe_forward_gelu_mlp",
    "comfy_moe_ln_modulate",
    "comfy_moe_gate_residual",
    "comfy_moe_ln_modulate_gate",
    "comfy_moe_combine_block",
    "comfy_moe_ffn_block",
    "comfy_moe_read_status",
    "comfy_moe_quantize_e4m3",
    "comfy_moe_stochastic_round_e4m3",
    "comfy_moe_quantize_weight_e4m3",
    "comfy_attn_rmsnorm_rope",
    "comfy_attn_forward",
    "comfy_moe_grouped_linear",
    "comfy_moe_ep_dispatch",
    "comfy_moe_ep_signal",
    "comfy_moe_ep_wait",
    "comfy_moe_ep_wait_budget",
    "comfy_moe_ep_combine",
)


class FfnWeights(Structure):
    """struct ComfyMoeFfnWeights"""

    _fields_ = [
        ("w1", c_void_p),
        ("w3", c_void_p),
        ("w2", c_void_p),
        ("ld13", c_int64),
        ("ld2", c_int64),
        ("hidden", c_int32),
        ("max_sms", c_int32),
        ("scale_w1", c_void_p),
        ("scale_w3", c_void_p),
        ("scale_w2", c_void_p),
        ("scale_in13", c_void_p),
        ("scale_in2", c_void_p),
    ]


class Layer(Structure):
    """struct ComfyMoeLayer"""

    _fields_ = [
        ("dim", c_int32),
        ("n_experts", c_int32),
        ("top_k", c_int32),
        ("w_dtype", c_int32),
        ("gate_dtype", c_int32),
        ("reserved", c_int32),
        ("w_gate", c_void_p),
        ("experts", FfnWeights * MAX_EXPERTS),
        ("shared", FfnWeights),
    ]


class MlpWeights(Structure):
    """struct ComfyMoeMlpWeights"""

    _fields_ = [
        ("w1", c_void_p),
        ("b1", c_void_p),
        ("w2", c_void_p),
        ("b2", c_void_p),
        ("ld1", c_int64),
        ("ld2", c_int64),
        ("hidden", c_int32),
        ("reserved", c_int32),
    ]


class MlpLayer(Structure):
    """struct ComfyMoeMlpLayer"""

    _fields_ = [
        ("dim", c_int32),
        ("n_experts", c_int32),
        ("top_k", c_int32),
        ("gate_dtype", c_int32),
        ("w_gate", c_void_p),
        ("experts", MlpWeights * MAX_EXPERTS),
        ("shared", MlpWeights),
    ]


class LinearGroup(Structure):
    """struct ComfyMoeLinearGroup"""

    _fields_ = [
        ("x", c_void_p),
        ("w", c_void_p),
        ("bias", c_void_p),
        ("out", c_void_p),
        ("ld_x", c_int64),
        ("ld_w", c_int64),
        ("ld_out", c_int64),
        ("rows", c_int32),
        ("in_features", c_int32),
        ("out_features", c_int32),
        ("reserved", c_int32),
    ]


class GroupedOptions(Structure):
    """struct ComfyMoeGroupedOptions"""

    _fields_ = [
        ("passes", c_int32),
        ("reserved", c_int32),
        ("y_out", POINTER(c_void_p)),
        ("y_row_shift", c_void_p),
        ("y_rows_cap", c_int64),
        ("arrive_flags", c_void_p),
        ("group_source", POINTER(c_int32)),
        ("arrive_epoch", c_uint32),
        ("reserved2", c_uint32),
        ("arrive_budget_cycles", c_int64),
    ]


class PeerPlan(Structure):
    """struct ComfyMoePeerPlan"""

    _fields_ = [
        ("world", c_int32),
        ("rank", c_int32),
        ("n_experts", c_int32),
        ("hidden_splits", c_int32),
        ("owner0", c_int32 * MAX_EXPERTS),
        ("owner1", c_int32 * MAX_EXPERTS),
        ("cap_rows", c_int64),
        ("peer_recv", c_void_p * MAX_RANKS),
        ("peer_y", c_void_p * MAX_RANKS),
        ("peer_flags", c_void_p * MAX_RANKS),
    ]


class Workspace(Structure):
    """struct ComfyMoeWorkspace"""

    _fields_ = [
        ("topk_idx", c_void_p),
        ("topk_weight", c_void_p),
        ("block_counts", c_void_p),
        ("block_offsets", c_void_p),
        ("expert_counts", c_void_p),
        ("expert_offsets", c_void_p),
        ("row_map", c_void_p),
        ("status", c_void_p),
        ("x_perm", c_void_p),
        ("x_q", c_void_p),
        ("h_perm", c_void_p),
        ("y_perm", c_void_p),
        ("h_shared", c_void_p),
        ("y_shared", c_void_p),
        ("rows_cap", c_int64),
        ("x_mod", c_void_p),
    ]


class MoeError(RuntimeError):
    def __init__(self, fn: str, code: int, text: str):
        super().__init__(f"{fn} failed with code {code}: {text}")
        self.code = code


_lib = None


def lib_path() -> str:
    """Path of the shared library; COMFY_B200_LIB overrides it (comparison builds)."""
    return os.environ.get("COMFY_B200_LIB") or _build.LIB_PATH


def load(build_if_missing: bool = False) -> ctypes.CDLL:
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        if build_if_missing:
            _build.build()
        else:
            raise ImportError(
                f"{path} is missing: the sm_100a kernels are not built. "
                "Run `python -m comfyui_b200.build` (needs nvcc); there is no fallback path."
            )
    lib = ctypes.CDLL(path)
    lib.comfy_moe_abi_version.restype = c_int
    lib.comfy_moe_error_string.restype = c_char_p
    lib.comfy_moe_error_string.argtypes = [c_int]
    lib.comfy_moe_plan_sizes.argtypes = [c_int, c_int, c_int, POINTER(c_int64), POINTER(c_int)]
    lib.comfy_moe_gate_topk.argtypes = [
        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
        c_float, c_void_p,
    ]
    lib.comfy_moe_route_count.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p]
    lib.comfy_moe_route_plan.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
    lib.comfy_moe_permute.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p, c_void_p,
    ]
    lib.comfy_moe_plan_permute.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
    ]
    lib.comfy_moe_route_static.argtypes = [
        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
    ]
    lib.comfy_moe_validate_routing.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_void_p,
                                               c_void_p]
    lib.comfy_moe_grouped_swiglu.argtypes = [
        c_int, c_int, POINTER(FfnWeights), POINTER(FfnWeights), c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
    ]
    lib.comfy_moe_grouped_gelu_mlp.argtypes = [
        c_int, POINTER(MlpWeights), POINTER(MlpWeights), c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
    ]
    lib.comfy_moe_forward_gelu_mlp.argtypes = [POINTER(MlpLayer), POINTER(Workspace), c_void_p, c_int, c_void_p,
                                               c_void_p]
    lib.comfy_moe_combine.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]
    lib.comfy_moe_combine_partials.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                               c_void_p]
    lib.comfy_moe_forward.argtypes = [POINTER(Layer), POINTER(Workspace), c_void_p, c_int, c_void_p, c_void_p]
    lib.comfy_moe_ln_modulate.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_float, c_void_p,
                                          c_void_p]
    lib.comfy_moe_ln_modulate_gate.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_int, c_int,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p,
    ]
    lib.comfy_moe_gate_residual.argtypes = [c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
    lib.comfy_moe_combine_block.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int,
                                            c_int, c_int, c_void_p, c_void_p]
    lib.comfy_moe_ffn_block.argtypes = [POINTER(Layer), POINTER(Workspace), c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_int64, c_int, c_int, c_float, c_void_p, c_void_p]
    lib.comfy_moe_read_status.argtypes = [c_void_p, c_void_p, POINTER(c_int32)]
    lib.comfy_moe_ep_dispatch.argtypes = [
        POINTER(PeerPlan), c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
    ]
    lib.comfy_moe_grouped_swiglu_scatter.argtypes = [
        c_int, c_int, POINTER(FfnWeights), c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, POINTER(c_void_p),
        c_void_p, c_int64, c_void_p, c_void_p,
    ]
    lib.comfy_moe_grouped_swiglu_ex.argtypes = [
        c_int, c_int, POINTER(FfnWeights), POINTER(FfnWeights), c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, POINTER(GroupedOptions), c_void_p, c_void_p,
    ]
    lib.comfy_moe_quantize_e4m3.argtypes = [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]
    lib.comfy_attn_rmsnorm_rope.argtypes = [c_void_p, c_int64, c_void_p, c_float, c_void_p, c_int64, c_int, c_int, c_int,
                                            c_int, c_int, c_int, c_void_p, c_int64, c_int, c_void_p]
    lib.comfy_attn_forward.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                       c_void_p, c_void_p]
    lib.comfy_moe_grouped_linear.argtypes = [c_int, POINTER(LinearGroup), c_void_p, c_void_p]
    lib.comfy_moe_stochastic_round_e4m3.argtypes = [c_void_p, c_int, c_void_p, c_int64, c_void_p, c_void_p]
    lib.comfy_moe_quantize_weight_e4m3.argtypes = [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p]
    lib.comfy_moe_ep_signal.argtypes = [POINTER(PeerPlan), c_int, c_uint32, c_void_p]
    lib.comfy_moe_ep_wait.argtypes = [POINTER(PeerPlan), c_int, c_uint32, c_void_p, c_void_p]
    lib.comfy_moe_ep_wait_budget.argtypes = [POINTER(PeerPlan), c_int, c_uint32, c_int64, c_void_p, c_void_p]
    lib.comfy_moe_ep_combine.argtypes = [POINTER(PeerPlan), c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                         c_void_p, c_void_p]
    for name in EXPORTS:
        if name not in ("comfy_moe_error_string",):
            getattr(lib, name).restype = c_int
    if lib.comfy_moe_abi_version() != ABI_VERSION:
        raise ImportError(f"{path}: ABI version {lib.comfy_moe_abi_version()} != expected {ABI_VERSION}; rebuild it")
    _lib = lib
    return lib


def check(fn: str, code: int) -> None:
    if code != OK:
        raise MoeError(fn, code, load().comfy_moe_error_string(code).decode())
