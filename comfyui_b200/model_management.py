"""The three helpers of ComfyUI's ``comfy/model_management.py`` that the MoE feed-forward touches.

Only what the hot path needs is here: ``cast_to`` (``model_management.py:1055-1072``, used by the
gate for its bare Parameter), ``supports_fp8_compute`` (``:1353-1375``, decides whether scaled-fp8
Linears multiply in fp8) and the offload-stream hooks ``cast_bias_weight`` calls (``:1012-1053``).
Device selection, VRAM accounting and model loading are out of scope.
"""
from __future__ import annotations

from typing import Optional

import torch

# Set by an embedding application that wants weights copied on side streams (the reference's
# --async-offload).  With the default of one stream, casts run on the current stream.
NUM_STREAMS = 1
FORCE_FP8_COMPUTE = False      # the reference's --supports-fp8-compute
DETERMINISTIC = False          # the reference's --deterministic: blocking copies only

_streams = {}
_cursor = {}


def is_device_cuda(device) -> bool:
    return getattr(device, "type", None) == "cuda"


def device_supports_non_blocking(device) -> bool:
    if DETERMINISTIC:
        return False
    return getattr(device, "type", "cpu") in ("cuda", "cpu")


def get_offload_stream(device) -> Optional["torch.cuda.Stream"]:
    """Round-robin side stream for weight copies, or None when offloading is synchronous."""
    if NUM_STREAMS <= 1 or not is_device_cuda(device):
        return None
    pool = _streams.get(device)
    if pool is None:
        pool = [torch.cuda.Stream(device=device, priority=0) for _ in range(NUM_STREAMS)]
        _streams[device] = pool
    i = _cursor.get(device, 0)
    chosen = pool[i]
    nxt = (i + 1) % len(pool)
    # the stream handed out next must not overtake work already queued on the compute stream
    pool[nxt].wait_stream(torch.cuda.current_stream())
    _cursor[device] = nxt
    return chosen


def sync_stream(device, stream) -> None:
    if stream is not None and is_device_cuda(device):
        torch.cuda.current_stream().wait_stream(stream)


def cast_to(weight: torch.Tensor, dtype=None, device=None, non_blocking: bool = False, copy: bool = False,
            stream=None) -> torch.Tensor:
    """Return ``weight`` in ``dtype`` on ``device``; the tensor itself when nothing has to change and no
    copy was asked for."""
    same_device = device is None or weight.device == device
    if same_device and not copy and (dtype is None or weight.dtype == dtype):
        return weight

    def run():
        if same_device:
            return weight.to(dtype=dtype, copy=copy)
        r = torch.empty_like(weight, dtype=dtype, device=device)
        r.copy_(weight, non_blocking=non_blocking)
        return r

    if stream is not None:
        with stream:
            return run()
    return run()


def supports_fp8_compute(device=None) -> bool:
    """True when fp8 tensor-core matmuls are worth using on ``device`` (Ada sm_89 and everything from
    Hopper up; B200 is sm_100)."""
    if FORCE_FP8_COMPUTE:
        return True
    if not torch.cuda.is_available():
        return False
    if device is not None and not is_device_cuda(torch.device(device)):
        return False
    major, minor = torch.cuda.get_device_capability(device)
    return major >= 9 or (major == 8 and minor >= 9)


def is_sm100(device) -> bool:
    """The hand-written kernels are built for sm_100a only."""
    if not (torch.cuda.is_available() and is_device_cuda(device)):
        return False
    return torch.cuda.get_device_capability(device)[0] == 10
