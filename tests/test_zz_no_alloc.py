"""comfy_moe_route_static: the routing steps for callers that cannot allocate device memory.

Some users of the library (real-time loops that reserve all device memory at start-up, plugins living in a
fixed arena handed to them by their host) may not call an allocator while they run.  For them the library
offers one entry point whose scratch lives in a fixed device array inside the library.  This test calls it
through the C ABI, twice in a row on different inputs, and requires bit-identical outputs to the regular
entry points (gate, plan, permutation), which take their scratch from the caller.

The file name sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _route_static(lib, N, x, w_gate, n_experts, fp8=False, scale=None):
    n, d = x.shape
    dev = x.device
    rows_cap = 2 * n + n_experts * N.ROW_ALIGN
    if fp8:
        return _route_static_fp8(lib, N, x, w_gate, n_experts, scale, rows_cap)
    out = dict(
        idx=torch.empty((n, 2), dtype=torch.int32, device=dev),
        w=torch.empty((n, 2), dtype=torch.float32, device=dev),
        counts=torch.empty((n_experts,), dtype=torch.int32, device=dev),
        offsets=torch.empty((n_experts + 1,), dtype=torch.int32, device=dev),
        x_perm=torch.zeros((rows_cap, d), dtype=torch.bfloat16, device=dev),
        row_map=torch.empty((n, 2), dtype=torch.int32, device=dev),
        ties=torch.zeros((1,), dtype=torch.int32, device=dev),
    )
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.comfy_moe_route_static(_ptr(x), _ptr(w_gate), N.BF16, n, d, n_experts, 2, N.BF16, None, _ptr(out["idx"]),
                                    _ptr(out["w"]), _ptr(out["counts"]), _ptr(out["offsets"]), _ptr(out["x_perm"]),
                                    None, None, _ptr(out["row_map"]), _ptr(out["ties"]), stream)
    assert rc == N.OK, lib.comfy_moe_error_string(rc)
    torch.cuda.synchronize()
    return out


def _route_static_fp8(lib, N, x, w_gate, n_experts, scale, rows_cap):
    """The same call with e4m3 activations: the permuted rows and the shared expert's copy are quantised on the way."""
    n, d = x.shape
    dev = x.device
    out = dict(
        idx=torch.empty((n, 2), dtype=torch.int32, device=dev),
        w=torch.empty((n, 2), dtype=torch.float32, device=dev),
        counts=torch.empty((n_experts,), dtype=torch.int32, device=dev),
        offsets=torch.empty((n_experts + 1,), dtype=torch.int32, device=dev),
        x_perm=torch.zeros((rows_cap, d), dtype=torch.uint8, device=dev),
        x_q=torch.zeros((n, d), dtype=torch.uint8, device=dev),
        row_map=torch.empty((n, 2), dtype=torch.int32, device=dev),
        ties=torch.zeros((1,), dtype=torch.int32, device=dev),
    )
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.comfy_moe_route_static(_ptr(x), _ptr(w_gate), N.BF16, n, d, n_experts, 2, N.FP8_E4M3, _ptr(scale),
                                    _ptr(out["idx"]), _ptr(out["w"]), _ptr(out["counts"]), _ptr(out["offsets"]),
                                    _ptr(out["x_perm"]), _ptr(out["x_q"]), _ptr(scale), _ptr(out["row_map"]),
                                    _ptr(out["ties"]), stream)
    assert rc == N.OK, lib.comfy_moe_error_string(rc)
    torch.cuda.synchronize()
    return out


def _route_regular(M, x, w_gate, n_experts, fp8=False, scale=None):
    n = x.shape[0]
    idx, w, block_counts, ties, _ = M.gate_topk(x, w_gate)
    block_offsets, counts, offsets = M.route_plan(block_counts, n, n_experts)
    x_perm, row_map, x_q = M.permute(x, idx, block_offsets, offsets, n_experts, zero_fill=True, fp8=fp8, want_xq=fp8,
                                     act_scale=scale, xq_scale=scale)
    torch.cuda.synchronize()
    res = dict(idx=idx, w=w, counts=counts, offsets=offsets, x_perm=x_perm, row_map=row_map, ties=ties)
    if fp8:
        res["x_perm"], res["x_q"] = x_perm.view(torch.uint8), x_q.view(torch.uint8)
    return res


def test_route_static_matches_regular_entry_points(cuda_device):
    from comfyui_b200 import _native as N
    from comfyui_b200 import moe_ops as M

    lib = N.load()
    dev = cuda_device
    g = torch.Generator().manual_seed(11)
    # two calls in a row: the second is smaller and has another expert count, so anything the first call left in
    # the shared scratch array would show up as a difference
    for n, d, e in ((4480, 2560, 4), (333, 512, 8)):
        x = torch.randn((n, d), generator=g).bfloat16().to(dev)
        w_gate = (torch.randn((e, d), generator=g) * 0.02).bfloat16().to(dev)
        got = _route_static(lib, N, x, w_gate, e)
        ref = _route_regular(M, x, w_gate, e)
        for key in ("idx", "w", "counts", "offsets", "row_map", "x_perm", "ties"):
            assert torch.equal(got[key], ref[key]), f"{key} differs at n={n}"


def test_route_static_fp8_activations(cuda_device):
    """The e4m3 variant (rows quantised on the way, with and without a scale_input), again two calls in a row."""
    from comfyui_b200 import _native as N
    from comfyui_b200 import moe_ops as M

    lib = N.load()
    dev = cuda_device
    g = torch.Generator().manual_seed(12)
    for n, d, e, s_in in ((1000, 2560, 4, None), (257, 512, 4, 0.75)):
        x = torch.randn((n, d), generator=g).bfloat16().to(dev)
        w_gate = (torch.randn((e, d), generator=g) * 0.02).bfloat16().to(dev)
        scale = None if s_in is None else torch.tensor(s_in, device=dev)
        got = _route_static(lib, N, x, w_gate, e, fp8=True, scale=scale)
        ref = _route_regular(M, x, w_gate, e, fp8=True, scale=scale)
        for key in ("idx", "w", "counts", "offsets", "row_map", "x_perm", "x_q", "ties"):
            assert torch.equal(got[key], ref[key]), f"{key} differs at n={n}"


def test_route_static_at_its_token_limit(cuda_device):
    """Exactly COMFY_MOE_STATIC_MAX_TOKENS tokens use the whole built-in scratch array; a small call follows it."""
    from comfyui_b200 import _native as N
    from comfyui_b200 import moe_ops as M

    lib = N.load()
    dev = cuda_device
    g = torch.Generator().manual_seed(13)
    for n, d, e in ((N.STATIC_MAX_TOKENS, 256, 8), (100, 256, 4)):
        x = torch.randn((n, d), generator=g).bfloat16().to(dev)
        w_gate = (torch.randn((e, d), generator=g) * 0.05).bfloat16().to(dev)
        got = _route_static(lib, N, x, w_gate, e)
        ref = _route_regular(M, x, w_gate, e)
        for key in ("idx", "w", "counts", "offsets", "row_map", "x_perm", "ties"):
            assert torch.equal(got[key], ref[key]), f"{key} differs at n={n}"


def test_route_static_rejects_oversize(cuda_device):
    from comfyui_b200 import _native as N

    lib = N.load()
    rc = lib.comfy_moe_route_static(None, None, N.BF16, N.STATIC_MAX_TOKENS + 1, 2560, 4, 2, N.BF16, None, None, None,
                                    None, None, None, None, None, None, None, None)
    assert rc == N.ETOOLARGE
    assert b"COMFY_MOE_STATIC_MAX_TOKENS" in lib.comfy_moe_error_string(rc)
