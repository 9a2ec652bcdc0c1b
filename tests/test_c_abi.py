"""The C-ABI shared library: builds for sm_100a, loads without a GPU and exports what the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from comfyui_b200 import _native, build

    build.build()
    return _native.load()


def _declared_functions():
    names = []
    inc = os.path.join(ROOT, "include")
    for fn in sorted(os.listdir(inc)):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names += re.findall(r"\b(comfy_(?:moe|attn)_\w+)\s*\(", text)
    return sorted(set(names))


def test_every_declared_symbol_is_exported(lib):
    declared = _declared_functions()
    assert len(declared) >= 11
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"


def test_binding_lists_match_header(lib):
    from comfyui_b200 import _native

    assert sorted(_native.EXPORTS) == _declared_functions()
    assert lib.comfy_moe_abi_version() == _native.ABI_VERSION


def test_struct_layouts_match_header():
    """ctypes mirrors of the C structs: sizes follow from the header's field lists (LP64)."""
    from comfyui_b200 import _native as N

    assert ctypes.sizeof(N.FfnWeights) == 3 * 8 + 2 * 8 + 2 * 4 + 5 * 8
    assert ctypes.sizeof(N.Layer) == 6 * 4 + 8 + (N.MAX_EXPERTS + 1) * ctypes.sizeof(N.FfnWeights)
    assert ctypes.sizeof(N.Workspace) == 16 * 8
    assert ctypes.sizeof(N.MlpWeights) == 4 * 8 + 2 * 8 + 2 * 4
    assert ctypes.sizeof(N.MlpLayer) == 4 * 4 + 8 + (N.MAX_EXPERTS + 1) * ctypes.sizeof(N.MlpWeights)
    assert ctypes.sizeof(N.PeerPlan) == 4 * 4 + 2 * 4 * N.MAX_EXPERTS + 8 + 3 * 8 * N.MAX_RANKS
    assert N.FfnWeights.max_sms.offset == 3 * 8 + 2 * 8 + 4
    assert ctypes.sizeof(N.LinearGroup) == 4 * 8 + 3 * 8 + 4 * 4


def test_plan_sizes(lib):
    rows, blocks = ctypes.c_int64(), ctypes.c_int()
    assert lib.comfy_moe_plan_sizes(8192, 4, 2, rows, blocks) == 0
    assert rows.value == 2 * 8192 + 4 * 128 and blocks.value == 256
    assert lib.comfy_moe_plan_sizes(1, 4, 2, rows, blocks) == 0
    assert rows.value == 2 + 512 and blocks.value == 1
    assert lib.comfy_moe_plan_sizes(0, 4, 2, rows, blocks) == 0 and blocks.value == 0
    assert lib.comfy_moe_plan_sizes(10, 9, 2, rows, blocks) != 0      # more experts than the kernels cover
    assert lib.comfy_moe_plan_sizes(10, 4, 3, rows, blocks) != 0      # top-k other than 2
    assert lib.comfy_moe_plan_sizes(-1, 4, 2, rows, blocks) != 0


def test_argument_validation_needs_no_gpu(lib):
    """Bad arguments are rejected on the host before any CUDA call."""
    from comfyui_b200 import _native as N

    assert lib.comfy_moe_gate_topk(None, None, 0, 16, 256, 4, 2, None, None, None, None, None, 1e-6, None) == N.EINVAL
    assert lib.comfy_moe_gate_topk(None, None, 0, 0, 256, 4, 2, None, None, None, None, None, 1e-6, None) == N.OK
    assert lib.comfy_moe_combine(None, None, None, None, 8, 256, None, None) == N.EINVAL
    assert lib.comfy_moe_permute(None, None, None, None, -1, 256, 4, 0, None, None, None, None, None, None, None) == N.EINVAL
    assert lib.comfy_moe_forward(None, None, None, 8, None, None) == N.EINVAL
    assert lib.comfy_moe_read_status(None, None, None) == N.EINVAL
    for code in range(6):
        assert len(lib.comfy_moe_error_string(code)) > 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    """No fallback: when the shared object is absent the loader raises and says how to build it."""
    from comfyui_b200 import _native, build

    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(build, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="comfyui_b200.build"):
        _native.load()


def test_kernels_refuse_cpu_tensors(lib):
    import torch

    from comfyui_b200 import moe_ops

    x = torch.zeros(8, 256, dtype=torch.bfloat16)
    w = torch.zeros(4, 256, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="no CPU path"):
        moe_ops.gate_topk(x, w)
