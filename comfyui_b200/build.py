"""Builds libcomfy_b200_moe.so in-tree with nvcc for sm_100a.

Run as ``python -m comfyui_b200.build``.  The library has no dependency on libtorch or libcuda at
link time (the tensor-map encoder is looked up through the CUDA runtime), so it also loads on a
machine without a GPU, where only its symbols can be inspected.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_NAME = "libcomfy_b200_moe.so"
LIB_PATH = os.path.join(PKG_DIR, LIB_NAME)

SOURCES = [
    "moe_route.cu",
    "moe_combine.cu",
    "moe_block_glue.cu",
    "moe_grouped_gemm_sm100.cu",
    "moe_peer.cu",
    "attn_glue.cu",
    "attn_fwd_sm100.cu",
    "weight_ingest.cu",
    "moe_c_api.cu",
]
HEADERS = ["moe_common.cuh", "ptx_sm100.cuh", os.path.join("..", "..", "include", "comfy_b200_moe.h")]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the CUDA extension cannot be built")
    return cand


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every kernel for sm_100a into one shared library; returns its path."""
    if not force and not _stale():
        return LIB_PATH
    cmd = [
        _nvcc(),
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-O3", "-std=c++17", "-lineinfo",
        "-shared", "-Xcompiler", "-fPIC",
        "-o", LIB_PATH,
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stdout + res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
