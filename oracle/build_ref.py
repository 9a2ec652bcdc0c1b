"""Recipe for oracle/_ref: the unmodified reference, where it can run, as a checker and CPU baseline.

TEST INFRASTRUCTURE, like everything under oracle/: only tests, the smoke check and bench.py's CPU legs may use what
this builds; the product never does.

The reference's code for this path is pure Python over PyTorch, so "building" it means collecting the files the path
imports.  This script imports ``comfy.ldm.hidream.model`` (and the Hunyuan3D-2.1 MoE block) from the reference tree
in a child process, records which of the tree's modules that import really loaded (18 files, about 235 KB), and
copies exactly those, byte for byte, to ``oracle/_ref/`` with their relative paths.  ``oracle/_ref/`` is git-ignored:
no reference source enters the history; the directory travels to a GPU box like any other build output, where
``oracle/ref_runner.py`` imports it to time the reference's own ``MOEFeedForwardSwiGLU`` on the host cores.

    python -m oracle.build_ref [reference_root]        # default: $COMFY_REFERENCE_ROOT, else ~/reference
"""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

_PROBE = r"""
import json, os, sys
root = sys.argv[1]
sys.path.insert(0, root)
import comfy.options
comfy.options.args_parsing = False
from comfy.cli_args import args
args.cpu = True
import comfy.model_management, comfy.ops, comfy.float                     # noqa: E402,F401
import comfy.ldm.hidream.model                                            # noqa: E402,F401
import comfy.ldm.hunyuan3dv2_1.hunyuandit                                 # noqa: E402,F401
files = sorted({os.path.relpath(m.__file__, root) for m in list(sys.modules.values())
                if getattr(m, "__file__", None) and os.path.abspath(m.__file__).startswith(os.path.abspath(root) + os.sep)})
print(json.dumps(files))
"""


def reference_root(arg: str | None = None) -> str:
    return arg or os.environ.get("COMFY_REFERENCE_ROOT") or os.path.join(os.path.expanduser("~"), "reference")


def build(root: str | None = None, quiet: bool = True) -> list[str]:
    """Copies the import closure of the path out of the reference tree.  Returns the relative paths copied."""
    root = reference_root(root)
    if not os.path.isdir(os.path.join(root, "comfy")):
        raise FileNotFoundError(f"no reference tree at {root}")
    res = subprocess.run([sys.executable, "-c", _PROBE, root], capture_output=True, text=True, cwd="/tmp")
    if res.returncode != 0:
        raise RuntimeError("importing the reference failed:\n" + res.stderr[-2000:])
    files = json.loads(res.stdout.strip().splitlines()[-1])
    if os.path.isdir(OUT):
        shutil.rmtree(OUT)
    for rel in files:
        dst = os.path.join(OUT, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(root, rel), dst)
    with open(os.path.join(OUT, "MANIFEST.json"), "w") as f:
        json.dump({"reference_root": root, "files": files}, f, indent=1)
    if not quiet:
        print(f"oracle/_ref: {len(files)} files of the reference copied")
    return files


def available() -> bool:
    return os.path.exists(os.path.join(OUT, "MANIFEST.json"))


if __name__ == "__main__":
    build(sys.argv[1] if len(sys.argv) > 1 else None, quiet=False)
