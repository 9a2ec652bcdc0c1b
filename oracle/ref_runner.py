"""Runs the UNMODIFIED reference modules collected under oracle/_ref (see build_ref.py) on the host cores.

TEST INFRASTRUCTURE: used by tests (oracle against reference on fresh inputs), by bench.py's CPU legs (the timed CPU
baseline, kind "reference") and nowhere in the product.  Nothing here reads the reference's own tree: a GPU box has
only the collected copy.

    python -m oracle.ref_runner --tokens 1024 --steps 5 --warmup 1 [--config1]      # prints one JSON object
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

from . import build_ref

_loaded = None


def load():
    """Imports the collected reference in CPU mode.  Returns (comfy.ops, comfy.ldm.hidream.model)."""
    global _loaded
    if _loaded is None:
        if not build_ref.available():
            raise FileNotFoundError("oracle/_ref is not built (python -m oracle.build_ref, needs the reference tree)")
        if build_ref.OUT not in sys.path:
            sys.path.insert(0, build_ref.OUT)
        import comfy.options

        comfy.options.args_parsing = False
        from comfy.cli_args import args

        args.cpu = True
        import comfy.ldm.hidream.model as model
        import comfy.ops as ops

        _loaded = (ops, model)
    return _loaded


def all_threads() -> int:
    torch.set_num_threads(os.cpu_count() or 1)
    return torch.get_num_threads()


def make_module(dim: int, hidden_dim: int, n_experts: int, dtype: torch.dtype, state: dict):
    """The reference's MOEFeedForwardSwiGLU on the CPU with the given state dict (strict)."""
    ops, model = load()
    m = model.MOEFeedForwardSwiGLU(dim, hidden_dim, n_experts, 2, dtype=dtype, device="cpu",
                                   operations=ops.disable_weight_init).eval()
    m.load_state_dict({k: v.to(dtype) for k, v in state.items()}, strict=True)
    return m


def time_layer(n_tokens: int, steps: int, warmup: int, dtype: torch.dtype = torch.bfloat16, dim: int = 2560,
               hidden_dim: int = 10240, n_experts: int = 4, bench_tokens: int = 8192):
    """tokens/s of the reference layer (gate in fp32, moe_infer, shared expert) on the first n_tokens of the seeded
    bench input, all host threads."""
    from . import hidream_moe_oracle as O

    cores = all_threads()
    m = make_module(dim, hidden_dim, n_experts, dtype, O.make_layer(dim, hidden_dim, n_experts, seed=0))
    gate32 = None
    x = O.make_input(bench_tokens, dim, seed=1).to(dtype)[:n_tokens].contiguous().view(1, n_tokens, dim)

    def call():
        nonlocal gate32
        if dtype == torch.float32:
            idx, w, _ = m.gate(x)
        else:
            if gate32 is None:
                import copy

                gate32 = copy.deepcopy(m.gate).float()
            idx, w, _ = gate32(x.float())
        x2 = x.view(-1, dim)
        return m.moe_infer(x2, idx.view(-1), w.to(dtype).view(-1, 1)) + m.shared_experts(x2)

    with torch.no_grad():
        for _ in range(warmup):
            call()
        t0 = time.perf_counter()
        for _ in range(steps):
            call()
        dt = (time.perf_counter() - t0) / max(steps, 1)
    return {"tokens_per_s": n_tokens / dt, "s_per_step": dt, "cores": cores, "tokens": n_tokens, "steps": steps}


def time_config1(reps: int = 3, dim: int = 2560, hidden_dim: int = 10240, n_experts: int = 4, n: int = 4096):
    """Benchmark configuration 1: fp32, [1, 4096, 2560]; the module's forward as shipped, and moe_infer + shared."""
    from . import hidream_moe_oracle as O

    cores = all_threads()
    m = make_module(dim, hidden_dim, n_experts, torch.float32, O.make_layer(dim, hidden_dim, n_experts, seed=0))
    x = O.make_input(n, dim, seed=1).view(1, n, dim)

    def infer():
        idx, w, _ = m.gate(x)
        x2 = x.view(-1, dim)
        return m.moe_infer(x2, idx.view(-1), w.view(-1, 1)) + m.shared_experts(x2)

    out = {"workload": "benchmark configuration 1: fp32, 4096 tokens, dim 2560, 4 experts top-2 + shared",
           "cores": cores, "reps": reps}
    flops = 2 * 2 * 3 * dim * 6912 + 2 * 3 * dim * 3584 + 2 * dim * n_experts
    with torch.no_grad():
        for name, fn in (("forward", lambda: m(x)), ("moe_infer_plus_shared", infer)):
            fn()
            best = None
            for _ in range(reps):
                t0 = time.perf_counter()
                fn()
                dt = time.perf_counter() - t0
                best = dt if best is None else min(best, dt)
            out[name] = {"s_per_call": best, "tokens_per_s": n / best, "tflops": flops * n / best / 1e12}
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--config1", action="store_true")
    ap.add_argument("--config1-reps", type=int, default=2)
    a = ap.parse_args()
    res = {"layer": time_layer(a.tokens, a.steps, a.warmup)}
    if a.config1:
        res["config1_fp32"] = time_config1(a.config1_reps)
    print(json.dumps(res))


if __name__ == "__main__":
    main()
