#!/usr/bin/env python
"""Benchmark of the HiDream MoE feed-forward layer: tokens/s of one full layer call.

    python bench.py --gpus N --steps K --warmup W            # this repository's sm_100a kernels
    python bench.py --impl reference --steps K --warmup W    # the reference algorithm on the host cores

A step is one call of the layer (gate -> plan -> permute -> grouped SwiGLU GEMM x2 -> combine, shared expert
included) on synthetic data: dim 2560, 4 routed experts of hidden 6912 (top-2), shared expert of hidden 3584,
bf16, 8192 tokens per GPU, weights N(0, 0.02^2), inputs N(0, 1), seeded.  With N > 1 the routed experts are
expert-parallel (rows dispatched and results returned by the kernels themselves over NVLink peer memory; the one
collective is an NCCL all-gather of the routing histograms), every rank owns 8192 tokens (weak scaling) and runs
the shared expert on them.

One JSON line is printed by rank 0.  `value` is measured with the inputs resident in HBM; `e2e` is the same
metric through the module call with pinned-host input and output copies inside the timed region; `roofline`
describes the grouped GEMM (both passes) against the measured bf16 tensor peak; `cpu_baseline` is the CPU
oracle (a restatement of the reference's PyTorch code) timed on this machine's host cores.  After the headline
loop, and outside its timed region, the default run adds sub-objects to the same line: `sustained` (the same
loop for more than a second, at the power-capped clock), `fp8` (benchmark configuration 3, same measurements),
`config5` (131 072 tokens in total, skewed router, strong scaling) and, with N > 1, `ep_parity` (every rank
compares the expert-parallel output of its tokens with the single-GPU layer).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

DIM, HIDDEN_DIM, N_EXPERTS, TOP_K = 2560, 4 * 2560, 4, 2
HIDDEN, HIDDEN_SHARED = 6912, 3584
TOKENS_PER_GPU = 8192
METRIC = "MoE-FFN tokens/s (HiDream MOEFeedForwardSwiGLU layer, dim 2560, 4 experts top-2 + shared)"
FLOPS_PER_TOKEN_GEMM = 2 * TOP_K * 3 * DIM * HIDDEN + 2 * 3 * DIM * HIDDEN_SHARED
FLOPS_PER_TOKEN = FLOPS_PER_TOKEN_GEMM + 2 * DIM * N_EXPERTS
CPU_SAMPLE_TOKENS = 1024


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(source="measured", hbm_gbs=p["hbm_gbs"], tflops_burst=p["bf16_tflops"],
                    tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]))
    return dict(source="fallback", hbm_gbs=6650.0, tflops_burst=1590.0, tflops_sustained=1400.0)


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    REASONS = {
        0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
        0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
    }

    def __init__(self, index: int, period_s: float = 0.01):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.period, self._stop, self._thread, self._h, self._nv = period_s, threading.Event(), None, None, None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------ CPU arm
def use_all_host_threads() -> int:
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the CPU arm is meant to use every host core at
    every N, so the thread count is set explicitly."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    return torch.get_num_threads()


def oracle_cpu_tokens_per_s(n_tokens: int, steps: int, warmup: int, dtype: str = "bf16"):
    """The CPU oracle on `n_tokens` of the bench workload, all host threads.  Returns (tokens/s, s/step, cores)."""
    from oracle import hidream_moe_oracle as O

    cores = use_all_host_threads()
    layer = {k: v.bfloat16() for k, v in O.make_layer(DIM, HIDDEN_DIM, N_EXPERTS, seed=0).items()}
    mode = O.PLAIN
    if dtype == "fp8":
        layer, mode = O.quantize_layer_fp8(layer), O.FP8_MATMUL
    x = O.make_input(TOKENS_PER_GPU, DIM, seed=1).bfloat16()[:n_tokens].contiguous()
    with torch.no_grad():
        for _ in range(warmup):
            O.moe_layer(x, layer, mode=mode, gate_in_fp32=True)
        t0 = time.perf_counter()
        for _ in range(steps):
            O.moe_layer(x, layer, mode=mode, gate_in_fp32=True)
        dt = (time.perf_counter() - t0) / max(steps, 1)
    return n_tokens / dt, dt, cores


def oracle_cpu_config1(reps: int = 3):
    """Benchmark configuration 1 on the host cores: the layer in fp32 on [1, 4096, 2560], timed both ways the
    reference can run it: `forward` (the masked branch it really takes) and `moe_infer` + shared expert.  Best of
    `reps` after one warm-up call each."""
    from oracle import hidream_moe_oracle as O

    cores = use_all_host_threads()
    n = 4096
    layer = O.make_layer(DIM, HIDDEN_DIM, N_EXPERTS, seed=0)
    x = O.make_input(n, DIM, seed=1)

    def forward():
        return O.moe_layer(x, layer, gate_in_fp32=True, branch="masked")

    def infer():
        idx, w = O.gate(x, layer["gate.weight"])
        return O.moe_infer(x, idx.reshape(-1), w.reshape(-1, 1), layer) + O.swiglu_ffn(x, layer, "shared_experts")

    out = {"workload": "benchmark configuration 1: fp32, 4096 tokens, dim 2560, 4 experts top-2 + shared", "cores": cores,
           "reps": reps}
    with torch.no_grad():
        for name, fn in (("forward", forward), ("moe_infer_plus_shared", infer)):
            fn()
            best = min(_timed(fn) for _ in range(reps))
            out[name] = {"s_per_call": best, "tokens_per_s": n / best,
                         "tflops": FLOPS_PER_TOKEN * n / best / 1e12}
    return out


def _timed(fn) -> float:
    t0 = time.perf_counter()
    fn()
    return time.perf_counter() - t0


def cpu_arm(n_tokens: int, steps: int, warmup: int, dtype: str):
    """The layer on the host cores: the unmodified reference modules when oracle/_ref holds them (bf16 / fp32; its
    fp8 path, torch._scaled_mm on the CPU, would take hours), else the oracle's restatement.
    Returns (tokens/s, s/step, cores, kind, description)."""
    from oracle import build_ref

    if dtype == "bf16" and build_ref.available():
        from oracle import ref_runner

        r = ref_runner.time_layer(n_tokens, steps, warmup)
        return (r["tokens_per_s"], r["s_per_step"], r["cores"], "reference",
                "the reference's own MoEGate (on x.float()), moe_infer and shared expert, unmodified modules collected "
                "under oracle/_ref, bf16 on the CPU")
    value, dt, cores = oracle_cpu_tokens_per_s(n_tokens, steps, warmup, dtype)
    return (value, dt, cores, "port", "CPU oracle (oracle/hidream_moe_oracle.py: the reference's gate + moe_infer + "
                                      "shared expert restated in PyTorch)")


def cpu_config1(reps: int):
    from oracle import build_ref

    if build_ref.available():
        from oracle import ref_runner

        out = ref_runner.time_config1(reps)
        out["kind"] = "reference"
        return out
    out = oracle_cpu_config1(reps)
    out["kind"] = "port"
    return out


def cpu_baseline_object(dtype: str, reps: int):
    value, dt, cores, kind, what = cpu_arm(CPU_SAMPLE_TOKENS, reps, 2, dtype)
    return {
        "value": value, "unit": "tokens/s", "cores": cores, "kind": kind,
        "sample": f"{reps} calls on the first {CPU_SAMPLE_TOKENS} of the {TOKENS_PER_GPU} bench tokens ({dtype}): {what}, "
                  f"{cores} host threads",
        "config1_fp32": cpu_config1(reps=2),
    }


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    value, dt, cores, kind, what = cpu_arm(CPU_SAMPLE_TOKENS, args.steps, max(args.warmup, 1), args.dtype)
    sample = (f"each step = the first {CPU_SAMPLE_TOKENS} of the {TOKENS_PER_GPU} bench tokens: {what}, {cores} host "
              "threads at every N")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
        "config": workload_config(args.gpus, args.dtype),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "host": {"os_cpu_count": os.cpu_count(), "torch_threads": cores},
        "config1_fp32": cpu_config1(reps=3),
    }
    print(json.dumps(line))


def ep_transport() -> str:
    if os.environ.get("COMFY_B200_EP_TRANSPORT", "peer") == "nccl":
        return "NCCL point-to-point dispatch and combine"
    return "dispatch and combine by the kernels over NVLink peer memory, NCCL all-gather of the routing histograms"


def workload_config(n_gpus: int, dtype: str = "bf16", tokens_per_gpu: int = TOKENS_PER_GPU, config5: bool = False):
    if config5:
        return {
            "workload": "benchmark configuration 5: HiDream MoE FFN layer, bf16, 8 x 16384 tokens in total, skewed router "
                        f"(gate.weight[0, 0] = {SKEW_BIAS} on a constant input feature: expert 0 takes about 60 % of the "
                        "top-1 picks), fp32 gate",
            "tokens_per_gpu": tokens_per_gpu, "global_tokens": tokens_per_gpu * n_gpus, "dim": DIM, "experts": N_EXPERTS,
            "top_k": TOP_K, "hidden": HIDDEN, "hidden_shared": HIDDEN_SHARED,
            "parallelism": "single GPU" if n_gpus == 1 else f"expert-parallel x{n_gpus} ({ep_transport()}), shared "
                                                            "expert data-parallel",
            "l2": "no flush: one step touches gigabytes of activations",
        }
    what = ("benchmark configuration 2: HiDream MoE FFN layer, bf16 weights and activations, 2 x 4096 tokens per GPU, fp32 gate"
            if dtype == "bf16" else
            "benchmark configuration 3: HiDream MoE FFN layer, expert and shared weights e4m3 with per-tensor fp32 scales, bf16 "
            "activations quantised to e4m3 for the matmuls, 2 x 4096 tokens per GPU, fp32 gate")
    return {
        "workload": what,
        "tokens_per_gpu": TOKENS_PER_GPU, "global_tokens": TOKENS_PER_GPU * n_gpus, "dim": DIM, "experts": N_EXPERTS,
        "top_k": TOP_K, "hidden": HIDDEN, "hidden_shared": HIDDEN_SHARED,
        "parallelism": "single GPU" if n_gpus == 1 else f"expert-parallel x{n_gpus} ({ep_transport()}), shared expert "
                                                        "data-parallel",
        "l2": "no flush: one step touches 0.48 GB of weights and 0.6 GB of activations, far more than the 126 MB L2",
    }


# ------------------------------------------------------------------------------------------ GPU arm
SKEW_BIAS = 1.16          # config 5: expert 0 wins about 60 % of the top-1 picks
CONFIG5_TOKENS = 131072   # 8 images of 2048 x 2048 (16384 tokens each)


def make_synthetic(dev, seed_w: int = 0, seed_x: int = 1, fp8: bool = False, n_tokens: int = TOKENS_PER_GPU,
                   skew: bool = False):
    """Seeded synthetic weights and input, generated on the host exactly like the oracle's recipe (same
    generator, same draw order) without importing it, then moved to the device."""
    g = torch.Generator().manual_seed(seed_w)
    state = {}

    def draw(name, shape):
        state[name] = (torch.randn(shape, generator=g, dtype=torch.float32) * 0.02).bfloat16().to(dev)

    for prefix, h in [("shared_experts", HIDDEN_SHARED)] + [(f"experts.{e}", HIDDEN) for e in range(N_EXPERTS)]:
        draw(prefix + ".w1.weight", (h, DIM))
        draw(prefix + ".w2.weight", (DIM, h))
        draw(prefix + ".w3.weight", (h, DIM))
    draw("gate.weight", (N_EXPERTS, DIM))
    if fp8:
        # per-tensor scaled e4m3 (benchmark configuration 3): s = max|w| / 448, wq = (w / s).to(e4m3); the gate stays bf16
        for k in [k for k in state if k != "gate.weight"]:
            w = state[k].float()
            sc = (w.abs().max() / 448.0).reshape(())
            state[k] = (w / sc).to(torch.float8_e4m3fn)
            state[k[: -len(".weight")] + ".scale_weight"] = sc.to(torch.float32)
    gx = torch.Generator().manual_seed(seed_x)
    x = torch.randn((n_tokens, DIM), generator=gx, dtype=torch.float32).bfloat16()
    if skew:
        # the gate has no bias term: a constant input feature and one weight column stand in for it
        x[:, 0] = 1
        state["gate.weight"][:, 0] = 0
        state["gate.weight"][0, 0] = SKEW_BIAS
    return state, x


def timed_region_peak(peaks, timed_ms: float, fp8: bool):
    """Tensor-peak denominator that matches how long the timed region ran: the measured burst figure for a region
    under a second (the GPU has not reached its power-capped clock yet), the sustained one beyond."""
    burst = timed_ms < 1000.0
    peak = (peaks["tflops_burst"] if burst else peaks["tflops_sustained"]) * (2.0 if fp8 else 1.0)
    label = (f"{peaks['source']}: cuBLAS bf16 {'burst' if burst else 'sustained'} figure "
             f"({peaks['tflops_burst']} burst / {peaks['tflops_sustained']} sustained), chosen because the timed region "
             f"lasted {timed_ms:.0f} ms" + ("; x 2 for fp8 (no measured fp8 figure exists)" if fp8 else ""))
    return peak, label


class Arm:
    """One workload on this rank: the module, its input, and the callable that runs one layer call."""

    def __init__(self, dev, world, rank, fp8: bool, config5: bool):
        import torch.distributed as dist

        from comfyui_b200 import ops
        from comfyui_b200.ldm.hidream.model import MOEFeedForwardSwiGLU

        self.dev, self.world, self.rank, self.fp8, self.config5 = dev, world, rank, fp8, config5
        self.n = n = CONFIG5_TOKENS // world if config5 else TOKENS_PER_GPU
        state, self.x_host = make_synthetic(dev, seed_w=0, seed_x=1 + rank, fp8=fp8, n_tokens=n, skew=config5)
        operations = ops.disable_weight_init if not fp8 else ops.scaled_fp8_ops(
            fp8_matrix_mult=True, scale_input=False, override_dtype=torch.float8_e4m3fn)
        self.module = MOEFeedForwardSwiGLU(DIM, HIDDEN_DIM, N_EXPERTS, TOP_K, dtype=torch.bfloat16, device=dev,
                                           operations=operations).eval()
        self.module.load_state_dict(state, strict=True)
        self.x = self.x_host.to(dev).view(2, n // 2, DIM)
        self.runner = None
        if world > 1:
            from comfyui_b200.expert_parallel import ExpertParallelMoE, PeerExpertParallelMoE

            # default: rows move over peer memory inside the kernels; COMFY_B200_EP_TRANSPORT=nccl selects the
            # host-planned NCCL exchange (bf16 only)
            transport = os.environ.get("COMFY_B200_EP_TRANSPORT", "peer")
            if transport != "nccl":
                try:        # the same answer on every rank: a missing module, not a failed rendezvous
                    import torch.distributed._symmetric_memory as symm_mem

                    symm_mem.empty, symm_mem.rendezvous
                except (ImportError, AttributeError):
                    transport = "nccl"
                    os.environ["COMFY_B200_EP_TRANSPORT"] = "nccl"     # workload_config() names the transport used
            if transport == "nccl":
                self.runner = ExpertParallelMoE(self.module, dist.group.WORLD)
            else:
                self.runner = PeerExpertParallelMoE(self.module, dist.group.WORLD, max_tokens=n)
            self.step = lambda inp: self.runner(inp)                      # noqa: E731
            self.launches_per_step = self.runner.launches_per_step
        else:
            assert ops._layer_pack(self.module, self.x) is not None, "bench: layer not eligible for the sm_100a kernels"
            self.step = lambda inp: self.module(inp)                      # noqa: E731
            self.launches_per_step = 5   # gate, plan + permute, GEMM pass 1, GEMM pass 2, combine

    def check(self):
        if self.runner is not None and hasattr(self.runner, "check"):
            self.runner.check()          # no flag wait ran out, every routed row fitted its receive buffer

    def routing(self):
        """Realised routing of the last call: slots per expert over all GPUs, rows each GPU's routed experts process."""
        from comfyui_b200 import ops, torch_ops

        if self.world > 1:
            r = self.runner
            last = r.last_counts_host if hasattr(r, "last_counts_host") else r.last_counts
            per_expert = [sum(c[e] for c in last) for e in range(N_EXPERTS)]
            owners = [r.place.owners(e) for e in range(N_EXPERTS)]
            rows = [sum(per_expert[e] for e in range(N_EXPERTS) if q in owners[e]) for q in range(self.world)]
        else:
            layer = ops._layer_pack(self.module, self.x)
            per_expert = torch_ops._workspace(layer, self.n).expert_counts.tolist()
            rows = [sum(per_expert)]
        return {"slots_per_expert": per_expert, "share_of_expert_0": per_expert[0] / max(sum(per_expert), 1),
                "routed_rows_per_gpu": rows}


def time_steps(arm, steps: int, barrier, local_rank: int):
    """Milliseconds for exactly `steps` layer calls (inputs resident in HBM) between two CUDA events on the launching
    stream, with the SM clock sampled meanwhile."""
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        ev0.record()
        for _ in range(steps):
            arm.step(arm.x)
        ev1.record()
        barrier()
    return ev0.elapsed_time(ev1), clocks.summary()


def clocks_of_all_ranks(clocks: dict, dev, world: int) -> dict:
    """Adds every rank's median SM clock under load to rank 0's clock record: the step time of a multi-GPU run is set by
    the slowest GPU, and GPUs under the same power cap do not all settle at the same clock."""
    import torch.distributed as dist

    if world > 1:
        mine = torch.tensor([float(clocks.get("sm_mhz") or 0.0)], dtype=torch.float64, device=dev)
        every = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        clocks = dict(clocks, sm_mhz_per_rank=[float(t.item()) for t in every])
    return clocks


def max_over_ranks(values, dev, world):
    import torch.distributed as dist

    t = torch.tensor(values, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def measure(arm, args, barrier, local_rank, peaks, *, steps: int, warmup: int, e2e: bool, sustained: bool,
            stages: bool, gpu_bar: bool):
    """All figures of one workload as a dict (identical on every rank; only rank 0 prints it)."""
    from comfyui_b200 import moe_ops, ops

    dev, world, n, fp8 = arm.dev, arm.world, arm.n, arm.fp8
    res = {}
    with torch.inference_mode():
        for _ in range(max(warmup, 3)):
            arm.step(arm.x)
        ms_total, clocks = time_steps(arm, steps, barrier, local_rank)
        clocks = clocks_of_all_ranks(clocks, dev, world)
        arm.check()
        st = None
        if world == 1 and stages:
            # per-stage timing of the same work through the stage-level C ABI, straight after the headline loop so
            # that both see the GPU in the same state (the sustained loops further down heat it up)
            st = time_stages(arm.module, arm.x.view(n, DIM), steps, moe_ops, ops)
        ms_e2e = 0.0
        if e2e:
            # end to end: every step copies its input from pinned host memory and its output back to pinned host
            # memory.  The copies run on their own streams with two buffers each, the way a serving loop would feed
            # the layer: step i's upload and step i-1's download overlap step i's compute; nothing is skipped.
            x_pinned = arm.x_host.pin_memory()
            out_pinned = torch.empty_like(arm.x_host).pin_memory()
            ms_e2e = time_end_to_end(arm.step, x_pinned, out_pinned, n, dev, steps, barrier)
        ms_total, ms_e2e = max_over_ranks([ms_total, ms_e2e], dev, world)
        ms_step = ms_total / steps
        res.update({
            "value": n * world / (ms_step * 1e-3), "unit": "tokens/s", "steps": steps, "ms_per_step": ms_step,
            "dtype": "fp8" if fp8 else "bf16", "clocks": clocks,
            "layer_tflops": FLOPS_PER_TOKEN * n * world / (ms_step * 1e-3) / 1e12,
            "layer_frac_of_nominal": FLOPS_PER_TOKEN * n / (ms_step * 1e-3) / 1e12 / (4500.0 if fp8 else 2250.0),
        })
        if e2e:
            e2e_s = ms_e2e / steps * 1e-3
            res["e2e"] = {"value": n * world / e2e_s, "unit": "tokens/s",
                          "h2d_bytes_per_step": arm.x_host.numel() * 2, "d2h_bytes_per_step": arm.x_host.numel() * 2,
                          "ms_per_step": ms_e2e / steps,
                          # both copies of a step overlap the compute of its neighbours, so a step cannot be shorter than
                          # the slower of one copy direction and the compute: the achieved rate names the limiter
                          "host_link_gbs_per_direction_per_gpu": arm.x_host.numel() * 2 / e2e_s / 1e9}
        if arm.config5:
            res["routing"] = arm.routing()

        if sustained:
            # the same loop for at least 1.2 s: the GPU settles at its power-capped clock
            k_long = max(steps, int(1200.0 / ms_step) + 1)
            ms_long, clocks_long = time_steps(arm, k_long, barrier, local_rank)
            clocks_long = clocks_of_all_ranks(clocks_long, dev, world)
            (ms_long,) = max_over_ranks([ms_long], dev, world)
            ms_l = ms_long / k_long
            res["sustained"] = {
                "steps": k_long, "timed_region_ms": ms_long, "ms_per_step": ms_l, "value": n * world / (ms_l * 1e-3),
                "unit": "tokens/s", "layer_tflops_per_gpu": FLOPS_PER_TOKEN * n / (ms_l * 1e-3) / 1e12,
                "layer_frac_of_nominal": FLOPS_PER_TOKEN * n / (ms_l * 1e-3) / 1e12 / (4500.0 if fp8 else 2250.0),
                "clocks": clocks_long,
            }

        if world > 1:
            # no per-kernel timing in the multi-GPU loop: the grouped GEMM's FLOPs per GPU over the WHOLE step (routing,
            # exchange, flag waits and combine included), i.e. a lower bound on what the kernel itself reaches
            peak, label = timed_region_peak(peaks, ms_total, fp8)
            achieved = FLOPS_PER_TOKEN_GEMM * n / (ms_step * 1e-3) / 1e12
            res["roofline"] = {
                "bound": "tensor", "kernel": "grouped_gemm_kernel (per GPU; time = the whole expert-parallel step)",
                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": label,
                "frac_of_nominal": achieved / (4500.0 if fp8 else 2250.0), "traffic": None,
            }
        elif st is not None:
            gemm_ms = st["grouped_gemm_ms"]
            achieved = FLOPS_PER_TOKEN_GEMM * n / (gemm_ms * 1e-3) / 1e12
            peak, label = timed_region_peak(peaks, st["timed_region_ms"], fp8)
            roof = {
                "bound": "tensor", "kernel": "grouped_gemm_kernel (pass 1 SwiGLU + pass 2, one C-ABI call)",
                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": label,
                "frac_of_burst": achieved / (peaks["tflops_burst"] * (2.0 if fp8 else 1.0)),
                "frac_of_sustained": achieved / (peaks["tflops_sustained"] * (2.0 if fp8 else 1.0)),
                "frac_of_nominal": achieved / (4500.0 if fp8 else 2250.0), "traffic": None,
            }
            if not arm.config5:
                # DRAM bytes of the two launches are not measured in this run: they come from the ncu capture of this
                # same workload that the named file summarises
                roof["traffic"] = TRAFFIC_FROM_CAPTURE["fp8" if fp8 else "bf16"]["traffic"]
                roof["algorithmic_bytes"] = TRAFFIC_FROM_CAPTURE["fp8" if fp8 else "bf16"]["algorithmic_bytes"]
                roof["traffic_source"] = TRAFFIC_FROM_CAPTURE["fp8" if fp8 else "bf16"]["source"]
            res["roofline"] = roof
            res["stages"] = st
            hbm = peaks["hbm_gbs"]
            res["hbm_kernels"] = {
                k: {"achieved_gbs": st[k + "_bytes"] / (st[k + "_ms"] * 1e-3) / 1e9,
                    "frac": st[k + "_bytes"] / (st[k + "_ms"] * 1e-3) / 1e9 / hbm, "peak_gbs": hbm}
                for k in ("gate", "permute", "combine")
            }
            if sustained:
                k_long = max(steps, int(1200.0 / max(sum(st[k + "_ms"] for k in STAGE_NAMES), 1e-3)) + 1)
                with ClockSampler(local_rank) as clocks_st:
                    st_long = time_stages(arm.module, arm.x.view(n, DIM), k_long, moe_ops, ops)
                a_long = FLOPS_PER_TOKEN_GEMM * n / (st_long["grouped_gemm_ms"] * 1e-3) / 1e12
                mult = 2.0 if fp8 else 1.0
                res["sustained"]["grouped_gemm"] = {
                    "steps": k_long, "timed_region_ms": st_long["timed_region_ms"], "ms": st_long["grouped_gemm_ms"],
                    "tflops": a_long, "frac_of_sustained_peak": a_long / (peaks["tflops_sustained"] * mult),
                    "frac_of_nominal": a_long / (4500.0 if fp8 else 2250.0),
                    "peak_source": f"{peaks['source']}: cuBLAS bf16 sustained {peaks['tflops_sustained']} TFLOP/s"
                                   + (" x 2 for fp8" if fp8 else ""),
                    "clocks": clocks_st.summary(),
                }
            if gpu_bar:
                res["gpu_bar"] = time_stock_composition(arm.module, arm.x, ops)
    return res


# dram__bytes_read.sum + dram__bytes_write.sum of the two grouped-GEMM launches of one layer call at 8192 tokens, from
# ncu captures of exactly this workload (not measured by bench.py itself)
TRAFFIC_FROM_CAPTURE = {
    "bf16": {"traffic": 1.576e9, "algorithmic_bytes": 1.30e9, "source": "profiles/grouped_gemm_bf16_8192tokens.md"},
    "fp8": {"traffic": 0.658e9, "algorithmic_bytes": 0.71e9, "source": "profiles/grouped_gemm_fp8_8192tokens.md"},
}
STAGE_NAMES = ["gate", "plan", "permute", "grouped_gemm", "combine"]


def expert_parallel_parity(arm):
    """Every rank runs its own tokens through the single-GPU layer with the full weights it holds anyway and compares
    the expert-parallel result with it.  Without a hidden split: bit for bit.  With one (8 GPUs) every routed result is
    the bf16 sum of two bf16 partial results instead of one rounding of one fp32 sum, so where the two partial sums
    cancel a few elements in a million leave the element-wise bf16 tolerance; the criterion there is the relative RMS
    difference (measured 2.6e-3 at these shapes) and the share of elements outside rtol = atol = 2e-2 (measured 1.5e-6),
    both reported."""
    import torch.distributed as dist

    from comfyui_b200 import ops

    with torch.inference_mode():
        ep = arm.runner(arm.x).clone()
        arm.check()
        assert ops._layer_pack(arm.module, arm.x) is not None
        single = arm.module(arm.x)
        torch.cuda.synchronize()
    split = getattr(arm.runner.place, "hidden_splits", 1) > 1
    exact = bool(torch.equal(ep, single))
    a, b = ep.float(), single.float()
    err = (a - b).abs()
    diff = float(err.max())
    rel_rms = float((a - b).norm() / b.norm())
    outside = float((err > 2e-2 + 2e-2 * b.abs()).float().mean())
    ok = (rel_rms < 5e-3 and outside < 1e-4) if split else exact
    t = torch.tensor([0.0 if ok else 1.0, 0.0 if exact else 1.0, diff, rel_rms, outside], dtype=torch.float64,
                     device=arm.dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    bad, inexact, diff, rel_rms, outside = t.tolist()
    return {"ok": bad == 0.0, "bit_identical": inexact == 0.0, "max_abs_diff": diff, "rel_rms": rel_rms,
            "share_outside_rtol_atol_2e-2": outside,
            "criterion": ("rel-RMS < 5e-3 and less than 1e-4 of the elements outside rtol = atol = 2e-2 (hidden dimension "
                          "split over two GPUs: the sum of two bf16 partial results)") if split else "torch.equal",
            "against": "the single-GPU layer on the same rank, same tokens, full weights", "tokens_per_gpu": arm.n}


def run_gpu_arm(args) -> None:
    import torch.distributed as dist

    from comfyui_b200 import _native

    _native.load()   # no fallback: fail here if the extension is not built
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torchrun --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    peaks = measured_peaks()
    fp8 = args.dtype == "fp8"
    config5 = args.workload == "config5"
    extras = args.workload == "hidream" and not args.headline_only
    warmup = max(args.warmup, 3)

    arm = Arm(dev, world, rank, fp8, config5)
    res = measure(arm, args, barrier, local_rank, peaks, steps=args.steps, warmup=warmup, e2e=True,
                  sustained=extras, stages=True, gpu_bar=not args.no_cpu_baseline)
    line = {
        "metric": METRIC, "value": res.pop("value"), "unit": res.pop("unit"), "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": res.pop("ms_per_step"), "higher_is_better": True,
        "scaling": "strong" if config5 else "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
        "config": workload_config(world, args.dtype, arm.n, config5),
        "gpu_launches": arm.launches_per_step * args.steps,
    }
    res.pop("steps"), res.pop("dtype")
    line.update(res)

    if extras:
        # Sub-objects of the same line, measured after the headline and outside its timed region: expert-parallel
        # parity, the other dtype (benchmark configuration 3 when the headline is configuration 2), configuration 5.
        if world > 1:
            line["ep_parity"] = {args.dtype: expert_parallel_parity(arm)}
        del arm
        torch.cuda.empty_cache()
        other = "bf16" if fp8 else "fp8"
        arm2 = Arm(dev, world, rank, not fp8, False)
        sub = measure(arm2, args, barrier, local_rank, peaks, steps=args.steps, warmup=warmup, e2e=True,
                      sustained=True, stages=True, gpu_bar=False)
        sub["config"] = workload_config(world, other, arm2.n, False)["workload"]
        sub["gpu_launches"] = arm2.launches_per_step * args.steps
        line[other] = sub
        if world > 1:
            line["ep_parity"][other] = expert_parallel_parity(arm2)
        del arm2
        torch.cuda.empty_cache()
        arm5 = Arm(dev, world, rank, False, True)
        k5 = max(3, min(args.steps, 10 if world == 1 else 20))
        sub = measure(arm5, args, barrier, local_rank, peaks, steps=k5, warmup=3, e2e=False, sustained=False,
                      stages=True, gpu_bar=False)
        sub["config"] = workload_config(world, "bf16", arm5.n, True)["workload"]
        sub["scaling"] = "strong"
        sub["tokens_per_gpu"] = arm5.n
        sub["gpu_launches"] = arm5.launches_per_step * k5
        line["config5"] = sub
        if world > 1:
            line["ep_parity"]["config5"] = expert_parallel_parity(arm5)
        arm = arm5

    if extras and world == 1:
        del arm
        torch.cuda.empty_cache()
        arm = None
        sub = measure_config4(dev, "bf16", steps=5, local_rank=local_rank)
        sub.pop("metric"), sub.pop("higher_is_better"), sub.pop("data")
        line["config4"] = sub

    if world == 1 and not args.no_cpu_baseline and rank == 0:
        line["cpu_baseline"] = cpu_baseline_object(args.dtype, reps=10)

    if (args.timeline or args.timeline_dir) and arm is not None:
        with torch.inference_mode():
            if args.timeline_dir:           # every rank writes its own file
                os.makedirs(args.timeline_dir, exist_ok=True)
                tag = f"{arm.world}gpus_{'fp8' if arm.fp8 else 'bf16'}{'_config5' if arm.config5 else ''}"
                path = os.path.join(args.timeline_dir, f"timeline_{tag}_rank{rank}.txt")
                print_timeline(arm.step, arm.x, path, rank)
                counts = getattr(arm.runner, "last_counts_host", None) if arm.world > 1 else None
                if counts is not None:      # how much work each expert (and so each rank) had in that step
                    per_expert = [sum(c[e] for c in counts) for e in range(len(counts[0]))]
                    with open(path, "a") as f:
                        print(f"rank {rank}: routed rows per expert over all ranks' tokens: {per_expert}", file=f)
            elif rank == 0:
                print_timeline(arm.step, arm.x)
            else:
                for _ in range(3):          # the other ranks take the same three steps
                    arm.step(arm.x)
                torch.cuda.synchronize()

    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def time_end_to_end(step, x_pinned, out_pinned, n, dev, steps, barrier):
    """Milliseconds for `steps` layer calls including, for every call, the host->device copy of its input and the
    device->host copy of its output (pinned memory both ways)."""
    compute = torch.cuda.current_stream()
    up, down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    x_dev = [torch.empty((2, n // 2, DIM), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    outs_pinned = [out_pinned, torch.empty_like(out_pinned).pin_memory()]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]

    def run(count):
        for i in range(count):
            b = i % 2
            with torch.cuda.stream(up):
                if i >= 2:
                    up.wait_event(in_free[b])                 # compute has finished reading this input buffer
                x_dev[b].view(n, DIM).copy_(x_pinned, non_blocking=True)
                in_ready[b].record(up)
            compute.wait_event(in_ready[b])
            y = step(x_dev[b])
            in_free[b].record(compute)
            produced = torch.cuda.Event()
            produced.record(compute)
            with torch.cuda.stream(down):
                down.wait_event(produced)
                if i >= 2:
                    down.wait_event(out_done[b])
                outs_pinned[b].copy_(y.view(n, DIM), non_blocking=True)
                out_done[b].record(down)
            y.record_stream(down)
        compute.wait_stream(up)
        compute.wait_stream(down)

    run(4)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run(steps)
    e1.record()
    barrier()
    return e0.elapsed_time(e1)


def time_stages(module, x2, steps, moe_ops, ops):
    """Average duration of every kernel of the layer: the launches of comfy_moe_forward (which fuses plan and permute into one), issued through
    the stage-level C-ABI entry points on a pre-allocated workspace with a CUDA event between stages.  All steps are
    queued before the one synchronisation at the end, so the events are not separated by host latency."""
    import ctypes

    from comfyui_b200 import _native as N

    lib = N.load()
    layer = ops._layer_pack(module, x2)
    n, d = x2.shape
    e = layer.n_experts
    ws = moe_ops.Workspace.for_layer(layer, n)
    out = torch.empty_like(x2)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    P = lambda t: ctypes.c_void_p(t.data_ptr())      # noqa: E731
    experts = (N.FfnWeights * e)()
    for i, pack in enumerate(layer.experts):
        pack.fill(experts[i])
    shared = layer.shared.struct()
    names = STAGE_NAMES
    act = N.FP8_E4M3 if layer.fp8 else N.BF16

    def one_step(marks):
        rc = 0
        marks[0].record()
        rc |= lib.comfy_moe_gate_topk(P(x2), P(layer.gate), N.BF16 if layer.gate.dtype == torch.bfloat16 else N.FP32, n, d,
                                      e, 2, P(ws.topk_idx), P(ws.topk_weight), P(ws.block_counts), None, None, 1e-6,
                                      stream)
        marks[1].record()
        rc |= lib.comfy_moe_route_plan(P(ws.block_counts), n, e, P(ws.block_offsets), P(ws.expert_counts),
                                       P(ws.expert_offsets), stream)
        marks[2].record()
        rc |= lib.comfy_moe_permute(P(x2), P(ws.topk_idx), P(ws.block_offsets), P(ws.expert_offsets), n, d, e, act,
                                    None, P(ws.x_perm), P(ws.x_q) if layer.fp8 else None, None, P(ws.row_map), None,
                                    stream)
        marks[3].record()
        rc |= lib.comfy_moe_grouped_swiglu(act, e, experts, ctypes.byref(shared), P(ws.expert_offsets),
                                           P(ws.expert_counts), ws.rows_cap, n, d, P(ws.x_perm), P(ws.h_perm),
                                           P(ws.y_perm), P(ws.x_q) if layer.fp8 else P(x2), P(ws.h_shared),
                                           P(ws.y_shared), P(ws.status), stream)
        marks[4].record()
        rc |= lib.comfy_moe_combine(P(ws.y_perm), P(ws.row_map), P(ws.topk_weight), P(ws.y_shared), n, d, P(out), stream)
        marks[5].record()
        if rc:
            raise RuntimeError("stage-level C-ABI call failed")

    def ev():
        return torch.cuda.Event(enable_timing=True)

    for _ in range(3):
        one_step([ev() for _ in range(6)])
    torch.cuda.synchronize()
    all_marks = [[ev() for _ in range(6)] for _ in range(steps)]
    for marks in all_marks:
        one_step(marks)
    torch.cuda.synchronize()
    res = {"steps": steps, "timed_region_ms": all_marks[0][0].elapsed_time(all_marks[-1][5])}
    for i, k in enumerate(names):
        res[k + "_ms"] = sum(m[i].elapsed_time(m[i + 1]) for m in all_marks) / steps
    res["gate_bytes"] = n * d * 2 + e * d * 2 + n * 2 * 8
    res["permute_bytes"] = n * d * 2 + (n * 2 * d * 2 if not layer.fp8 else n * 3 * d)
    res["combine_bytes"] = n * 2 * d * 2 + n * d * 2 + n * d * 2
    return res


def print_timeline(step, x, path=None, rank: int = 0) -> None:
    """Kernel timeline of one step on this rank (torch.profiler / CUPTI): start offset, duration, stream, kernel name.
    Three steps are profiled and the middle one is shown, followed by the wall time of each of the three steps on this
    rank.  Goes to `path` when given (one file per rank), else to stderr."""
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            step(x)
        torch.cuda.synchronize()
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    evs.sort(key=lambda e: e.time_range.start)
    out = open(path, "w") if path else sys.stderr
    try:
        gates = [i for i, e in enumerate(evs) if "gate_topk" in e.name]
        if len(gates) < 3:
            print("timeline: no gate kernels found", file=out)
            return
        lo, hi = gates[1], gates[2]
        # the side stream's first kernels of the step may start before the gate: include what began up to 50 us earlier
        while lo > 0 and evs[lo - 1].time_range.start > evs[gates[1]].time_range.start - 50:
            lo -= 1
        t0 = evs[gates[1]].time_range.start
        print(f"rank {rank}: timeline of one step (offset us from the gate's start, duration us, stream, kernel)", file=out)
        for e in evs[lo:hi]:
            if e.time_range.start < evs[gates[2]].time_range.start - 50 or "gate_topk" in e.name:
                print(f"{e.time_range.start - t0:9.1f} {e.time_range.elapsed_us():8.1f}  s{getattr(e, 'device_resource_id', '?')}  "
                      f"{e.name[:110]}", file=out)
        ends = [evs[gates[i + 1]].time_range.start - evs[gates[i]].time_range.start for i in range(2)]
        print(f"rank {rank}: gate-to-gate step times under the profiler: {ends[0]:.1f} us, {ends[1]:.1f} us", file=out)
    finally:
        if path:
            out.close()


def time_stock_composition(module, x, ops, steps: int = 10):
    """The same module with the sm_100a kernels switched off: forward() then runs the composition the reference
    ships (masked branch, one library GEMM per Linear, boolean-mask gathers, host syncs), and moe_infer the sorted
    variant.  This is what the layer costs on this GPU today; it is reported next to the headline, never as it."""
    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    n = x.shape[0] * x.shape[1]
    x2 = x.view(n, x.shape[-1])
    saved = ops.ENABLE_SM100_KERNELS
    ops.ENABLE_SM100_KERNELS = False
    try:
        ms_forward = timed(lambda: module(x))

        def infer():
            idx, w, _ = module.gate(x)
            return module.moe_infer(x2, idx.view(-1), w.view(-1, 1)) + module.shared_experts(x2)

        ms_infer = timed(infer)
    finally:
        ops.ENABLE_SM100_KERNELS = saved
    return {"what": "same module and weights, sm_100a kernels off: stock PyTorch composition on this GPU",
            "forward_ms": ms_forward, "forward_tokens_per_s": n / (ms_forward * 1e-3),
            "moe_infer_ms": ms_infer, "moe_infer_tokens_per_s": n / (ms_infer * 1e-3), "steps": steps}


def run_hunyuan3d(args) -> None:
    """Side workload (not the headline): the Hunyuan3D-2.1 MoE block, hidden size 2048, 8 experts top-2 + shared,
    GELU feed-forwards of inner width 8192 with biases, 2 x 4096 latent tokens, bf16, one GPU."""
    from comfyui_b200 import _native, ops
    from comfyui_b200.ldm.hunyuan3dv2_1.hunyuandit import MoEBlock

    _native.load()
    dev = torch.device("cuda", 0)
    dim, inner, e, n = 2048, 8192, 8, 8192
    mod = MoEBlock(dim, num_experts=e, moe_top_k=2, ff_inner_dim=inner, operations=ops.disable_weight_init, device=dev,
                   dtype=torch.bfloat16).eval()
    g = torch.Generator().manual_seed(0)
    with torch.no_grad():
        for name, p in mod.named_parameters():      # weights N(0, 0.02^2), biases five times wider, seeded
            std = 0.1 if name.endswith("bias") else 0.02
            p.copy_((torch.randn(p.shape, generator=g, dtype=torch.float32) * std).to(torch.bfloat16))
    gx = torch.Generator().manual_seed(1)
    x = torch.randn((n, dim), generator=gx, dtype=torch.float32).bfloat16().to(dev).view(2, n // 2, dim)
    flops = n * (2 * 2 * 2 * dim * inner + 2 * 2 * dim * inner + 2 * dim * e)

    def timed(steps, warmup):
        for _ in range(warmup):
            mod(x)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            mod(x)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    with torch.inference_mode():
        assert ops.hunyuan3d_moe_forward(mod, x) is not None, "bench: layer not eligible for the sm_100a kernels"
        with ClockSampler(0) as clocks:
            ms = timed(args.steps, max(args.warmup, 3))
        ops.ENABLE_SM100_KERNELS = False
        try:
            ms_stock = timed(10, 3)
        finally:
            ops.ENABLE_SM100_KERNELS = True
    print(json.dumps({
        "metric": "MoE tokens/s (Hunyuan3D-2.1 MoEBlock, hidden 2048, 8 experts top-2 + shared, inner 8192)",
        "value": n / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "Hunyuan3D-2.1 MoE block, 2 x 4096 tokens, bf16, fp32 gate", "tokens": n, "dim": dim,
                   "experts": e, "top_k": 2, "inner": inner},
        "gpu_launches": 5 * args.steps, "clocks": clocks.summary(),
        "layer_tflops": flops / (ms * 1e-3) / 1e12, "layer_frac_of_nominal": flops / (ms * 1e-3) / 1e12 / 2250.0,
        "gpu_bar": {"what": "same module and weights, sm_100a kernels off: stock PyTorch composition on this GPU",
                    "forward_ms": ms_stock, "forward_tokens_per_s": n / (ms_stock * 1e-3)},
    }))


HIDREAM_I1 = dict(patch_size=2, in_channels=16, out_channels=16, num_layers=16, num_single_layers=32,
                  attention_head_dim=128, num_attention_heads=20, caption_channels=[4096, 4096], text_emb_dim=2048,
                  num_routed_experts=4, num_activated_experts=2, axes_dims_rope=[64, 32, 32], max_resolution=[128, 128],
                  llama_layers=list(range(32)) + [31] * 16)


def measure_config4(dev, dtype: str, steps: int, n_double: int = 16, n_single: int = 32, local_rank: int = 0):
    """Benchmark configuration 4: one denoising step of a HiDream-I1-shaped transformer (16 double-stream + 32
    single-stream blocks, 20 heads x 128, MoE feed-forward on the image tokens), random-init weights, latent
    [2, 16, 128, 128], T5 states [2, 128, 4096], per-layer Llama states [2, 32, 128, 4096], pooled [2, 2048]; the whole
    model call (embedders, text projections, blocks, final layer).  Timed with the kernels and, on the same modules
    and weights, as PyTorch composes it on this GPU."""
    from comfyui_b200 import ops
    from comfyui_b200.ldm.hidream.model import HiDreamImageTransformer2DModel

    fp8 = dtype == "fp8"
    operations = ops.disable_weight_init if not fp8 else ops.scaled_fp8_ops(
        fp8_matrix_mult=True, scale_input=False, override_dtype=torch.float8_e4m3fn)
    cfg = dict(HIDREAM_I1, num_layers=n_double, num_single_layers=n_single)
    cfg["llama_layers"] = HIDREAM_I1["llama_layers"][:n_double + n_single]
    torch.manual_seed(0)
    model = HiDreamImageTransformer2DModel(**cfg, dtype=torch.bfloat16, device=dev, operations=operations).eval()
    with torch.no_grad():
        for mod in model.modules():
            w = getattr(mod, "weight", None)
            if isinstance(mod, torch.nn.Linear) and w is not None and w.dtype == torch.float8_e4m3fn:
                # scaled fp8 checkpoint convention: s = max|w| / 448, weight = (w / s) in e4m3, scale_weight = s
                full = torch.randn(w.shape, device=dev) * 0.02
                sc = full.abs().max() / 448.0
                w.copy_((full / sc).to(torch.float8_e4m3fn))
                mod.scale_weight.fill_(float(sc))
                if mod.bias is not None:
                    mod.bias.copy_((torch.randn(mod.bias.shape, device=dev) * 0.02).to(mod.bias.dtype))
        for name, p in model.named_parameters():
            if p.dtype == torch.float8_e4m3fn or name.endswith("scale_weight"):
                continue
            if "rms_norm" in name:
                p.fill_(1.0)
            else:
                p.normal_(0.0, 0.02)
    n_params = sum(p.numel() for p in model.parameters())
    b = 2
    x = torch.randn((b, 16, 128, 128), device=dev).bfloat16()
    t = torch.tensor([500.0, 500.0], device=dev)
    y = torch.randn((b, 2048), device=dev).bfloat16()
    context = torch.randn((b, 128, 4096), device=dev).bfloat16()
    llama = torch.randn((b, 32, 128, 4096), device=dev).bfloat16()

    def timed(count, warmup):
        for _ in range(warmup):
            model(x, t, y, context, llama)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(count):
            out = model(x, t, y, context, llama)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / count, out

    with torch.inference_mode():
        with ClockSampler(local_rank) as clocks:
            ms, out = timed(steps, 2)
        ops.check_device_status()
        finite = bool(torch.isfinite(out.float()).all())
        from comfyui_b200.ldm.hidream import model as hidream

        ops.ENABLE_SM100_KERNELS = False
        stock_gate = hidream.MoEGate.forward
        try:
            ms_stock, out_stock = timed(max(steps // 2, 2), 1)
            rel_as_shipped = float((out.float() - out_stock.float()).norm() / out_stock.float().norm())

            # one more stock step with the routing convention of the kernels (MoEGate on the fp32 copy of its input,
            # weights cast back): what is left is arithmetic, not a different choice of experts
            def gate_on_fp32_copy(self, hidden_states):
                idx, w, aux = stock_gate(self, hidden_states.float())
                return idx, w.to(hidden_states.dtype), aux

            hidream.MoEGate.forward = gate_on_fp32_copy
            out_same_routing = model(x, t, y, context, llama)
            rel = float((out.float() - out_same_routing.float()).norm() / out_same_routing.float().norm())
            # the yardstick for the two figures above: how far two runs of the STOCK composition drift apart on this
            # workload when every element of the input latent moves to a neighbouring bf16 value (one unit in the last
            # place, up or down at random): 48 blocks of random weights with top-2 routing amplify rounding-level
            # differences, whoever makes them
            gen = torch.Generator(device=dev).manual_seed(7)
            step = torch.randint(0, 2, x.shape, generator=gen, device=dev, dtype=torch.int16) * 2 - 1
            x_moved = (x.view(torch.int16) + step).view(torch.bfloat16)
            out_other = model(x_moved, t, y, context, llama)
            rel_noise = float((out_other.float() - out_same_routing.float()).norm() / out_same_routing.float().norm())
        finally:
            hidream.MoEGate.forward = stock_gate
            ops.ENABLE_SM100_KERNELS = True
    del model
    torch.cuda.empty_cache()
    return {
        "metric": "one denoising step, ms (HiDream-I1-shaped transformer, whole model call)", "value": ms, "unit": "ms",
        "steps": steps, "ms_per_step": ms, "higher_is_better": False, "dtype": dtype, "data": "synthetic",
        "config": {"workload": f"benchmark configuration 4: {n_double} double-stream + {n_single} single-stream blocks, "
                               "latent [2, 16, 128, 128] (2 x 4096 image tokens), T5 [2, 128, 4096], Llama "
                               "[2, 32, 128, 4096], pooled [2, 2048], random-init "
                               + ("scaled fp8 e4m3 Linears (fp8 matrix multiplication), bf16 activations" if fp8 else "bf16"),
                   "parameters": n_params, "dim": 2560, "heads": 20, "head_dim": 128, "experts": 4, "top_k": 2},
        "clocks": clocks.summary(), "output_finite": finite,
        "gpu_bar": {"what": "same modules and weights, sm_100a kernels off: stock PyTorch composition on this GPU",
                    "ms_per_step": ms_stock},
        "speedup_vs_stock": ms_stock / ms,
        # relative RMS difference of the step output between the kernels and the stock composition: with the gate of
        # both on the fp32 copy of its input, and against the composition as shipped (bf16 gate: a few tokens per
        # thousand and layer pick other experts, and 48 layers of random weights spread that over the image)
        "rel_rms_vs_stock_output": {"same_routing_convention": rel, "as_shipped": rel_as_shipped,
                                    "stock_vs_stock_with_input_moved_by_one_bf16_ulp": rel_noise},
    }


def run_dit(args) -> None:
    """Side workload: benchmark configuration 4 on one GPU (see measure_config4)."""
    from comfyui_b200 import _native

    _native.load()
    dev = torch.device("cuda", 0)
    res = measure_config4(dev, args.dtype, min(args.steps, 10), args.double_blocks, args.single_blocks)
    res.update({"n_gpus": 1, "warmup": 2})
    print(json.dumps(res))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--double-blocks", type=int, default=16, help="dit: number of double-stream blocks")
    ap.add_argument("--single-blocks", type=int, default=32, help="dit: number of single-stream blocks")
    ap.add_argument("--workload", default="hidream", choices=["hidream", "config5", "hunyuan3d", "dit", "dit_body"],
                    help="hidream = the headline layer (8192 tokens per GPU, weak scaling); config5 = 131072 tokens in "
                         "total with a skewed router (strong scaling); hunyuan3d = the sibling GELU-MLP MoE block "
                         "(one GPU, bf16); dit = benchmark configuration 4, one denoising step of the whole HiDream-I1-shaped "
                         "transformer (one GPU; dit_body is an alias)")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8"],
                    help="bf16 (benchmark configuration 2, the default) or per-tensor scaled fp8 e4m3 expert weights (configuration 3)")
    ap.add_argument("--timeline", action="store_true",
                    help="after the timing, print the kernel timeline of one step on rank 0 to stderr (torch.profiler)")
    ap.add_argument("--timeline-dir", default=None,
                    help="like --timeline, but every rank writes its timeline to a file of its own in this directory")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU oracle and the stock-composition timings (profiling runs)")
    ap.add_argument("--headline-only", action="store_true",
                    help="hidream workload: skip the sub-objects (sustained loop, the other dtype, configuration 5, "
                         "expert-parallel parity) that the default run adds to the line")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "hunyuan3d":
        run_hunyuan3d(args)
    elif args.workload in ("dit", "dit_body"):
        run_dit(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
