#!/usr/bin/env python
"""Benchmark of the HiDream MoE feed-forward layer: tokens/s of one full layer call.

    python bench.py --gpus N --steps K --warmup W            # this repository's sm_100a kernels
    python bench.py --impl reference --steps K --warmup W    # the reference algorithm on the host cores

A step is one call of the layer (gate -> plan -> permute -> grouped SwiGLU GEMM x2 -> combine, shared expert
included) on synthetic data: dim 2560, 4 routed experts of hidden 6912 (top-2), shared expert of hidden 3584,
bf16, 8192 tokens per GPU, weights N(0, 0.02^2), inputs N(0, 1), seeded.  With N > 1 the routed experts are
expert-parallel (NCCL all-to-all dispatch and combine), every rank owns 8192 tokens (weak scaling) and runs the
shared expert on them.

One JSON line is printed by rank 0.  `value` is measured with the inputs resident in HBM; `e2e` is the same
metric through the module call with pinned-host input and output copies inside the timed region; `roofline`
describes the grouped GEMM (both passes) against the measured bf16 tensor peak; `cpu_baseline` is the CPU
oracle (a restatement of the reference's PyTorch code) timed on this machine's host cores.
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
def oracle_cpu_tokens_per_s(n_tokens: int, steps: int, warmup: int, dtype: str = "bf16"):
    """The CPU oracle on `n_tokens` of the bench workload, all host threads.  Returns (tokens/s, s/step, cores)."""
    from oracle import hidream_moe_oracle as O

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
    return n_tokens / dt, dt, torch.get_num_threads()


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    value, dt, cores = oracle_cpu_tokens_per_s(CPU_SAMPLE_TOKENS, args.steps, max(args.warmup, 1), args.dtype)
    sample = (f"each step = the first {CPU_SAMPLE_TOKENS} of the {TOKENS_PER_GPU} bench tokens through the CPU oracle "
              f"(oracle/hidream_moe_oracle.py: the reference's gate + moe_infer + shared expert in PyTorch)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
        "config": workload_config(args.gpus, args.dtype),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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


def run_gpu_arm(args) -> None:
    import torch.distributed as dist

    from comfyui_b200 import _native, moe_ops, ops
    from comfyui_b200.ldm.hidream.model import MOEFeedForwardSwiGLU

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

    fp8 = args.dtype == "fp8"
    config5 = args.workload == "config5"
    n = CONFIG5_TOKENS // world if config5 else TOKENS_PER_GPU
    state, x_host = make_synthetic(dev, seed_w=0, seed_x=1 + rank, fp8=fp8, n_tokens=n, skew=config5)
    operations = ops.disable_weight_init if not fp8 else ops.scaled_fp8_ops(
        fp8_matrix_mult=True, scale_input=False, override_dtype=torch.float8_e4m3fn)
    module = MOEFeedForwardSwiGLU(DIM, HIDDEN_DIM, N_EXPERTS, TOP_K, dtype=torch.bfloat16, device=dev,
                                  operations=operations).eval()
    module.load_state_dict(state, strict=True)
    x_pinned = x_host.pin_memory()
    out_pinned = torch.empty_like(x_host).pin_memory()
    x = x_host.to(dev).view(2, n // 2, DIM)

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
            runner = ExpertParallelMoE(module, dist.group.WORLD)
        else:
            runner = PeerExpertParallelMoE(module, dist.group.WORLD, max_tokens=n)
        step = lambda inp: runner(inp)                      # noqa: E731
        launches_per_step = runner.launches_per_step
    else:
        assert ops._layer_pack(module, x) is not None, "bench: layer not eligible for the sm_100a kernels"
        step = lambda inp: module(inp)                      # noqa: E731
        launches_per_step = 5   # gate, plan + permute, GEMM pass 1, GEMM pass 2, combine

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.inference_mode():
        for _ in range(max(args.warmup, 3)):
            step(x)
        # ---- device-resident timing: exactly K steps between two events
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clocks:
            ev0.record()
            for _ in range(args.steps):
                step(x)
            ev1.record()
            barrier()
        ms_total = ev0.elapsed_time(ev1)
        if world > 1 and hasattr(runner, "check"):
            runner.check()          # no flag wait ran out, every routed row fitted its receive buffer

        # ---- end to end: every step copies its input from pinned host memory and its output back to pinned host
        # memory.  The copies run on their own streams with two buffers each, the way a serving loop would feed
        # the layer: step i's upload and step i-1's download overlap step i's compute; nothing is skipped.
        ms_e2e = time_end_to_end(step, x_pinned, out_pinned, n, dev, args.steps, barrier)

        # ---- per-stage timing of the same work through the stage-level C ABI (single GPU only)
        stages = None
        gpu_bar = None
        if world == 1:
            stages = time_stages(module, x.view(n, DIM), args.steps, moe_ops, ops)
            if not args.no_cpu_baseline:
                gpu_bar = time_stock_composition(module, x, ops)


        if args.timeline and rank == 0:
            print_timeline(step, x)
        elif args.timeline:
            for _ in range(3):          # the other ranks take the same three steps
                step(x)
            torch.cuda.synchronize()

    times = torch.tensor([ms_total, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e = times.tolist()

    if rank == 0:
        peaks = measured_peaks()
        ms_step = ms_total / args.steps
        value = n * world / (ms_step * 1e-3)
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if config5 else "weak",
            "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "config": workload_config(world, args.dtype, n, config5),
            "e2e": {"value": n * world / (ms_e2e / args.steps * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": x_pinned.numel() * 2, "d2h_bytes_per_step": out_pinned.numel() * 2},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks.summary(),
            "layer_tflops": FLOPS_PER_TOKEN * n * world / (ms_step * 1e-3) / 1e12,
            "layer_frac_of_nominal": FLOPS_PER_TOKEN * n / (ms_step * 1e-3) / 1e12 / (4500.0 if fp8 else 2250.0),
        }
        if world > 1:
            # no per-kernel timing in the multi-GPU loop: the grouped GEMM's FLOPs per GPU over the WHOLE step (routing,
            # exchange, flag waits and combine included), i.e. a lower bound on what the kernel itself reaches
            peak = peaks["tflops_sustained"] * (2.0 if fp8 else 1.0)
            achieved = FLOPS_PER_TOKEN_GEMM * n / (ms_step * 1e-3) / 1e12
            line["roofline"] = {
                "bound": "tensor", "kernel": "grouped_gemm_kernel (per GPU; time = the whole expert-parallel step)",
                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "peak_source": f"{peaks['source']}: sustained cuBLAS bf16 (burst {peaks['tflops_burst']})"
                               + (" x 2 for fp8" if fp8 else ""),
                "frac_of_nominal": achieved / (4500.0 if fp8 else 2250.0), "traffic": None,
            }
        if config5:
            # realised routing: slots per expert over all GPUs, and the rows each GPU's routed experts process
            if world > 1:
                last = runner.last_counts_host if hasattr(runner, "last_counts_host") else runner.last_counts
                per_expert = [sum(c[e] for c in last) for e in range(N_EXPERTS)]
                owners = [runner.place.owners(e) for e in range(N_EXPERTS)]
                rows = [sum(per_expert[e] for e in range(N_EXPERTS) if r in owners[e]) for r in range(world)]
            else:
                from comfyui_b200 import torch_ops

                layer = ops._layer_pack(module, x)
                per_expert = torch_ops._workspace(layer, n).expert_counts.tolist()
                rows = [sum(per_expert)]
            line["routing"] = {"slots_per_expert": per_expert, "share_of_expert_0": per_expert[0] / sum(per_expert),
                               "routed_rows_per_gpu": rows}
        if stages is not None:
            gemm_ms = stages["grouped_gemm_ms"]
            achieved = FLOPS_PER_TOKEN_GEMM * n / (gemm_ms * 1e-3) / 1e12
            # fp8: no measured fp8 denominator exists; twice the measured bf16 figure is used and named as such
            peak = peaks["tflops_sustained"] * (2.0 if fp8 else 1.0)
            line["roofline"] = {
                "bound": "tensor", "kernel": "grouped_gemm_kernel (pass 1 SwiGLU + pass 2, one C-ABI call)",
                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "peak_source": f"{peaks['source']}: sustained cuBLAS bf16 (burst {peaks['tflops_burst']})"
                               + (" x 2 for fp8" if fp8 else ""),
                "frac_of_burst": achieved / (peaks["tflops_burst"] * (2.0 if fp8 else 1.0)),
                "frac_of_nominal": achieved / (4500.0 if fp8 else 2250.0),
                # dram__bytes_read + dram__bytes_write of the two launches, from the ncu capture summarised in
                # profiles/grouped_gemm_{bf16,fp8}_8192tokens.md (same workload)
                "traffic": 0.658e9 if fp8 else 1.587e9, "algorithmic_bytes": 0.71e9 if fp8 else 1.30e9,
            }
            line["stages"] = stages
            line["gpu_bar"] = gpu_bar
            hbm = peaks["hbm_gbs"]
            line["hbm_kernels"] = {
                k: {"achieved_gbs": stages[k + "_bytes"] / (stages[k + "_ms"] * 1e-3) / 1e9,
                    "frac": stages[k + "_bytes"] / (stages[k + "_ms"] * 1e-3) / 1e9 / hbm, "peak_gbs": hbm}
                for k in ("gate", "permute", "combine")
            }
            if not args.no_cpu_baseline:
                cpu_value, cpu_dt, cores = oracle_cpu_tokens_per_s(CPU_SAMPLE_TOKENS, 20, 2, args.dtype)
                line["cpu_baseline"] = {
                    "value": cpu_value, "unit": "tokens/s", "cores": cores, "kind": "port",
                    "sample": f"20 calls on the first {CPU_SAMPLE_TOKENS} of the {n} bench tokens, CPU oracle "
                              "(PyTorch, all host threads)",
                }
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
    names = ["gate", "plan", "permute", "grouped_gemm", "combine"]
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
                                    None, P(ws.x_perm), P(ws.x_q) if layer.fp8 else None, None, P(ws.row_map), stream)
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
    res = {}
    for i, k in enumerate(names):
        res[k + "_ms"] = sum(m[i].elapsed_time(m[i + 1]) for m in all_marks) / steps
    res["gate_bytes"] = n * d * 2 + e * d * 2 + n * 2 * 8
    res["permute_bytes"] = n * d * 2 + (n * 2 * d * 2 if not layer.fp8 else n * 3 * d)
    res["combine_bytes"] = n * 2 * d * 2 + n * d * 2 + n * d * 2
    return res


def print_timeline(step, x) -> None:
    """Kernel timeline of one step on this rank (torch.profiler / CUPTI), printed to stderr: start offset, duration,
    kernel name.  Three steps are profiled and the middle one is shown."""
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            step(x)
        torch.cuda.synchronize()
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    evs.sort(key=lambda e: e.time_range.start)
    gates = [i for i, e in enumerate(evs) if "gate_topk" in e.name]
    if len(gates) < 3:
        print("timeline: no gate kernels found", file=sys.stderr)
        return
    lo, hi = gates[1], gates[2]
    t0 = evs[lo].time_range.start
    print("timeline of one step (offset us, duration us, kernel):", file=sys.stderr)
    for e in evs[lo:hi]:
        print(f"{e.time_range.start - t0:9.1f} {e.time_range.elapsed_us():8.1f}  {e.name[:100]}", file=sys.stderr)


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


def run_dit_body(args) -> None:
    """Side workload (not the headline): the transformer body of benchmark configuration 4, i.e. 16 double-stream and 32
    single-stream HiDream blocks (dim 2560, 20 heads x 128, MoE feed-forward on the image tokens), random-init bf16,
    2 x 4096 image tokens + 2 x 384 text tokens (128 T5 + 2 x 128 Llama), one pass = one denoising step without the
    embedders and the final layer.  Timed with the kernels and, on the same modules, as PyTorch composes it."""
    from comfyui_b200 import _native, ops
    from comfyui_b200.ldm.hidream import model as M

    _native.load()
    dev = torch.device("cuda", 0)
    dim, heads, head_dim, b, s_img, s_txt = 2560, 20, 128, 2, 4096, 384
    n_double, n_single = args.double_blocks, args.single_blocks
    torch.manual_seed(0)

    fp8 = args.dtype == "fp8"
    operations = ops.disable_weight_init if not fp8 else ops.scaled_fp8_ops(
        fp8_matrix_mult=True, scale_input=False, override_dtype=torch.float8_e4m3fn)

    def build(single):
        cls = M.HiDreamImageSingleTransformerBlock if single else M.HiDreamImageTransformerBlock
        blk = cls(dim, heads, head_dim, 4, 2, dtype=torch.bfloat16, device=dev, operations=operations).eval()
        with torch.no_grad():
            for mod in blk.modules():
                w = getattr(mod, "weight", None)
                if isinstance(mod, torch.nn.Linear) and w is not None and w.dtype == torch.float8_e4m3fn:
                    # scaled fp8 checkpoint convention: s = max|w| / 448, weight = (w / s) in e4m3, scale_weight = s
                    full = torch.randn(w.shape, device=dev) * 0.02
                    sc = full.abs().max() / 448.0
                    w.copy_((full / sc).to(torch.float8_e4m3fn))
                    mod.scale_weight.fill_(float(sc))
                    if mod.bias is not None:
                        mod.bias.copy_((torch.randn(mod.bias.shape, device=dev) * 0.02).to(mod.bias.dtype))
            for name, p in blk.named_parameters():
                if p.dtype == torch.float8_e4m3fn or name.endswith("scale_weight"):
                    continue
                if "rms_norm" in name:
                    p.fill_(1.0)
                else:
                    p.normal_(0.0, 0.02)
        return blk

    doubles = [build(False) for _ in range(n_double)]
    singles = [build(True) for _ in range(n_single)]
    img = torch.randn((b, s_img, dim), device=dev).bfloat16()
    txt = torch.randn((b, s_txt, dim), device=dev).bfloat16()
    ada = torch.randn((b, dim), device=dev).bfloat16()
    # the model's position ids: (0, row, column) for the 64 x 64 patches, zeros for text tokens
    ids = torch.zeros((b, s_img + s_txt, 3), device=dev)
    ids[:, :s_img, 1] = torch.arange(64, device=dev).repeat_interleave(64)
    ids[:, :s_img, 2] = torch.arange(64, device=dev).repeat(64)
    omega = [1.0 / (10000 ** torch.linspace(0, (d - 2) / d, steps=d // 2, dtype=torch.float64, device=dev))
             for d in (64, 32, 32)]
    ang = torch.cat([ids[..., i, None].float() * omega[i].float() for i in range(3)], dim=-1)
    rope = torch.stack([ang.cos(), -ang.sin(), ang.sin(), ang.cos()], dim=-1).reshape(b, s_img + s_txt, 1, 64, 2, 2)
    rope = rope.float().contiguous()

    def step():
        x, t = img, txt
        for blk in doubles:
            x, t = blk(x, None, t, ada, rope)
        seq = torch.cat([x, t], dim=1)
        for blk in singles:
            seq = blk(seq, None, None, ada, rope)
        return seq

    def timed(steps, warmup):
        for _ in range(warmup):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    steps = min(args.steps, 10)
    with torch.inference_mode():
        with ClockSampler(0) as clocks:
            ms = timed(steps, 3)
        ops.ENABLE_SM100_KERNELS = False
        try:
            ms_stock = timed(max(steps // 2, 2), 2)
        finally:
            ops.ENABLE_SM100_KERNELS = True
    print(json.dumps({
        "metric": "denoising-step body, ms (HiDream-I1 transformer blocks)", "value": ms, "unit": "ms",
        "n_gpus": 1, "steps": steps, "warmup": 3, "ms_per_step": ms, "higher_is_better": False, "dtype": args.dtype,
        "data": "synthetic",
        "config": {"workload": f"benchmark configuration 4 without embedders and final layer: {n_double} double-stream + "
                               f"{n_single} single-stream blocks, 2 x (4096 image + 384 text) tokens, random-init "
                               + ("scaled fp8 e4m3 Linears (fp8 matrix multiplication), bf16 activations" if fp8 else "bf16"),
                   "dim": dim, "heads": heads, "head_dim": head_dim, "experts": 4, "top_k": 2},
        "clocks": clocks.summary(),
        "gpu_bar": {"what": "same modules and weights, sm_100a kernels off: stock PyTorch composition on this GPU",
                    "ms_per_step": ms_stock},
        "speedup_vs_stock": ms_stock / ms,
    }))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--double-blocks", type=int, default=16, help="dit_body: number of double-stream blocks")
    ap.add_argument("--single-blocks", type=int, default=32, help="dit_body: number of single-stream blocks")
    ap.add_argument("--workload", default="hidream", choices=["hidream", "config5", "hunyuan3d", "dit_body"],
                    help="hidream = the headline layer (8192 tokens per GPU, weak scaling); config5 = 131072 tokens in "
                         "total with a skewed router (strong scaling); hunyuan3d = the sibling GELU-MLP MoE block "
                         "(one GPU, bf16)")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8"],
                    help="bf16 (benchmark configuration 2, the default) or per-tensor scaled fp8 e4m3 expert weights (configuration 3)")
    ap.add_argument("--timeline", action="store_true",
                    help="after the timing, print the kernel timeline of one step on rank 0 to stderr (torch.profiler)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU oracle and the stock-composition timings (profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "hunyuan3d":
        run_hunyuan3d(args)
    elif args.workload == "dit_body":
        run_dit_body(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
