"""Expert parallelism over peer memory.

Single GPU: the ranks of a 2-, 4- or 8-way placement are emulated on one device (every rank's receive / result /
flag buffers are ordinary allocations of that device, the phases of a step are run rank after rank), which checks
the dispatch addressing, the flag kernels, the grouped GEMM on received rows and the peer combine against the
single-GPU layer.  Flags are always raised before they are waited for, so no kernel ever waits on another launch.

Several GPUs (skipped with fewer): child processes, one per GPU, symmetric memory, NCCL only for the histogram
all-gather.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import hidream_moe_oracle as O

pytestmark = pytest.mark.gpu

DIM, HIDDEN_DIM, E = 512, 2048, 4


def _module(dev, fp8=False, n_experts=E):
    from comfyui_b200 import ops
    from comfyui_b200.ldm.hidream.model import MOEFeedForwardSwiGLU

    layer = {k: v.bfloat16() for k, v in O.make_layer(DIM, HIDDEN_DIM, n_experts, seed=0).items()}
    operations = ops.disable_weight_init
    if fp8:
        layer = O.quantize_layer_fp8(layer)
        operations = ops.scaled_fp8_ops(fp8_matrix_mult=True, scale_input=False, override_dtype=torch.float8_e4m3fn)
    module = MOEFeedForwardSwiGLU(DIM, HIDDEN_DIM, n_experts, 2, dtype=torch.bfloat16, device=dev,
                                  operations=operations).eval()
    module.load_state_dict({k: v.to(dev) for k, v in layer.items()}, strict=True)
    return module


@pytest.mark.parametrize("push", [True, False], ids=["push", "pull"])
@pytest.mark.parametrize("world,fp8", [(2, False), (4, False), (8, False), (2, True), (8, True)])
def test_emulated_ranks_on_one_gpu(cuda_device, world, fp8, push):
    from comfyui_b200 import moe_ops as M
    from comfyui_b200.expert_parallel import PeerBuffers, PeerExpertParallelMoE, Placement

    dev = cuda_device
    module = _module(dev, fp8)
    place = Placement(world, E)
    tokens = [1000, 700, 333, 1, 512, 129, 64, 2048][:world]
    xs = [O.make_input(n, DIM, seed=100 + r).bfloat16().to(dev) for r, n in enumerate(tokens)]
    cap_rows = sum(tokens) * min(2, place.experts_per_rank)
    act = torch.float8_e4m3fn if fp8 else torch.bfloat16
    bufs = PeerBuffers.emulate(place, cap_rows, 2 * max(tokens), DIM, act, dev)
    ranks = [PeerExpertParallelMoE(module, buffers=bufs[r], place=place, rank=r, push_results=push)
             for r in range(world)]
    with torch.inference_mode():
        for step in range(2):           # the second step re-uses every buffer and flag
            counts = []
            for x in xs:
                _, _, bc, _, _ = M.gate_topk(x, module.gate.weight)
                counts.append(M.route_plan(bc, x.shape[0], E)[1])
            counts_all = torch.stack(counts).contiguous()
            for r in range(world):
                ranks[r].phase_route(xs[r], counts_all=counts_all)
            for r in range(world):
                ranks[r].phase_experts()
            outs = [ranks[r].phase_combine() for r in range(world)]
            for r in range(world):
                ranks[r].check()
                single = module(xs[r].view(1, -1, DIM)).view(-1, DIM)
                if place.hidden_splits == 1:
                    assert torch.equal(outs[r], single), f"step {step} rank {r}"
                else:
                    torch.testing.assert_close(outs[r].float(), single.float(), rtol=2e-2, atol=2e-2)
    assert counts_all.sum(dim=1).tolist() == [2 * t for t in tokens]


def test_a_wait_that_runs_out_reports_and_returns(cuda_device):
    """The bounded wait on its real path: rank 0 of an emulated pair waits for an "arrived" flag that nobody raises,
    with a budget of about a millisecond.  The kernel gives up, leaves code 7 in the status word and returns; the host
    turns that into ETIMEOUT; the GPU and the buffers stay usable (a complete step follows on the same buffers)."""
    import ctypes

    from comfyui_b200 import _native as N
    from comfyui_b200 import moe_ops as M
    from comfyui_b200.expert_parallel import PeerBuffers, PeerExpertParallelMoE, Placement

    dev = cuda_device
    lib = N.load()
    place = Placement(2, E)
    bufs = PeerBuffers.emulate(place, 4096, 2048, DIM, torch.bfloat16, dev)
    status = torch.zeros((N.STATUS_WORDS,), dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = lib.comfy_moe_ep_wait_budget(bufs[0].plan, N.EP_ARRIVED, 1, 2_000_000, ctypes.c_void_p(status.data_ptr()), stream)
    t1.record()
    assert rc == N.OK
    with pytest.raises(N.MoeError) as err:
        M.read_status(status)
    assert err.value.code == N.ETIMEOUT and "status word = 7" in str(err.value)
    assert 0.2 < t0.elapsed_time(t1) < 100.0            # it waited for its budget (about 1 ms), not for two seconds
    M.read_status(status)                               # reported once, then clean
    assert lib.comfy_moe_ep_wait_budget(bufs[0].plan, N.EP_ARRIVED, 1, 0, ctypes.c_void_p(status.data_ptr()),
                                        stream) == N.EINVAL
    # the same buffers then carry a normal step
    module = _module(dev)
    ranks = [PeerExpertParallelMoE(module, buffers=bufs[r], place=place, rank=r) for r in range(2)]
    xs = [O.make_input(n, DIM, seed=40 + r).bfloat16().to(dev) for r, n in enumerate((300, 200))]
    with torch.inference_mode():
        counts = []
        for x in xs:
            _, _, bc, _, _ = M.gate_topk(x, module.gate.weight)
            counts.append(M.route_plan(bc, x.shape[0], E)[1])
        counts_all = torch.stack(counts).contiguous()
        for r in range(2):
            ranks[r].phase_route(xs[r], counts_all=counts_all)
        for r in range(2):
            ranks[r].phase_experts()
        for r in range(2):
            out = ranks[r].phase_combine()
            ranks[r].check()
            assert torch.equal(out, module(xs[r].view(1, -1, DIM)).view(-1, DIM))


def test_two_layers_share_the_buffers(cuda_device):
    """The layers of a model use one set of buffers and one epoch counter, one after the other."""
    from comfyui_b200 import moe_ops as M
    from comfyui_b200.expert_parallel import PeerBuffers, PeerExpertParallelMoE, Placement

    dev, world = cuda_device, 2
    place = Placement(world, E)
    tokens = [400, 250]
    xs = [O.make_input(n, DIM, seed=70 + r).bfloat16().to(dev) for r, n in enumerate(tokens)]
    bufs = PeerBuffers.emulate(place, 2 * sum(tokens), 2 * max(tokens), DIM, torch.bfloat16, dev)
    mods = []
    for seed in (0, 1):
        m = _module(dev)
        with torch.no_grad():
            for p in m.parameters():
                p.mul_(1.0 + 0.25 * seed)
        mods.append(m)
    layers = [[PeerExpertParallelMoE(m, buffers=bufs[r], place=place, rank=r) for r in range(world)] for m in mods]
    with torch.inference_mode():
        for which in (0, 1, 0, 1):
            mod, ranks = mods[which], layers[which]
            counts = [M.route_plan(M.gate_topk(x, mod.gate.weight)[2], x.shape[0], E)[1] for x in xs]
            counts_all = torch.stack(counts).contiguous()
            for r in range(world):
                ranks[r].phase_route(xs[r], counts_all=counts_all)
            for r in range(world):
                ranks[r].phase_experts()
            outs = [ranks[r].phase_combine() for r in range(world)]
            for r in range(world):
                ranks[r].check()
                assert torch.equal(outs[r], mod(xs[r].view(1, -1, DIM)).view(-1, DIM)), f"layer {which} rank {r}"
    assert bufs[0].epoch == 4 and bufs[1].epoch == 4


def test_rank_without_tokens(cuda_device):
    """A rank that owns experts but has no tokens of its own still serves the others (and gets an empty output)."""
    from comfyui_b200 import moe_ops as M
    from comfyui_b200.expert_parallel import PeerBuffers, PeerExpertParallelMoE, Placement

    dev = cuda_device
    module = _module(dev)
    place = Placement(2, E)
    tokens = [0, 300]
    xs = [O.make_input(n, DIM, seed=50 + r).bfloat16().to(dev) for r, n in enumerate(tokens)]
    bufs = PeerBuffers.emulate(place, 1024, 1024, DIM, torch.bfloat16, dev)
    ranks = [PeerExpertParallelMoE(module, buffers=bufs[r], place=place, rank=r) for r in range(2)]
    with torch.inference_mode():
        counts = []
        for x in xs:
            _, _, bc, _, _ = M.gate_topk(x, module.gate.weight)
            counts.append(M.route_plan(bc, x.shape[0], E)[1])
        counts_all = torch.stack(counts).contiguous()
        assert counts_all[0].sum().item() == 0
        for r in range(2):
            ranks[r].phase_route(xs[r], counts_all=counts_all)
        for r in range(2):
            ranks[r].phase_experts()
        outs = [ranks[r].phase_combine() for r in range(2)]
        for r in range(2):
            ranks[r].check()
        assert outs[0].shape == (0, DIM)
        assert torch.equal(outs[1], module(xs[1].view(1, -1, DIM)).view(-1, DIM))


def test_receive_buffer_too_small_is_reported(cuda_device):
    """Rows that do not fit the receive buffers are not written; the status word says so."""
    from comfyui_b200 import _native as N, moe_ops as M
    from comfyui_b200.expert_parallel import PeerBuffers, PeerExpertParallelMoE, Placement

    dev = cuda_device
    module = _module(dev)
    place = Placement(2, E)
    xs = [O.make_input(256, DIM, seed=7 + r).bfloat16().to(dev) for r in range(2)]
    bufs = PeerBuffers.emulate(place, 128, 512, DIM, torch.bfloat16, dev)  # 1024 routed rows will not fit
    ranks = [PeerExpertParallelMoE(module, buffers=bufs[r], place=place, rank=r) for r in range(2)]
    with torch.inference_mode():
        counts = [M.route_plan(M.gate_topk(x, module.gate.weight)[2], 256, E)[1] for x in xs]
        counts_all = torch.stack(counts).contiguous()
        for r in range(2):
            ranks[r].phase_route(xs[r], counts_all=counts_all)
        for r in range(2):
            ranks[r].phase_experts()
        for r in range(2):
            ranks[r].phase_combine()
        with pytest.raises(N.MoeError) as err:
            ranks[0].check()
        assert err.value.code == N.ETOOLARGE


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, tokens, fp8, push, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from comfyui_b200.expert_parallel import PeerExpertParallelMoE

        module = _module(dev, fp8)
        n = tokens[rank]
        x = O.make_input(n, DIM, seed=100 + rank).bfloat16().to(dev).view(1, n, DIM)
        # one case leaves the capacity to the constructor's own agreement between the ranks (their counts differ)
        ep = PeerExpertParallelMoE(module, max_tokens=None if (world == 2 and fp8) else max(tokens), push_results=push)
        with torch.inference_mode():
            outs = [ep(x) for _ in range(3)]
            ep.check()
            single = module(x)
        torch.cuda.synchronize()
        dist.barrier()
        torch.save({"outs": [o.cpu() for o in outs], "single": single.cpu(), "counts": ep.last_counts_host},
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,fp8,push", [(2, False, True), (2, False, False), (2, True, True), (4, False, True),
                                            (8, False, True), (8, True, True)])
def test_peer_expert_parallel_on_gpus(tmp_path, cuda_device, world, fp8, push):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    tokens = [1000, 700, 333, 1, 512, 129, 64, 2048][:world]
    mp.spawn(_worker, args=(world, _free_port(), tokens, fp8, push, str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        r = torch.load(tmp_path / f"rank{rank}.pt")
        for o in r["outs"][1:]:
            assert torch.equal(o, r["outs"][0])
        if world <= E:
            assert torch.equal(r["outs"][0], r["single"]), f"rank {rank}"
        else:
            torch.testing.assert_close(r["outs"][0].float(), r["single"].float(), rtol=2e-2, atol=2e-2)
        assert [sum(c) for c in r["counts"]] == [2 * t for t in tokens]
