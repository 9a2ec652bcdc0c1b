"""Host logic of the expert-parallel layer under gloo on the CPU (world sizes 2 and 4).

The kernels cannot run here, so a CPU stand-in with the same interface (built on the oracle's arithmetic) is
plugged into ExpertParallelMoE: what is tested is the placement, the count exchange, the split sizes, the
ordering of the point-to-point transfers, the receive layout handed to the grouped GEMM and the way partial
results of hidden-split experts come back.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from comfyui_b200.expert_parallel import ExpertParallelMoE, Placement, exchange_plan
from oracle import hidream_moe_oracle as O

DIM, HIDDEN_DIM = 128, 512


class OracleKernels:
    """CPU stand-in for CudaKernels: same methods, PyTorch arithmetic with the kernels' rounding points."""

    def __init__(self, layer, place, rank):
        self.layer, self.place, self.rank = layer, place, rank
        self.n_experts = layer["gate.weight"].shape[0]
        self.local = []
        part, splits = place.hidden_part(rank), place.hidden_splits
        for e in place.local_experts(rank):
            w1, w2, w3 = (layer[f"experts.{e}.{k}.weight"] for k in ("w1", "w2", "w3"))
            h = w1.shape[0] // splits
            lo, hi = part * h, (part + 1) * h
            self.local.append({"f.w1.weight": w1[lo:hi], "f.w3.weight": w3[lo:hi], "f.w2.weight": w2[:, lo:hi]})

    def route(self, x):
        idx, w = O.gate(x.float(), self.layer["gate.weight"].float())
        idx = idx.sort(dim=1).values.to(torch.int32)      # any fixed pair order will do
        w = torch.gather(O.gate_scores_fp64(x, self.layer["gate.weight"]).float(), 1, idx.long())
        flat = idx.flatten().long()
        counts = torch.bincount(flat, minlength=self.n_experts).to(torch.int32)
        offsets = torch.zeros(self.n_experts + 1, dtype=torch.int32)
        for e in range(self.n_experts):
            offsets[e + 1] = offsets[e] + -(-int(counts[e]) // 128) * 128
        rows_cap = 2 * x.shape[0] + 128 * self.n_experts
        x_perm = torch.zeros((rows_cap, x.shape[1]), dtype=x.dtype)
        row_map = torch.empty_like(flat, dtype=torch.int32)
        for e in range(self.n_experts):
            slots = (flat == e).nonzero().flatten()          # ascending slot index: the stable order
            dest = offsets[e] + torch.arange(slots.numel(), dtype=torch.int32)
            row_map[slots] = dest
            x_perm[dest.long()] = x[slots // 2]
        return idx, w, counts, offsets, x_perm, row_map.view(-1, 2)

    def shared_expert(self, x):
        return O.swiglu_ffn(x, self.layer, "shared_experts")

    def routed_experts(self, rows, group_start, group_count):
        y = torch.zeros((rows.shape[0], rows.shape[1]), dtype=rows.dtype)
        for j, (s, c) in enumerate(zip(group_start, group_count)):
            if c:
                y[s:s + c] = O.swiglu_ffn(rows[s:s + c], self.local[j], "f")
        return y

    def combine(self, partials, row_map, w, y_shared):
        y = partials[0] if len(partials) == 1 else (partials[0].float() + partials[1].float()).to(partials[0].dtype)
        wb = w.to(y.dtype)
        contrib = y[row_map.long()] * wb.unsqueeze(-1)
        routed = (contrib[:, 0].float() + contrib[:, 1].float()).to(y.dtype)
        return routed + y_shared

    def empty_rows(self, rows, dim, like):
        return torch.zeros((max(rows, 1), dim), dtype=like.dtype)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_experts, tokens_per_rank, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        layer = {k: v.bfloat16() for k, v in O.make_layer(DIM, HIDDEN_DIM, n_experts, seed=0).items()}
        n = tokens_per_rank[rank]
        x = O.make_input(n, DIM, seed=100 + rank).bfloat16()

        class _Module:      # ExpertParallelMoE only needs the expert count from the module when kernels are given
            experts = [None] * n_experts

        place = Placement(world, n_experts)
        ep = ExpertParallelMoE(_Module(), kernels=OracleKernels(layer, place, rank))
        out = ep(x.view(1, n, DIM)).view(n, DIM)
        # single-process answer for the same tokens, same routing convention as the stand-in
        k = OracleKernels(layer, Placement(1, n_experts), 0)
        idx, w, _, _, _, _ = k.route(x)
        ref, _, _ = O.moe_layer(x, layer, routing=(idx.long(), w.bfloat16()))
        torch.save({"out": out, "ref": ref, "counts": ep.last_counts}, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n_experts,tokens", [
    (2, 4, [96, 40]),          # two experts per rank, ragged token counts
    (4, 4, [33, 0, 64, 7]),    # one expert per rank, one rank without tokens
    (4, 2, [50, 50, 20, 31]),  # more ranks than experts: every expert's hidden dimension split over two ranks
])
def test_expert_parallel_matches_single_process(tmp_path, world, n_experts, tokens):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, n_experts, tokens, str(tmp_path)), nprocs=world, join=True)
    split = world > n_experts
    for rank in range(world):
        r = torch.load(tmp_path / f"rank{rank}.pt")
        assert r["out"].shape == r["ref"].shape
        if tokens[rank] == 0:
            continue
        if split:
            # two partial sums rounded to bf16 and added: one extra rounding against the single-GPU result
            torch.testing.assert_close(r["out"].float(), r["ref"].float(), rtol=2e-2, atol=2e-2)
        else:
            assert torch.equal(r["out"], r["ref"]), f"rank {rank} differs"
        assert [sum(c) for c in r["counts"]] == [2 * t for t in tokens]


def test_placement_and_exchange_plan():
    p = Placement(2, 4)
    assert p.local_experts(0) == [0, 1] and p.local_experts(1) == [2, 3] and p.owners(2) == [1]
    p = Placement(4, 4)
    assert p.local_experts(3) == [3] and p.hidden_splits == 1
    p = Placement(8, 4)
    assert p.local_experts(5) == [2] and p.hidden_part(5) == 1 and p.owners(2) == [4, 5] and p.hidden_splits == 2
    p1 = Placement(1, 4)
    assert p1.local_experts(0) == [0, 1, 2, 3]
    with pytest.raises(ValueError):
        Placement(3, 4)
    counts = [[5, 1, 0, 2], [3, 3, 3, 3]]
    recv_start, rows, gstart, gcount = exchange_plan(counts, 1, Placement(2, 4))
    assert recv_start == [[0, 0], [3, 5]] and rows == 8 and gstart == [0, 3] and gcount == [3, 5]
    recv_start, rows, gstart, gcount = exchange_plan(counts, 0, Placement(2, 4))
    assert recv_start == [[0, 5], [8, 9]] and rows == 12 and gcount == [8, 4]


def _dropout_worker(rank, world, port, out_dir):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    layer = {k: v.bfloat16() for k, v in O.make_layer(DIM, HIDDEN_DIM, 4, seed=0).items()}

    class _Module:
        experts = [None] * 4

    ep = ExpertParallelMoE(_Module(), kernels=OracleKernels(layer, Placement(world, 4), rank))
    x = O.make_input(16, DIM, seed=rank).bfloat16()
    ep(x)                                                   # one healthy step
    if rank == 1:
        # this rank leaves between steps, with nothing of its own in flight
        torch.save({"left": True}, os.path.join(out_dir, "rank1.pt"))
        os._exit(0)
    try:
        ep(x)
        outcome = "completed"
    except Exception as exc:                                # the count exchange cannot complete without the peer
        outcome = type(exc).__name__
    torch.save({"outcome": outcome}, os.path.join(out_dir, "rank0.pt"))
    os._exit(0)


def test_rank_leaving_between_steps_is_detected(tmp_path):
    """Failure detection on the host: a rank that exits between two layer calls makes the survivor's next count
    exchange raise (connection loss or the process-group timeout) instead of hanging."""
    port = _free_port()
    ctx = mp.spawn(_dropout_worker, args=(2, port, str(tmp_path)), nprocs=2, join=False)
    for p in ctx.processes:
        p.join(timeout=120)
        assert not p.is_alive(), "a rank hung after its peer left"
    assert torch.load(tmp_path / "rank1.pt")["left"]
    assert torch.load(tmp_path / "rank0.pt")["outcome"] != "completed"


def test_peer_buffer_layout_and_plan():
    """Host side of the peer-memory transport: buffer layout, owner tables and peer addresses (no GPU needed)."""
    from comfyui_b200.expert_parallel import PeerBuffers, Placement

    for world, splits in ((2, 1), (4, 1), (8, 2)):
        place = Placement(world, 4)
        cap, ret, dim = 384, 256, 512
        off_recv, off_y, off_ret, total = PeerBuffers.layout(cap, ret, dim, torch.bfloat16, place.hidden_splits)
        assert off_recv == 256 and off_y >= off_recv + cap * dim * 2 and off_ret >= off_y + cap * dim * 2
        assert total >= off_ret + splits * ret * dim * 2 and all(o % 256 == 0 for o in (off_recv, off_y, off_ret))
        bufs = [torch.zeros(total, dtype=torch.uint8) for _ in range(world)]
        bases = [b.data_ptr() for b in bufs]
        for rank in range(world):
            pb = PeerBuffers(place, rank, cap, ret, dim, torch.bfloat16, bases, bufs[rank])
            assert pb.recv.shape == (cap, dim) and pb.y.shape == (cap, dim) and pb.ret.shape == (splits, ret, dim)
            assert pb.recv.data_ptr() == bases[rank] + off_recv and pb.ret.data_ptr() == bases[rank] + off_ret
            plan = pb.plan
            assert (plan.world, plan.rank, plan.n_experts, plan.hidden_splits, plan.cap_rows) == (world, rank, 4, splits, cap)
            for e in range(4):
                owners = place.owners(e)
                assert plan.owner0[e] == owners[0] and plan.owner1[e] == (owners[1] if splits == 2 else -1)
            assert [plan.peer_recv[r] for r in range(world)] == [b + off_recv for b in bases]
            assert [plan.peer_flags[r] for r in range(world)] == bases
            # this rank's results go into the return buffer of its own hidden part at every rank
            part = place.hidden_part(rank)
            assert pb.peer_ret == [b + off_ret + part * ret * dim * 2 for b in bases]
        # fp8 activations halve the receive buffer only
        assert PeerBuffers.layout(cap, ret, dim, torch.float8_e4m3fn, splits)[1] == off_recv + cap * dim


def test_receive_layout_of_both_transports_agree():
    """The NCCL transport plans the receive buffer on the host (exchange_plan); the peer-memory transport's dispatch
    kernel derives a row's place from the all-gathered histograms alone.  Both are "local experts in order, each
    holding the rows of source 0, 1, ..."; this restates the kernel's formula and checks it against the host plan."""
    from comfyui_b200.expert_parallel import Placement, exchange_plan

    def kernel_row_base(counts, place, q, e, source):          # recv_row_base of csrc/moe_peer.cu
        row = 0
        for f in range(e):
            if q in place.owners(f):
                row += sum(counts[s][f] for s in range(place.world))
        return row + sum(counts[s][e] for s in range(source))

    g = torch.Generator().manual_seed(0)
    for world in (2, 4, 8):
        place = Placement(world, 4)
        counts = torch.randint(0, 500, (world, 4), generator=g).tolist()
        counts[1] = [0, 0, 0, 0]                                # a rank without tokens
        for rank in range(world):
            recv_start, recv_rows, group_start, group_count = exchange_plan(counts, rank, place)
            for j, e in enumerate(place.local_experts(rank)):
                assert group_start[j] == kernel_row_base(counts, place, rank, e, 0)
                assert group_count[j] == sum(counts[s][e] for s in range(world))
                for s in range(world):
                    assert recv_start[j][s] == kernel_row_base(counts, place, rank, e, s)
            assert recv_rows == sum(sum(counts[s][e] for s in range(world)) for e in place.local_experts(rank))
