"""Expert-parallel execution of one HiDream MoE feed-forward across the GPUs of one node.

The reference is single-process and has no counterpart to this file; the partitioning follows from the layer
(``comfy/ldm/hidream/model.py:287-346``): rows are independent, the only coupling is that a token's two experts may
live on another GPU.

* Tokens are data-parallel: every rank owns its own ``[n, D]`` slice, runs the gate, the shared expert (weights
  replicated) and the final combine on it.
* Routed experts are expert-parallel.  With E experts on G ranks: G <= E -> E/G consecutive experts per rank;
  G = 2E -> expert e lives on ranks 2e and 2e+1, each holding one half of the hidden dimension (rows of w1/w3,
  columns of w2, passed to the kernels as strided views without copying); the two partial outputs are summed by the
  token's owner.
* One exchange each way, with two transports:

  ``PeerExpertParallelMoE`` (the default of ``bench.py``): every rank's receive and return buffers live in symmetric
  memory mapped into all peers; the dispatch kernel writes each routed row straight into its expert's rank, the expert
  GEMM writes each result straight back into the token owner's return buffer, epoch flags in peer memory order the
  steps, and the only collective is an NCCL all-gather of the E-bin histograms.  No host synchronisation.

  ``ExpertParallelMoE``: the histograms are all-gathered and read on the host (one synchronisation per call, like the
  reference's ``bincount().cpu()``), then rows travel as point-to-point transfers batched into one NCCL group (an
  all-to-all with exact per-pair row counts).  The permutation kernel already wrote the rows grouped by expert, i.e.
  by destination, so the send side needs no packing; received rows land in local HBM ordered (local expert, source
  rank), which the grouped GEMM consumes in place.  Its arithmetic is delegated to a ``kernels`` object: ``CudaKernels``
  (the sm_100a kernels through the C ABI) in production; the CPU tests plug in a stand-in so the exchange logic can
  run under gloo.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


@dataclass
class Placement:
    """Which routed experts (and which hidden slice of them) a rank computes."""

    world: int
    n_experts: int

    def __post_init__(self):
        g, e = self.world, self.n_experts
        if g <= e:
            if e % g:
                raise ValueError(f"{e} experts do not divide over {g} ranks")
            self.experts_per_rank, self.hidden_splits = e // g, 1
        else:
            if g % e:
                raise ValueError(f"{g} ranks do not divide over {e} experts")
            self.experts_per_rank, self.hidden_splits = 1, g // e

    def local_experts(self, rank: int) -> List[int]:
        first = (rank // self.hidden_splits) * self.experts_per_rank
        return list(range(first, first + self.experts_per_rank))

    def hidden_part(self, rank: int) -> int:
        return rank % self.hidden_splits

    def owners(self, expert: int) -> List[int]:
        first = (expert // self.experts_per_rank) * self.hidden_splits
        return list(range(first, first + self.hidden_splits))


def exchange_plan(counts: Sequence[Sequence[int]], rank: int, place: Placement):
    """Pure host arithmetic of one exchange.  ``counts[s][e]`` = routed slots of source rank s for expert e.

    Returns (recv_start, recv_rows, group_start, group_count):
      recv_start[j][s]  first row, in this rank's receive buffer, of the rows source s sends for local expert j;
      recv_rows         total rows received;
      group_start[j], group_count[j]  the row range local expert j computes on (all sources, contiguous).
    """
    local = place.local_experts(rank)
    recv_start, group_start, group_count = [], [], []
    row = 0
    for e in local:
        group_start.append(row)
        starts = []
        for s in range(place.world):
            starts.append(row)
            row += int(counts[s][e])
        recv_start.append(starts)
        group_count.append(row - group_start[-1])
    return recv_start, row, group_start, group_count


class CudaKernels:
    """The sm_100a kernels behind the C ABI, bound to one loaded MOEFeedForwardSwiGLU module."""

    def __init__(self, module, place: Placement, rank: int, allow_fp8: bool = False):
        from . import moe_ops, ops

        self.M = moe_ops
        self.module = module
        dev = module.gate.weight.device
        self.gate_w = module.gate.weight.detach()
        self.n_experts = len(module.experts)
        self.shared = ops._ffn_pack(module.shared_experts, dev, moe_ops)
        if self.shared is None:
            raise ValueError("shared expert weights are not eligible for the sm_100a kernels")
        part, splits = place.hidden_part(rank), place.hidden_splits
        self.local = []
        for e in place.local_experts(rank):
            ffn = module.experts[e]
            full = ops._ffn_pack(ffn, dev, moe_ops)
            if full is None:
                raise ValueError(f"expert {e} weights are not eligible for the sm_100a kernels")
            if splits == 1:
                self.local.append(full)
            else:
                h = full.hidden // splits
                if h % 128:
                    raise ValueError("hidden slice must be a multiple of 128")
                lo, hi = part * h, (part + 1) * h
                self.local.append(moe_ops.FfnPack(full.w1[lo:hi], full.w3[lo:hi], full.w2[:, lo:hi],
                                                  scale_w1=full.scale_w1, scale_w3=full.scale_w3,
                                                  scale_w2=full.scale_w2, scale_in13=full.scale_in13,
                                                  scale_in2=full.scale_in2))
        self.fp8 = self.shared.w1.dtype == torch.float8_e4m3fn
        self._limited = {}
        if self.fp8:
            # every rank quantises the rows it sends with ONE activation scale, and the expert's rank dequantises with
            # its own scale_input: all routed experts (local or not) must therefore carry the same scale_input
            scales = []
            for e in range(self.n_experts):
                pack = ops._ffn_pack(module.experts[e], dev, moe_ops)
                if pack is None:
                    raise ValueError(f"expert {e} weights are not eligible for the sm_100a kernels")
                scales.append(None if pack.scale_in13 is None else float(pack.scale_in13))
            if len(set(scales)) != 1:
                raise ValueError("expert-parallel fp8 needs one scale_input shared by w1/w3 of all routed experts "
                                 f"(found {scales}): the dispatch quantises each row once for whichever rank computes it")
        if self.fp8 and not allow_fp8:
            raise ValueError("the NCCL transport covers bf16 weights; scaled fp8 runs on the peer-memory transport")

    launches_local = 3      # gate, plan, permutation

    def route(self, x):
        M = self.M
        n = x.shape[0]
        idx, w, block_counts, _, _ = M.gate_topk(x, self.gate_w)
        block_offsets, counts, offsets = M.route_plan(block_counts, n, self.n_experts)
        x_perm, row_map, _ = M.permute(x, idx, block_offsets, offsets, self.n_experts)
        return idx, w, counts, offsets, x_perm, row_map

    def shared_expert(self, x, max_sms: int = 0):
        pack = self.shared
        if max_sms > 0:
            import dataclasses

            pack = self._limited.get(max_sms)
            if pack is None:
                pack = dataclasses.replace(self.shared, max_sms=max_sms)
                self._limited[max_sms] = pack
        _, y, _, _ = self.M.grouped_swiglu([], pack, None, None, None, x, check_status=False)
        return y

    def routed_experts(self, rows, group_start, group_count):
        dev = rows.device
        start = torch.tensor(group_start, dtype=torch.int32).to(dev, non_blocking=True)
        count = torch.tensor(group_count, dtype=torch.int32).to(dev, non_blocking=True)
        y, _, _, _ = self.M.grouped_swiglu(self.local, None, start, count, rows, None, check_status=False)
        return y

    def combine(self, partials, row_map, w, y_shared):
        return self.M.combine(partials[0], row_map, w, y_shared, y_perm_b=partials[1] if len(partials) > 1 else None)

    def empty_rows(self, rows, dim, like):
        return torch.empty((max(rows, 1), dim), dtype=like.dtype, device=like.device)


class ExpertParallelMoE:
    """Callable: ``out = ep(x)`` with x this rank's tokens ``[B, S, D]`` or ``[n, D]`` (bf16 on the GPU)."""

    def __init__(self, module, group=None, kernels=None):
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.n_experts = len(module.experts)
        self.place = Placement(self.world, self.n_experts)
        self.kernels = kernels if kernels is not None else CudaKernels(module, self.place, self.rank)
        self.last_counts = None          # [world][E] routed slots of the last call, for reporting
        self._side = None                # side stream for the count exchange and the dispatch (CUDA only)
        self._pinned = None
        # gate, plan, permute, shared GEMM x2, routed GEMM x2, combine
        self.launches_per_step = 8

    # -- communication helpers ------------------------------------------------------------------
    def _peer(self, r: int) -> int:
        return dist.get_global_rank(self.group, r) if self.group is not dist.group.WORLD else r

    def _gather_counts(self, counts: torch.Tensor) -> List[List[int]]:
        flat = torch.empty((self.world * self.n_experts,), dtype=counts.dtype, device=counts.device)
        dist.all_gather_into_tensor(flat, counts.contiguous(), group=self.group)
        return flat.view(self.world, self.n_experts).cpu().tolist()      # the one host sync of the call

    def _exchange(self, sends: List[Tuple[torch.Tensor, int]], recvs: List[Tuple[torch.Tensor, int]]):
        ops = []
        for t, peer in sends:
            if t.shape[0]:
                ops.append(dist.P2POp(dist.isend, t, self._peer(peer), group=self.group))
        for t, peer in recvs:
            if t.shape[0]:
                ops.append(dist.P2POp(dist.irecv, t, self._peer(peer), group=self.group))
        return dist.batch_isend_irecv(ops) if ops else []

    # -- one layer call -------------------------------------------------------------------------
    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        k, place, rank = self.kernels, self.place, self.rank
        dim = x2.shape[1]
        cuda = x2.is_cuda

        idx, w, counts_dev, offsets_dev, x_perm, row_map = k.route(x2)

        # The count exchange, the host's planning and the dispatch run on a side stream that only depends on the
        # routing kernels, so the shared expert (main stream) computes underneath them.
        if cuda:
            main = torch.cuda.current_stream()
            if self._side is None:
                self._side = torch.cuda.Stream(device=x2.device)
                self._pinned = torch.empty((self.world * self.n_experts,), dtype=torch.int32).pin_memory()
            side = self._side
            side.wait_stream(main)
            with torch.cuda.stream(side):
                flat = torch.empty((self.world * self.n_experts,), dtype=counts_dev.dtype, device=x2.device)
                dist.all_gather_into_tensor(flat, counts_dev.contiguous(), group=self.group)
                self._pinned.copy_(flat, non_blocking=True)
                done = torch.cuda.Event()
                done.record(side)
            y_shared = k.shared_expert(x2)
            done.synchronize()                                     # the one host synchronisation of the call
            counts = self._pinned.view(self.world, self.n_experts).tolist()
        else:
            counts = self._gather_counts(counts_dev)
            y_shared = k.shared_expert(x2)
        self.last_counts = counts
        mine = counts[rank]
        # first row of every expert in my permuted buffer: expert blocks start on multiples of 128 rows
        my_offset, row = [], 0
        for e in range(self.n_experts):
            my_offset.append(row)
            row += -(-mine[e] // 128) * 128

        recv_start, recv_rows, group_start, group_count = exchange_plan(counts, rank, place)
        recv = k.empty_rows(recv_rows, dim, x_perm)
        local = place.local_experts(rank)

        # dispatch: my rows of expert e go to every rank that computes (a slice of) e
        sends, recvs, copies = [], [], []
        for e in range(self.n_experts):
            rows = x_perm[my_offset[e]: my_offset[e] + mine[e]]
            for q in place.owners(e):
                if q != rank:
                    sends.append((rows, q))
        for j, e in enumerate(local):
            for s in range(self.world):
                dst = recv[recv_start[j][s]: recv_start[j][s] + counts[s][e]]
                if s == rank:
                    copies.append((dst, x_perm[my_offset[e]: my_offset[e] + mine[e]]))
                else:
                    recvs.append((dst, s))
        if cuda:
            recv.record_stream(side)
            x_perm.record_stream(side)
            with torch.cuda.stream(side):
                for dst, src in copies:
                    dst.copy_(src)
                for h in self._exchange(sends, recvs):
                    h.wait()
            main.wait_stream(side)
        else:
            for dst, src in copies:
                dst.copy_(src)
            for h in self._exchange(sends, recvs):
                h.wait()

        y_recv = k.routed_experts(recv, group_start, group_count)

        # return: partial outputs go back to the rows' owners, into buffers laid out like x_perm
        partials = [k.empty_rows(x_perm.shape[0], dim, y_recv) for _ in range(place.hidden_splits)]
        sends, recvs = [], []
        for j, e in enumerate(local):
            for s in range(self.world):
                src = y_recv[recv_start[j][s]: recv_start[j][s] + counts[s][e]]
                if s == rank:
                    partials[place.hidden_part(rank)][my_offset[e]: my_offset[e] + mine[e]].copy_(src)
                else:
                    sends.append((src, s))
        for e in range(self.n_experts):
            for q in place.owners(e):
                if q != rank:
                    dst = partials[place.hidden_part(q)][my_offset[e]: my_offset[e] + mine[e]]
                    recvs.append((dst, q))
        for h in self._exchange(sends, recvs):
            h.wait()

        out = k.combine(partials, row_map, w, y_shared)
        return out.view(shape)


# ====================================================================================================
# Peer-memory transport: dispatch and combine by the kernels themselves over NVLink, no host synchronisation
# ====================================================================================================
def _align(v: int, a: int = 256) -> int:
    return (v + a - 1) // a * a


class PeerBuffers:
    """One rank's receive buffer, result buffer, return buffers and flag block, plus every peer's as mapped in this
    process.

    ``create`` allocates them in symmetric memory (``torch.distributed._symmetric_memory``: one allocation per rank,
    exchanged and mapped at a rendezvous, done once per shape).  ``emulate`` builds the same structure for several
    ranks living on ONE device, which is how the addressing logic is tested without a second GPU.

    recv [cap_rows, dim]           rows other ranks routed to this rank's experts (activation dtype)
    y    [cap_rows, dim] bf16      this rank's expert outputs, read by the peers (pull variant of the return path)
    ret  [splits, ret_rows, dim]   expert outputs for this rank's own slots, written by the owners (push variant)"""

    FLAG_BYTES = 256

    def __init__(self, place: Placement, rank: int, cap_rows: int, ret_rows: int, dim: int, act_dtype: torch.dtype,
                 bases: List[int], mine: torch.Tensor, keep=None):
        from . import _native as N

        self.place, self.rank, self.cap_rows, self.ret_rows = place, rank, cap_rows, ret_rows
        self.dim, self.act_dtype = dim, act_dtype
        off_recv, off_y, off_ret, total = self.layout(cap_rows, ret_rows, dim, act_dtype, place.hidden_splits)
        es = 1 if act_dtype == torch.float8_e4m3fn else 2
        self._keep = (mine, keep)
        raw = mine.view(torch.uint8)
        self.flags = raw[: self.FLAG_BYTES].view(torch.int32)
        self.recv = raw[off_recv: off_recv + cap_rows * dim * es].view(act_dtype).view(cap_rows, dim)
        self.y = raw[off_y: off_y + cap_rows * dim * 2].view(torch.bfloat16).view(cap_rows, dim)
        ret_bytes = place.hidden_splits * ret_rows * dim * 2
        self.ret = raw[off_ret: off_ret + ret_bytes].view(torch.bfloat16).view(place.hidden_splits, ret_rows, dim)
        plan = N.PeerPlan()
        plan.world, plan.rank, plan.n_experts, plan.hidden_splits = place.world, rank, place.n_experts, place.hidden_splits
        for e in range(place.n_experts):
            owners = place.owners(e)
            plan.owner0[e] = owners[0]
            plan.owner1[e] = owners[1] if len(owners) > 1 else -1
        plan.cap_rows = cap_rows
        for r, base in enumerate(bases):
            plan.peer_flags[r] = base
            plan.peer_recv[r] = base + off_recv
            plan.peer_y[r] = base + off_y
        self.plan = plan
        self.epoch = 0       # steps taken on these buffers; the flags carry it, so it belongs to the buffers
        # where this rank's partial results go at every rank: that rank's return buffer of this rank's hidden part
        part_bytes = ret_rows * dim * 2
        self.peer_ret = [base + off_ret + place.hidden_part(rank) * part_bytes for base in bases]

    @classmethod
    def layout(cls, cap_rows: int, ret_rows: int, dim: int, act_dtype: torch.dtype, splits: int):
        es = 1 if act_dtype == torch.float8_e4m3fn else 2
        off_recv = cls.FLAG_BYTES
        off_y = off_recv + _align(cap_rows * dim * es)
        off_ret = off_y + _align(cap_rows * dim * 2)
        return off_recv, off_y, off_ret, off_ret + _align(splits * ret_rows * dim * 2)

    _shared = {}

    @classmethod
    def shared(cls, place: Placement, rank: int, cap_rows: int, ret_rows: int, dim: int, act_dtype: torch.dtype,
               device, group) -> "PeerBuffers":
        """Buffers for this shape, created once and then shared by every layer that asks for them (the layers of a
        model run one after the other on one stream, and the step order that makes single buffers safe holds across
        layers just as it does across calls of one layer)."""
        key = (id(group), place.world, place.n_experts, rank, cap_rows, ret_rows, dim, act_dtype, str(device))
        got = cls._shared.get(key)
        if got is None:
            got = cls.create(place, rank, cap_rows, ret_rows, dim, act_dtype, device, group)
            cls._shared[key] = got
        return got

    @classmethod
    def create(cls, place: Placement, rank: int, cap_rows: int, ret_rows: int, dim: int, act_dtype: torch.dtype,
               device, group):
        import os

        # plain peer mappings are all the kernels need; no NVLink multicast object is bound to the buffers
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        total = cls.layout(cap_rows, ret_rows, dim, act_dtype, place.hidden_splits)[3]
        buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        handle = symm_mem.rendezvous(buf, group)
        buf[: cls.FLAG_BYTES].zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)           # every rank's flags are zero before anyone raises one
        return cls(place, rank, cap_rows, ret_rows, dim, act_dtype, [int(p) for p in handle.buffer_ptrs], buf,
                   keep=handle)

    @classmethod
    def emulate(cls, place: Placement, cap_rows: int, ret_rows: int, dim: int, act_dtype: torch.dtype,
                device) -> List["PeerBuffers"]:
        total = cls.layout(cap_rows, ret_rows, dim, act_dtype, place.hidden_splits)[3]
        bufs = [torch.zeros(total, dtype=torch.uint8, device=device) for _ in range(place.world)]
        bases = [b.data_ptr() for b in bufs]
        return [cls(place, r, cap_rows, ret_rows, dim, act_dtype, bases, bufs[r], keep=bufs)
                for r in range(place.world)]


class PeerExpertParallelMoE:
    """``out = ep(x)``: the expert-parallel layer with the rows moved by the kernels over peer memory.

    Two streams, no host synchronisation.  Main: gate -> plan -> all-gather of the 4-bin histograms (NCCL, device to
    device) -> dispatch kernel (writes rows into the owners' receive buffers) -> "arrived" flag -> routed experts'
    first pass (every group waits inside the kernel for its own source's flag) -> second pass of routed and shared
    expert together (results written into the token owners' return buffers) -> "done" flag -> wait -> combine.
    Side: the shared expert's first pass, started after the gate, joined before the common second pass.
    The three ``phase_*`` methods are the step cut where ranks depend on one another, so a test can drive several
    ranks that live on one GPU in lock step.

    Buffer capacity is fixed by the first call: ``max_tokens`` if given, else the largest token count any rank brings to
    that call (one all-reduce inside the rendezvous that maps the buffers).  A later call with more tokens than that
    raises here for the caller's own return buffers and reports through the status word for a peer's receive buffer."""

    _tensors = {}       # scratch tensors by shape, shared by all layers (see _scratch)

    def __init__(self, module, group=None, *, max_tokens: Optional[int] = None, buffers: Optional[PeerBuffers] = None,
                 place: Optional[Placement] = None, rank: Optional[int] = None, push_results: Optional[bool] = None):
        import os

        from . import _native as N, moe_ops

        if push_results is None:
            push_results = os.environ.get("COMFY_B200_EP_RETURN", "push") != "pull"
        # push: the expert GEMM writes every result row into the return buffer of the rank that owns the token
        # while it computes; pull: results stay with the expert's rank and the combine kernel fetches them
        self.push = push_results
        self._side = None

        self.N, self.M = N, moe_ops
        self.lib = N.load()
        self.module = module
        self.group = group
        if buffers is None:
            self.group = group if group is not None else dist.group.WORLD
            rank, world = dist.get_rank(self.group), dist.get_world_size(self.group)
            place = Placement(world, len(module.experts))
        self.rank, self.place, self.world = rank, place, place.world
        self.n_experts = place.n_experts
        self.kernels = CudaKernels(module, place, rank, allow_fp8=True)
        self.fp8 = self.kernels.fp8
        # SMs kept free for the routing kernels while the shared expert's first pass runs beside them (0 = run them in
        # turn); COMFY_B200_EP_FRONT_SMS overrides.  16 let the dispatch end with that pass on 2 and 4 GPUs (188 against
        # 196 us at 8192 tokens); with a hidden split every routed row goes to two GPUs, and on 8 GPUs 32 (bf16) and 24
        # (fp8, half the bytes) measured better: 1.707 against 1.773 ms per step, 1.054 against 1.066.
        default_front = 16 if place.hidden_splits == 1 else (24 if self.fp8 else 32)
        self.front_sms = int(os.environ.get("COMFY_B200_EP_FRONT_SMS", default_front))
        self.buffers = buffers
        self.max_tokens = max_tokens
        self.last_counts = None
        self._state = None
        self._scratch_cache = {}
        self._h_ws = None
        # gate, plan, dispatch, 2 flags, 2 waits, shared GEMM x2, routed GEMM x2, combine (+ the shared expert's
        # input quantiser for fp8 when it runs beside the routing kernels)
        # (push: gate, plan, dispatch, flag, shared first pass, routed first pass, common second pass, flag, wait,
        # combine = 10)
        self.launches_per_step = (10 if self.push else 12) + (1 if (self.fp8 and self.front_sms > 0) else 0)

    def _ensure_buffers(self, n: int, dim: int, device):
        if self.buffers is not None:
            return
        cap_tokens = self.max_tokens
        if cap_tokens is None:
            # ranks may bring different token counts: size every rank's buffers for the largest
            largest = torch.tensor([n], dtype=torch.int64, device=device)
            dist.all_reduce(largest, op=dist.ReduceOp.MAX, group=self.group)
            cap_tokens = int(largest.item())
        # a token sends at most one slot to a given expert: world * tokens rows per local expert at most
        cap_rows = self.world * cap_tokens * min(2, self.place.experts_per_rank)
        act = torch.float8_e4m3fn if self.fp8 else torch.bfloat16
        self.buffers = PeerBuffers.shared(self.place, self.rank, cap_rows, 2 * cap_tokens, dim, act, device, self.group)

    # -- per-shape scratch: every tensor and every ctypes argument of a step, made once -----------------
    def _scratch(self, n: int, dim: int, device):
        key = (n, dim, str(device))
        sc = self._scratch_cache.get(key)
        if sc is not None:
            return sc
        import ctypes

        N, k, b = self.N, self.kernels, self.buffers
        if 2 * n > b.ret_rows:
            raise ValueError(f"{n} tokens do not fit the return buffers ({b.ret_rows} rows); pass max_tokens")
        e, world = self.n_experts, self.world
        i32 = dict(dtype=torch.int32, device=device)
        n_blocks = max((n + N.TOKENS_PER_BLOCK - 1) // N.TOKENS_PER_BLOCK, 1)
        n_groups = self.place.experts_per_rank * (world if self.push else 1)
        act = torch.float8_e4m3fn if self.fp8 else torch.bfloat16
        sc = type("Scratch", (), {})()
        # the tensors are shared by every layer of the same shape on these buffers (layers run one after the other on
        # one stream); what is per layer are the weight structs further down
        hidden = k.local[0].hidden
        tkey = (id(b), n, dim, e, world, n_groups, k.shared.hidden, hidden, self.fp8, str(device))
        t = PeerExpertParallelMoE._tensors.get(tkey)
        if t is None:
            t = dict(
                idx=torch.empty((n, 2), **i32), w=torch.empty((n, 2), dtype=torch.float32, device=device),
                block_counts=torch.empty((n_blocks, e), **i32), block_offsets=torch.empty((n_blocks, e), **i32),
                counts=torch.empty((e,), **i32), offsets=torch.empty((e + 1,), **i32),
                counts_all=torch.empty((world, e), **i32), row_map=torch.empty((n, 2), **i32),
                groups=torch.zeros((3, n_groups), **i32),              # start, count, output row shift
                status=torch.zeros((N.STATUS_WORDS,), **i32),           # device status, near-ties, e4m3 overflows
                x_q=torch.empty((n, dim), dtype=act, device=device) if self.fp8 else None,
                h_shared=torch.empty((max(n, 1), k.shared.hidden), dtype=act, device=device),
                y_shared=torch.empty((max(n, 1), dim), dtype=torch.bfloat16, device=device),
                h_ws=torch.empty((b.cap_rows, hidden), dtype=b.act_dtype, device=b.recv.device))
            PeerExpertParallelMoE._tensors[tkey] = t
            moe_ops_status = self.M._status_words
            moe_ops_status.add(t["status"])
        for name, value in t.items():
            setattr(sc, name, value)
        self._h_ws = t["h_ws"]
        P = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())                    # noqa: E731
        sc.p = {name: P(getattr(sc, name)) for name in ("idx", "w", "block_counts", "block_offsets", "counts",
                                                        "offsets", "counts_all", "row_map", "status", "x_q",
                                                        "h_shared", "y_shared")}
        sc.p["near"] = ctypes.c_void_p(sc.status.data_ptr() + 4)
        sc.p["overflow"] = ctypes.c_void_p(sc.status.data_ptr() + 8)
        sc.p["g_start"], sc.p["g_count"], sc.p["g_shift"] = (P(sc.groups[i]) for i in range(3))
        sc.p["recv"], sc.p["y"], sc.p["h_ws"] = P(b.recv), P(b.y), P(self._h_ws)
        sc.p["ret0"] = P(b.ret[0])
        sc.p["ret1"] = P(b.ret[1]) if self.place.hidden_splits == 2 else None
        sc.p["gate_w"] = P(k.gate_w)
        sc.gate_dtype = N.BF16 if k.gate_w.dtype == torch.bfloat16 else N.FP32
        sc.p["in13"] = P(k.local[0].scale_in13) if self.fp8 else None
        sc.p["in13_shared"] = P(k.shared.scale_in13) if self.fp8 else None
        # weights: the shared expert (all SMs, and on all but front_sms), the local experts once per group
        sc.shared = k.shared.struct()
        sc.shared_limited = k.shared.struct()
        sc.shared_limited.max_sms = max(self._sm_count(device) - self.front_sms, 2) if self.front_sms > 0 else 0
        per_group = [pack for pack in k.local for _ in range(world if self.push else 1)]
        sc.group_weights = (N.FfnWeights * len(per_group))()
        for i, pack in enumerate(per_group):
            pack.fill(sc.group_weights[i])
        sc.n_groups = len(per_group)
        sc.y_out = None
        if self.push:
            # group j * world + p holds local expert j's rows from source rank (rank + p) % world (own rows first)
            sources = [(self.rank + pos) % world for _ in k.local for pos in range(world)]
            sc.y_out = (ctypes.c_void_p * len(per_group))(*[int(b.peer_ret[s]) for s in sources])
            sc.group_source = (ctypes.c_int32 * len(per_group))(*sources)
            flags = b.flags.data_ptr() + 4 * N.EP_ARRIVED * N.MAX_RANKS
            # first pass over the routed groups: every group waits, inside the kernel, for its own source's rows only
            sc.opt_routed_p1 = N.GroupedOptions(passes=1, arrive_flags=flags, group_source=sc.group_source)
            # second pass: routed groups (results into the token owners' return buffers) and the shared expert together
            sc.opt_p2 = N.GroupedOptions(passes=2, y_out=sc.y_out, y_row_shift=sc.p["g_shift"].value,
                                         y_rows_cap=b.ret_rows)
            sc.opt_shared_p1 = N.GroupedOptions(passes=1)
        self._scratch_cache[key] = sc
        return sc

    @staticmethod
    def _stream_ptr():
        import ctypes

        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def _shared_expert(self, sc, x_in: torch.Tensor, n: int, dim: int, limited: bool):
        import ctypes

        N = self.N
        w = sc.shared_limited if limited else sc.shared
        N.check("comfy_moe_grouped_swiglu", self.lib.comfy_moe_grouped_swiglu(
            N.FP8_E4M3 if self.fp8 else N.BF16, 0, None, ctypes.byref(w), None, None, 0, n, dim, None, None, None,
            ctypes.c_void_p(x_in.data_ptr()), sc.p["h_shared"], sc.p["y_shared"], sc.p["status"], self._stream_ptr()))

    # -- the three phases of a step ---------------------------------------------------------------
    def phase_route(self, x2: torch.Tensor, counts_all: Optional[torch.Tensor] = None, want_xq: bool = True,
                    after_gate=None):
        """Gate, plan, histogram exchange, dispatch, "arrived" flag.  ``counts_all`` [world, E] replaces the
        collective in single-GPU emulation; ``after_gate`` is called once the gate kernel has been launched (the
        caller's hook for starting work on another stream that should not compete with the gate for SMs)."""
        import ctypes

        N, lib = self.N, self.lib
        n, dim = x2.shape
        self._ensure_buffers(n, dim, x2.device)
        b = self.buffers
        sc = self._scratch(n, dim, x2.device)
        p = sc.p
        b.epoch += 1
        sc.status[1:2].zero_()    # the near-tie counter only: the status word is sticky until check() has read it
        S = self._stream_ptr()
        px = ctypes.c_void_p(x2.data_ptr())
        if n > 0:
            N.check("comfy_moe_gate_topk", lib.comfy_moe_gate_topk(px, p["gate_w"], sc.gate_dtype, n, dim, self.n_experts,
                                                                  2, p["idx"], p["w"], p["block_counts"], p["near"], None,
                                                                  1e-6, S))
        if after_gate is not None:
            after_gate()
        N.check("comfy_moe_route_plan", lib.comfy_moe_route_plan(p["block_counts"], n, self.n_experts,
                                                                 p["block_offsets"], p["counts"], p["offsets"], S))
        if counts_all is not None:
            sc.counts_all.copy_(counts_all)
        else:
            dist.all_gather_into_tensor(sc.counts_all.view(-1), sc.counts, group=self.group)
        N.check("comfy_moe_ep_dispatch", lib.comfy_moe_ep_dispatch(
            b.plan, px, p["idx"], p["block_offsets"], p["counts_all"], n, dim, N.FP8_E4M3 if self.fp8 else N.BF16,
            p["in13"], p["x_q"] if want_xq else None, p["in13_shared"], p["row_map"], p["g_start"], p["g_count"],
            p["g_shift"] if self.push else None, p["status"], S))
        N.check("comfy_moe_ep_signal", lib.comfy_moe_ep_signal(b.plan, N.EP_ARRIVED, b.epoch, S))
        self._state = (sc, x2)

    def _shared_first_pass(self, sc, x_in: torch.Tensor, n: int, dim: int, limited: bool):
        """h_shared = silu(x w1) * (x w3) of the shared expert; its second pass rides in the routed groups' launch."""
        import ctypes

        N = self.N
        w = sc.shared_limited if limited else sc.shared
        N.check("comfy_moe_grouped_swiglu_ex", self.lib.comfy_moe_grouped_swiglu_ex(
            N.FP8_E4M3 if self.fp8 else N.BF16, 0, None, ctypes.byref(w), None, None, 0, n, dim, None, None, None,
            ctypes.c_void_p(x_in.data_ptr()), sc.p["h_shared"], sc.p["y_shared"], ctypes.byref(sc.opt_shared_p1),
            sc.p["status"], self._stream_ptr()))

    def phase_experts(self, shared_done: bool = False, join=None):
        """Push variant: first pass of the shared expert (unless the caller already ran it beside the routing kernels),
        first pass of the local routed experts, each group starting as soon as ITS source rank's rows have arrived (the
        wait sits inside the kernel), then one second pass over routed groups and shared expert together; ``join`` is
        called between the two passes (the caller's stream join with the shared expert's first pass).
        Pull variant: shared expert, wait for every rank's rows, routed experts into the local result buffer."""
        import ctypes

        N, lib, b = self.N, self.lib, self.buffers
        sc, x2 = self._state
        p = sc.p
        n, dim = x2.shape
        act = N.FP8_E4M3 if self.fp8 else N.BF16
        x_in = sc.x_q if self.fp8 else x2
        if self.push:
            if not shared_done and n > 0:
                self._shared_first_pass(sc, x_in, n, dim, limited=False)
            S = self._stream_ptr()
            sc.opt_routed_p1.arrive_epoch = b.epoch
            N.check("comfy_moe_grouped_swiglu_ex", lib.comfy_moe_grouped_swiglu_ex(
                act, sc.n_groups, sc.group_weights, None, p["g_start"], p["g_count"], b.cap_rows, 0, dim, p["recv"],
                p["h_ws"], p["ret0"], None, None, None, ctypes.byref(sc.opt_routed_p1), p["status"], S))
            if join is not None:
                join()
            S = self._stream_ptr()
            N.check("comfy_moe_grouped_swiglu_ex", lib.comfy_moe_grouped_swiglu_ex(
                act, sc.n_groups, sc.group_weights, ctypes.byref(sc.shared) if n > 0 else None, p["g_start"],
                p["g_count"], b.cap_rows, n, dim, p["recv"], p["h_ws"], p["ret0"],
                ctypes.c_void_p(x_in.data_ptr()) if n > 0 else None, p["h_shared"], p["y_shared"],
                ctypes.byref(sc.opt_p2), p["status"], S))
            N.check("comfy_moe_ep_signal", lib.comfy_moe_ep_signal(b.plan, N.EP_DONE, b.epoch, S))
            return
        if not shared_done and n > 0:
            self._shared_expert(sc, x_in, n, dim, limited=False)
        S = self._stream_ptr()
        N.check("comfy_moe_ep_wait", lib.comfy_moe_ep_wait(b.plan, N.EP_ARRIVED, b.epoch, p["status"], S))
        if False:
            pass
        else:
            N.check("comfy_moe_grouped_swiglu", lib.comfy_moe_grouped_swiglu(
                act, sc.n_groups, sc.group_weights, None, p["g_start"], p["g_count"], b.cap_rows, 0, dim, p["recv"],
                p["h_ws"], p["y"], None, None, None, p["status"], S))
        N.check("comfy_moe_ep_signal", lib.comfy_moe_ep_signal(b.plan, N.EP_DONE, b.epoch, S))

    def phase_combine(self) -> torch.Tensor:
        """After every rank's results are in place: the weighted combine (local for the push variant of the return
        path, reading the owners' result buffers for the pull variant)."""
        import ctypes

        N, lib, b = self.N, self.lib, self.buffers
        sc, x2 = self._state
        p = sc.p
        n, dim = x2.shape
        S = self._stream_ptr()
        N.check("comfy_moe_ep_wait", lib.comfy_moe_ep_wait(b.plan, N.EP_DONE, b.epoch, p["status"], S))
        out = torch.empty((n, dim), dtype=torch.bfloat16, device=x2.device)
        po = ctypes.c_void_p(out.data_ptr())
        if n == 0:
            pass
        elif not self.push:
            N.check("comfy_moe_ep_combine", lib.comfy_moe_ep_combine(b.plan, p["idx"], p["row_map"], p["w"],
                                                                    p["y_shared"], n, dim, po, S))
        elif p["ret1"] is not None:
            N.check("comfy_moe_combine_partials", lib.comfy_moe_combine_partials(p["ret0"], p["ret1"], p["row_map"],
                                                                                p["w"], p["y_shared"], n, dim, po, S))
        else:
            N.check("comfy_moe_combine", lib.comfy_moe_combine(p["ret0"], p["row_map"], p["w"], p["y_shared"], n, dim,
                                                              po, S))
        self.last_status = sc.status
        self._last_counts_dev = sc.counts_all
        return out

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        n, dim = x2.shape
        if self.front_sms <= 0 or n == 0:
            self.phase_route(x2)
            self.phase_experts()
            return self.phase_combine().view(shape)
        # The shared expert needs only x, so it runs on a side stream, on all but `front_sms` SMs, beside the routing
        # plan, the histogram all-gather and the dispatch kernel (NVLink-bound), which take the SMs left free; the
        # routed experts follow.  The gate goes first and alone: it is a memory-bound pass over all tokens that takes
        # 20 us on the whole GPU and over 100 us on sixteen SMs.  For fp8 the shared expert's input is quantised by a
        # kernel of its own (the dispatch kernel's quantised copy would come too late).
        self._ensure_buffers(n, dim, x2.device)
        sc = self._scratch(n, dim, x2.device)
        main = torch.cuda.current_stream()
        if self._side is None:
            self._side = torch.cuda.Stream(device=x2.device)
        side = self._side

        def start_shared_expert():
            side.wait_stream(main)              # behind the gate (and whatever produced x)
            with torch.cuda.stream(side):
                if self.fp8:
                    self.N.check("comfy_moe_quantize_e4m3", self.lib.comfy_moe_quantize_e4m3(
                        x2.data_ptr(), sc.p["in13_shared"], x2.numel(), sc.p["x_q"],
                        sc.p["overflow"], self._stream_ptr()))
                if self.push:
                    self._shared_first_pass(sc, sc.x_q if self.fp8 else x2, n, dim, limited=True)
                else:
                    self._shared_expert(sc, sc.x_q if self.fp8 else x2, n, dim, limited=True)

        self.phase_route(x2, want_xq=False, after_gate=start_shared_expert)
        if self.push:
            # the routed first pass queues up behind the local dispatch only: it takes SMs as the shared expert's
            # first pass lets go of them; the streams join before the common second pass
            self.phase_experts(shared_done=True, join=lambda: main.wait_stream(side))
        else:
            main.wait_stream(side)
            self.phase_experts(shared_done=True)
        return self.phase_combine().view(shape)

    def _sm_count(self, device) -> int:
        return torch.cuda.get_device_properties(device).multi_processor_count

    @property
    def last_counts_host(self) -> List[List[int]]:
        """[world][E] routed slots of the last call (one device-to-host copy; for reporting only)."""
        return self._last_counts_dev.tolist()

    def check(self) -> None:
        """Synchronises and raises if a flag wait ran out or the rows did not fit the receive buffers."""
        self.M.read_status(self.last_status)
