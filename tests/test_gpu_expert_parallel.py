"""Expert-parallel layer on real GPUs (needs at least two B200s on the node; skipped otherwise).

Child processes, one per GPU, NCCL.  Every rank compares its expert-parallel output with the single-GPU kernels run
on the same tokens: without a hidden split the two must agree bit for bit (rows are independent and see the same
arithmetic wherever they are computed).
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


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, tokens, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from comfyui_b200 import ops
        from comfyui_b200.expert_parallel import ExpertParallelMoE
        from comfyui_b200.ldm.hidream.model import MOEFeedForwardSwiGLU

        layer = {k: v.bfloat16().to(dev) for k, v in O.make_layer(DIM, HIDDEN_DIM, E, seed=0).items()}
        module = MOEFeedForwardSwiGLU(DIM, HIDDEN_DIM, E, 2, dtype=torch.bfloat16, device=dev,
                                      operations=ops.disable_weight_init).eval()
        module.load_state_dict(layer, strict=True)
        n = tokens[rank]
        x = O.make_input(n, DIM, seed=100 + rank).bfloat16().to(dev).view(1, n, DIM)
        ep = ExpertParallelMoE(module)
        with torch.inference_mode():
            out = ep(x)
            again = ep(x)
            single = module(x)
        torch.cuda.synchronize()
        torch.save({"out": out.cpu(), "again": again.cpu(), "single": single.cpu(), "counts": ep.last_counts},
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_on_gpus(tmp_path, cuda_device, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    tokens = [1000, 700, 333, 1, 512, 129, 64, 2048][:world]
    mp.spawn(_worker, args=(world, _free_port(), tokens, str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        r = torch.load(tmp_path / f"rank{rank}.pt")
        assert torch.equal(r["out"], r["again"])
        if world <= E:
            assert torch.equal(r["out"], r["single"]), f"rank {rank}"
        else:
            torch.testing.assert_close(r["out"].float(), r["single"].float(), rtol=2e-2, atol=2e-2)
        assert [sum(c) for c in r["counts"]] == [2 * t for t in tokens]
