"""Two-GPU check of the pipelined Ulysses path: every rank's output shard must equal, byte for byte, the
same rows of a single-GPU call on the full tensors (the exchanges only move data). Skipped on one GPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, heads_per_step, exchange, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import spargeattn_b200 as S
    from spargeattn_b200 import ops
    from spargeattn_b200.sharding import close_peer_exchanges, ulysses_attention
    B, H, N, D = 1, 8, 4096, 128
    g = torch.Generator().manual_seed(5)
    walk = lambda: torch.cumsum(torch.randn(B, H, N, D, generator=g), dim=2) * 0.1
    q = (torch.randn(B, H, N, D, generator=g) + walk()).to(torch.bfloat16).cuda()
    k = (torch.randn(B, H, N, D, generator=g) + walk() + torch.randn(D, generator=g) * 3).to(torch.bfloat16).cuda()
    v = (torch.randn(B, H, N, D, generator=g) + walk()).to(torch.bfloat16).cuda()
    topk = torch.linspace(0.3, 0.7, H).cuda()
    ref = S.spas_sage2_attn_meansim_topk_cuda(q, k, v, topk=topk)
    n = N // world
    sl = slice(rank * n, (rank + 1) * n)
    for _ in range(2):
        o = ulysses_attention(q[:, :, sl].contiguous(), k[:, :, sl].contiguous(), v[:, :, sl].contiguous(),
                              topk=topk, heads_per_step=heads_per_step, exchange=exchange)
        torch.cuda.synchronize()
        ops.check_device_status()
        result[(rank, heads_per_step)] = result.get((rank, heads_per_step), True) and bool(torch.equal(o, ref[:, :, sl]))
    close_peer_exchanges()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["peer", "p2p", "a2a"])
@pytest.mark.parametrize("heads_per_step", [1, 4])
def test_ulysses_two_gpus_equals_single_gpu(heads_per_step, exchange):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mgr = mp.Manager()
    result = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), heads_per_step, exchange, result), nprocs=world, join=True)
    assert all(result[(r, heads_per_step)] for r in range(world)), dict(result)
