"""CPU tests (gloo, world_size 2) of the multi-GPU host logic: head partitioning and the Ulysses
all-to-all pair around a stand-in attention function."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from spargeattn_b200.sharding import partition_heads


def test_partition_heads_balances_and_covers():
    costs = [5, 1, 1, 1, 4, 2, 2, 3, 3, 2, 6, 1]
    for world in (1, 2, 4, 8):
        parts = partition_heads(costs, world)
        assert sorted(i for p in parts for i in p) == list(range(len(costs)))
        loads = [sum(costs[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(costs)
    assert partition_heads([1.0] * 12, 8) == [[0, 8], [1, 9], [2, 10], [3, 11], [4], [5], [6], [7]]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ref_attention(q, k, v, topk=None, **kw):
    o = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float())
    if topk is not None:                       # per-head knob: make the result depend on it
        o = o * topk.view(1, -1, 1, 1)
    return o.to(q.dtype)


def _worker(rank, world, port, q, k, v, topk, out_dict):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from spargeattn_b200.sharding import head_to_seq_shard, seq_to_head_shard, ulysses_attention
    n = q.shape[2] // world
    sl = slice(rank * n, (rank + 1) * n)
    qs, ks, vs = q[:, :, sl].contiguous(), k[:, :, sl].contiguous(), v[:, :, sl].contiguous()
    # round trip of the two exchanges is the identity
    assert torch.equal(head_to_seq_shard(seq_to_head_shard(qs)), qs)
    # after the first exchange a rank holds full-length heads
    qh = seq_to_head_shard(qs)
    hs = q.shape[1] // world
    assert torch.equal(qh, q[:, rank * hs:(rank + 1) * hs])
    o = ulysses_attention(qs, ks, vs, attention=_ref_attention, topk=topk)
    o2 = ulysses_attention(qs, ks, vs, attention=_ref_attention, topk=topk, heads_per_step=2)
    assert torch.equal(o, o2)
    o3 = ulysses_attention(qs, ks, vs, attention=_ref_attention, topk=topk, exchange="a2a")
    assert torch.allclose(o, o3, atol=1e-6)
    out_dict[rank] = o
    dist.barrier()
    dist.destroy_process_group()


def test_ulysses_matches_single_process():
    world = 2
    g = torch.Generator().manual_seed(0)
    B, H, N, D = 2, 4, 64, 16
    q, k, v = (torch.randn(B, H, N, D, generator=g) for _ in range(3))
    topk = torch.tensor([0.5, 1.0, 1.5, 2.0])
    ref = _ref_attention(q, k, v, topk=topk)
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), q, k, v, topk, out), nprocs=world, join=True)
    n = N // world
    for r in range(world):
        assert torch.allclose(out[r], ref[:, :, r * n:(r + 1) * n], atol=1e-6)
