"""CPU tests (gloo, world_size 2) of the multi-GPU host logic: head partitioning and the Ulysses
all-to-all pair around a stand-in attention function."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import pytest

from spargeattn_b200.sharding import partition_heads, partition_rows


def test_partition_heads_balances_and_covers():
    costs = [5, 1, 1, 1, 4, 2, 2, 3, 3, 2, 6, 1]
    for world in (1, 2, 4, 8):
        parts = partition_heads(costs, world)
        assert sorted(i for p in parts for i in p) == list(range(len(costs)))
        loads = [sum(costs[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(costs)
    assert partition_heads([1.0] * 12, 8) == [[0, 8], [1, 9], [2, 10], [3, 11], [4], [5], [6], [7]]


@pytest.mark.parametrize("B,H,nq,world", [(1, 12, 256, 1), (1, 12, 256, 2), (1, 12, 256, 4), (1, 12, 256, 8), (2, 30, 139, 8),
                                          (1, 32, 256, 8), (1, 24, 931, 8), (1, 12, 256, 5), (1, 3, 7, 4), (1, 1, 1, 3)])
def test_partition_rows_covers_every_cell_once_and_balances(B, H, nq, world):
    """Row sharding: every (batch, head, query block) cell belongs to exactly one rank, each rank's share of a
    head is one contiguous range, and no rank has more than one cell above the even share."""
    units = partition_rows(B, H, nq, world)
    assert len(units) == world
    seen = set()
    for us in units:
        for (b, h, first, count) in us:
            assert 0 <= b < B and 0 <= h < H and count > 0 and 0 <= first and first + count <= nq
            for i in range(first, first + count):
                assert (b, h, i) not in seen
                seen.add((b, h, i))
        heads = [(b, h) for (b, h, _, _) in us]
        assert len(heads) == len(set(heads))                       # one range per head and rank
    assert len(seen) == B * H * nq
    loads = [sum(c for (_, _, _, c) in us) for us in units]
    assert max(loads) - min(loads) <= 1 or B * H * nq < world
    # twelve heads on eight ranks: one and a half heads each, the split heads cut in the middle
    if (B, H, nq, world) == (1, 12, 256, 8):
        assert units[0] == [(0, 0, 0, 256), (0, 1, 0, 128)] and units[1] == [(0, 1, 128, 128), (0, 2, 0, 256)]


def test_partition_rows_weighted_for_causal_rows():
    """Causal rows grow with the row index: equal cost means late rows are spread thinner than early ones."""
    nq = 256
    cost = [min(256, 2 * (i + 1)) for i in range(nq)]
    units = partition_rows(1, 12, nq, 8, cost)
    loads = [sum(sum(cost[a:a + n]) for (_, _, a, n) in us) for us in units]
    assert sum(loads) == 12 * sum(cost)
    assert max(loads) - min(loads) <= max(cost)
    assert units[0][1][3] > 128                                    # the first half-head takes more than half the rows


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


def _leaving_worker(rank, world, port, port2, q, k, v, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from spargeattn_b200.sharding import StepMonitor, ulysses_attention
    store = dist.TCPStore("127.0.0.1", port2, world, is_master=(rank == 0), wait_for_workers=False)
    mon = StepMonitor(store, rank, world, timeout_s=2.0)
    n = q.shape[2] // world
    sl = slice(rank * n, (rank + 1) * n)
    qs, ks, vs = q[:, :, sl].contiguous(), k[:, :, sl].contiguous(), v[:, :, sl].contiguous()
    import time
    mon.enter(0)
    ulysses_attention(qs, ks, vs, attention=_ref_attention)          # step 0: everyone is there
    if rank == 1:                                                    # leaves between two steps, nothing in flight
        result[rank] = "left"
        time.sleep(4.0)                                              # keep its sockets open: the others must not rely on a reset
        return
    t0 = time.monotonic()
    try:
        mon.enter(1)
        ulysses_attention(qs, ks, vs, attention=_ref_attention)
        result[rank] = "no error"
    except RuntimeError as e:
        result[rank] = (str(e), time.monotonic() - t0)


def test_rank_leaving_between_steps_is_named_before_the_next_collective():
    """Failure detection on the host: a rank that stops between two steps is reported by name within the monitor's
    limit, and the survivor has not entered the exchange it would have blocked in."""
    world = 2
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(1, 4, 32, 16, generator=g) for _ in range(3))
    mgr = mp.Manager()
    res = mgr.dict()
    mp.spawn(_leaving_worker, args=(world, _free_port(), _free_port(), q, k, v, res), nprocs=world, join=True)
    assert res[1] == "left"
    msg, waited = res[0]
    assert "rank(s) [1] did not reach step 1" in msg and "reported by rank 0" in msg
    assert 1.5 < waited < 4.0


def test_ulysses_rejects_unsupported_arguments_before_any_exchange():
    from spargeattn_b200.sharding import ulysses_attention
    x = torch.zeros(1, 2, 4, 8)
    with pytest.raises(ValueError):
        ulysses_attention(x, x, x, attention=_ref_attention, return_sparsity=True)
    with pytest.raises(ValueError):
        ulysses_attention(x, x, x, attention=_ref_attention, tensor_layout="NHD")
