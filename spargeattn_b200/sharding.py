"""Multi-GPU use of the sparse-attention path: one process per GPU, torch.distributed for the plumbing.

Two schemes, both outside the kernels:

* head sharding -- every (batch, head) pair is independent end to end (predictor, quantisers,
  attention), so ranks simply own disjoint sets of heads: no collective on the data path.
  `partition_heads` balances the sets by an estimate of each head's live blocks.
* Ulysses sequence parallelism -- each rank holds N/G tokens of all heads; one all-to-all turns that
  into all N tokens of H/G heads, the single-GPU path runs unchanged, and a second all-to-all
  returns the output to the sequence-sharded layout.  Pooling and quantisation happen after the
  exchange on full-length heads, so results are identical to a single-GPU run.  The received
  chunks land in this GPU's own memory before any kernel reads them.
"""
from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


def partition_heads(costs: Sequence[float], world_size: int) -> List[List[int]]:
    """Longest-processing-time assignment of head indices to ranks. costs[i] = expected work of head i."""
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    loads = [0.0] * world_size
    owned: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda j: (loads[j], j))
        owned[r].append(i)
        loads[r] += costs[i]
    return [sorted(o) for o in owned]


def _a2a(x: torch.Tensor, group) -> torch.Tensor:
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x, group=group)
    return out


def seq_to_head_shard(x: torch.Tensor, group=None) -> torch.Tensor:
    """[B, H, N/G, D] on every rank (rank r holds tokens r*N/G ...) -> [B, H/G, N, D] (rank r holds heads r*H/G ...)."""
    G = dist.get_world_size(group)
    B, H, n, D = x.shape
    assert H % G == 0, "number of heads must be divisible by the sequence-parallel size"
    # chunk g of the send buffer = my tokens of head group g
    send = x.reshape(B, G, H // G, n, D).permute(1, 0, 2, 3, 4).contiguous()
    recv = _a2a(send, group)                                  # chunk s = rank s's tokens of my head group
    return recv.permute(1, 2, 0, 3, 4).reshape(B, H // G, G * n, D).contiguous()


def head_to_seq_shard(x: torch.Tensor, group=None) -> torch.Tensor:
    """Inverse of seq_to_head_shard: [B, H/G, N, D] -> [B, H, N/G, D]."""
    G = dist.get_world_size(group)
    B, h, N, D = x.shape
    assert N % G == 0
    send = x.reshape(B, h, G, N // G, D).permute(2, 0, 1, 3, 4).contiguous()   # chunk s = token slice s of my heads
    recv = _a2a(send, group)                                                   # chunk g = my token slice of head group g
    return recv.permute(1, 0, 2, 3, 4).reshape(B, G * h, N // G, D).contiguous()


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, attention: Optional[Callable] = None,
                      group=None, **kwargs) -> torch.Tensor:
    """Sequence-parallel wrapper: q, k, v are [B, H, N/G, D] shards; returns the [B, H, N/G, D] output shard.
    `attention` defaults to spas_sage2_attn_meansim_topk_cuda; per-head knobs given as [H] tensors are sliced."""
    if attention is None:
        from .core import spas_sage2_attn_meansim_topk_cuda as attention
    G = dist.get_world_size(group)
    r = dist.get_rank(group)
    H = q.shape[1]
    hs = H // G
    for name, val in list(kwargs.items()):
        if isinstance(val, torch.Tensor) and val.dim() == 1 and val.numel() == H:
            kwargs[name] = val[r * hs:(r + 1) * hs]
    qh, kh, vh = (seq_to_head_shard(t, group) for t in (q, k, v))
    oh = attention(qh, kh, vh, **kwargs)
    return head_to_seq_shard(oh.contiguous(), group)
