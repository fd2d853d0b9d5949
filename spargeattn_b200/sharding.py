"""Multi-GPU use of the sparse-attention path: one process per GPU, torch.distributed for the plumbing.

Two schemes, both outside the kernels:

* head sharding -- every (batch, head) pair is independent end to end (predictor, quantisers,
  attention), so ranks simply own disjoint sets of heads: no collective on the data path.
  `partition_heads` balances the sets by an estimate of each head's live blocks.
* Ulysses sequence parallelism -- each rank holds N/G tokens of all heads; one all-to-all turns that
  into all N tokens of H/G heads, the single-GPU path runs unchanged, and a second all-to-all
  returns the output to the sequence-sharded layout.  Pooling and quantisation happen after the
  exchange on full-length heads, so results are identical to a single-GPU run.  The received
  chunks land in this GPU's own memory before any kernel reads them.  `ulysses_attention` does the
  exchanges head by head on a second stream so that they overlap the attention of the other heads.
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


def partition_rows(B: int, H: int, nq: int, world_size: int, row_cost: Optional[Sequence[float]] = None):
    """Row sharding of a [B, H] set of heads over `world_size` ranks with no collective: the (batch, head, query
    block) cells are laid end to end and cut into `world_size` contiguous runs of equal cost, so a rank owns
    whole heads plus at most two partial ones, each as a contiguous range of 128-row query blocks
    (12 heads on 8 ranks: one and a half heads each). Keys and values of a partially owned head are needed by
    both owners; they prepare them independently.

    row_cost[i]: expected work of query block i (its number of live key blocks); default: equal.
    Returns, per rank, a list of units (b, h, first_query_block, n_query_blocks); every cell appears once."""
    cost = [1.0] * nq if row_cost is None else [float(c) for c in row_cost]
    assert len(cost) == nq and world_size >= 1
    per_head = sum(cost)
    total = per_head * B * H
    units: List[List[tuple]] = [[] for _ in range(world_size)]
    acc, r = 0.0, 0
    for bh in range(B * H):
        start = 0
        for i in range(nq):
            # cell (bh, i) goes to the rank in whose share its midpoint falls
            mid = acc + cost[i] / 2.0
            owner = min(world_size - 1, int(mid * world_size / total)) if total > 0 else 0
            if owner != r:
                if i > start:
                    units[r].append((bh // H, bh % H, start, i - start))
                start, r = i, owner
            acc += cost[i]
        units[r].append((bh // H, bh % H, start, nq - start))
    return units


def attention_units(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_block_ranges: torch.Tensor,
                    q_blocks_max: Optional[int] = None, **kwargs) -> torch.Tensor:
    """spas_sage2_attn_meansim_topk_cuda on the heads a rank touches, computing only each head's owned query
    blocks. q, k, v: [B, Hloc, N, D] (HND); q_block_ranges: int32 [B, Hloc, 2] = (first block, count), on the
    device or the host; q_blocks_max: the largest count (pass it with device-resident ranges, otherwise it is
    read back from them, which synchronises). Rows outside the ranges are not written. kwargs: topk, is_causal,
    simthreshd1, pvthreshd, attention_sink, scale, smooth_k (as the public function)."""
    from . import core
    assert kwargs.get("tensor_layout", "HND") == "HND" and not kwargs.get("return_sparsity", False)
    ranges = q_block_ranges.to(device=q.device, dtype=torch.int32).contiguous()
    qmax = int(q_block_ranges[..., 1].max()) if q_blocks_max is None else int(q_blocks_max)
    return core._meansim_attention(q, k, v, kwargs.get("is_causal", False), kwargs.get("scale"), kwargs.get("smooth_k", True),
                                   kwargs.get("simthreshd1", -0.1), kwargs.get("cdfthreshd"), kwargs.get("topk", 0.5),
                                   kwargs.get("pvthreshd", 50), kwargs.get("attention_sink", False), "HND", False,
                                   bool(kwargs.get("is_causal", False)) and core.SAGE2_TOKEN_LEVEL_CAUSAL,
                                   q_block_ranges=ranges, q_blocks_max=qmax)


class StepMonitor:
    """Host-side liveness check for multi-rank loops, run between steps (no kernel or collective in flight).

    Before a step every rank announces it in a key-value store (any torch.distributed store: the TCPStore the
    job was launched with, or one made for the purpose) and then waits, with a limit, until every rank has
    announced it. A rank that raised, exited or hangs does not announce: the others get a RuntimeError that
    names it *before* they enqueue a collective that could never complete, and can tear down in order. The
    reference has no counterpart (it runs single-GPU)."""

    def __init__(self, store, rank: int, world_size: int, timeout_s: float = 30.0, prefix: str = "sparge/step"):
        self.store, self.rank, self.world, self.timeout, self.prefix = store, rank, world_size, timeout_s, prefix

    def enter(self, step: int) -> None:
        import time
        # counters only grow: add() returns the current value without blocking, so a missing peer cannot stall us
        self.store.add(f"{self.prefix}/{self.rank}", 1)
        deadline = time.monotonic() + self.timeout
        want = step + 1
        missing = list(range(self.world))
        while missing:
            missing = [r for r in missing if self.store.add(f"{self.prefix}/{r}", 0) < want]
            if not missing:
                return
            if time.monotonic() > deadline:
                raise RuntimeError(f"rank(s) {missing} did not reach step {step} within {self.timeout:g} s "
                                   f"(reported by rank {self.rank}); no collective of that step has been started")
            time.sleep(0.005)


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


def _exchange(send_chunks, recv_chunks, group) -> None:
    """Chunk g of `send_chunks` goes to rank g of the group; chunk s of `recv_chunks` comes from rank s.
    All chunks are contiguous tensors of one size: nothing is staged, the data lands where it is used."""
    G = dist.get_world_size(group)
    r = dist.get_rank(group)
    recv_chunks[r].copy_(send_chunks[r])
    ops = []
    for g in range(G):
        if g == r:
            continue
        peer = dist.get_global_rank(group, g) if group is not None else g
        ops.append(dist.P2POp(dist.isend, send_chunks[g], peer, group))
        ops.append(dist.P2POp(dist.irecv, recv_chunks[g], peer, group))
    for req in dist.batch_isend_irecv(ops) if ops else []:
        req.wait()


class PeerExchange:
    """Per-rank exchange buffers that the other ranks of a single-node group map into their address space
    (CUDA IPC through the C ABI's sparge_peer_* calls), so that the sequence<->head exchanges become
    copy-engine transfers over NVLink: ranks pull their heads' token slices out of the peers' input buffers
    and push output slices into the peers' output buffers. No SM is used by the transfers, so they overlap
    the attention kernels; the only collectives left are two one-element all-reduces per call that order
    the copies across ranks (everyone has staged / everyone has pushed).

    Collective: every rank of `group` must construct it, call `ensure` with the same sizes, and `close`."""

    def __init__(self, group=None):
        import ctypes
        from . import _cabi
        self._ct, self._lib, self._check = ctypes, _cabi.lib, _cabi.check
        self.group = group
        self.G = dist.get_world_size(group)
        self.r = dist.get_rank(group)
        self.in_bytes = self.out_bytes = 0
        self.local_in = self.local_out = None
        self.peer_in = {}
        self.peer_out = {}
        self.flag = None

    def _alloc(self, nbytes):
        ptr, handle = self._ct.c_void_p(), self._ct.create_string_buffer(64)
        self._check(self._lib.sparge_peer_alloc(nbytes, self._ct.byref(ptr), handle), "sparge_peer_alloc")
        return ptr.value, handle.raw

    def _open_all(self, handle):
        handles = [None] * self.G
        dist.all_gather_object(handles, handle, group=self.group)
        mapped = {}
        for s in range(self.G):
            if s != self.r:
                p = self._ct.c_void_p()
                self._check(self._lib.sparge_peer_open(handles[s], self._ct.byref(p)), "sparge_peer_open")
                mapped[s] = p.value
        return mapped

    def ensure(self, in_bytes: int, out_bytes: int, device) -> None:
        if in_bytes <= self.in_bytes and out_bytes <= self.out_bytes:
            return
        self.close()
        self.flag = torch.zeros(1, dtype=torch.int32, device=device)
        self.local_in, h_in = self._alloc(in_bytes)
        self.local_out, h_out = self._alloc(out_bytes)
        self.peer_in = self._open_all(h_in)
        self.peer_out = self._open_all(h_out)
        self.in_bytes, self.out_bytes = in_bytes, out_bytes

    def fence(self) -> None:
        """Stream-ordered rendezvous of all ranks on the current stream."""
        dist.all_reduce(self.flag, group=self.group)

    def copy(self, dst, src, nbytes, stream) -> None:
        self._check(self._lib.sparge_copy_async(dst, src, nbytes, stream.cuda_stream), "sparge_copy_async")

    def copy2d(self, dst, dpitch, src, spitch, width, height, stream) -> None:
        self._check(self._lib.sparge_copy2d_async(dst, dpitch, src, spitch, width, height, stream.cuda_stream),
                    "sparge_copy2d_async")

    def close(self) -> None:
        """Unmap the peers' buffers, wait until every rank has done so, then free this rank's buffers."""
        if self.local_in is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for table in (self.peer_in, self.peer_out):
            for p in table.values():
                self._lib.sparge_peer_close(p)
            table.clear()
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._lib.sparge_peer_free(self.local_in)
        self._lib.sparge_peer_free(self.local_out)
        self.local_in = self.local_out = None
        self.in_bytes = self.out_bytes = 0


_PEER_EXCHANGES = {}


def peer_exchange(group=None) -> PeerExchange:
    """The process-wide PeerExchange of a group (created on first use by every rank)."""
    if group not in _PEER_EXCHANGES:            # keyed by the group object itself (None = default group)
        _PEER_EXCHANGES[group] = PeerExchange(group)
    return _PEER_EXCHANGES[group]


def close_peer_exchanges() -> None:
    """Collective tear-down of every PeerExchange; call before destroying the process group."""
    for ex in _PEER_EXCHANGES.values():
        ex.close()
    _PEER_EXCHANGES.clear()


def auto_heads_per_step(B: int, N: int, heads: int, device) -> int:
    """Smallest step whose attention launch still fills the GPU for about a dozen waves of CTAs (two per SM):
    shorter launches lose more to their partial last wave than the extra overlap gains."""
    device = torch.device(device)
    slots = 2 * torch.cuda.get_device_properties(device).multi_processor_count if device.type == "cuda" else 1
    per_head = B * ((N + 127) // 128)
    return next((c for c in range(1, heads + 1) if c * per_head >= 12 * slots), heads)


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, attention: Optional[Callable] = None,
                      group=None, heads_per_step: Optional[int] = None, exchange: str = "auto", **kwargs) -> torch.Tensor:
    """Sequence-parallel wrapper: q, k, v are [B, H, N/G, D] shards; returns the [B, H, N/G, D] output shard.
    `attention` defaults to spas_sage2_attn_meansim_topk_cuda; per-head knobs given as [H] tensors are sliced.

    The H/G heads a rank owns are processed `heads_per_step` at a time (None: chosen from the problem size). On CUDA the exchanges run on a second
    stream: while the attention of one step runs, the inputs of the next step arrive and the output of the
    previous step leaves, so only the first input exchange and the last output exchange are exposed. Every
    exchange writes straight into its final place ([N, D] per head going in, the caller-layout shard coming
    back); no permuted staging copies are made.

    `exchange`: "peer" moves the data with copy-engine transfers between IPC-mapped buffers (PeerExchange; one
    node, NCCL group, CUDA tensors), "p2p" with batched send/recv of the process group (any backend), "a2a"
    with one all_to_all_single per tensor and no pipelining; "auto" picks "peer" (2 ranks) or "a2a" (more) for
    CUDA tensors on an NCCL group and "p2p" otherwise."""
    if attention is None:
        from .core import spas_sage2_attn_meansim_topk_cuda as attention
    # checked before the first collective: an exception later would leave the other ranks waiting in an exchange
    if kwargs.get("return_sparsity", False):
        raise ValueError("ulysses_attention returns the output shard only: return_sparsity is not supported")
    if kwargs.get("tensor_layout", "HND") != "HND":
        raise ValueError("ulysses_attention exchanges [B, H, N/G, D] shards: tensor_layout must be 'HND'")
    G = dist.get_world_size(group)
    r = dist.get_rank(group)
    B, H, n, D = q.shape
    assert H % G == 0, "number of heads must be divisible by the sequence-parallel size"
    hs = H // G
    if heads_per_step is None:
        heads_per_step = auto_heads_per_step(B, G * n, hs, q.device)
    step = max(1, min(int(heads_per_step), hs))
    q, k, v = (t if t.is_contiguous() else t.contiguous() for t in (q, k, v))
    out = torch.empty_like(q)
    cuda = q.is_cuda
    if exchange == "auto":
        # Two ranks hold enough heads each to pipeline the exchange behind the attention of other heads, which
        # the copy-engine peer transfers do without taking SMs; with more ranks and few heads per rank there is
        # nothing to pipeline and one all-to-all per tensor has the least overhead.
        if cuda and dist.get_backend(group) == "nccl":
            exchange = "peer" if G == 2 else "a2a"
        else:
            exchange = "p2p"
    if exchange == "a2a":                          # one all-to-all per tensor, nothing pipelined
        for name, val in list(kwargs.items()):
            if isinstance(val, torch.Tensor) and val.dim() == 1 and val.numel() == H:
                kwargs[name] = val[r * hs:(r + 1) * hs]
        qh, kh, vh = (seq_to_head_shard(t, group) for t in (q, k, v))
        return head_to_seq_shard(attention(qh, kh, vh, **kwargs).contiguous(), group)
    if exchange not in ("peer", "p2p"):
        raise ValueError("exchange must be 'auto', 'peer', 'p2p' or 'a2a'")
    if exchange == "peer" and not cuda:
        raise ValueError("exchange='peer' needs CUDA tensors")
    main = torch.cuda.current_stream(q.device) if cuda else None
    steps = [(j0, min(j0 + step, hs)) for j0 in range(0, hs, step)]
    full = [tuple(torch.empty(B, j1 - j0, G * n, D, dtype=t.dtype, device=t.device) for t in (q, k, v))
            for (j0, j1) in steps]
    outs = [None] * len(steps)
    ev_in = [torch.cuda.Event() if cuda else None for _ in steps]

    def exchange_in(i):
        j0, j1 = steps[i]
        for src, dst in zip((q, k, v), full[i]):
            for b in range(B):
                for j in range(j0, j1):
                    _exchange([src[b, g * hs + j] for g in range(G)],
                              [dst[b, j - j0, s * n:(s + 1) * n] for s in range(G)], group)

    def exchange_out(i):
        j0, j1 = steps[i]
        o = outs[i]
        for b in range(B):
            for j in range(j0, j1):
                _exchange([o[b, j - j0, s * n:(s + 1) * n] for s in range(G)],
                          [out[b, g * hs + j] for g in range(G)], group)

    if exchange == "peer":
        px = peer_exchange(group)
        es = q.element_size()
        shard = B * H * n * D * es                     # one tensor's shard on one rank
        px.ensure(3 * shard, shard, q.device)
        row, full_row = n * D * es, G * n * D * es     # one head's token slice / one full-length head

        # Transfers with different peers go to different streams, so that several copy engines and all the
        # NVLink ports work at once; `stream` (the exchange stream) forks to the lanes and joins them again.
        lanes = _side_streams(q.device)[3:]

        def fork(stream):
            ev = torch.cuda.Event()
            ev.record(stream)
            for lane in lanes:
                lane.wait_event(ev)

        def join(stream):
            for lane in lanes:
                ev = torch.cuda.Event()
                ev.record(lane)
                stream.wait_event(ev)

        def lane_of(s_, stream):
            return stream if s_ == r else lanes[s_ % len(lanes)]

        def exchange_in(i, stream):                    # noqa: F811 - replaces the send/recv version
            j0, j1 = steps[i]
            fork(stream)
            for t, (src, dst) in enumerate(zip((q, k, v), full[i])):
                for b in range(B):
                    head0 = ((b * H) + r * hs + j0) * row
                    for s_ in range(G):
                        base = src.data_ptr() if s_ == r else px.peer_in[s_] + t * shard
                        px.copy2d(dst.data_ptr() + b * (j1 - j0) * full_row + s_ * row, full_row,
                                  base + head0, row, row, j1 - j0, lane_of(s_, stream))
            join(stream)

        def stage(i, stream):
            """Copy the slices that the peers will pull for their step i into my exchange buffer."""
            if i >= len(steps):
                return
            j0, j1 = steps[i]
            for t, src in enumerate((q, k, v)):
                if len(steps) == 1:                    # everything at once: one copy per tensor
                    px.copy(px.local_in + t * shard, src.data_ptr(), shard, stream)
                    continue
                for b in range(B):
                    for s_ in range(G):
                        if s_ != r:
                            ofs = ((b * H) + s_ * hs + j0) * row
                            px.copy(px.local_in + t * shard + ofs, src.data_ptr() + ofs, (j1 - j0) * row, stream)

        def exchange_out(i, stream):                   # noqa: F811
            j0, j1 = steps[i]
            o = outs[i]
            fork(stream)
            for b in range(B):
                head0 = ((b * H) + r * hs + j0) * row
                for s_ in range(G):
                    base = px.local_out if s_ == r else px.peer_out[s_]
                    px.copy2d(base + head0, row, o.data_ptr() + b * (j1 - j0) * full_row + s_ * row, full_row,
                              row, j1 - j0, lane_of(s_, stream))
            join(stream)
    else:
        px = None
        _in, _out = exchange_in, exchange_out
        exchange_in = lambda i, stream=None: _in(i)
        exchange_out = lambda i, stream=None: _out(i)

    def head_kwargs(i):
        j0, j1 = steps[i]
        kw = dict(kwargs)
        for name, val in kwargs.items():
            if isinstance(val, torch.Tensor) and val.dim() == 1 and val.numel() == H:
                kw[name] = val[r * hs + j0:r * hs + j1]
        return kw

    if not cuda:
        for i in range(len(steps)):
            exchange_in(i)
            outs[i] = attention(*full[i], **head_kwargs(i)).contiguous()
            exchange_out(i)
        return out

    # Streams: `comm` carries every exchange; the attention of step i runs on compute stream i % 2, so the
    # last CTAs of one step and the first CTAs of the next share the SMs instead of leaving them idle.
    work = _side_streams(q.device)
    comm, compute = work[0], work[1:3]
    comm.wait_stream(main)                      # inputs and the buffers above are ready
    for cs in compute:
        cs.wait_stream(main)
    with torch.cuda.stream(comm):
        if px is not None:
            # stage the slices of the first step where the peers can read them; nobody pulls a slice before
            # every rank has staged it (one-element all-reduce = stream-ordered rendezvous)
            stage(0, comm)
            px.fence()
        exchange_in(0, comm)
        ev_in[0].record(comm)
        if px is not None and len(steps) > 1:
            for i in range(1, len(steps)):
                stage(i, comm)
            px.fence()
        if len(steps) > 1:
            exchange_in(1, comm)
            ev_in[1].record(comm)
    for i in range(len(steps)):
        cs = compute[i % len(compute)]
        with torch.cuda.stream(cs):
            cs.wait_event(ev_in[i])
            o = attention(*full[i], **head_kwargs(i))
            outs[i] = o if o.is_contiguous() else o.contiguous()
            outs[i].record_stream(comm)
            done = torch.cuda.Event()
            done.record(cs)
        with torch.cuda.stream(comm):
            comm.wait_event(done)
            exchange_out(i, comm)
            if i + 2 < len(steps):
                exchange_in(i + 2, comm)
                ev_in[i + 2].record(comm)
    if px is not None:
        with torch.cuda.stream(comm):
            px.fence()                                 # every rank's pushes have landed
            px.copy(out.data_ptr(), px.local_out, shard, comm)
    main.wait_stream(comm)
    for cs in compute:
        main.wait_stream(cs)
    return out


_SIDE_STREAMS = {}


def _side_streams(device):
    """One exchange stream, two compute streams and four transfer lanes per device, created once."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = [torch.cuda.Stream(device=key, priority=-1)] + [torch.cuda.Stream(device=key) for _ in range(6)]
    return _SIDE_STREAMS[key]
