"""Host-buffer front end: q, k, v in (pinned) host memory, output back in host memory.

Every (batch, head) pair is independent end to end, so the call is cut into head chunks and run as a
three-stage pipeline on three CUDA streams -- upload chunk i+1, compute chunk i, download chunk i-1 --
which hides most of the PCIe time behind the kernels. Results are identical to one call on the whole
tensors. With `units` (the row sharding of sharding.partition_rows) a head may be owned in part: only its
owned query rows are uploaded, computed and downloaded, its keys and values in full. The reference has no counterpart (its callers hold q, k, v on the device already); this exists
for callers that stage activations in host memory and for the end-to-end measurement of bench.py.
"""
from typing import Optional

import torch

from . import core


class _Pipe:
    def __init__(self, device):
        self.up = torch.cuda.Stream(device)
        self.run = torch.cuda.Stream(device)
        self.down = torch.cuda.Stream(device)
        self.bufs = {}

    def buffers(self, key, shape, dtype, device, n):
        k = (key, tuple(shape), dtype)
        if k not in self.bufs:
            self.bufs[k] = [torch.empty(shape, dtype=dtype, device=device) for _ in range(n)]
        return self.bufs[k]


_pipes = {}
_unit_ranges = {}


def _ranges_on_device(units, dev):
    """int32 [len(units), 2] = (first query block, count) per unit, copied to the device once per unit list."""
    key = (dev.index, tuple(units))
    if key not in _unit_ranges:
        _unit_ranges[key] = torch.tensor([[a, n] for (_, _, a, n) in units], dtype=torch.int32).to(dev)
    return _unit_ranges[key]


def spas_sage2_attn_meansim_topk_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None,
                                      device=None, heads_per_chunk: int = 2, units=None, **kwargs) -> torch.Tensor:
    """q, k, v: CPU tensors [B, H, N, D] (HND), ideally pinned. Returns a CPU tensor of q's shape and 16-bit dtype.
    kwargs are those of spas_sage2_attn_meansim_topk_cuda; per-head knobs given as [H] tensors are sliced per chunk.

    units: a rank's share under row sharding, a list of (b, h, first_query_block, n_query_blocks) as
    sharding.partition_rows returns it; then q, k, v are [1, len(units), N, D] with head i belonging to unit i,
    only the owned rows of q are read and only the owned rows of the result are written."""
    assert not q.is_cuda and q.dim() == 4, "host front end takes CPU tensors [B,H,N,D]"
    assert kwargs.get("tensor_layout", "HND") == "HND" and not kwargs.get("return_sparsity", False)
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B, H, N, D = q.shape
    if units is not None:
        assert B == 1 and H == len(units), "with units, q/k/v hold one head per unit: [1, len(units), N, D]"
        from . import sharding
        ranges = _ranges_on_device(units, dev)
    odt = torch.float16 if q.dtype in (torch.float32, torch.float16) else torch.bfloat16
    if out is None:
        out = torch.empty(B, H, N, D, dtype=odt).pin_memory()
    pipe = _pipes.setdefault(dev.index, _Pipe(dev))
    hc = max(1, min(heads_per_chunk, H))
    chunks = [(b, h0, min(h0 + hc, H)) for b in range(B) for h0 in range(0, H, hc)]
    # Uploads run back to back, so the call ends one compute and one download after the last upload: the last
    # chunk goes head by head, which makes that tail as short as it can be.
    b, h0, h1 = chunks.pop()
    chunks += [(b, h, h + 1) for h in range(h0, h1)]
    nbuf = 3
    dq = pipe.buffers("q", (1, hc, N, D), q.dtype, dev, nbuf)
    dk = pipe.buffers("k", (1, hc, N, D), k.dtype, dev, nbuf)
    dv = pipe.buffers("v", (1, hc, N, D), v.dtype, dev, nbuf)
    do = pipe.buffers("o", (1, hc, N, D), odt, dev, nbuf)
    cur = torch.cuda.current_stream(dev)
    start = torch.cuda.Event()
    start.record(cur)
    for s in (pipe.up, pipe.run, pipe.down):
        s.wait_event(start)
    uploaded = [torch.cuda.Event() for _ in chunks]
    computed = [torch.cuda.Event() for _ in chunks]
    downloaded = [torch.cuda.Event() for _ in chunks]
    for i, (b, h0, h1) in enumerate(chunks):
        slot, n = i % nbuf, h1 - h0
        with torch.cuda.stream(pipe.up):
            if i >= nbuf:
                pipe.up.wait_event(computed[i - nbuf])          # the input slot is free once its chunk was computed
            if units is None:
                dq[slot][:, :n].copy_(q[b:b + 1, h0:h1], non_blocking=True)
            else:
                for j, (_, _, a, cnt) in enumerate(units[h0:h1]):      # owned query rows only
                    r0, r1 = a * 128, min((a + cnt) * 128, N)
                    dq[slot][0, j, r0:r1].copy_(q[0, h0 + j, r0:r1], non_blocking=True)
            dk[slot][:, :n].copy_(k[b:b + 1, h0:h1], non_blocking=True)
            dv[slot][:, :n].copy_(v[b:b + 1, h0:h1], non_blocking=True)
            uploaded[i].record(pipe.up)
        with torch.cuda.stream(pipe.run):
            pipe.run.wait_event(uploaded[i])
            if i >= nbuf:
                pipe.run.wait_event(downloaded[i - nbuf])       # the output slot is free once it was downloaded
            kw = dict(kwargs)
            for name, val in kwargs.items():
                if isinstance(val, torch.Tensor) and val.dim() == 1 and val.numel() == H:
                    kw[name] = val[h0:h1]
            if units is None:
                o = core.spas_sage2_attn_meansim_topk_cuda(dq[slot][:, :n], dk[slot][:, :n], dv[slot][:, :n], **kw)
            else:
                o = sharding.attention_units(dq[slot][:, :n], dk[slot][:, :n], dv[slot][:, :n], ranges[h0:h1].view(1, n, 2),
                                             max(c for (_, _, _, c) in units[h0:h1]), **kw)
            do[slot][:, :n].copy_(o)
            computed[i].record(pipe.run)
        with torch.cuda.stream(pipe.down):
            pipe.down.wait_event(computed[i])
            if units is None:
                out[b:b + 1, h0:h1].copy_(do[slot][:, :n], non_blocking=True)
            else:
                for j, (_, _, a, cnt) in enumerate(units[h0:h1]):
                    r0, r1 = a * 128, min((a + cnt) * 128, N)
                    out[0, h0 + j, r0:r1].copy_(do[slot][0, j, r0:r1], non_blocking=True)
            downloaded[i].record(pipe.down)
    cur.wait_event(downloaded[-1])
    cur.wait_event(computed[-1])
    return out
