"""Host-buffer front end: q, k, v in (pinned) host memory, output back in host memory.

Every (batch, head) pair is independent end to end, so the call is cut into head chunks and run as a
three-stage pipeline on three CUDA streams -- upload chunk i+1, compute chunk i, download chunk i-1 --
which hides most of the PCIe time behind the kernels. Results are identical to one call on the whole
tensors. The reference has no counterpart (its callers hold q, k, v on the device already); this exists
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


def spas_sage2_attn_meansim_topk_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None,
                                      device=None, heads_per_chunk: int = 2, **kwargs) -> torch.Tensor:
    """q, k, v: CPU tensors [B, H, N, D] (HND), ideally pinned. Returns a CPU tensor of q's shape and 16-bit dtype.
    kwargs are those of spas_sage2_attn_meansim_topk_cuda; per-head knobs given as [H] tensors are sliced per chunk."""
    assert not q.is_cuda and q.dim() == 4, "host front end takes CPU tensors [B,H,N,D]"
    assert kwargs.get("tensor_layout", "HND") == "HND" and not kwargs.get("return_sparsity", False)
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B, H, N, D = q.shape
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
            dq[slot][:, :n].copy_(q[b:b + 1, h0:h1], non_blocking=True)
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
            o = core.spas_sage2_attn_meansim_topk_cuda(dq[slot][:, :n], dk[slot][:, :n], dv[slot][:, :n], **kw)
            do[slot][:, :n].copy_(o)
            computed[i].record(pipe.run)
        with torch.cuda.stream(pipe.down):
            pipe.down.wait_event(computed[i])
            out[b:b + 1, h0:h1].copy_(do[slot][:, :n], non_blocking=True)
            downloaded[i].record(pipe.down)
    cur.wait_event(downloaded[-1])
    cur.wait_event(computed[-1])
    return out
