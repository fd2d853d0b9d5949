"""Seeded synthetic q/k/v generators shaped like video-DiT and LLM-prefill activations.

They stand in for real model activations in tests and benchmarks: tokens laid out on a
(T, H, W) latent grid get a spatially smooth component so that pooled 128/64-token blocks are
self-similar and the block predictor has structure to find; K gets a per-channel bias, which is
what K mean-smoothing exists to remove."""
import math
from typing import Optional, Tuple

import torch


def _gauss_kernel(sigma: float, device, dtype) -> torch.Tensor:
    radius = max(1, int(math.ceil(3 * sigma)))
    x = torch.arange(-radius, radius + 1, device=device, dtype=dtype)
    k = torch.exp(-0.5 * (x / sigma) ** 2)
    return k / k.sum()


def _blur_axis(x: torch.Tensor, kernel: torch.Tensor, axis: int) -> torch.Tensor:
    """1-D convolution along `axis` with reflect padding (falls back to replicate on short axes)."""
    r = (kernel.numel() - 1) // 2
    x = x.movedim(axis, -1)
    shp = x.shape
    flat = x.reshape(-1, 1, shp[-1])
    mode = "reflect" if shp[-1] > r else "replicate"
    flat = torch.nn.functional.pad(flat, (r, r), mode=mode)
    out = torch.nn.functional.conv1d(flat, kernel.view(1, 1, -1))
    return out.reshape(shp).movedim(-1, axis)


def smoothed_grid(heads: int, grid: Tuple[int, int, int], dim: int, gen: torch.Generator, device, sigma: float = 2.0,
                  amplitude: float = 2.0) -> torch.Tensor:
    """[heads, T*H*W, dim] fp32:  N(0,1) + amplitude * (3-D Gaussian-blurred N(0,1), unit std)."""
    T, Hh, W = grid
    base = torch.randn(heads, T, Hh, W, dim, generator=gen, device=device)
    sm = torch.randn(heads, T, Hh, W, dim, generator=gen, device=device)
    kern = _gauss_kernel(sigma, device, sm.dtype)
    for axis in (1, 2, 3):
        sm = _blur_axis(sm, kern, axis)
    sm = sm / sm.std()
    return (base + amplitude * sm).reshape(heads, T * Hh * W, dim)


def video_qkv(B: int, H: int, grid: Tuple[int, int, int], D: int, seed: int, device="cpu", text_tokens: int = 0,
              text_first: bool = True, dtype=torch.bfloat16, k_bias_std: float = 3.0):
    """q, k, v of shape [B, H, text_tokens + T*H*W, D]."""
    gen = torch.Generator(device=device).manual_seed(seed)
    outs = []
    for name in ("q", "k", "v"):
        x = smoothed_grid(B * H, grid, D, gen, device)
        if text_tokens:
            txt = torch.randn(B * H, text_tokens, D, generator=gen, device=device)
            x = torch.cat([txt, x], dim=1) if text_first else torch.cat([x, txt], dim=1)
        if name == "k":
            x = x + k_bias_std * torch.randn(D, generator=gen, device=device)
        outs.append(x.reshape(B, H, -1, D).to(dtype))
    return tuple(outs)


def _rope(x: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate-half rotary embedding over positions 0..N-1; x is [..., N, D]."""
    N, D = x.shape[-2:]
    inv = theta ** (-torch.arange(0, D, 2, device=x.device, dtype=torch.float32) / D)
    ang = torch.arange(N, device=x.device, dtype=torch.float32)[:, None] * inv[None, :]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
    x1, x2 = x[..., : D // 2], x[..., D // 2:]
    return x * cos + torch.cat([-x2, x1], -1) * sin


def llm_prefill_qkv(B: int, H: int, N: int, D: int, seed: int, device="cpu", dtype=torch.bfloat16,
                    theta: float = 500000.0, sink_tokens: int = 16, sink_gain: float = 4.0):
    """Causal-prefill shaped inputs: q, k ~ N(0,1) with RoPE, a `sink` prefix whose keys are larger."""
    gen = torch.Generator(device=device).manual_seed(seed)
    q = _rope(torch.randn(B, H, N, D, generator=gen, device=device), theta)
    k = _rope(torch.randn(B, H, N, D, generator=gen, device=device), theta)
    k[..., :sink_tokens, :] *= sink_gain
    v = torch.randn(B, H, N, D, generator=gen, device=device)
    return q.to(dtype), k.to(dtype), v.to(dtype)


def bernoulli_block_mask(B: int, H: int, N: int, p: float, seed: int, device="cpu") -> torch.Tensor:
    """int32 [B,H,nq,nk] Bernoulli(p) block mask with the diagonal blocks (2q, 2q+1) forced live."""
    gen = torch.Generator(device=device).manual_seed(seed)
    nq, nk = (N + 127) // 128, (N + 63) // 64
    m = (torch.rand(B, H, nq, nk, generator=gen, device=device) < p).to(torch.int32)
    qi = torch.arange(nq, device=device)
    for off in (0, 1):
        kj = (2 * qi + off).clamp(max=nk - 1)
        m[:, :, qi, kj] = 1
    return m


# The five workload shapes the benchmarks and tests refer to by index.
WORKLOADS = {
    0: dict(name="small_noncausal", kind="video", B=1, H=4, D=64, grid=(8, 16, 16), text=0, topk=0.5, causal=False),
    1: dict(name="cogvideox2b", kind="video", B=2, H=30, D=64, grid=(13, 30, 45), text=226, text_first=True, topk=0.5,
            causal=False),
    2: dict(name="wan2.1_1.3b_480p", kind="video", B=1, H=12, D=128, grid=(21, 39, 40), text=0, topk=0.5, causal=False),
    3: dict(name="llama3_8b_prefill_32k", kind="llm", B=1, H=32, D=128, N=32768, topk=0.5, causal=True),
    4: dict(name="hunyuanvideo_720p", kind="video", B=1, H=24, D=128, grid=(33, 45, 80), text=256, text_first=False,
            topk=0.4, causal=False, ulysses=True),
}


def workload_heads_qkv(idx: int, heads, device="cpu", dtype=torch.bfloat16):
    """Inputs of the listed (batch, head) pairs of workload `idx` as [1, len(heads), N, D] tensors. Every head has
    its own seed, so a rank that owns some heads of a sharded run generates exactly the data another rank (or a
    single-GPU run) would generate for them."""
    w = WORKLOADS[idx]
    qs, ks, vs = [], [], []
    for (b, h) in heads:
        seed = 1000003 * (idx + 1) + 1009 * b + h
        if w["kind"] == "llm":
            q, k, v = llm_prefill_qkv(1, 1, w["N"], w["D"], seed, device, dtype)
        else:
            q, k, v = video_qkv(1, 1, w["grid"], w["D"], seed, device, w.get("text", 0), w.get("text_first", True), dtype)
        qs.append(q)
        ks.append(k)
        vs.append(v)
    return torch.cat(qs, 1), torch.cat(ks, 1), torch.cat(vs, 1)


def workload_shape(idx: int) -> Tuple[int, int, int, int]:
    """(B, H, N, D) of workload `idx`."""
    w = WORKLOADS[idx]
    if w["kind"] == "llm":
        n = w["N"]
    else:
        t, hh, ww = w["grid"]
        n = t * hh * ww + w.get("text", 0)
    return w["B"], w["H"], n, w["D"]


def workload_qkv(idx: int, device="cpu", heads: Optional[int] = None, dtype=torch.bfloat16):
    """Inputs of workload `idx`; `heads` overrides H (a head shard of the same workload)."""
    w = WORKLOADS[idx]
    H = heads if heads is not None else w["H"]
    seed = idx
    if w["kind"] == "llm":
        return llm_prefill_qkv(w["B"], H, w["N"], w["D"], seed, device, dtype)
    return video_qkv(w["B"], H, w["grid"], w["D"], seed, device, w.get("text", 0), w.get("text_first", True), dtype)
