"""CPU oracle for the SpargeAttn sparse-attention hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch on the CPU, the arithmetic of the reference's
`spas_sage2_attn_meansim_topk_cuda` / `block_sparse_sage2_attn_cuda` path.  Only tests,
the smoke check and the CPU-baseline leg of the benchmark may import it; the product
(`spargeattn_b200`) never does and fails loudly without its CUDA library.

Parity status: the reference ships no tests, golden vectors or stored input/output pairs for this
path, so this restatement is pinned against outputs of the reference itself instead:
  (a) the compiled reference (oracle/build_ref.py) run on a B200 by tests/golden/make_ref_gpu_golden.py:
      fixtures tests/golden/ref_gpu_*.pt in bf16 and fp16 hold its K mean, pooled values, flags, INT8 Q/K,
      scales, block map, LUT, counts, FP8 V bytes and V scales, and its attention output;
  (b) the reference's Triton kernels run under the Triton CPU interpreter for fp16 inputs
      (tests/golden/make_golden.py, fixtures ref_predictor_*.pt).
tests/test_oracle_golden.py states what is bit-exact against (a) and (b) and bounds the rest (pooled
values can differ in the last bit of a handful of entries because the compiled kernel's reduction
order is Triton's own; the attention output is compared at cosine >= 0.999, relative L1 <= 1e-2).

Where the reference leaves a summation order or a division instruction to a library
(Triton reductions, cuBLAS, torch softmax/sort), this file pins one choice, stated at each
function, and the CUDA kernels implement the same choice so that they can be compared
bit for bit:
  * the K mean and the softmax accumulate in fp64 (order-free to ~1e-16) and are rounded to
    fp32 once; block pooling and row norms use short fp32 running sums in a fixed order,
    combined in fp64 / by a fixed butterfly (see pool_sim_quant);
  * the Q/K block scale is fma(max|x|, RN(1/127), 1e-7) -- the compiled reference contracts
    `max / 127. + 1e-7` that way (bit-exact on every fixture scale); the element quotient x / scale
    is IEEE (the reference's approximate quotient gave the same INT8 on every compared element);
  * the V scale is amax * RN(1/2.25) and the V multiplier 2.25 * (1 / amax): csrc/fused is built with
    --use_fast_math, i.e. dividend times the hardware reciprocal of the divisor. The hardware
    reciprocal has no published bit-level definition: `quant_v` takes the device's value as an
    optional input and otherwise uses the correctly rounded reciprocal (differs from the device
    in about 2 of 10^4 FP8 bytes);
  * the pooled score is an fp32 FMA chain over ascending channel index;
  * the row softmax is evaluated in fp64, rounded to fp32, then to the 16-bit dtype;
  * top-k uses a stable descending order (ties -> lower block index);
  * the cdf mode's cumulative sum is the one torch computes on a CUDA device in the 16-bit type
    (aten_device_cumsum), and its count the upper-bound search torch runs (searchsorted_right).

Reference files are cited as path:line relative to the reference project root.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

BLKQ = 128
BLKK = 64
S_FP8_OFFSET = 8.807          # csrc/qattn/attn_utils.cuh:28-30
V_SCALE_MAX = 2.25            # spas_sage_attn/core.py:151
LOG2E = 1.4426950408889634    # csrc/math.cuh
MASK_VALUE = -5000000.0       # csrc/qattn/attn_utils.cuh:348-352


# ----------------------------------------------------------------------------- helpers
def hyperparameter_check(hyper, H: int) -> torch.Tensor:
    """spas_sage_attn/utils.py:38-50 -- scalar / 0-d / 1-d -> fp32 [H]."""
    if type(hyper) in (float, int):
        return torch.full((H,), float(hyper), dtype=torch.float32)
    if isinstance(hyper, torch.Tensor):
        assert hyper.dim() <= 1, "Hyperparameter tensor must be 1D"
        if hyper.dim() == 0:
            return torch.full((H,), hyper.item(), dtype=torch.float32)
        assert hyper.numel() == H, f"Hyperparameter tensor must have {H} elements, but has {hyper.numel()}"
        return hyper.to(torch.float32).cpu()
    raise ValueError("Hyperparameter must be a float or a tensor")


def precision_metric(a: torch.Tensor, b: torch.Tensor) -> dict:
    """spas_sage_attn/utils.py:25-36 -- cosine similarity, relative L1, RMSE (b is the reference)."""
    x, xx = a.double().reshape(1, -1), b.double().reshape(1, -1)
    sim = torch.nn.functional.cosine_similarity(x, xx).item()
    l1 = ((x - xx).abs().sum() / xx.abs().sum()).item()
    rmse = torch.sqrt(torch.mean((x - xx) ** 2)).item()
    return {"Cossim": sim, "L1": l1, "RMSE": rmse}


def e4m3_round(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> e4m3 value (returned as fp32): one round-to-nearest-even, saturating to +-448, as
    `cvt.rn.satfinite.e4m3x2.f32` does (csrc/numeric_conversion.cuh:48-63; checked exhaustively on a
    B200 for every fp32 in [2^-12, 512)).  Written out by hand because torch's CPU float8 cast does
    not saturate."""
    x = x.to(torch.float32)
    a = x.abs().clamp(max=448.0)
    # exponent of the e4m3 bucket: normal numbers have 3 mantissa bits, subnormals a fixed 2^-9 step
    _, ex = torch.frexp(torch.where(a > 0, a, torch.ones_like(a)))     # a = mant * 2^ex, mant in [0.5, 1)
    e = (ex - 1).to(torch.float32).clamp(min=-6.0)
    step = torch.exp2(e - 3.0)
    q = torch.round(a / step) * step          # torch.round is half-to-even; a/step is exact (power of two)
    q = q.clamp(max=448.0)
    return torch.copysign(torch.where(a > 0, q, torch.zeros_like(a)), x)   # keeps the sign of -0 and of underflow


def e4m3_bits(x: torch.Tensor) -> torch.Tensor:
    """e4m3-representable fp32 values -> their uint8 bit patterns."""
    return x.to(torch.float32).to(torch.float8_e4m3fn).view(torch.uint8)


def e4m3_from_bits(b: torch.Tensor) -> torch.Tensor:
    return b.view(torch.float8_e4m3fn).to(torch.float32)


def fma_f32(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """Correctly rounded fp32 fused multiply-add a * b + c (one rounding), elementwise.
    The product of two fp32 numbers is exact in fp64; the fp64 sum is made exact with a two-sum error
    term, which decides the (rare) case where the fp64 sum lands on an fp32 rounding midpoint."""
    p = a.double() * b.double()
    cd = c.double().expand_as(p)
    s = p + cd
    bb = s - p
    err = (p - (s - bb)) + (cd - bb)                       # s + err == p + c exactly
    r = s.float()
    rd = r.double()
    up = torch.nextafter(r, torch.full_like(r, float("inf"))).double()
    dn = torch.nextafter(r, torch.full_like(r, float("-inf"))).double()
    tie_up = (s - rd == (up - rd) / 2) & (s > rd)          # s exactly half way towards the next fp32
    tie_dn = (rd - s == (rd - dn) / 2) & (s < rd)
    r = torch.where(tie_up & (err > 0), up.float(), r)     # true sum above the midpoint: round up
    r = torch.where(tie_dn & (err < 0), dn.float(), r)
    return r


# ----------------------------------------------------------------------------- K mean
def k_mean(k: torch.Tensor) -> torch.Tensor:
    """spas_sage_attn/core.py:119-120 `km = k.mean(dim=-2, keepdim=True)` in k's dtype.

    Pinned: exact (fp64) sum over tokens, divided by N in fp64, rounded to fp32, then to the
    16-bit dtype.  torch's own reduction accumulates in fp32 in a library-chosen order."""
    n = k.shape[-2]
    return (k.double().sum(dim=-2, keepdim=True) / float(n)).float().to(k.dtype)


# ----------------------------------------------------------------------------- pool / sim / quant
def _blocks(x: torch.Tensor, bs: int) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """[B,H,N,D] -> zero-padded [B,H,nb,bs,D] plus a row-validity mask [nb,bs]."""
    B, H, N, D = x.shape
    nb = (N + bs - 1) // bs
    pad = nb * bs - N
    if pad:
        x = torch.cat([x, torch.zeros(B, H, pad, D, dtype=x.dtype)], dim=2)
    valid = (torch.arange(nb * bs) < N).view(nb, bs)
    return x.view(B, H, nb, bs, D), valid, nb


def pool_sim_quant(x: torch.Tensor, km: Optional[torch.Tensor], bs: int, simthreshd1: torch.Tensor,
                   want_pool: bool = True):
    """spas_sage_attn/utils.py:161-214 (fused pool + self-similarity + per-block INT8) and
    utils.py:89-159 (`qk_quantize`, quantiser only).

    x: [B,H,N,D] fp16/bf16.  km: [B,H,1,D] in x's dtype or None.  Returns
    (pool [B,H,nb,D] x.dtype, sim [B,H,nb] bool, x_int8 [B,H,N,D], scale [B,H,nb] fp32)."""
    B, H, N, D = x.shape
    xb, valid, nb = _blocks(x, bs)
    if km is not None:
        # utils.py:185-188: subtraction in the 16-bit dtype, padded rows re-zeroed
        xb = (xb - km.view(B, H, 1, 1, D)).to(x.dtype)
        xb = torch.where(valid.view(1, 1, nb, bs, 1), xb, torch.zeros((), dtype=x.dtype))
    x32 = xb.float()

    # utils.py:206-210 -- scale = max|x| / 127 + 1e-7 (one FMA in the compiled kernel); round half away from zero
    amax = x32.abs().amax(dim=(-1, -2))
    scale = fma_f32(amax, torch.tensor(1.0, dtype=torch.float32) / 127.0, torch.tensor(1e-7, dtype=torch.float32))
    y = x32 / scale.view(B, H, nb, 1, 1)
    y = y + torch.where(y >= 0, 0.5, -0.5).to(torch.float32)
    x_int8 = y.to(torch.int8).view(B, H, nb * bs, D)[:, :, :N].contiguous()
    if not want_pool:
        return None, None, x_int8, scale

    # Pinned reduction orders (the CUDA kernel uses the same ones, see csrc/pool_quant.cu):
    #   rows:     fp32 running sum over each run of 8 consecutive rows, fp64 across the runs
    #   channels: fp32 running sum of squares over each run of 8 consecutive channels, then an
    #             fp32 butterfly (partner = index xor D/16, ..., xor 1) across the D/8 runs
    def rows8(t):                                                     # [B,H,nb,bs,D] fp32 -> [B,H,nb,D] fp64
        g = t.view(B, H, nb, bs // 8, 8, D)
        acc = g[..., 0, :].clone()
        for i in range(1, 8):
            acc = acc + g[..., i, :]
        return acc.double().sum(dim=-2)

    # utils.py:182,192 -- pool = sum over rows / BS_  (BS_ = rows actually present)
    bs_ = valid.sum(-1).to(torch.float32)                            # [nb]
    pool = (rows8(x32).float() / bs_.view(1, 1, nb, 1)).to(x.dtype)

    # utils.py:193-199 -- x_hat = fp16(x / ||x||), sim = sum_ij <x_hat_i, x_hat_j> / BS_^2 > thr
    # using  sum_ij <a_i, a_j> = || sum_i a_i ||^2 ; the division is one IEEE reciprocal per row
    # followed by a multiplication per element.
    sq = (x32 * x32).view(B, H, nb, bs, D // 8, 8)                    # products of 16-bit values are exact
    part = sq[..., 0].clone()
    for i in range(1, 8):
        part = part + sq[..., i]
    tpr = D // 8
    o = tpr // 2
    while o >= 1:
        part = part + part[..., torch.arange(tpr) ^ o]
        o //= 2
    nrm = part[..., :1].sqrt()                                        # [B,H,nb,bs,1]
    rinv = torch.ones_like(nrm) / nrm
    xhat = (x32 * rinv).to(torch.float16)                             # 0 * inf -> NaN on empty rows
    zero_row = (nrm.squeeze(-1) == 0).any(dim=-1)
    xhat = torch.where(nrm == 0, torch.zeros((), dtype=torch.float16), xhat)
    ssum = rows8(xhat.float())                                        # [B,H,nb,D] fp64
    total = (ssum * ssum).sum(dim=-1).float()
    simval = total / (bs_ * bs_).view(1, 1, nb)
    sim = simval > simthreshd1.view(1, H, 1)
    full = (valid.sum(-1) == bs).view(1, 1, nb)
    sim = sim & full & ~zero_row                                     # explicit form of the reference's NaN rule
    return pool, sim, x_int8, scale


# ----------------------------------------------------------------------------- predictor
def pooled_probs(pq: torch.Tensor, pk: torch.Tensor, sim_k: torch.Tensor, is_causal: bool) -> torch.Tensor:
    """spas_sage_attn/utils.py:386-396 -- pooled score map and its row softmax, in the 16-bit dtype."""
    B, H, nq, D = pq.shape
    nk = pk.shape[2]
    dt = pq.dtype
    a, b = pq.float(), pk.float()
    acc = torch.zeros(B, H, nq, nk, dtype=torch.float32)
    for d in range(D):  # fp32 FMA chain, ascending d (16-bit x 16-bit products are exact in fp32)
        acc = acc + a[..., :, d:d + 1] * b[..., :, d].unsqueeze(-2)
    s = acc.to(dt)
    s = (s.float() * torch.tensor(D ** -0.5, dtype=torch.float32)).to(dt)
    s = s.masked_fill(~sim_k.view(B, H, 1, nk), float("-inf"))
    if is_causal:
        qi = torch.arange(nq).view(nq, 1)
        kj = torch.arange(nk).view(1, nk)
        s = s.masked_fill((kj >= (qi + 1) * (BLKQ // BLKK)).view(1, 1, nq, nk), float("-inf"))
    s64 = s.double()
    m = s64.amax(dim=-1, keepdim=True)
    e = torch.exp(s64 - m)
    p = (e / e.sum(dim=-1, keepdim=True)).float().to(dt)
    p = torch.where(torch.isinf(m), torch.zeros((), dtype=dt), p)     # row with no candidate
    return p


def select_blocks(p: torch.Tensor, sim_q: torch.Tensor, sim_k: torch.Tensor, topk: Optional[torch.Tensor],
                  cdfthreshd: Optional[torch.Tensor], is_causal: bool, attention_sink: bool) -> torch.Tensor:
    """spas_sage_attn/utils.py:397-415 and :282-292 -- final boolean block map [B,H,nq,nk]."""
    B, H, nq, nk = p.shape
    order = torch.sort(p.float(), dim=-1, descending=True, stable=True)
    if cdfthreshd is not None:
        # utils.py:398-403: torch.cumsum of the sorted probabilities in the 16-bit dtype, then
        # torch.searchsorted(cdf, threshold, right=True). The reference runs on a CUDA device, where cumsum is
        # ATen's chunked Sklansky scan with every combine rounded to the 16-bit type (aten_device_cumsum): its
        # rounding decides the count on long rows, so that scan is restated here, not a mathematically exact sum.
        cdf = aten_device_cumsum(order.values.to(p.dtype).reshape(B * H * nq, nk)).float()
        thr = cdfthreshd.to(torch.float32).view(1, H, 1).expand(B, H, nq).reshape(-1)
        n_sel = searchsorted_right(cdf, thr).view(B, H, nq)
    else:
        n_sel = (topk.to(torch.float32) * nk).to(torch.int64).view(1, H, 1).expand(B, H, nq)
    n_sel = n_sel.clamp(min=1, max=nk)                                # utils.py:289 (>= 1)
    rank = torch.empty_like(order.indices)
    rank.scatter_(-1, order.indices, torch.arange(nk).expand(B, H, nq, nk).contiguous())
    sel = rank < n_sel.unsqueeze(-1)
    fmap = sel | ~sim_k.view(B, H, 1, nk) | ~sim_q.view(B, H, nq, 1)
    if is_causal:
        qi = torch.arange(nq).view(nq, 1)
        kj = torch.arange(nk).view(1, nk)
        fmap = fmap & (kj < (qi + 1) * (BLKQ // BLKK)).view(1, 1, nq, nk)
    if attention_sink:
        fmap = fmap.clone()
        fmap[..., 0] = True
    return fmap


def aten_scan_log_threads_x(num_rows: int, row_size: int) -> int:
    """get_log_num_threads_x_inner_scan of ATen/native/cuda/ScanUtils.cuh (torch 2.11), in its uint32 arithmetic."""
    lx = 0
    while (1 << lx) < row_size:
        lx += 1
    ly = 0
    while (1 << ly) < num_rows:
        ly += 1
    v = ((9 + ((lx - ly) & 0xFFFFFFFF)) & 0xFFFFFFFF) // 2
    return min(max(4, v), 9)


def aten_device_cumsum(x: torch.Tensor) -> torch.Tensor:
    """torch.cumsum(x, -1) of a contiguous [rows, n] fp16/bf16 matrix as ATen computes it on a CUDA device
    (tensor_kernel_scan_innermost_dim with std::plus<scalar_t>, ATen/native/cuda/ScanUtils.cuh): the row is cut
    into chunks of 2 * nx values (nx from aten_scan_log_threads_x); the total of the previous chunks is added to
    the first value of a chunk; log2(nx) + 1 Sklansky steps combine the chunk, and every addition is rounded to
    the 16-bit type. Checked bit for bit against recorded device results (tests/golden/ref_gpu_cdf_*.pt)."""
    R, n = x.shape
    dt = x.dtype
    lg = aten_scan_log_threads_x(R, n)
    nx = 1 << lg
    W = 2 * nx
    out = torch.empty_like(x)
    total = torch.zeros(R, dtype=dt)
    t = torch.arange(nx)
    for c0 in range(0, n, W):
        w = min(W, n - c0)
        buf = torch.zeros(R, W, dtype=dt)
        buf[:, :w] = x[:, c0:c0 + w]
        buf[:, 0] = (buf[:, 0].float() + total.float()).to(dt)
        for m in range(lg + 1):
            s = 1 << m
            a = ((t >> m) << (m + 1)) | s
            ti, si = a + (t % s), a - 1
            buf[:, ti] = (buf[:, ti].float() + buf[:, si].float()).to(dt)
        out[:, c0:c0 + w] = buf[:, :w]
        total = buf[:, W - 1].clone()
    return out


def searchsorted_right(cdf: torch.Tensor, thr: torch.Tensor) -> torch.Tensor:
    """torch.searchsorted(cdf, thr, right=True) per row as the upper-bound binary search torch runs (cdf [rows, n]
    fp32 values, thr [rows] fp32). Written out because a rounded cumulative sum need not be monotone, and then the
    result is whatever that particular search visits."""
    R, n = cdf.shape
    start = torch.zeros(R, dtype=torch.long)
    end = torch.full((R,), n, dtype=torch.long)
    rows = torch.arange(R)
    while bool((start < end).any()):
        act = start < end
        mid = start + ((end - start) >> 1)
        go = ~(cdf[rows, mid.clamp(max=n - 1)] > thr)
        start = torch.where(act & go, mid + 1, start)
        end = torch.where(act & ~go, mid, end)
    return start


def block_map_to_lut(block_map: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """spas_sage_attn/utils.py:54-87 -- delta-encoded LUT (first entry absolute, zero tail) + counts."""
    bm = block_map != 0
    B, H, nq, nk = bm.shape
    valid = bm.sum(-1).to(torch.int32)
    idx = torch.arange(nk).expand(B, H, nq, nk)
    key = torch.where(bm, idx, idx + nk)                               # live first, ascending
    order = torch.sort(key, dim=-1, stable=True).indices
    pos = torch.gather(idx, -1, order)
    prev = torch.cat([torch.zeros(B, H, nq, 1, dtype=pos.dtype), pos[..., :-1]], dim=-1)
    lut = pos - prev
    live = torch.arange(nk).view(1, 1, 1, nk) < valid.unsqueeze(-1)
    lut = torch.where(live, lut, torch.zeros_like(lut)).to(torch.int32)
    return lut, valid


def block_map_to_mask(block_map: torch.Tensor, nq_tokens: int, nk_tokens: int) -> torch.Tensor:
    """spas_sage_attn/utils.py:424-432 -- expand a block map to a token mask, cropped to the lengths."""
    m = (block_map != 0).repeat_interleave(BLKQ, dim=-2).repeat_interleave(BLKK, dim=-1)
    return m[..., :nq_tokens, :nk_tokens]


def predictor(q, k, km, is_causal=False, simthreshd1=-0.1, cdfthreshd=None, topk=0.5, attention_sink=False):
    """spas_sage_attn/utils.py:371-421 `get_block_map_meansim_fuse_quant`.
    Returns dict(map, lut, valid, q_int8, q_scale, k_int8, k_scale, pq, pk, sim_q, sim_k, p)."""
    assert (cdfthreshd is None) != (topk is None), "Only one of cdfthreshd and topk can be set."
    H = q.shape[1]
    thr = hyperparameter_check(simthreshd1, H)
    tk = hyperparameter_check(topk, H) if topk is not None else None
    cdf = hyperparameter_check(cdfthreshd, H) if cdfthreshd is not None else None
    pq, sim_q, q8, qs = pool_sim_quant(q, None, BLKQ, thr)
    pk, sim_k, k8, ks = pool_sim_quant(k, km, BLKK, thr)
    p = pooled_probs(pq, pk, sim_k, is_causal)
    fmap = select_blocks(p, sim_q, sim_k, tk, cdf, is_causal, attention_sink)
    lut, valid = block_map_to_lut(fmap)
    return dict(map=fmap, lut=lut, valid=valid, q_int8=q8, q_scale=qs, k_int8=k8, k_scale=ks,
                pq=pq, pk=pk, sim_q=sim_q, sim_k=sim_k, p=p)


# ----------------------------------------------------------------------------- V quantisation
def quant_v(v: torch.Tensor, recip_scale: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """spas_sage_attn/core.py:115-117,143-151 + csrc/fused/fused.cu:80-191 (built with --use_fast_math).

    v: [B,H,N,D] any float dtype.  Returns (v8 [B,H,N_pad128,D] as e4m3 values in fp32, zero rows
    beyond N; v_scale [B,H,D] fp32).  The reference stores the same numbers transposed to
    [B,H,D,N_pad] with a 16-token permutation that only serves its mma.sync register layout.

    fused.cu:150 `scale = amax / scale_max` and :163 `recp_scale = scale_max / amax` are approximate
    quotients (dividend times hardware reciprocal).  The first equals amax * RN(1/2.25) on every fixture
    value.  For the second pass `recip_scale` [B,H,D] = the device's quotient 2.25 / amax to reproduce the
    reference bit for bit; without it the correctly rounded reciprocal stands in."""
    B, H, N, D = v.shape
    v16 = v.to(torch.float16).float()
    amax = v16.abs().amax(dim=-2)                                     # [B,H,D]
    v_scale = amax * (torch.tensor(1.0, dtype=torch.float32) / V_SCALE_MAX)
    if recip_scale is None:
        r = V_SCALE_MAX * (torch.ones_like(amax) / amax)
    else:
        r = recip_scale.to(torch.float32).reshape(B, H, D)
    r = torch.where(amax > 0, r, torch.zeros_like(r))                 # all-zero channel: emit zeros, not NaN
    v8 = e4m3_round(v16 * r.unsqueeze(-2))
    npad = (N + 127) // 128 * 128
    out = torch.zeros(B, H, npad, D, dtype=torch.float32)
    out[:, :, :N] = v8
    return out, v_scale


# ----------------------------------------------------------------------------- attention
def per_warp_int8(q, k, BLKQ=128, WARPQ=32, BLKK=64, WARPK=64):
    """spas_sage_attn/quant_per_block.py:102-148 (kernel :21-48, sm_scale = 1): one scale per WARPQ = 32 query rows
    (ceil(N/128) * 4 per head; a group past the end gets 1e-7) and per WARPK = 64 keys; no mean subtraction.
    HND layout.  Returns (q_int8, q_scale [B,H,nq*4], k_int8, k_scale [B,H,nk])."""
    B, H, N, D = q.shape
    _, _, q8, qs = pool_sim_quant(q, None, WARPQ, None, want_pool=False)
    groups = (N + BLKQ - 1) // BLKQ * (BLKQ // WARPQ)
    qs = torch.cat([qs, torch.full((B, H, groups - qs.shape[-1]), 1e-7, dtype=torch.float32)], -1)
    _, _, k8, ks = pool_sim_quant(k, None, WARPK, None, want_pool=False)
    return q8, qs, k8, ks


def per_thread_int8(q, k, BLKQ=128, WARPQ=32, BLKK=64, WARPK=64):
    """Quantiser for qk_quant_gran = 3.  The reference ships none (its kernel only documents the layout,
    csrc/qattn/qk_int_sv_f8_cuda_sm89.cuh:116-136, scale shapes qk_int_sv_f8_cuda_sm89.cu:349-353): this one uses the
    arithmetic of quant_per_block_int8_kernel on the row / key sets that share a scale -- rows r, r+8, r+16, r+24
    of a 32-row group (entry (row // 32) * 8 + row % 8), keys 2t, 2t+1 of every 8 of a 64-key block (entry
    block * 4 + (key % 8) // 2).  Returns (q_int8, q_scale [B,H,nq*32], k_int8, k_scale [B,H,nk*4])."""
    B, H, N, D = q.shape

    def quant(x, pad_to, shape, reduce_dims, group_of):
        n_pad = (N + pad_to - 1) // pad_to * pad_to
        x32 = torch.cat([x.float(), torch.zeros(B, H, n_pad - N, D)], 2)
        amax = x32.abs().amax(-1).view(B, H, *shape).amax(dim=reduce_dims).reshape(B, H, -1)
        scale = fma_f32(amax, torch.tensor(1.0, dtype=torch.float32) / 127.0, torch.tensor(1e-7, dtype=torch.float32))
        y = x32 / scale[:, :, group_of(torch.arange(n_pad))].unsqueeze(-1)
        y = y + torch.where(y >= 0, 0.5, -0.5).to(torch.float32)
        return y.to(torch.int8)[:, :, :N].contiguous(), scale

    # rows as (group of 32, which 8, row % 8); keys as (block of 64, which 8, pair in the 8, which of the pair)
    q8, qs = quant(q, BLKQ, (-1, WARPQ // 8, 8), 3, lambda r: (r // WARPQ) * 8 + r % 8)
    k8, ks = quant(k, BLKK, (-1, WARPK // 8, 4, 2), (3, 5), lambda n: (n // WARPK) * 4 + (n % 8) // 2)
    return q8, qs, k8, ks


def granular_scales(q_scale, k_scale, b, h, i, j, rows, cols, qk_quant_gran):
    """Per-row and per-column dequantisation factors of scores tile (query block i, key block j) for the three
    granularities of csrc/qattn/qk_int_sv_f8_cuda_sm89.cuh:106-136: 1 one scalar each; 2 one Q scale per 32 rows;
    3 Q entry (row // 32) * 8 + row % 8 of the block's 32, K entry (key % 8) // 2 of the block's 4 (the mma.sync
    accumulator layout of the reference: a thread owns rows r, r + 8 and key pairs 2t, 2t + 1 of every 8)."""
    if qk_quant_gran == 1:
        return q_scale[b, h, i].expand(rows), k_scale[b, h, j].expand(cols)
    r = torch.arange(rows)
    if qk_quant_gran == 2:
        return q_scale[b, h, i * 4 + r // 32], k_scale[b, h, j].expand(cols)
    n = torch.arange(cols)
    return q_scale[b, h, i * 32 + (r // 32) * 8 + r % 8], k_scale[b, h, j * 4 + (n % 8) // 2]


def attention_blockwise(q8, q_scale, k8, k_scale, v8, v_scale, block_map, sm_scale: float, pvthreshd,
                        token_causal: bool = False, out_dtype=torch.bfloat16, pv_skip: bool = True, q_blocks=None,
                        qk_quant_gran: int = 1, pv_threshold_mode: int = 1, group_counts=None, pv_fp16: bool = False):
    """Oracle B: block-online emulation of csrc/qattn/qk_int_sv_f8_cuda_sm89.cuh:42-755 with the
    helpers of csrc/qattn/attn_utils.cuh (update_mo :418-466, exponentiate_r :391-415,
    RS_32_to_8 :581-596, normalize_d :757-811).  fp32 PV accumulation.

    q8,k8: int8 [B,H,N,D]; q_scale [B,H,nq]; k_scale [B,H,nk]; v8: e4m3 values fp32 [B,H,N_pad,D];
    v_scale [B,H,D]; block_map bool [B,H,nq,nk]; pvthreshd fp32 [H].
    `q_blocks`: optional list of query-block indices; only those 128-row blocks are evaluated (the other
    rows of the result stay zero), so that a sample of a long sequence can be checked in seconds.
    `qk_quant_gran` 1/2/3: scale layouts of `granular_scales` (q_scale / k_scale then have 1/4/32 and 1/1/4
    entries per block).  `pv_threshold_mode` 1: the skip test reduces over the 128-row block
    (PVThresholdMode::kPerBlock, sm89.cuh:322-345); 2: every 32-row group decides for itself (kPerWarp: the
    warp-level reduction of :317-320 only).  `group_counts`: optional int32 [B,H,nq*4] tensor that receives,
    per 32-row group, the number of P.V products kept (the reference's PV_Count, sm89.cuh:355-358,650-656).
    `pv_fp16`: the fp16-PV kernel of the Sage1 signatures (csrc/qattn/qk_int_sv_f16_cuda_sm80.cuh): v8 then holds
    the fp16 values of V (as fp32), v_scale is ignored, P = 2^(t - m) without the FP8 offset is rounded to fp16."""
    B, H, N, D = q8.shape
    nq, nk = block_map.shape[-2:]
    c = sm_scale * LOG2E
    o = torch.zeros(B, H, N, D, dtype=torch.float32)
    skipped = 0
    for b in range(B):
        for h in range(H):
            kf = k8[b, h].float()
            for i in (range(nq) if q_blocks is None else q_blocks):
                r0, r1 = i * BLKQ, min((i + 1) * BLKQ, N)
                qf = q8[b, h, r0:r1].float()
                rows = r1 - r0
                m = torch.full((rows,), MASK_VALUE, dtype=torch.float32)
                # Rows of a partial last query block beyond N take part in the skip test's maximum over the block
                # (update_mo has no row mask, attn_utils.cuh:418-466).  The reference leaves them unfilled in shared
                # memory (predicated load without fill, attn_utils.cuh:133), so what they hold is not defined; the
                # CUDA kernel under test zero-fills them, and zeros are modelled here: zero scores, running maximum 0
                # after the first block, difference 0, hence no skip in a partial query block with a positive
                # threshold.  m_pad is that running maximum.
                m_pad = MASK_VALUE
                d = torch.ones(rows, dtype=torch.float32)
                acc = torch.zeros(rows, D, dtype=torch.float32)
                live = torch.nonzero(block_map[b, h, i]).flatten().tolist()
                for n_it, j in enumerate(live):
                    c0, c1 = j * BLKK, min((j + 1) * BLKK, N)
                    s = qf @ kf[c0:c1].t()                              # exact: |S| < 2^24
                    rs, cs = granular_scales(q_scale, k_scale, b, h, i, j, rows, c1 - c0, qk_quant_gran)
                    t = s * ((c * rs).view(-1, 1) * cs.view(1, -1))
                    if token_causal:
                        qi = torch.arange(r0, r1).view(-1, 1)
                        kj = torch.arange(c0, c1).view(1, -1)
                        t = torch.where(kj > qi, torch.full_like(t, MASK_VALUE), t)
                    rowmax = t.amax(dim=-1)
                    m_new = torch.maximum(m, rowmax)
                    is_tail = n_it >= len(live) - 2                    # last two live blocks never skip
                    keep = torch.ones(rows, dtype=torch.bool)
                    pad_delta = (0.0 - m_pad) if rows < BLKQ else float("-inf")
                    m_pad = max(m_pad, 0.0)
                    if pv_skip and not is_tail:
                        if pv_threshold_mode == 1:
                            delta = max((rowmax - m).max().item(), pad_delta)
                            if delta + float(pvthreshd[h]) <= 0:
                                skipped += 1
                                continue
                        else:                                          # each 32-row group on its own
                            for g0 in range(0, rows, 32):
                                g_delta = (rowmax - m)[g0:g0 + 32].max().item()
                                if g0 + 32 > rows:                     # the group that also holds padded rows
                                    g_delta = max(g_delta, pad_delta)
                                if g_delta + float(pvthreshd[h]) <= 0:
                                    keep[g0:g0 + 32] = False
                                    skipped += 1
                    if group_counts is not None:
                        for g0 in range(0, BLKQ, 32):                  # a group past the end counts like its block
                            if g0 >= rows or bool(keep[g0]):
                                group_counts[b, h, i * 4 + g0 // 32] += 1
                    alpha = torch.exp2(m - m_new)
                    if pv_fp16:
                        p = torch.exp2(t - m_new.unsqueeze(-1))
                        p_lo = p.to(torch.float16).float()
                    else:
                        p = torch.exp2(t - m_new.unsqueeze(-1) + S_FP8_OFFSET)
                        p_lo = e4m3_round(p)
                    d_new = d * alpha + p.sum(dim=-1)
                    acc_new = acc * alpha.unsqueeze(-1) + p_lo @ v8[b, h, c0:c1]
                    # a group that drops the block keeps its state (its maximum cannot have risen: delta < 0)
                    m = torch.where(keep, m_new, m)
                    d = torch.where(keep, d_new, d)
                    acc = torch.where(keep.unsqueeze(-1), acc_new, acc)
                if live:
                    o[b, h, r0:r1] = acc / d.unsqueeze(-1) * (1.0 if pv_fp16 else v_scale[b, h].view(1, D))
    return o.to(out_dtype), skipped


def attention_blockwise_sampled(q8, q_scale, k8, k_scale, v8, v_scale, block_map, sm_scale: float, pvthreshd,
                                q_blocks, token_causal: bool = False, out_dtype=torch.bfloat16, pv_skip: bool = True,
                                pv_fp16: bool = False):
    """`attention_blockwise` restricted to the query blocks in `q_blocks`, evaluated for all (batch, head,
    query block) samples at once: the loop runs over the position in each sample's live list, not over
    samples, so a few dozen blocks of a 100k-token sequence take seconds.  Same arithmetic, same visiting
    order (ascending key block), same skip rule.  Returns [B,H,len(q_blocks)*128,D] (rows beyond N are zero)
    and the number of skipped blocks."""
    B, H, N, D = q8.shape
    nq, nk = block_map.shape[-2:]
    c = sm_scale * LOG2E
    qb = torch.as_tensor(list(q_blocks), dtype=torch.long)
    nb = qb.numel()
    S = B * H * nb
    bi = torch.arange(B).view(B, 1, 1).expand(B, H, nb).reshape(S)
    hi = torch.arange(H).view(1, H, 1).expand(B, H, nb).reshape(S)
    qi = qb.view(1, 1, nb).expand(B, H, nb).reshape(S)
    pad_q = nq * BLKQ - N
    q8p = torch.cat([q8, torch.zeros(B, H, pad_q, D, dtype=q8.dtype)], 2) if pad_q else q8
    pad_k = nk * BLKK - N
    k8p = torch.cat([k8, torch.zeros(B, H, pad_k, D, dtype=k8.dtype)], 2) if pad_k else k8
    v8p = v8 if v8.shape[2] >= nk * BLKK else torch.cat([v8, torch.zeros(B, H, nk * BLKK - v8.shape[2], D)], 2)
    qf = q8p.view(B, H, nq, BLKQ, D)[bi, hi, qi].float()                      # [S,128,D]
    kblk = k8p.view(B, H, nk, BLKK, D)
    vblk = v8p[:, :, :nk * BLKK].reshape(B, H, nk, BLKK, D)
    bm = block_map[bi, hi, qi]                                                # [S,nk]
    cnt = bm.sum(-1)
    order = torch.sort(torch.where(bm, torch.arange(nk).expand(S, nk), torch.arange(nk).expand(S, nk) + nk), dim=-1).values
    qrow = qi.view(S, 1) * BLKQ + torch.arange(BLKQ).view(1, BLKQ)             # [S,128]
    row_ok = qrow < N
    qsc = q_scale[bi, hi, qi]
    thr = pvthreshd[hi]
    m = torch.full((S, BLKQ), MASK_VALUE, dtype=torch.float32)
    d = torch.ones(S, BLKQ, dtype=torch.float32)
    acc = torch.zeros(S, BLKQ, D, dtype=torch.float32)
    skipped = 0
    for n_it in range(int(cnt.max()) if S else 0):
        act = n_it < cnt
        j = torch.where(act, order[:, n_it], torch.zeros_like(cnt))
        s = torch.matmul(qf, kblk[bi, hi, j].float().transpose(-1, -2))        # exact: |S| < 2^24
        t = s * (c * qsc * k_scale[bi, hi, j]).view(S, 1, 1)
        kidx = j.view(S, 1) * BLKK + torch.arange(BLKK).view(1, BLKK)          # [S,64]
        dead = (kidx >= N).view(S, 1, BLKK)
        if token_causal:
            dead = dead | (kidx.view(S, 1, BLKK) > qrow.view(S, BLKQ, 1))
        t = torch.where(dead, torch.full_like(t, MASK_VALUE), t)
        rowmax = t.amax(dim=-1)
        m_new = torch.maximum(m, rowmax)
        upd = act.clone()
        if pv_skip:
            # padded rows of a partial last query block take part as zero rows (see attention_blockwise)
            delta = (rowmax - m).amax(dim=-1)
            skip = act & (n_it < cnt - 2) & (delta + thr <= 0)
            skipped += int(skip.sum())
            upd = upd & ~skip
        alpha = torch.exp2(m - m_new)
        p = torch.exp2(t - m_new.unsqueeze(-1) + (0.0 if pv_fp16 else S_FP8_OFFSET))
        p = torch.where(dead, torch.zeros_like(p), p)
        d_new = d * alpha + p.sum(dim=-1)
        p_lo = p.to(torch.float16).float() if pv_fp16 else e4m3_round(p)      # pv_fp16: see attention_blockwise
        acc_new = acc * alpha.unsqueeze(-1) + torch.matmul(p_lo, vblk[bi, hi, j])
        u1, u2 = upd.view(S, 1), upd.view(S, 1, 1)
        m = torch.where(u1, m_new, m)
        d = torch.where(u1, d_new, d)
        acc = torch.where(u2, acc_new, acc)
    o = acc / d.unsqueeze(-1) * (1.0 if pv_fp16 else v_scale[bi, hi].view(S, 1, D))
    o = torch.where((row_ok & (cnt > 0).view(S, 1)).unsqueeze(-1), o, torch.zeros_like(o))
    return o.view(B, H, nb * BLKQ, D).to(out_dtype), skipped


def attention_dense_masked(q8, q_scale, k8, k_scale, v8, v_scale, block_map, sm_scale: float,
                           token_causal: bool = False, out_dtype=torch.bfloat16, q_chunk: int = 1024):
    """Oracle A: fp32 softmax attention on the de-quantised operands with the 128x64 block map
    expanded to tokens (spas_sage_attn/utils.py:424-432).  No fp8 rounding of P, no PV skip.
    Also the CPU baseline that the benchmark times."""
    B, H, N, D = q8.shape                                             # N: query rows given (a prefix is allowed)
    NK = k8.shape[2]
    nq, nk = block_map.shape[-2:]
    qd = q8.float() * q_scale.repeat_interleave(BLKQ, dim=-1)[..., :N].unsqueeze(-1)
    kd = k8.float() * k_scale.repeat_interleave(BLKK, dim=-1)[..., :NK].unsqueeze(-1)
    vd = v8[:, :, :NK] * v_scale.unsqueeze(-2)
    o = torch.zeros(B, H, N, D, dtype=torch.float32)
    for r0 in range(0, N, q_chunk):
        r1 = min(r0 + q_chunk, N)
        assert r0 % BLKQ == 0
        bm = block_map[:, :, r0 // BLKQ:(r1 + BLKQ - 1) // BLKQ]
        mask = block_map_to_mask(bm, r1 - r0, NK)
        if token_causal:
            qi = torch.arange(r0, r1).view(-1, 1)
            kj = torch.arange(NK).view(1, -1)
            mask = mask & (kj <= qi)
        s = torch.matmul(qd[:, :, r0:r1], kd.transpose(-1, -2)) * sm_scale
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        p = torch.nan_to_num(p, nan=0.0)                                # rows with no live block -> zeros
        o[:, :, r0:r1] = torch.matmul(p, vd)
    return o.to(out_dtype)


# ----------------------------------------------------------------------------- public API mirrors
def _prologue(q, k, v, tensor_layout):
    """spas_sage_attn/core.py:107-117 -- layout, N>=128 check, dtype normalisation."""
    assert tensor_layout in ["HND", "NHD"]
    if tensor_layout == "NHD":
        q, k, v = (t.transpose(-2, -3) for t in (q, k, v))
    assert q.size(-2) >= 128, "seq_len should be not less than 128."
    dt = torch.float16 if q.dtype in (torch.float32, torch.float16) else torch.bfloat16
    return q.contiguous().to(dt), k.contiguous().to(dt), v.contiguous().to(torch.float16), dt


def spas_sage2_attn_meansim_topk(q, k, v, is_causal=False, scale=None, smooth_k=True, simthreshd1=-0.1,
                                 cdfthreshd=None, topk=0.5, pvthreshd=50, attention_sink=False,
                                 tensor_layout="HND", return_sparsity=False, token_causal=False,
                                 blockwise=True, return_parts=False, pv_fp16=False):
    """spas_sage_attn/core.py:105-169 (and :39-103 when `cdfthreshd` is given instead of `topk`).
    `token_causal=False` reproduces the reference, which never forwards is_causal to its kernel.
    `token_causal=True, pv_fp16=True` is the Sage1-signature path (core.py:235-319): fp16 V, fp16 P.V, is_causal
    forwarded to the kernel."""
    q, k, v, dt = _prologue(q, k, v, tensor_layout)
    H, D = q.shape[1], q.shape[-1]
    assert D in (64, 128)
    km = k_mean(k) if smooth_k else None
    pr = predictor(q, k, km, is_causal, simthreshd1, cdfthreshd, topk, attention_sink)
    sm_scale = scale if scale is not None else 1.0 / math.sqrt(D)
    pv = hyperparameter_check(pvthreshd, H)
    v8, vs = (v.to(torch.float16).float(), None) if pv_fp16 else quant_v(v)
    if blockwise:
        o, _ = attention_blockwise(pr["q_int8"], pr["q_scale"], pr["k_int8"], pr["k_scale"], v8, vs, pr["map"],
                                   sm_scale, pv, token_causal and is_causal, dt, pv_fp16=pv_fp16)
    else:
        assert not pv_fp16
        o = attention_dense_masked(pr["q_int8"], pr["q_scale"], pr["k_int8"], pr["k_scale"], v8, vs, pr["map"],
                                   sm_scale, token_causal and is_causal, dt)
    if tensor_layout == "NHD":
        o = o.transpose(-2, -3)
    nq, nk = pr["map"].shape[-2:]
    B = q.shape[0]
    denom = (nk * nq * B * H) if not is_causal else ((nk + 2) // 2 * nq * B * H)   # core.py:162-167
    sparsity = 1.0 - float(pr["valid"].float().sum()) / denom
    out = (o, sparsity) if return_sparsity else o
    if return_parts:
        pr.update(v8=v8, v_scale=vs, km=km)
        return out, pr
    return out


def block_sparse_sage2_attn(q, k, v, mask_id, scale=None, smooth_k=True, pvthreshd=50, tensor_layout="HND",
                            return_sparsity=False, blockwise=True, return_parts=False):
    """spas_sage_attn/core.py:171-233."""
    q, k, v, dt = _prologue(q, k, v, tensor_layout)
    B, H, N, D = q.shape
    assert D in (64, 128)
    km = k_mean(k) if smooth_k else None
    dummy = torch.zeros(H)
    _, _, q8, qs = pool_sim_quant(q, None, BLKQ, dummy, want_pool=False)
    _, _, k8, ks = pool_sim_quant(k, km, BLKK, dummy, want_pool=False)
    assert mask_id.dim() == 4
    fmap = mask_id != 0
    lut, valid = block_map_to_lut(fmap)
    sm_scale = scale if scale is not None else 1.0 / math.sqrt(D)
    pv = hyperparameter_check(pvthreshd, H)
    v8, vs = quant_v(v)
    if blockwise:
        o, _ = attention_blockwise(q8, qs, k8, ks, v8, vs, fmap, sm_scale, pv, False, dt)
    else:
        o = attention_dense_masked(q8, qs, k8, ks, v8, vs, fmap, sm_scale, False, dt)
    if tensor_layout == "NHD":
        o = o.transpose(-2, -3)
    nq, nk = fmap.shape[-2:]
    sparsity = 1.0 - float(valid.float().sum()) / ((nk + 2) // 2 * nq * B * H)     # core.py:229-231
    out = (o, sparsity) if return_sparsity else o
    if return_parts:
        return out, dict(map=fmap, lut=lut, valid=valid, q_int8=q8, q_scale=qs, k_int8=k8, k_scale=ks,
                         v8=v8, v_scale=vs, km=km)
    return out
