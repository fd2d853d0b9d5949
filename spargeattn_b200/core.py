"""Public operator API: the five functions of the reference's spas_sage_attn/core.py with the same
names, signatures, defaults, assertions and return values, served by the sm_100a kernels.

Differences from the reference, all deliberate:
  * work is queued on PyTorch's current stream (the reference launches on the legacy default
    stream, csrc/qattn/qk_int_sv_f8_cuda_sm89.cuh:780);
  * V is consumed in its 16-bit input type and rounded to fp16 inside the quantiser instead of
    being cast by torch first (same values, two fewer passes over V);
  * `smooth_k=False` works (the reference raises NameError: `km` is undefined, core.py:119-128);
  * query rows whose block row has no live block are zeros, not uninitialised memory;
  * an all-zero V channel yields zeros instead of NaN.
"""
import torch

from . import ops

# The reference's Sage2 entry points pass the literal False in the kernel's is_causal slot
# (spas_sage_attn/core.py:154-158, :221-225): causality is enforced per block by the predictor
# only, and rows inside a diagonal block still see later keys of that block.  False keeps that
# behaviour; True additionally masks key > query inside the kernel.
SAGE2_TOKEN_LEVEL_CAUSAL = False

# The Sage1-signature entry points of the reference (core.py:235-319) keep V in fp16 and run an fp16 P.V kernel.
# True: they run the fp16-PV variant of the attention kernel here as well (about 1.2x the FP8 kernel's time);
# False: they share the FP8-PV kernel of the Sage2 entry points (faster; output within cosine 0.9996 but only
# 1.4-2.4 % relative L1 of the reference's, because V and P are rounded to e4m3).
SAGE1_FP16_PV = True


_knob_cache = {}


def hyperparameter_check(hyper, H, device):
    """spas_sage_attn/utils.py:38-50. Scalar knobs are materialised once per (value, H, device) and reused:
    the tensors are read-only inputs of the kernels, and small calls are otherwise launch-bound."""
    if type(hyper) == float or type(hyper) == int:
        key = (float(hyper), H, str(device))
        cached = _knob_cache.get(key)
        if cached is None:
            # built on the host and copied with a blocking transfer: the cached tensor is complete before any
            # stream can read it (a fill kernel queued on the stream of the first caller would not be ordered
            # with later callers on other streams). The first use of a knob value should precede graph capture.
            cached = torch.full((H,), float(hyper), dtype=torch.float32).to(device)
            if len(_knob_cache) < 256:
                _knob_cache[key] = cached
        return cached
    elif isinstance(hyper, torch.Tensor):
        assert len(hyper.shape) <= 1, "Hyperparameter tensor must be 1D"
        if len(hyper.shape) == 0:
            hyper = torch.full((H,), hyper.item(), device=device)
        assert hyper.numel() == H, f"Hyperparameter tensor must have {H} elements, but has {hyper.numel()}"
        hyper = hyper.to(device)
    else:
        print(hyper)
        raise ValueError("Hyperparameter must be a float or a tensor")
    return hyper.to(torch.float32).contiguous()


# A PV block is skipped when every row's new maximum is at least pvthreshd (in log2 units) below
# the running one (qk_int_sv_f8_cuda_sm89.cuh:353).  From 8.807 + 10 = 18.8 upward every probability
# of such a block rounds to zero in e4m3 anyway, so with a scalar threshold this large the kernel
# variant without the test produces the same output (the denominators differ by < 2^-30 relative).
PV_SKIP_NEVER_FIRES_FROM = 30.0


def _pv_threshold_tensor(pvthreshd, H, device):
    if type(pvthreshd) in (int, float) and float(pvthreshd) >= PV_SKIP_NEVER_FIRES_FROM:
        return None
    return hyperparameter_check(pvthreshd, H, device)


def _prologue(q, k, v, tensor_layout):
    """spas_sage_attn/core.py:107-117."""
    assert tensor_layout in ['HND', 'NHD']
    if tensor_layout == 'NHD':
        q, k, v = (t.transpose(-2, -3) for t in (q, k, v))
    assert q.size(-2) >= 128, "seq_len should be not less than 128."
    torch.cuda.set_device(v.device)
    dtype = q.dtype
    qk_dtype = torch.float16 if dtype in (torch.float32, torch.float16) else torch.bfloat16

    def prep(t, want):
        # The kernels read any [B,H,N,D] view with a contiguous last dimension in place (an "NHD" tensor seen
        # through transpose is such a view); only other layouts / dtypes are copied, as the reference always does.
        if want is not None and t.dtype != want:
            t = t.to(want)
        return t if ops.strided_ok(t) else t.contiguous()

    q, k = prep(q, qk_dtype), prep(k, qk_dtype)
    v = prep(v, None if v.dtype in (torch.float16, torch.bfloat16) else torch.float16)
    return q, k, v


def _empty_like_layout(q):
    """Output buffer [B,H,N,D] in q's memory format (HND-contiguous, or NHD storage seen through a transpose)."""
    B, H, N, D = q.shape
    if q.stride(1) == D and q.stride(2) == H * D and q.stride(0) == N * H * D:
        return torch.empty(B, N, H, D, dtype=q.dtype, device=q.device).transpose(1, 2)
    return torch.empty(B, H, N, D, dtype=q.dtype, device=q.device)


_SIDE_STREAMS = {}
# The three preparation chains of a call (K mean -> K pooling / quantisation; Q pooling / quantisation; V quantiser)
# are independent until the selection and the attention kernel. For a share of a few heads (what a rank owns under
# row sharding on many GPUs) no single one of these kernels fills the GPU, and running the chains on three streams
# shortens the call; for a whole multi-head problem every kernel fills all CTA slots by itself and the extra
# streams only add event traffic (measured: 3.006 against 3.03 ms for 12 heads of 32 760 tokens, 56.4 against 55.6 ms
# for 24 heads of 119 056), and a handful of short launches is bound by the host's launch rate, which events
# worsen. Hence the window, in (batch * heads * tokens) rows.
CONCURRENT_PREP_MIN_ROWS = 16384
CONCURRENT_PREP_MAX_ROWS = 163840
# Below the window the whole path is issued by one C call (sparge_meansim_forward): 0.14 ms of a [1, 4, 2048, 64] call
# were the interpreter walking through nine wrappers.
SINGLE_CALL_MAX_ROWS = CONCURRENT_PREP_MIN_ROWS


def _side_streams(device):
    """Two streams per device for the independent preparation steps of one call, created once."""
    key = torch.device(device).index
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = (torch.cuda.Stream(device), torch.cuda.Stream(device))
    return _SIDE_STREAMS[key]


def _run_beside(side, fn):
    """Runs the kernels of fn() on stream `side`, ordered after everything enqueued on the current stream so far.
    Returns (result, event): the caller makes the current stream wait for the event before it uses the result.
    The outputs are allocated from the current stream's pool (only the launches move), so they are recycled like
    any other tensor of that stream."""
    main = torch.cuda.current_stream(side.device)
    start = torch.cuda.Event()
    start.record(main)
    side.wait_event(start)
    with ops.launch_on(side):
        out = fn()
    done = torch.cuda.Event()
    done.record(side)
    return out, done


def get_block_map_meansim_fuse_quant(q, k, km=None, is_causal=False, BLKQ=128, BLKK=64, simthreshd1=0.1,
                                     cdfthreshd=0.9, topk=None, is_sparse=True, return_lut=False,
                                     attention_sink=False, best_first=False, q_stream=None):
    """spas_sage_attn/utils.py:371-421. `best_first` (not in the reference) reorders each LUT row so that the
    block with the largest pooled probability is visited first; the selected set is unchanged. `q_stream`: a
    second stream on which Q is pooled and quantised while the current one does the same for K."""
    assert (cdfthreshd is None and topk is not None) \
        or (cdfthreshd is not None and topk is None), "Only one of cdfthreshd and topk can be set."
    assert BLKQ == 128 and BLKK == 64, "this build fixes the sparsity block at 128 x 64"
    Headnum = q.size(1)
    simthreshd1 = hyperparameter_check(simthreshd1, Headnum, q.device)
    if cdfthreshd is not None:
        cdfthreshd = hyperparameter_check(cdfthreshd, Headnum, q.device)
    if topk is not None:
        topk = hyperparameter_check(topk, Headnum, q.device)
    if q_stream is None:
        pooled_q, sim_q, q_int8, q_scale = ops.pool_sim_quant(q, None, BLKQ, simthreshd1)
        pooled_k, sim_k, k_int8, k_scale = ops.pool_sim_quant(k, km, BLKK, simthreshd1)
    else:
        (pooled_q, sim_q, q_int8, q_scale), q_done = _run_beside(q_stream, lambda: ops.pool_sim_quant(q, None, BLKQ, simthreshd1))
        pooled_k, sim_k, k_int8, k_scale = ops.pool_sim_quant(k, km, BLKK, simthreshd1)
        torch.cuda.current_stream(q.device).wait_event(q_done)
    lut, valid_block_num, final_map = ops.select_blocks(pooled_q, pooled_k, sim_q, sim_k, topk, cdfthreshd, is_causal,
                                                        attention_sink, want_mask=not return_lut,
                                                        best_first=best_first and return_lut)
    if not return_lut:
        return final_map.bool(), q_int8, q_scale, k_int8, k_scale
    return lut, valid_block_num, q_int8, q_scale, k_int8, k_scale


def get_vanilla_qk_quant(q, k, km=None, BLKQ=128, BLKK=64):
    """spas_sage_attn/utils.py:265-268."""
    _, _, q_int8, q_scale = ops.pool_sim_quant(q, None, BLKQ, None)
    _, _, k_int8, k_scale = ops.pool_sim_quant(k, km, BLKK, None)
    return q_int8, q_scale, k_int8, k_scale


def per_warp_int8(q, k, BLKQ=128, WARPQ=32, BLKK=64, WARPK=64, tensor_layout="HND"):
    """spas_sage_attn/quant_per_block.py:102-148 -- INT8 Q with one scale per 32 rows, K with one per 64 keys (the
    operands of qk_quant_gran = 2); no mean subtraction. Returns (q_int8, q_scale [B,H,ceil(N/128)*4,1], k_int8,
    k_scale [B,H,ceil(N/64),1]); the INT8 tensors have the inputs' shape."""
    assert (BLKQ, WARPQ, BLKK, WARPK) == (128, 32, 64, 64), "the attention kernel's tiling: 128/32 query rows, 64 keys"
    if tensor_layout not in ("HND", "NHD"):
        raise ValueError(f"Unknown tensor layout: {tensor_layout}")
    if tensor_layout == "NHD":
        q, k = q.transpose(1, 2), k.transpose(1, 2)
    _, _, q_int8, q_scale = ops.pool_sim_quant(q, None, WARPQ, None)
    _, _, k_int8, k_scale = ops.pool_sim_quant(k, None, WARPK, None)
    if tensor_layout == "NHD":
        q_int8, k_int8 = q_int8.transpose(1, 2), k_int8.transpose(1, 2)
    return q_int8, q_scale.unsqueeze(-1), k_int8, k_scale.unsqueeze(-1)


def block_map_lut_triton(block_map):
    """spas_sage_attn/utils.py:76-87 (name kept for callers; nothing here uses Triton)."""
    return ops.mask_to_lut(block_map)


def _sparsity(valid_block_num, lut, causal_denominator):
    """spas_sage_attn/core.py:162-167, :229-231."""
    if not causal_denominator:
        denom = lut.size(3) * lut.size(2) * lut.size(0) * lut.size(1)
    else:
        denom = (lut.size(3) + 2) // 2 * lut.size(2) * lut.size(0) * lut.size(1)
    return (1 - (valid_block_num.float().sum()) / denom).item()


def _meansim_attention(q, k, v, is_causal, scale, smooth_k, simthreshd1, cdfthreshd, topk, pvthreshd, attention_sink,
                       tensor_layout, return_sparsity, kernel_causal, q_block_ranges=None, q_blocks_max=0,
                       pv_fp16=False):
    """The path of spas_sage_attn/core.py:105-169. `q_block_ranges` (int32 [B,H,2]: first 128-row query block, count)
    makes the attention kernel compute only those rows of each head (the multi-GPU row sharding); everything
    before the attention kernel still covers the whole head, since every query block needs all keys.
    `pv_fp16`: V stays fp16 and the kernel multiplies fp16 P by fp16 V (core.py:246-263, the Sage1 signatures)."""
    q, k, v = _prologue(q, k, v, tensor_layout)
    headdim = q.size(-1)
    assert headdim in [64, 128], "headdim should be in [64, 128]. For other headdim, you can use padding and specify the softmax scale."
    rows = q.size(0) * q.size(1) * q.size(2)
    if rows < SINGLE_CALL_MAX_ROWS and q_block_ranges is None and not pv_fp16:
        # a handful of short launches: issued by one C call, the interpreter's share of the time is what matters here
        B_, H_, N_, _ = q.shape
        thr = hyperparameter_check(simthreshd1, H_, q.device)
        cdf = None if cdfthreshd is None else hyperparameter_check(cdfthreshd, H_, q.device)
        tk = None if topk is None else hyperparameter_check(topk, H_, q.device)
        assert (cdf is None) != (tk is None), "Only one of cdfthreshd and topk can be set."
        pv = _pv_threshold_tensor(pvthreshd, H_, q.device)
        o, ws, offs = ops.meansim_forward(q, k, v, _empty_like_layout(q), thr, cdf, tk, pv,
                                          scale if scale is not None else 1.0 / (headdim ** 0.5), bool(is_causal),
                                          kernel_causal, attention_sink, smooth_k)
        if tensor_layout == 'NHD':
            o = o.transpose(-2, -3)
        if return_sparsity:
            nq, nk = (N_ + 127) // 128, (N_ + 63) // 64
            valid = ws[offs["valid"]:offs["valid"] + B_ * H_ * nq * 4].view(torch.int32)
            denom = nk * nq * B_ * H_ if is_causal is False else (nk + 2) // 2 * nq * B_ * H_     # core.py:162-167
            return o, (1 - valid.float().sum() / denom).item()
        return o
    beside = CONCURRENT_PREP_MIN_ROWS <= rows <= CONCURRENT_PREP_MAX_ROWS
    s_q, s_v = _side_streams(q.device) if beside else (None, None)
    if pv_fp16:
        v16 = v.to(torch.float16).contiguous()             # core.py:246-248: V is cast to fp16 whatever the input type
    elif beside:
        (v_fp8, v_scale), v_done = _run_beside(s_v, lambda: ops.quant_v(v))
    km = ops.k_mean(k) if smooth_k else None
    pvthreshd = _pv_threshold_tensor(pvthreshd, q.size(-3), q.device)
    # The PV-skip rule depends on the visiting order (it exempts the last two live blocks), so the
    # best-first order is used only when the skip test is compiled out.
    lut, valid_block_num, q_int8, q_scale, k_int8, k_scale = get_block_map_meansim_fuse_quant(
        q, k, km, is_causal=is_causal, simthreshd1=simthreshd1, cdfthreshd=cdfthreshd, topk=topk, return_lut=True,
        attention_sink=attention_sink, BLKQ=128, BLKK=64, best_first=pvthreshd is None, q_stream=s_q)
    if scale is None:
        scale = 1.0 / (headdim ** 0.5)
    if pv_fp16:
        o = ops.attn_fwd_f16pv(q_int8, k_int8, v16, lut, valid_block_num, pvthreshd, q_scale, k_scale, scale,
                               kernel_causal, q.dtype, out=_empty_like_layout(q), q_block_ranges=q_block_ranges,
                               q_blocks_max=q_blocks_max)
    else:
        if beside:
            torch.cuda.current_stream(q.device).wait_event(v_done)
        else:
            v_fp8, v_scale = ops.quant_v(v)
        o = ops.attn_fwd(q_int8, k_int8, v_fp8, lut, valid_block_num, pvthreshd, q_scale, k_scale, v_scale, scale,
                         kernel_causal, q.dtype, out=_empty_like_layout(q), q_block_ranges=q_block_ranges,
                         q_blocks_max=q_blocks_max)
    if tensor_layout == 'NHD':
        o = o.transpose(-2, -3)
    if return_sparsity:
        return o, _sparsity(valid_block_num, lut, is_causal is not False)
    return o


@torch.compiler.disable
def spas_sage2_attn_meansim_cuda(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, smooth_k=True,
                                 simthreshd1=0.6, cdfthreshd=0.98, pvthreshd=50, attention_sink=False,
                                 tensor_layout="HND", output_dtype=torch.float16, return_sparsity=False):
    """spas_sage_attn/core.py:39-103 -- cdf-threshold selection, INT8 QK / FP8 PV."""
    return _meansim_attention(q, k, v, is_causal, scale, smooth_k, simthreshd1, cdfthreshd, None, pvthreshd,
                              attention_sink, tensor_layout, return_sparsity,
                              bool(is_causal) and SAGE2_TOKEN_LEVEL_CAUSAL)


@torch.compiler.disable
def spas_sage2_attn_meansim_topk_cuda(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None,
                                      smooth_k=True, simthreshd1=-0.1, cdfthreshd=None, topk=0.5, pvthreshd=50,
                                      attention_sink=False, tensor_layout="HND", output_dtype=torch.float16,
                                      return_sparsity=False):
    """spas_sage_attn/core.py:105-169 -- top-k selection, INT8 QK / FP8 PV."""
    return _meansim_attention(q, k, v, is_causal, scale, smooth_k, simthreshd1, cdfthreshd, topk, pvthreshd,
                              attention_sink, tensor_layout, return_sparsity,
                              bool(is_causal) and SAGE2_TOKEN_LEVEL_CAUSAL)


@torch.compiler.disable
def block_sparse_sage2_attn_cuda(q, k, v, mask_id=None, dropout_p=0.0, scale=None, smooth_k=True, pvthreshd=50,
                                 attention_sink=False, tensor_layout="HND", output_dtype=torch.float16,
                                 return_sparsity=False):
    """spas_sage_attn/core.py:171-233 -- attention under a user-supplied 128x64 block mask."""
    q, k, v = _prologue(q, k, v, tensor_layout)
    km = ops.k_mean(k) if smooth_k else None
    headdim = q.size(-1)
    q_int8, q_scale, k_int8, k_scale = get_vanilla_qk_quant(q, k, km, 128, 64)
    assert mask_id is not None, "mask_id is required"
    lut, valid_block_num = block_map_lut_triton(block_map=mask_id)
    if scale is None:
        scale = 1.0 / (headdim ** 0.5)
    assert headdim in [64, 128], "headdim should be in [64, 128]. For other headdim, you can use padding and specify the softmax scale."
    pvthreshd = _pv_threshold_tensor(pvthreshd, q.size(-3), q.device)
    v_fp8, v_scale = ops.quant_v(v)
    o = ops.attn_fwd(q_int8, k_int8, v_fp8, lut, valid_block_num, pvthreshd, q_scale, k_scale, v_scale, scale, False,
                     q.dtype, out=_empty_like_layout(q))
    if tensor_layout == 'NHD':
        o = o.transpose(-2, -3)
    if return_sparsity:
        return o, _sparsity(valid_block_num, lut, True)   # core.py:229-231 always uses the causal denominator
    return o


@torch.compiler.disable
def spas_sage_attn_meansim_cuda(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, smooth_k=True,
                                simthreshd1=0.6, cdfthreshd=0.98, pvthreshd=50, attention_sink=False,
                                tensor_layout="HND", output_dtype=torch.float16, return_sparsity=False):
    """spas_sage_attn/core.py:235-276 -- Sage1 signature (cdf selection).  The reference runs its fp16-PV
    mma.sync kernel here on unquantised fp16 V and forwards is_causal to it; this build runs the fp16-PV
    variant of the tcgen05 kernel (SAGE1_FP16_PV = False: the FP8-PV kernel) with token-level causal masking."""
    return _meansim_attention(q, k, v, is_causal, scale, smooth_k, simthreshd1, cdfthreshd, None, pvthreshd,
                              attention_sink, tensor_layout, return_sparsity, bool(is_causal), pv_fp16=SAGE1_FP16_PV)


@torch.compiler.disable
def spas_sage_attn_meansim_topk_cuda(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None,
                                     smooth_k=True, simthreshd1=-0.1, cdfthreshd=None, topk=0.5, pvthreshd=50,
                                     attention_sink=False, tensor_layout="HND", output_dtype=torch.float16,
                                     return_sparsity=False):
    """spas_sage_attn/core.py:278-319 -- Sage1 signature (top-k selection), token-level causal, fp16 P.V."""
    return _meansim_attention(q, k, v, is_causal, scale, smooth_k, simthreshd1, cdfthreshd, topk, pvthreshd,
                              attention_sink, tensor_layout, return_sparsity, bool(is_causal), pv_fp16=SAGE1_FP16_PV)
