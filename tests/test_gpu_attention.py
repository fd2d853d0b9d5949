"""GPU parity of the tcgen05 attention kernel and of the public API against the CPU oracle.

Tolerance (floating point): cosine similarity >= 0.999 and relative L1 <= 1e-2 against the
oracle's block-online emulation evaluated with the same mask and the same quantised operands."""
import pytest
import torch

import sparge_oracle as O

pytestmark = pytest.mark.gpu

COS_MIN = 0.999
L1_MAX = 1e-2


def _check(o_gpu, o_ref):
    m = O.precision_metric(o_gpu.float().cpu(), o_ref.float())
    assert m["Cossim"] >= COS_MIN and m["L1"] <= L1_MAX, m
    return m


def _inputs(B, H, N, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    walk = lambda: torch.cumsum(torch.randn(B, H, N, D, generator=g), dim=2) * 0.1
    q = (torch.randn(B, H, N, D, generator=g) + walk()).to(dtype)
    k = (torch.randn(B, H, N, D, generator=g) + walk() + torch.randn(D, generator=g) * 3).to(dtype)
    v = (torch.randn(B, H, N, D, generator=g) + walk()).to(dtype)
    return q, k, v


def _status_ok():
    from spargeattn_b200 import ops
    ops.check_device_status()


@pytest.mark.parametrize("shape", [(1, 2, 128, 64), (1, 2, 128, 128), (1, 2, 640, 64), (2, 2, 1000, 128),
                                   (1, 4, 2048, 64), (1, 2, 200, 128), (1, 1, 1500, 64)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_topk_api_matches_oracle(shape, dtype):
    import spargeattn_b200 as S
    B, H, N, D = shape
    q, k, v = _inputs(B, H, N, D, dtype, 10)
    (o_ref, sp_ref), parts = O.spas_sage2_attn_meansim_topk(q, k, v, topk=0.5, return_sparsity=True, return_parts=True)
    o, sp = S.spas_sage2_attn_meansim_topk_cuda(q.cuda(), k.cuda(), v.cuda(), topk=0.5, return_sparsity=True)
    _status_ok()
    assert o.dtype == dtype and o.shape == q.shape
    assert abs(sp - sp_ref) < 1e-6
    _check(o, o_ref)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("kernel_causal", [False, True])
def test_causal_variants(D, kernel_causal):
    """Sage2 API: block-level causality only (reference behaviour).  Sage1-signature API: the
    kernel also masks key > query."""
    import spargeattn_b200 as S
    B, H, N = 1, 2, 1100
    q, k, v = _inputs(B, H, N, D, torch.bfloat16, 11)
    o_ref = O.spas_sage2_attn_meansim_topk(q, k, v, is_causal=True, topk=0.5, token_causal=kernel_causal,
                                           pv_fp16=kernel_causal)           # the Sage1 signatures multiply in fp16
    fn = S.spas_sage_attn_meansim_topk_cuda if kernel_causal else S.spas_sage2_attn_meansim_topk_cuda
    o = fn(q.cuda(), k.cuda(), v.cuda(), is_causal=True, topk=0.5)
    _status_ok()
    _check(o, o_ref)


@pytest.mark.parametrize("D", [64, 128])
def test_block_sparse_api_matches_oracle(D):
    import spargeattn_b200 as S
    from spargeattn_b200.synthetic import bernoulli_block_mask
    B, H, N = 2, 2, 1200
    q, k, v = _inputs(B, H, N, D, torch.bfloat16, 12)
    mask = bernoulli_block_mask(B, H, N, 0.4, 3)
    mask[0, 1, 2] = 0                                     # a query block row with no live block -> zeros
    (o_ref, sp_ref), _ = O.block_sparse_sage2_attn(q, k, v, mask, return_sparsity=True, return_parts=True)
    o, sp = S.block_sparse_sage2_attn_cuda(q.cuda(), k.cuda(), v.cuda(), mask_id=mask.cuda(), return_sparsity=True)
    _status_ok()
    assert abs(sp - sp_ref) < 1e-6
    assert torch.count_nonzero(o[0, 1, 256:384]) == 0
    _check(o, o_ref)


@pytest.mark.parametrize("causal", [False, True])
def test_cdf_api_matches_oracle(causal):
    """spas_sage2_attn_meansim_cuda: cdf-threshold selection (what the reference's tuner calls)."""
    import spargeattn_b200 as S
    B, H, N, D = 1, 3, 1300, 128
    q, k, v = _inputs(B, H, N, D, torch.bfloat16, 17)
    cdf = torch.tensor([0.9, 0.95, 0.98])
    (o_ref, sp_ref), _ = O.spas_sage2_attn_meansim_topk(q, k, v, is_causal=causal, simthreshd1=0.6, cdfthreshd=cdf,
                                                        topk=None, return_sparsity=True, return_parts=True)
    o, sp = S.spas_sage2_attn_meansim_cuda(q.cuda(), k.cuda(), v.cuda(), is_causal=causal, simthreshd1=0.6,
                                           cdfthreshd=cdf, return_sparsity=True)
    _status_ok()
    assert abs(sp - sp_ref) < 1e-6
    _check(o, o_ref)


def test_nhd_layout_and_per_head_knobs():
    import spargeattn_b200 as S
    B, H, N, D = 1, 3, 700, 64
    q, k, v = _inputs(B, H, N, D, torch.float16, 13)
    topk = torch.tensor([0.3, 0.5, 0.9])
    o_ref = O.spas_sage2_attn_meansim_topk(q, k, v, topk=topk, simthreshd1=0.3, attention_sink=True)
    nhd = lambda t: t.transpose(1, 2).contiguous().cuda()
    o = S.spas_sage2_attn_meansim_topk_cuda(nhd(q), nhd(k), nhd(v), topk=topk, simthreshd1=0.3, attention_sink=True,
                                           tensor_layout="NHD")
    _status_ok()
    assert o.shape == (B, N, H, D)
    assert o.is_contiguous()                               # written in NHD directly, no permuted copy
    _check(o.transpose(1, 2), o_ref)
    # reading the NHD tensors in place gives the same bytes as the HND-contiguous call
    o_hnd = S.spas_sage2_attn_meansim_topk_cuda(q.cuda(), k.cuda(), v.cuda(), topk=topk, simthreshd1=0.3,
                                                attention_sink=True)
    assert torch.equal(o.transpose(1, 2), o_hnd)
    # a view that cannot be read in place (odd storage offset) is copied, as the reference does
    pad = torch.zeros(B, H, N, D + 1, dtype=q.dtype, device="cuda")
    pad[..., 1:] = q.cuda()
    o_odd = S.spas_sage2_attn_meansim_topk_cuda(pad[..., 1:], k.cuda(), v.cuda(), topk=topk, simthreshd1=0.3,
                                                attention_sink=True)
    assert torch.equal(o_odd, o_hnd)


def test_pv_threshold_skips_blocks():
    """A small pvthreshd makes the kernel skip PV blocks exactly where the oracle does (to tolerance)."""
    import spargeattn_b200 as S
    B, H, N, D = 1, 2, 2048, 64
    q, k, v = _inputs(B, H, N, D, torch.bfloat16, 14)
    q = q * 3                                              # peaky softmax so that skipping actually fires
    for thr in (50.0, 4.0):
        out, parts = O.spas_sage2_attn_meansim_topk(q, k, v, topk=0.6, pvthreshd=thr, return_parts=True)
        o = S.spas_sage2_attn_meansim_topk_cuda(q.cuda(), k.cuda(), v.cuda(), topk=0.6, pvthreshd=thr)
        _status_ok()
        _check(o, out)
    pv = O.hyperparameter_check(4.0, H)
    _, skipped = O.attention_blockwise(parts["q_int8"], parts["q_scale"], parts["k_int8"], parts["k_scale"],
                                       parts["v8"], parts["v_scale"], parts["map"], D ** -0.5, pv)
    assert skipped > 0, "test input does not exercise the skip path"


def test_dense_mask_matches_sdpa():
    """Size-independent property: with every block live the result is ordinary softmax attention."""
    import spargeattn_b200 as S
    B, H, N, D = 1, 4, 4096, 128
    q, k, v = _inputs(B, H, N, D, torch.bfloat16, 15)
    mask = torch.ones(B, H, N // 128, N // 64, dtype=torch.int32)
    o = S.block_sparse_sage2_attn_cuda(q.cuda(), k.cuda(), v.cuda(), mask_id=mask.cuda())
    _status_ok()
    ref = torch.nn.functional.scaled_dot_product_attention(q.cuda().float(), k.cuda().float(), v.cuda().float())
    m = O.precision_metric(o.float().cpu(), ref.cpu())
    assert m["Cossim"] >= 0.995 and m["L1"] <= 0.06, m    # quantisation error of INT8 QK / FP8 PV vs fp32


def test_linearity_in_v():
    """attn(q, k, 2v) == 2 attn(q, k, v) up to fp16 rounding: V scales are per channel and powers of two are exact."""
    import spargeattn_b200 as S
    B, H, N, D = 1, 2, 1024, 128
    q, k, v = _inputs(B, H, N, D, torch.float16, 16)
    o1 = S.spas_sage2_attn_meansim_topk_cuda(q.cuda(), k.cuda(), v.cuda(), topk=0.5)
    o2 = S.spas_sage2_attn_meansim_topk_cuda(q.cuda(), k.cuda(), (v * 2).cuda(), topk=0.5)
    _status_ok()
    assert torch.allclose(o2.float(), 2 * o1.float(), rtol=2e-3, atol=1e-4)


def test_host_front_end_matches_device_call():
    """Pipelined host-buffer entry point: same bytes as one call on device tensors."""
    import spargeattn_b200 as S
    from spargeattn_b200.host import spas_sage2_attn_meansim_topk_host
    B, H, N, D = 2, 5, 900, 64
    q, k, v = _inputs(B, H, N, D, torch.bfloat16, 18)
    topk = torch.tensor([0.3, 0.4, 0.5, 0.6, 0.7])
    ref = S.spas_sage2_attn_meansim_topk_cuda(q.cuda(), k.cuda(), v.cuda(), topk=topk)
    for hpc in (1, 2, 5):
        out = spas_sage2_attn_meansim_topk_host(q.pin_memory(), k.pin_memory(), v.pin_memory(), heads_per_chunk=hpc, topk=topk)
        torch.cuda.synchronize()
        assert torch.equal(out, ref.cpu())
    _status_ok()


def test_concurrent_preparation_gives_the_same_bytes():
    """Mid-sized calls run Q pooling and the V quantiser on side streams beside the K chain: same bytes as the
    one-stream order, also when calls follow each other on different streams."""
    import spargeattn_b200 as S
    from spargeattn_b200 import core
    B, H, N, D = 1, 2, 3000, 128
    q, k, v = (t.cuda() for t in _inputs(B, H, N, D, torch.bfloat16, 20))
    lo, hi, single = core.CONCURRENT_PREP_MIN_ROWS, core.CONCURRENT_PREP_MAX_ROWS, core.SINGLE_CALL_MAX_ROWS
    try:
        core.SINGLE_CALL_MAX_ROWS = 0                                                      # entry by entry
        core.CONCURRENT_PREP_MIN_ROWS, core.CONCURRENT_PREP_MAX_ROWS = 1 << 40, 0          # one stream
        ref = S.spas_sage2_attn_meansim_topk_cuda(q, k, v, topk=0.5)
        ref_c = S.spas_sage2_attn_meansim_topk_cuda(q, k, v, topk=0.5, is_causal=True, pvthreshd=4.0)
        core.CONCURRENT_PREP_MIN_ROWS, core.CONCURRENT_PREP_MAX_ROWS = 0, 1 << 40          # side streams
        outs = []
        other = torch.cuda.Stream()
        for i in range(6):
            with torch.cuda.stream(other if i % 2 else torch.cuda.current_stream()):
                if i % 2:
                    other.wait_stream(torch.cuda.default_stream())
                outs.append(S.spas_sage2_attn_meansim_topk_cuda(q, k, v, topk=0.5))
        out_c = S.spas_sage2_attn_meansim_topk_cuda(q, k, v, topk=0.5, is_causal=True, pvthreshd=4.0)
        torch.cuda.synchronize()
    finally:
        core.CONCURRENT_PREP_MIN_ROWS, core.CONCURRENT_PREP_MAX_ROWS, core.SINGLE_CALL_MAX_ROWS = lo, hi, single
    _status_ok()
    assert all(torch.equal(o, ref) for o in outs) and torch.equal(out_c, ref_c)


@pytest.mark.parametrize("kw", [dict(topk=0.5), dict(topk=0.3, is_causal=True, attention_sink=True), dict(topk=0.6, pvthreshd=4.0),
                                dict(cdfthreshd=0.9, simthreshd1=0.3), dict(topk=0.5, smooth_k=False), dict(topk=0.5, scale=0.07),
                                dict(topk=0.4, tensor_layout="NHD")])
@pytest.mark.parametrize("shape,dtype", [((2, 3, 1100, 64), torch.bfloat16), ((1, 2, 2048, 128), torch.float16)])
def test_single_call_path_equals_the_entry_by_entry_path(kw, shape, dtype):
    """Small problems are issued by one C call (sparge_meansim_forward) instead of nine wrappers: the same kernels in
    the same order on the same stream, so the bytes are the same, for every knob, with and without return_sparsity."""
    import spargeattn_b200 as S
    from spargeattn_b200 import core
    B, H, N, D = shape
    q, k, v = (t.cuda() for t in _inputs(B, H, N, D, dtype, 23))
    kw = dict(kw)
    if kw.get("tensor_layout") == "NHD":
        q, k, v = (t.transpose(1, 2).contiguous() for t in (q, k, v))
    fn = S.spas_sage2_attn_meansim_cuda if "cdfthreshd" in kw else S.spas_sage2_attn_meansim_topk_cuda
    assert B * H * N < core.SINGLE_CALL_MAX_ROWS
    one, sp_one = fn(q, k, v, return_sparsity=True, **kw)
    one2 = fn(q, k, v, **kw)
    single = core.SINGLE_CALL_MAX_ROWS
    try:
        core.SINGLE_CALL_MAX_ROWS = 0
        sep, sp_sep = fn(q, k, v, return_sparsity=True, **kw)
    finally:
        core.SINGLE_CALL_MAX_ROWS = single
    _status_ok()
    assert torch.equal(one, sep) and torch.equal(one2, sep) and sp_one == sp_sep
    assert one.shape == q.shape and one.stride() == sep.stride()


def test_host_front_end_with_partially_owned_heads():
    """Row-sharded host entry point: a rank's units (whole heads and parts of heads) give, on the rows it owns, the
    bytes of the full call; rows it does not own are neither read from q nor written to the result."""
    import spargeattn_b200 as S
    from spargeattn_b200.host import spas_sage2_attn_meansim_topk_host
    from spargeattn_b200.sharding import partition_rows
    B, H, N, D = 1, 3, 1500, 128
    q, k, v = _inputs(B, H, N, D, torch.bfloat16, 19)
    ref = S.spas_sage2_attn_meansim_topk_cuda(q.cuda(), k.cuda(), v.cuda(), topk=0.5).cpu()
    nq = (N + 127) // 128
    seen = torch.zeros(H, N, dtype=torch.bool)
    for units in partition_rows(B, H, nq, 4):
        heads = [h for (_, h, _, _) in units]
        hq, hk, hv = (t[:, heads].contiguous().pin_memory() for t in (q, k, v))
        for i, (_, _, a, n) in enumerate(units):           # rows of q outside the unit must not matter
            hq[0, i, :a * 128] = float("nan")
            hq[0, i, (a + n) * 128:] = float("nan")
        out = torch.full((1, len(units), N, D), -7.0, dtype=torch.bfloat16).pin_memory()
        for hpc in (1, 2):
            spas_sage2_attn_meansim_topk_host(hq, hk, hv, out=out, units=units, heads_per_chunk=hpc, topk=0.5)
            torch.cuda.synchronize()
            for i, (_, h, a, n) in enumerate(units):
                r0, r1 = a * 128, min((a + n) * 128, N)
                assert torch.equal(out[0, i, r0:r1], ref[0, h, r0:r1])
                assert (out[0, i, :r0] == -7.0).all() and (out[0, i, r1:] == -7.0).all()
                seen[h, r0:r1] = True
    assert seen.all()
    _status_ok()


@pytest.mark.parametrize("N", [128, 129, 191, 257])
def test_tiny_and_ragged_lengths(N):
    import spargeattn_b200 as S
    q, k, v = _inputs(1, 2, N, 64, torch.bfloat16, 19)
    o_ref = O.spas_sage2_attn_meansim_topk(q, k, v, topk=0.5)
    o = S.spas_sage2_attn_meansim_topk_cuda(q.cuda(), k.cuda(), v.cuda(), topk=0.5)
    _status_ok()
    _check(o, o_ref)


def test_degenerate_inputs_do_not_stall_or_poison():
    """All-zero tensors, huge magnitudes and a constant K: finite (or zero) outputs, no bounded wait expires."""
    import spargeattn_b200 as S
    B, H, N, D = 1, 2, 640, 128
    z = torch.zeros(B, H, N, D, dtype=torch.bfloat16, device="cuda")
    q, k, v = (t.cuda() for t in _inputs(B, H, N, D, torch.bfloat16, 20))
    o = S.spas_sage2_attn_meansim_topk_cuda(z, z, z, topk=0.5)
    assert torch.count_nonzero(o) == 0
    o = S.spas_sage2_attn_meansim_topk_cuda(q, k, z, topk=0.5)            # all-zero V -> zeros, not NaN
    assert torch.count_nonzero(o) == 0
    S.spas_sage2_attn_meansim_topk_cuda(q * 1e4, k * 1e4, v * 1e3, topk=0.5)   # scores beyond fp32 resolution: only no stall
    kc = torch.ones_like(k)                                                # constant K: smoothed K is all zero
    o = S.spas_sage2_attn_meansim_topk_cuda(q, kc, v, topk=0.5)
    assert torch.isfinite(o.float()).all()
    _status_ok()


@pytest.mark.parametrize("gain", [4.0, 20.0])
def test_large_score_scale_takes_the_exact_exponent_path(gain):
    """Per-block scales above 2^-7 leave the biased-FMA exponent path (its constant would be rounded too
    coarsely) for the exact int->float one; the result must stay within the usual tolerance."""
    import spargeattn_b200 as S
    q, k, v = _inputs(1, 2, 1024, 128, torch.bfloat16, 21)
    q, k = q * gain, k * gain
    o_ref = O.spas_sage2_attn_meansim_topk(q, k, v, topk=0.5)
    o = S.spas_sage2_attn_meansim_topk_cuda(q.cuda(), k.cuda(), v.cuda(), topk=0.5)
    _status_ok()
    _check(o, o_ref)


def test_return_pv_count_matches_oracle_skip_count():
    """`return_pv_count` diagnostic: entries = live blocks minus the blocks dropped by the pvthreshd test."""
    from spargeattn_b200 import ops
    B, H, N, D = 1, 2, 2048, 64
    q, k, v = _inputs(B, H, N, D, torch.bfloat16, 14)
    q = q * 3
    _, parts = O.spas_sage2_attn_meansim_topk(q, k, v, topk=0.6, pvthreshd=4.0, return_parts=True)
    pv = O.hyperparameter_check(4.0, H)
    _, skipped = O.attention_blockwise(parts["q_int8"], parts["q_scale"], parts["k_int8"], parts["k_scale"],
                                       parts["v8"], parts["v_scale"], parts["map"], D ** -0.5, pv)
    lut, valid = O.block_map_to_lut(parts["map"])
    dev = lambda t: t.cuda().contiguous()
    v8_bits = O.e4m3_bits(parts["v8"])
    args = (dev(parts["q_int8"]), dev(parts["k_int8"]), dev(v8_bits), dev(lut.int()), dev(valid.int()))
    scales = (dev(parts["q_scale"]), dev(parts["k_scale"]), dev(parts["v_scale"]))
    # without the test every live block is computed
    _, cnt = ops.attn_fwd(*args, None, *scales, D ** -0.5, False, torch.bfloat16, return_pv_count=True)
    cnt = cnt.cpu().view(B, H, -1, 4)
    assert (cnt == valid.int().unsqueeze(-1)).all()
    # with it: four equal entries per block, never above the live count, total = oracle's (decisions at the
    # threshold may differ by rounding of the running maximum: allow 1 %)
    _, cnt = ops.attn_fwd(*args, dev(pv), *scales, D ** -0.5, False, torch.bfloat16, return_pv_count=True)
    _status_ok()
    cnt = cnt.cpu().view(B, H, -1, 4)
    assert (cnt == cnt[..., :1]).all() and (cnt[..., 0] <= valid.int()).all() and (cnt[..., 0] >= valid.int().clamp(max=2)).all()
    gpu_skipped = int(valid.sum()) - int(cnt[..., 0].sum())
    assert skipped > 0 and abs(gpu_skipped - skipped) <= max(1, skipped // 100), (gpu_skipped, skipped)


@pytest.mark.parametrize("D,causal", [(128, False), (64, False), (128, True)])
def test_row_range_units_equal_the_full_call(D, causal):
    """The multi-GPU row sharding computes a range of query blocks per head: those rows must carry the same bytes
    as the full call, and rows outside the ranges must not be written."""
    import spargeattn_b200 as S
    from spargeattn_b200 import ops
    from spargeattn_b200.sharding import attention_units, partition_rows
    B, H, N = 1, 3, 1500
    q, k, v = (t.cuda() for t in _inputs(B, H, N, D, torch.bfloat16, 31))
    full = S.spas_sage2_attn_meansim_topk_cuda(q, k, v, topk=0.5, is_causal=causal)
    nq = (N + 127) // 128
    got = torch.full_like(full, float("nan"))
    for units in partition_rows(B, H, nq, 4):                      # what each of four ranks would compute
        heads = [h for (_, h, _, _) in units]
        ranges = torch.tensor([[a, n] for (_, _, a, n) in units], dtype=torch.int32).view(1, len(units), 2)
        o = attention_units(q[:, heads], k[:, heads], v[:, heads], ranges, topk=0.5, is_causal=causal)
        _status_ok()
        for i, (_, h, a, n) in enumerate(units):
            r0, r1 = a * 128, min((a + n) * 128, N)
            got[0, h, r0:r1] = o[0, i, r0:r1]
    assert torch.equal(got, full)
    # rows outside a range stay untouched
    buf_ranges = torch.tensor([[[2, 3]] * H], dtype=torch.int32)
    from spargeattn_b200 import core
    o = attention_units(q, k, v, buf_ranges, topk=0.5, is_causal=causal)
    assert torch.equal(o[:, :, 256:640], full[:, :, 256:640])


def _gran_case(N, D, dtype, seed, gran, topk=0.6, causal=False):
    """Operands for the attention entry with per-block / per-warp / per-thread Q/K scales: the block map of the
    predictor, the quantised operands of the granularity's quantiser, FP8 V -- all from the oracle."""
    B, H = 1, 2
    q, k, v = _inputs(B, H, N, D, dtype, seed)
    q = q * 3                                              # peaky softmax: the skip test has something to drop
    km = O.k_mean(k)
    pr = O.predictor(q, k, km, causal, torch.full((H,), -0.1), None, torch.full((H,), topk), False)
    ksm = (k - km).to(dtype)
    if gran == 1:
        q8, qs, k8, ks = pr["q_int8"], pr["q_scale"], pr["k_int8"], pr["k_scale"]
    elif gran == 2:
        q8, qs, k8, ks = O.per_warp_int8(q, ksm)
    else:
        q8, qs, k8, ks = O.per_thread_int8(q, ksm)
    v8, vs = O.quant_v(v)
    lut, valid = O.block_map_to_lut(pr["map"])
    return dict(q=q, ksm=ksm, q8=q8, qs=qs, k8=k8, ks=ks, v8=v8, vs=vs, map=pr["map"], lut=lut.int(), valid=valid.int(), H=H)


@pytest.mark.parametrize("gran", [2, 3])
@pytest.mark.parametrize("N,D,causal", [(1500, 64, False), (1000, 128, False), (900, 128, True)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_per_warp_and_per_thread_scales_match_oracle(gran, N, D, causal, dtype):
    """qk_quant_gran 2 and 3 (csrc/qattn/qk_int_sv_f8_cuda_sm89.cuh:106-136): the kernel applies one Q scale per
    32 rows, or per-thread Q and K scales, exactly where the reference's accumulator layout puts them."""
    from spargeattn_b200 import ops
    c = _gran_case(N, D, dtype, 51, gran, causal=causal)
    dev = lambda t: t.cuda().contiguous()
    o = ops.attn_fwd(dev(c["q8"]), dev(c["k8"]), dev(O.e4m3_bits(c["v8"])), dev(c["lut"]), dev(c["valid"]), None,
                     dev(c["qs"]), dev(c["ks"]), dev(c["vs"]), D ** -0.5, causal, dtype, qk_quant_gran=gran)
    _status_ok()
    ref, _ = O.attention_blockwise(c["q8"], c["qs"], c["k8"], c["ks"], c["v8"], c["vs"], c["map"], D ** -0.5, None,
                                   token_causal=causal, out_dtype=dtype, pv_skip=False, qk_quant_gran=gran)
    _check(o, ref)
    # the finer scales must matter for this input: reading them with the per-block layout gives another result
    if gran == 3:
        wrong, _ = O.attention_blockwise(c["q8"], c["qs"][..., ::32].contiguous(), c["k8"], c["ks"][..., ::4].contiguous(),
                                         c["v8"], c["vs"], c["map"], D ** -0.5, None, token_causal=causal,
                                         out_dtype=dtype, pv_skip=False)
        assert O.precision_metric(o.float().cpu(), wrong.float())["L1"] > 2e-2


def test_per_warp_quantiser_is_bit_exact_and_feeds_granularity_two():
    """per_warp_int8 (spas_sage_attn/quant_per_block.py:102-148): INT8 bytes and scales equal the oracle's, groups
    past the end of the sequence get 1e-7, NHD is a view of the same result; its output runs through the kernel."""
    from spargeattn_b200 import core, ops
    B, H, N, D = 1, 2, 1100, 128
    q, k, v = _inputs(B, H, N, D, torch.bfloat16, 52)
    q8, qs, k8, ks = core.per_warp_int8(q.cuda(), k.cuda())
    q8o, qso, k8o, kso = O.per_warp_int8(q, k)
    assert qs.shape == (B, H, (N + 127) // 128 * 4, 1) and ks.shape == (B, H, (N + 63) // 64, 1)
    assert torch.equal(q8.cpu(), q8o) and torch.equal(k8.cpu(), k8o)
    assert torch.equal(qs.cpu().squeeze(-1), qso) and torch.equal(ks.cpu().squeeze(-1), kso)
    assert float(qso[0, 0, -1]) == pytest.approx(1e-7) and (N + 31) // 32 < qso.shape[-1]
    q8n, qsn, k8n, ksn = core.per_warp_int8(q.transpose(1, 2).contiguous().cuda(), k.transpose(1, 2).contiguous().cuda(),
                                            tensor_layout="NHD")
    assert q8n.shape == (B, N, H, D) and torch.equal(q8n.transpose(1, 2), q8) and torch.equal(qsn, qs)
    with pytest.raises(ValueError):
        core.per_warp_int8(q.cuda(), k.cuda(), tensor_layout="HDN")
    with pytest.raises(ValueError):
        ops.attn_fwd(q8, k8, k8.view(torch.uint8), torch.zeros(B, H, 9, 18, dtype=torch.int32, device="cuda"),
                     torch.zeros(B, H, 9, dtype=torch.int32, device="cuda"), None, qs, ks,
                     torch.ones(B, H, D, device="cuda"), 1.0, False, torch.bfloat16, qk_quant_gran=4)


@pytest.mark.parametrize("gran", [1, 3])
def test_per_warp_pv_threshold_mode_matches_oracle(gran):
    """PVThresholdMode::kPerWarp: each 32-row group drops a block's P.V on its own. The output matches the oracle run
    in that mode, the per-group counts match its counts (decisions at the threshold may differ by rounding: 1 %),
    groups of one block differ from each other, and no group keeps more products than the per-block mode (which
    drops a block only when all four groups would)."""
    from spargeattn_b200 import ops
    N, D, dtype = 2048, 64, torch.bfloat16
    c = _gran_case(N, D, dtype, 14, gran)
    H = c["H"]
    pv = O.hyperparameter_check(4.0, H)
    dev = lambda t: t.cuda().contiguous()
    args = (dev(c["q8"]), dev(c["k8"]), dev(O.e4m3_bits(c["v8"])), dev(c["lut"]), dev(c["valid"]))
    scales = (dev(c["qs"]), dev(c["ks"]), dev(c["vs"]))
    o2, cnt2 = ops.attn_fwd(*args, dev(pv), *scales, D ** -0.5, False, dtype, return_pv_count=True, qk_quant_gran=gran,
                            pv_threshold_mode=2)
    _status_ok()
    o1, cnt1 = ops.attn_fwd(*args, dev(pv), *scales, D ** -0.5, False, dtype, return_pv_count=True, qk_quant_gran=gran,
                            pv_threshold_mode=1)
    o0, cnt0 = ops.attn_fwd(*args, dev(pv), *scales, D ** -0.5, False, dtype, return_pv_count=True, qk_quant_gran=gran,
                            pv_threshold_mode=0)
    _status_ok()
    counts = torch.zeros(1, H, c["valid"].shape[-1] * 4, dtype=torch.int32)
    ref, skipped = O.attention_blockwise(c["q8"], c["qs"], c["k8"], c["ks"], c["v8"], c["vs"], c["map"], D ** -0.5, pv,
                                         out_dtype=dtype, qk_quant_gran=gran, pv_threshold_mode=2, group_counts=counts)
    _check(o2, ref)
    cnt2, cnt1, cnt0 = cnt2.cpu(), cnt1.cpu(), cnt0.cpu()
    live4 = c["valid"].repeat_interleave(4, dim=-1)
    assert torch.equal(cnt0, live4)                                       # mode 0 ignores the threshold
    assert skipped > 0 and int((live4 - counts).sum()) == skipped
    assert abs(int(cnt2.sum()) - int(counts.sum())) <= max(1, skipped // 100), (int(cnt2.sum()), int(counts.sum()))
    assert (cnt2 != counts).float().mean().item() < 0.02
    assert (cnt2 <= cnt1).all() and (cnt1 <= live4).all()                 # the block drops only what every group drops
    per_block = cnt2.view(1, H, -1, 4)
    assert (per_block != per_block[..., :1]).any()                        # the four groups of a block decide differently
    assert int(cnt2.sum()) < int(cnt1.sum()) < int(live4.sum())           # both modes dropped something, per-warp more


def test_partial_last_query_block_never_skips():
    """The reference's skip test takes its maximum over all 128 rows of the Q tile (attn_utils.cuh:418-466 has no row
    mask); rows beyond N are left unfilled by its loader, so its decision in a partial last query block depends on
    stale shared memory. This kernel zero-fills them: zero scores, running maximum 0, difference 0, so the partial
    block keeps every product while full blocks of the same head drop some. Kernel and oracle agree on that."""
    from spargeattn_b200 import ops
    B, H, N, D = 1, 2, 2000, 64                       # 15 full query blocks + one of 80 rows
    q, k, v = _inputs(B, H, N, D, torch.bfloat16, 14)
    q = q * 3
    _, parts = O.spas_sage2_attn_meansim_topk(q, k, v, topk=0.6, pvthreshd=4.0, return_parts=True)
    pv = O.hyperparameter_check(4.0, H)
    nq = (N + 127) // 128
    counts = torch.zeros(B, H, nq * 4, dtype=torch.int32)
    ref, skipped = O.attention_blockwise(parts["q_int8"], parts["q_scale"], parts["k_int8"], parts["k_scale"], parts["v8"],
                                         parts["v_scale"], parts["map"], D ** -0.5, pv, group_counts=counts)
    lut, valid = O.block_map_to_lut(parts["map"])
    dev = lambda t: t.cuda().contiguous()
    o, cnt = ops.attn_fwd(dev(parts["q_int8"]), dev(parts["k_int8"]), dev(O.e4m3_bits(parts["v8"])), dev(lut.int()),
                          dev(valid.int()), dev(pv), dev(parts["q_scale"]), dev(parts["k_scale"]), dev(parts["v_scale"]),
                          D ** -0.5, False, torch.bfloat16, return_pv_count=True)
    _status_ok()
    _check(o, ref)
    cnt = cnt.cpu().view(B, H, nq, 4)
    counts = counts.view(B, H, nq, 4)
    live = valid.int()
    assert skipped > 0 and (cnt[:, :, :-1, 0] < live[:, :, :-1]).any()            # full blocks do drop products
    assert torch.equal(cnt[:, :, -1], live[:, :, -1:].expand(B, H, 4))            # the partial block keeps all
    assert torch.equal(counts[:, :, -1], live[:, :, -1:].expand(B, H, 4))
    assert abs(int(cnt.sum()) - int(counts.sum())) <= max(4, 4 * skipped // 100)


@pytest.mark.parametrize("N,D,causal,topk", [(1500, 128, False, 0.5), (1000, 64, False, 0.6), (900, 128, True, 0.5),
                                             (2100, 64, True, 0.4), (130, 128, False, 1.0), (4096, 128, False, 0.1)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fp16_pv_kernel_matches_oracle(N, D, causal, topk, dtype):
    """The fp16-PV variant (tcgen05 kind::f16; the arithmetic of the reference's Sage1 kernel): unquantised fp16 V,
    P rounded to fp16 without the FP8 offset. Against the oracle in that mode at the attention tolerance; it must
    also be markedly closer to an fp32 attention on the same INT8 Q/K than the FP8 kernel is."""
    from spargeattn_b200 import ops
    B, H = 1, 2
    q, k, v = _inputs(B, H, N, D, dtype, 61)
    km = O.k_mean(k)
    pr = O.predictor(q, k, km, causal, torch.full((H,), -0.1), None, torch.full((H,), topk), False)
    lut, valid = O.block_map_to_lut(pr["map"])
    v16 = v.to(torch.float16)
    dev = lambda t: t.cuda().contiguous()
    args = (dev(pr["q_int8"]), dev(pr["k_int8"]))
    o = ops.attn_fwd_f16pv(*args, dev(v16), dev(lut.int()), dev(valid.int()), None, dev(pr["q_scale"]), dev(pr["k_scale"]),
                           D ** -0.5, causal, dtype)
    _status_ok()
    ref, _ = O.attention_blockwise(pr["q_int8"], pr["q_scale"], pr["k_int8"], pr["k_scale"], v16.float(), None, pr["map"],
                                   D ** -0.5, None, token_causal=causal, out_dtype=dtype, pv_skip=False, pv_fp16=True)
    m = _check(o, ref)
    assert m["L1"] <= 3e-3, m                               # fp16 products: an order of magnitude inside the FP8 bar
    # against exact P and V (fp32 softmax on the de-quantised Q/K under the same mask): fp16 PV is closer than FP8 PV
    v8, vs = O.quant_v(v)
    exact = O.attention_dense_masked(pr["q_int8"], pr["q_scale"], pr["k_int8"], pr["k_scale"], v16.float(),
                                     torch.ones(B, H, D), pr["map"], D ** -0.5, token_causal=causal, out_dtype=torch.float32)
    o8 = ops.attn_fwd(*args, dev(O.e4m3_bits(v8)), dev(lut.int()), dev(valid.int()), None, dev(pr["q_scale"]),
                      dev(pr["k_scale"]), dev(vs), D ** -0.5, causal, dtype)
    e16 = O.precision_metric(o.float().cpu(), exact)["L1"]
    e8 = O.precision_metric(o8.float().cpu(), exact)["L1"]
    assert e16 < 0.5 * e8, (e16, e8)


def test_fp16_pv_skip_counts_and_sage1_api():
    """fp16-PV kernel with the skip test: counts against the oracle in that mode; and the Sage1-signature entry points
    (what the reference serves with its fp16-PV kernel) run it, token-level causal included."""
    import spargeattn_b200 as S
    from spargeattn_b200 import core, ops
    B, H, N, D = 1, 2, 2048, 64
    q, k, v = _inputs(B, H, N, D, torch.bfloat16, 14)
    q = q * 3
    km = O.k_mean(k)
    pr = O.predictor(q, k, km, False, torch.full((H,), -0.1), None, torch.full((H,), 0.6), False)
    lut, valid = O.block_map_to_lut(pr["map"])
    pv = O.hyperparameter_check(4.0, H)
    v16 = v.to(torch.float16)
    dev = lambda t: t.cuda().contiguous()
    o, cnt = ops.attn_fwd_f16pv(dev(pr["q_int8"]), dev(pr["k_int8"]), dev(v16), dev(lut.int()), dev(valid.int()), dev(pv),
                                dev(pr["q_scale"]), dev(pr["k_scale"]), D ** -0.5, False, torch.bfloat16, return_pv_count=True)
    _status_ok()
    counts = torch.zeros(B, H, valid.shape[-1] * 4, dtype=torch.int32)
    ref, skipped = O.attention_blockwise(pr["q_int8"], pr["q_scale"], pr["k_int8"], pr["k_scale"], v16.float(), None,
                                         pr["map"], D ** -0.5, pv, pv_fp16=True, group_counts=counts)
    _check(o, ref)
    assert skipped > 0 and abs(int(cnt.cpu().sum()) - int(counts.sum())) <= max(4, 4 * skipped // 100)
    # public Sage1 signatures: fp16 PV by default, the FP8 kernel when switched off; both near the same answer
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    for causal in (False, True):
        a = S.spas_sage_attn_meansim_topk_cuda(qc, kc, vc, topk=0.6, is_causal=causal)
        try:
            core.SAGE1_FP16_PV = False
            b = S.spas_sage_attn_meansim_topk_cuda(qc, kc, vc, topk=0.6, is_causal=causal)
        finally:
            core.SAGE1_FP16_PV = True
        _status_ok()
        m = O.precision_metric(a.float().cpu(), b.float().cpu())
        assert m["Cossim"] > 0.999 and 1e-4 < m["L1"] < 5e-2, m
        # cdf selection keeps a single block for many rows of blocks here; under the token-level causal mask some
        # rows then see no key at all: they are zeros, never NaN
        c = S.spas_sage_attn_meansim_cuda(qc, kc, vc, is_causal=causal, simthreshd1=0.3, cdfthreshd=0.95)
        assert torch.isfinite(c.float()).all()
        try:
            core.SAGE1_FP16_PV = False
            c8 = S.spas_sage_attn_meansim_cuda(qc, kc, vc, is_causal=causal, simthreshd1=0.3, cdfthreshd=0.95)
        finally:
            core.SAGE1_FP16_PV = True
        assert torch.isfinite(c8.float()).all()
        assert torch.equal((c.float().abs().sum(-1) == 0), (c8.float().abs().sum(-1) == 0))     # the same empty rows
