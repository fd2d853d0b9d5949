"""Runs the compiled, unmodified reference (``oracle/_ref``, built by ``oracle/build_ref.py``) on a CUDA
device and returns its intermediate tensors in this repository's layouts.  TEST INFRASTRUCTURE ONLY:
tests, the golden-fixture generator and the benchmark's reference leg use it; the product never does.

The reference package is called ``spas_sage_attn``; so is this repository's drop-in alias package.
``load()`` therefore imports the reference under that name from ``oracle/_ref`` *first* and refuses to
continue if Python resolved the name to anything else.  The product itself is ``spargeattn_b200`` and
can live in the same process.

Pieces follow spas_sage_attn/core.py:105-169 (top-k API) step by step so that every intermediate can be
compared: the predictor (utils.py:371-421), the V path (core.py:143-151 -> csrc/fused/fused.cu) and the
attention op (core.py:155-156 -> csrc/qattn/qk_int_sv_f8_cuda_sm89.cu:392-585).
"""
from __future__ import annotations

import contextlib
import importlib
import os
import sys
from typing import Optional

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")

# fused.cu:51-55: within each group of 16 tokens, input token t is stored at position PERM16[t]
PERM16 = [0, 1, 4, 5, 8, 9, 12, 13, 2, 3, 6, 7, 10, 11, 14, 15]


def available() -> bool:
    pkg = os.path.join(REF_ROOT, "spas_sage_attn")
    return os.path.isdir(pkg) and any(f.startswith("_qattn") for f in os.listdir(pkg)) \
        and any(f.startswith("_fused") for f in os.listdir(pkg))


_ref = None


def load():
    """Import the reference package (core, utils, the two extensions). Raises if it has not been built."""
    global _ref
    if _ref is not None:
        return _ref
    if not available():
        raise RuntimeError("oracle/_ref is missing: run `python oracle/build_ref.py` where the reference checkout is")
    if "spas_sage_attn" in sys.modules:
        mod = sys.modules["spas_sage_attn"]
        if not os.path.abspath(mod.__file__).startswith(REF_ROOT):
            raise RuntimeError("the alias package spas_sage_attn of this repository is already imported; "
                               "load the reference first or in a separate process")
    sys.path.insert(0, REF_ROOT)
    try:
        pkg = importlib.import_module("spas_sage_attn")
    finally:
        sys.path.remove(REF_ROOT)
    assert os.path.abspath(pkg.__file__).startswith(REF_ROOT), pkg.__file__
    _ref = dict(pkg=pkg, core=importlib.import_module("spas_sage_attn.core"),
                utils=importlib.import_module("spas_sage_attn.utils"),
                qattn=importlib.import_module("spas_sage_attn._qattn"),
                fused=importlib.import_module("spas_sage_attn._fused"))
    return _ref


@contextlib.contextmanager
def stable_sort(enabled: bool = True):
    """utils.py:397 sorts without `stable=True`; the contract of this build is 'ties go to the lower block
    index'.  Inside this context torch.sort is stable, so that the reference's block map is comparable
    bit for bit; outside it the reference runs untouched (used to count how many blocks its tie order flips)."""
    if not enabled:
        yield
        return
    orig = torch.sort

    def _sort(*a, **kw):
        kw.setdefault("stable", True)
        return orig(*a, **kw)

    torch.sort = _sort
    try:
        yield
    finally:
        torch.sort = orig


def prologue(q, k, v):
    """core.py:113-120 -- dtype normalisation and the K mean, exactly as the reference computes them."""
    if q.dtype in (torch.float32, torch.float16):
        q, k, v = q.contiguous().to(torch.float16), k.contiguous().to(torch.float16), v.contiguous().to(torch.float16)
    else:
        q, k, v = q.contiguous().to(torch.bfloat16), k.contiguous().to(torch.bfloat16), v.contiguous().to(torch.float16)
    km = k.mean(dim=-2, keepdim=True)
    return q, k, v, km


def predictor(q, k, km, is_causal=False, simthreshd1=-0.1, cdfthreshd=None, topk=0.5, attention_sink=False,
              stable: bool = True) -> dict:
    """utils.py:371-421 on the device; returns map (bool), lut, valid, q/k int8 + scales, pooled q/k and sim flags."""
    R = load()
    U = R["utils"]
    H = q.size(1)
    thr = U.hyperparameter_check(simthreshd1, H, q.device)
    pq, sim_q, q8, qs = U.get_pool_sim_triton_simmean_fuse_quant(q, None, 128, thr)
    pk, sim_k, k8, ks = U.get_pool_sim_triton_simmean_fuse_quant(k, km, 64, thr)
    with stable_sort(stable):
        fmap, q8b, qsb, k8b, ksb = U.get_block_map_meansim_fuse_quant(
            q, k, km, is_causal=is_causal, simthreshd1=simthreshd1, cdfthreshd=cdfthreshd, topk=topk,
            return_lut=False, attention_sink=attention_sink, BLKQ=128, BLKK=64)
    lut, valid = U.block_map_lut_triton(fmap)
    return dict(map=fmap.bool(), lut=lut, valid=valid, q_int8=q8b, q_scale=qsb, k_int8=k8b, k_scale=ksb,
                pq=pq, pk=pk, sim_q=sim_q, sim_k=sim_k)


def vanilla_quant(q, k, km):
    """utils.py:265-268 (`qk_quantize`, the block-sparse API's quantiser)."""
    return load()["utils"].get_vanilla_qk_quant(q, k, km, 128, 64)


def quant_v(v16: torch.Tensor):
    """core.py:143-151.  Returns (v_fp8 as the reference lays it out [B,H,D,N_pad], v_scale [B,H,D],
    v8 un-permuted and transposed back to this repository's token-major [B,H,N_pad,D] uint8 bytes)."""
    F = load()["fused"]
    b, h, n, d = v16.shape
    npad = (n + 127) // 128 * 128
    vt = torch.empty((b, h, d, npad), dtype=v16.dtype, device=v16.device)
    F.transpose_pad_permute_cuda(v16, vt, 1)
    v8 = torch.empty(vt.shape, dtype=torch.float8_e4m3fn, device=v16.device)
    vs = torch.empty((b, h, d), dtype=torch.float32, device=v16.device)
    F.scale_fuse_quant_cuda(vt, v8, vs, n, 2.25, 1)
    perm = torch.tensor(PERM16, device=v16.device)
    idx = (torch.arange(npad, device=v16.device).view(-1, 16)[:, :1] + perm.view(1, 16)).reshape(-1)
    token_major = v8.view(torch.uint8)[..., idx].transpose(-1, -2).contiguous()
    return v8, vs, token_major


def attention(q8, k8, v_fp8, lut, valid, pvthreshd, q_scale, k_scale, v_scale, sm_scale, out_dtype, is_causal=False,
              qk_quant_gran=1, return_pv_count=False):
    """core.py:155-156: the Sage2++ sm89 op (fp16 PV accumulation); the hot path passes per-block scales
    (qk_quant_gran = 1), the op also takes per-warp (2) and per-thread (3) ones."""
    Q = load()["qattn"]
    o = torch.empty(q8.shape, dtype=out_dtype, device=q8.device)
    cnt = Q.qk_int8_sv_f8_accum_f16_block_sparse_attn_inst_buf_fuse_v_scale_with_pv_threshold(
        q8, k8, v_fp8, o, lut, valid, pvthreshd, q_scale, k_scale, v_scale, 1, int(bool(is_causal)), int(qk_quant_gran),
        float(sm_scale), int(bool(return_pv_count)))
    return (o, cnt) if return_pv_count else o


def per_warp_int8(q, k):
    """quant_per_block.py:102-148 (Triton): INT8 Q with one scale per 32 rows, K with one per 64 keys."""
    import importlib
    mod = importlib.import_module(load()["core"].__package__ + ".quant_per_block")
    q8, qs, k8, ks = mod.per_warp_int8(q, k)
    return q8, qs.squeeze(-1).contiguous(), k8, ks.squeeze(-1).contiguous()


def api_topk(q, k, v, stable: bool = True, **kw):
    """The reference's public entry point, spas_sage2_attn_meansim_topk_cuda (core.py:105-169)."""
    with stable_sort(stable):
        return load()["core"].spas_sage2_attn_meansim_topk_cuda(q, k, v, **kw)


def api_block_sparse(q, k, v, mask_id, **kw):
    """block_sparse_sage2_attn_cuda (core.py:171-233)."""
    return load()["core"].block_sparse_sage2_attn_cuda(q, k, v, mask_id=mask_id, **kw)


def time_ms(fn, warmup: int = 3, steps: int = 10) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps
