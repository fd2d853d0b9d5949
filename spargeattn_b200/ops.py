"""Tensor-level wrappers over the C ABI: allocate outputs with torch, pass raw pointers and the
current CUDA stream.  These mirror the helper functions of the reference's
spas_sage_attn/utils.py (get_pool_sim_triton_simmean_fuse_quant :270-280, get_quant :255-263,
block_map_lut_triton :76-87) and the `_fused` / `_qattn` extension calls in core.py:143-158."""
import threading
from typing import Optional, Tuple

import torch

from . import _cabi

BLKQ, BLKK = 128, 64
_status_words = {}


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return _cabi.F16
    if t.dtype == torch.bfloat16:
        return _cabi.BF16
    raise ValueError(f"expected a float16 or bfloat16 tensor, got {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_launch = threading.local()


def _stream(t: torch.Tensor):
    s = getattr(_launch, "stream", None)
    return (s if s is not None else torch.cuda.current_stream(t.device)).cuda_stream


class launch_on:
    """Within this context the wrappers of this module launch their kernels on `stream` while their outputs are
    still allocated from the current stream's pool: the caller orders `stream` after the current stream before
    and the current stream after `stream` behind the block, so the tensors live and die like any other tensor
    of the current stream (no cross-stream bookkeeping in the allocator)."""

    def __init__(self, stream):
        self.stream = stream

    def __enter__(self):
        self.prev = getattr(_launch, "stream", None)
        _launch.stream = self.stream
        return self

    def __exit__(self, *exc):
        _launch.stream = self.prev
        return False


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("spargeattn_b200 runs on CUDA tensors only (no CPU path)")
        if t is not None and not t.is_contiguous():
            raise RuntimeError("expected a contiguous tensor")


def strided_ok(t: torch.Tensor) -> bool:
    """True if a [B,H,N,D] view can be read in place: last dim contiguous, 16-byte aligned rows."""
    return (t.dim() == 4 and t.stride(-1) == 1 and t.data_ptr() % 16 == 0
            and all(st % 8 == 0 and st >= 0 for st in t.stride()[:3]) and t.stride(2) > 0)


def _need_strided(t):
    if not t.is_cuda:
        raise RuntimeError("spargeattn_b200 runs on CUDA tensors only (no CPU path)")
    if not strided_ok(t):
        raise RuntimeError("expected a [B,H,N,D] view with contiguous last dimension, 16-byte aligned")


def device_status_word(device) -> torch.Tensor:
    """One int32 per device that sparge_attn_fwd writes when a bounded in-kernel wait expires."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _status_words:
        # host tensor + blocking copy: the word is zero on the device before any stream can launch a kernel on it
        _status_words[key] = torch.zeros(1, dtype=torch.int32).to(f"cuda:{key}")
    return _status_words[key]


def check_device_status(device=None) -> int:
    """Synchronising read of the device status word; raises if a kernel reported a timeout."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    code = int(device_status_word(dev).item())
    if code != 0:
        raise RuntimeError(f"sparge_attn_fwd reported device status {code} (a bounded wait expired)")
    return code


def k_mean(k: torch.Tensor) -> torch.Tensor:
    _need_strided(k)
    B, H, N, D = k.shape
    km = torch.empty(B, H, 1, D, dtype=k.dtype, device=k.device)
    nbytes = _cabi.lib.sparge_k_mean_scratch_bytes(B, H, N, D)
    scratch = torch.empty(max(nbytes, 8), dtype=torch.uint8, device=k.device)
    _cabi.check(_cabi.lib.sparge_k_mean_strided(_ptr(k), _ptr(km), _ptr(scratch), B, H, N, D, _dt(k), k.stride(0),
                                                k.stride(1), k.stride(2), _stream(k)), "sparge_k_mean")
    return km


def pool_sim_quant(x: torch.Tensor, km: Optional[torch.Tensor], block: int, simthreshd1: Optional[torch.Tensor]):
    """Returns (pool, sim, x_int8, scale); pool and sim are None when simthreshd1 is None."""
    _need_strided(x)
    _need_cuda(km, simthreshd1)
    B, H, N, D = x.shape
    # 32-row groups (per-warp granularity of Q, quantiser only) are counted per 128-row block: four each
    nb = (N + 127) // 128 * 4 if block == 32 else (N + block - 1) // block
    x8 = torch.empty(B, H, N, D, dtype=torch.int8, device=x.device)
    scale = torch.empty(B, H, nb, dtype=torch.float32, device=x.device)
    pool = sim = None
    if simthreshd1 is not None:
        pool = torch.empty(B, H, nb, D, dtype=x.dtype, device=x.device)
        sim = torch.empty(B, H, nb, dtype=torch.uint8, device=x.device)
    _cabi.check(_cabi.lib.sparge_pool_quant_strided(_ptr(x), _ptr(km), _ptr(simthreshd1), _ptr(pool), _ptr(sim),
                                                    _ptr(x8), _ptr(scale), B, H, N, D, block, _dt(x), x.stride(0),
                                                    x.stride(1), x.stride(2), _stream(x)), "sparge_pool_quant")
    return pool, sim, x8, scale


def select_blocks(pq, pk, sim_q, sim_k, topk: Optional[torch.Tensor], cdfthreshd: Optional[torch.Tensor],
                  is_causal: bool, attention_sink: bool, want_mask: bool = False, best_first: bool = False):
    """Returns (lut, valid, mask-or-None). best_first=False gives the reference's ascending LUT."""
    _need_cuda(pq, pk, sim_q, sim_k, topk, cdfthreshd)
    B, H, nq, D = pq.shape
    nk = pk.shape[2]
    lut = torch.empty(B, H, nq, nk, dtype=torch.int32, device=pq.device)
    valid = torch.empty(B, H, nq, dtype=torch.int32, device=pq.device)
    mask = torch.empty(B, H, nq, nk, dtype=torch.uint8, device=pq.device) if want_mask else None
    _cabi.check(_cabi.lib.sparge_select(_ptr(pq), _ptr(pk), _ptr(sim_q), _ptr(sim_k), _ptr(topk), _ptr(cdfthreshd),
                                        _ptr(mask), _ptr(lut), _ptr(valid), B, H, nq, nk, D, _dt(pq),
                                        int(bool(is_causal)), int(bool(attention_sink)), int(bool(best_first)),
                                        _stream(pq)), "sparge_select")
    return lut, valid, mask


def mask_to_lut(block_map: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    assert block_map.dim() == 4
    assert block_map.is_contiguous()
    _need_cuda(block_map)
    if block_map.dtype == torch.bool:
        block_map = block_map.view(torch.uint8)
    elif block_map.dtype.is_floating_point:
        block_map = (block_map != 0).view(torch.uint8)   # -0.0 must count as false
    B, H, nq, nk = block_map.shape
    lut = torch.empty(B, H, nq, nk, dtype=torch.int32, device=block_map.device)
    valid = torch.empty(B, H, nq, dtype=torch.int32, device=block_map.device)
    _cabi.check(_cabi.lib.sparge_mask_to_lut(_ptr(block_map), block_map.element_size(), _ptr(lut), _ptr(valid), B, H,
                                             nq, nk, _stream(block_map)), "sparge_mask_to_lut")
    return lut, valid


def quant_v(v: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """v [B,H,N,D] fp16/bf16 -> (v8 uint8 [B,H,N_pad,D] e4m3 bytes, v_scale [B,H,D])."""
    _need_strided(v)
    B, H, N, D = v.shape
    npad = (N + 127) // 128 * 128
    v8 = torch.empty(B, H, npad, D, dtype=torch.uint8, device=v.device)
    vs = torch.empty(B, H, D, dtype=torch.float32, device=v.device)
    _cabi.check(_cabi.lib.sparge_quant_v_strided(_ptr(v), _ptr(v8), _ptr(vs), B, H, N, D, _dt(v), v.stride(0), v.stride(1),
                                                 v.stride(2), _stream(v)), "sparge_quant_v")
    return v8, vs


def div_approx(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Elementwise a / b as the GPU's `div.approx.ftz.f32` evaluates it (fp32 CUDA tensors of one shape)."""
    _need_cuda(a, b)
    assert a.dtype == torch.float32 and b.dtype == torch.float32 and a.shape == b.shape
    out = torch.empty_like(a)
    _cabi.check(_cabi.lib.sparge_div_approx(_ptr(a), _ptr(b), _ptr(out), a.numel(), _stream(a)), "sparge_div_approx")
    return out


def attn_fwd(q8, k8, v8, lut, valid, pvthreshd: Optional[torch.Tensor], q_scale, k_scale, v_scale, sm_scale: float,
             is_causal: bool, out_dtype: torch.dtype, out: Optional[torch.Tensor] = None,
             return_pv_count: bool = False, q_block_ranges: Optional[torch.Tensor] = None, q_blocks_max: int = 0,
             qk_quant_gran: int = 1, pv_threshold_mode: Optional[int] = None):
    """Block-sparse attention. With `return_pv_count` also returns int32 [B, H, ceil(N/128)*4]: per 32-row group the
    number of P.V products computed (the `return_pv_count` diagnostic of csrc/qattn/qk_int_sv_f8_cuda_sm89.cu:526-584).
    `q_block_ranges` (int32 [B, H, 2] on the device: first query block, count) restricts each head to a range of
    128-row query blocks; the other rows of the output are left untouched. `q_blocks_max` >= the largest count.
    `qk_quant_gran` 1 / 2 / 3: per-block, per-warp or per-thread Q/K scales; `pv_threshold_mode` 0 none, 1 per block,
    2 per 32-row group (default: 1 when `pvthreshd` is given, else 0) -- csrc/qattn/attn_utils.cuh:45-63."""
    _need_cuda(q8, k8, v8, lut, valid, pvthreshd, q_scale, k_scale, v_scale, q_block_ranges)
    B, H, N, D = q8.shape
    if out is None:
        out = torch.empty(B, H, N, D, dtype=out_dtype, device=q8.device)
    _need_strided(out)
    status = device_status_word(q8.device)
    pv_count = torch.empty(B, H, (N + 127) // 128 * 4, dtype=torch.int32, device=q8.device) if return_pv_count else None
    if q_block_ranges is not None:
        assert q_block_ranges.dtype == torch.int32 and q_block_ranges.numel() == 2 * B * H and q_blocks_max > 0
    if pv_threshold_mode is None:
        pv_threshold_mode = 0 if pvthreshd is None else 1
    nq, nk = (N + 127) // 128, (N + 63) // 64
    want = {1: (nq, nk), 2: (nq * 4, nk), 3: (nq * 32, nk * 4)}.get(qk_quant_gran)
    if want is None:
        raise ValueError(f"Unsupported qk_quant_gran: {qk_quant_gran}")      # as DISPATCH_QK_QUANT_GRAN does
    assert q_scale.numel() == B * H * want[0] and k_scale.numel() == B * H * want[1], "scale shapes do not match qk_quant_gran"
    _cabi.check(_cabi.lib.sparge_attn_fwd_gran(_ptr(q8), _ptr(k8), _ptr(v8), _ptr(out), _ptr(lut), _ptr(valid),
                                               _ptr(pvthreshd), _ptr(q_scale), _ptr(k_scale), _ptr(v_scale),
                                               _ptr(status), B, H, N, D, _dt(out), int(bool(is_causal)),
                                               float(sm_scale), out.stride(0), out.stride(1), out.stride(2),
                                               _ptr(pv_count), _ptr(q_block_ranges), int(q_blocks_max),
                                               int(qk_quant_gran), int(pv_threshold_mode), _stream(q8)),
                "sparge_attn_fwd")
    return (out, pv_count) if return_pv_count else out


def attn_fwd_f16pv(q8, k8, v16, lut, valid, pvthreshd: Optional[torch.Tensor], q_scale, k_scale, sm_scale: float,
                   is_causal: bool, out_dtype: torch.dtype, out: Optional[torch.Tensor] = None,
                   return_pv_count: bool = False, q_block_ranges: Optional[torch.Tensor] = None, q_blocks_max: int = 0):
    """Block-sparse attention with fp16 P and V (the reference's fp16-PV op, core.py:263): v16 is fp16 [B,H,N,D],
    contiguous; everything else as attn_fwd with per-block scales."""
    _need_cuda(q8, k8, v16, lut, valid, pvthreshd, q_scale, k_scale, q_block_ranges)
    assert v16.dtype == torch.float16 and v16.is_contiguous(), "v must be a contiguous fp16 [B,H,N,D] tensor"
    B, H, N, D = q8.shape
    assert tuple(v16.shape) == (B, H, N, D)
    if out is None:
        out = torch.empty(B, H, N, D, dtype=out_dtype, device=q8.device)
    _need_strided(out)
    status = device_status_word(q8.device)
    pv_count = torch.empty(B, H, (N + 127) // 128 * 4, dtype=torch.int32, device=q8.device) if return_pv_count else None
    if q_block_ranges is not None:
        assert q_block_ranges.dtype == torch.int32 and q_block_ranges.numel() == 2 * B * H and q_blocks_max > 0
    _cabi.check(_cabi.lib.sparge_attn_fwd_f16pv(_ptr(q8), _ptr(k8), _ptr(v16), _ptr(out), _ptr(lut), _ptr(valid),
                                                _ptr(pvthreshd), _ptr(q_scale), _ptr(k_scale), _ptr(status), B, H, N, D,
                                                _dt(out), int(bool(is_causal)), float(sm_scale), out.stride(0),
                                                out.stride(1), out.stride(2), _ptr(pv_count), _ptr(q_block_ranges),
                                                int(q_blocks_max), _stream(q8)), "sparge_attn_fwd_f16pv")
    return (out, pv_count) if return_pv_count else out


_forward_ws = {}
WS_PARTS = ("km", "scratch", "pq", "pk", "sim_q", "sim_k", "q_int8", "k_int8", "q_scale", "k_scale", "lut", "valid", "v8", "v_scale")


def meansim_forward(q, k, v, out, simthreshd1, cdfthreshd, topk, pvthreshd, sm_scale: float, is_causal: bool,
                    kernel_causal: bool, attention_sink: bool, smooth_k: bool):
    """The whole path in one C call (sparge_meansim_forward). q, k, v, out: [B,H,N,D] views with a contiguous last
    dimension; the knob tensors are fp32 [H] on the device. Returns (out, workspace, offsets): the intermediates
    (WS_PARTS, byte offsets) stay valid until the next call of this function on the same stream."""
    import ctypes
    _need_strided(q), _need_strided(k), _need_strided(v), _need_strided(out)
    _need_cuda(simthreshd1, cdfthreshd, topk, pvthreshd)
    B, H, N, D = q.shape
    stream = _stream(q)
    key = (q.device.index, stream)
    nbytes = int(_cabi.lib.sparge_forward_workspace_bytes(B, H, N, D))
    ws = _forward_ws.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = _forward_ws[key] = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    st3 = lambda t: (ctypes.c_longlong * 3)(t.stride(0), t.stride(1), t.stride(2))
    _cabi.check(_cabi.lib.sparge_meansim_forward(
        _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(simthreshd1), _ptr(cdfthreshd), _ptr(topk), _ptr(pvthreshd), _ptr(ws),
        nbytes, _ptr(device_status_word(q.device)), B, H, N, D, _dt(q), _dt(v), int(bool(is_causal)), int(bool(kernel_causal)),
        int(bool(attention_sink)), int(bool(smooth_k)), float(sm_scale), st3(q), st3(k), st3(v), st3(out), stream),
        "sparge_meansim_forward")
    offs = (ctypes.c_size_t * len(WS_PARTS))()
    _cabi.check(_cabi.lib.sparge_forward_workspace_layout(B, H, N, D, offs, len(WS_PARTS)), "sparge_forward_workspace_layout")
    return out, ws, dict(zip(WS_PARTS, list(offs)))


def tensor_peak(kind: str = "i8", n: int = 128, ctas_per_sm: int = 2, target_ms: float = 50.0, device=None) -> dict:
    """Sustained tcgen05.mma rate of the current device for 8-bit operands (M = 128, N = n, K = 32 per
    instruction, operands resident in shared memory): {"tops", "ms", "kind", "n", "ctas_per_sm"}.
    A first short run sizes the timed one to about `target_ms`."""
    import ctypes
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    code = {"i8": 0, "f8": 1}[kind]
    status = device_status_word(dev)
    ms, nops = ctypes.c_float(), ctypes.c_double()
    stream = torch.cuda.current_stream(dev).cuda_stream

    def run(iters):
        _cabi.check(_cabi.lib.sparge_tensor_peak(code, n, ctas_per_sm, iters, _ptr(status), ctypes.byref(ms),
                                                 ctypes.byref(nops), stream), "sparge_tensor_peak")
        return float(ms.value), float(nops.value)

    with torch.cuda.device(dev):
        t, _ = run(4096)
        iters = int(max(4096, min(1 << 22, 4096 * target_ms / max(t, 1e-3))))
        t, total = run(iters)
    return {"tops": total / (t * 1e-3) / 1e12, "ms": t, "kind": kind, "n": n, "ctas_per_sm": ctas_per_sm}
