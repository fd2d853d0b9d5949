"""ctypes binding of libsparge_b200.so (the C ABI declared in include/sparge_b200.h).

There is no fallback: if the shared library has not been built, importing this module raises.
Build it with `python spargeattn_b200/build.py`.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsparge_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: the sm_100a CUDA library has not been built. "
        "Run `python spargeattn_b200/build.py` (needs nvcc); there is no CPU or PyTorch fallback.")

lib = ctypes.CDLL(LIB_PATH)

_p, _i, _f, _sz, _ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t, ctypes.c_longlong

# name -> (restype, argtypes); must list every symbol of include/sparge_b200.h
SIGNATURES = {
    "sparge_strerror": (ctypes.c_char_p, [_i]),
    "sparge_abi_version": (_i, []),
    "sparge_k_mean_scratch_bytes": (_sz, [_i, _i, _i, _i]),
    "sparge_k_mean": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _p]),
    "sparge_k_mean_static": (_i, [_p, _p, _i, _i, _i, _i, _i, _p]),
    "sparge_pool_quant": (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p]),
    "sparge_select": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _p]),
    "sparge_mask_to_lut": (_i, [_p, _i, _p, _p, _i, _i, _i, _i, _p]),
    "sparge_quant_v": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _p]),
    "sparge_k_mean_strided": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _ll, _ll, _ll, _p]),
    "sparge_pool_quant_strided": (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _ll, _ll, _ll, _p]),
    "sparge_quant_v_strided": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _ll, _ll, _ll, _p]),
    "sparge_attn_fwd_strided": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _ll, _ll, _ll, _p]),
    "sparge_attn_fwd_pv_count": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _ll, _ll, _ll, _p, _p]),
    "sparge_attn_fwd_rows": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _ll, _ll, _ll, _p, _p, _i, _p]),
    "sparge_attn_fwd_gran": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _ll, _ll, _ll, _p, _p, _i,
                                  _i, _i, _p]),
    "sparge_attn_fwd_f16pv": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _ll, _ll, _ll, _p, _p, _i, _p]),
    "sparge_forward_workspace_bytes": (ctypes.c_size_t, [_i, _i, _i, _i]),
    "sparge_forward_workspace_layout": (_i, [_i, _i, _i, _i, ctypes.POINTER(ctypes.c_size_t), _i]),
    "sparge_meansim_forward": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, ctypes.c_size_t, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i,
                                    _f, ctypes.POINTER(_ll), ctypes.POINTER(_ll), ctypes.POINTER(_ll), ctypes.POINTER(_ll), _p]),
    "sparge_peer_alloc": (_i, [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p]),
    "sparge_peer_free": (_i, [_p]),
    "sparge_peer_open": (_i, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]),
    "sparge_peer_close": (_i, [_p]),
    "sparge_copy_async": (_i, [_p, _p, ctypes.c_size_t, _p]),
    "sparge_copy2d_async": (_i, [_p, ctypes.c_size_t, _p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, _p]),
    "sparge_selftest_wait_expiry": (_i, [_p, ctypes.c_uint, ctypes.c_uint, _p]),
    "sparge_attn_fwd": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _p]),
    "sparge_div_approx": (_i, [_p, _p, _p, _i, _p]),
    "sparge_tensor_peak": (_i, [_i, _i, _i, _i, _p, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_double), _p]),
}
for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args

OK, ERR_INVALID_ARG, ERR_NULL, ERR_CUDA, ERR_TOO_LARGE, ERR_UNSUPPORTED = range(6)
F16, BF16 = 0, 1


def strerror(status: int) -> str:
    return lib.sparge_strerror(status).decode()


def check(status: int, what: str) -> None:
    """Map a status code to the exception class the reference raises for the same mistake:
    bad head_dim / dtype -> ValueError (csrc/pytorch_extensions_utils.cuh:45-98),
    everything else -> RuntimeError (TORCH_CHECK, :25-43)."""
    if status == OK:
        return
    msg = f"{what}: {strerror(status)} (status {status})"
    if status in (ERR_INVALID_ARG, ERR_TOO_LARGE):
        raise ValueError(msg)
    if status == ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(msg)
