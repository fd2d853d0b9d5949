"""CPU tests of the drop-in boundary: the shared library loads, exports every symbol the header
declares, and rejects bad arguments with a status code before touching the GPU."""
import ctypes
import inspect
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "sparge_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sparge_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from spargeattn_b200 import _cabi
    syms = _declared_symbols()
    assert len(syms) >= 9
    for s in syms:
        assert hasattr(_cabi.lib, s), f"{s} is declared in include/sparge_b200.h but not exported"
        assert s in _cabi.SIGNATURES, f"{s} has no ctypes signature"
    assert _cabi.lib.sparge_abi_version() == 1
    assert _cabi.strerror(0) == "ok"


def test_null_and_bad_arguments_return_status_codes():
    from spargeattn_b200 import _cabi
    L = _cabi.lib
    one = ctypes.c_void_p(16)     # never dereferenced: validation fails first
    assert L.sparge_k_mean(None, one, one, 1, 1, 128, 64, 0, None) == _cabi.ERR_NULL
    assert L.sparge_k_mean(one, one, one, 1, 1, 128, 96, 0, None) == _cabi.ERR_INVALID_ARG
    assert L.sparge_k_mean(one, one, one, 1, 1, 128, 64, 7, None) == _cabi.ERR_INVALID_ARG
    assert L.sparge_pool_quant(one, None, None, None, None, None, one, 1, 1, 128, 64, 128, 0, None) == _cabi.ERR_NULL
    assert L.sparge_pool_quant(one, None, None, None, None, one, one, 1, 1, 128, 64, 48, 0, None) == _cabi.ERR_INVALID_ARG
    # 32-row groups are a quantiser granularity (per-warp Q scales): no pooling / self-similarity for them
    assert L.sparge_pool_quant(one, None, one, one, one, one, one, 1, 1, 128, 64, 32, 0, None) == _cabi.ERR_UNSUPPORTED
    assert L.sparge_pool_quant(one, None, one, None, None, one, one, 1, 1, 128, 64, 64, 0, None) == _cabi.ERR_NULL
    assert L.sparge_select(one, one, one, one, one, one, None, one, one, 1, 1, 1, 2, 64, 0, 0, 0, 0, None) == _cabi.ERR_INVALID_ARG
    assert L.sparge_select(one, one, one, one, None, None, None, one, one, 1, 1, 1, 2, 64, 0, 0, 0, 0, None) == _cabi.ERR_INVALID_ARG
    assert L.sparge_mask_to_lut(one, 3, one, one, 1, 1, 1, 2, None) == _cabi.ERR_INVALID_ARG
    assert L.sparge_quant_v(one, one, None, 1, 1, 128, 64, 0, None) == _cabi.ERR_NULL
    assert L.sparge_quant_v(one, one, one, 70000, 1, 128, 64, 0, None) == _cabi.ERR_TOO_LARGE
    assert L.sparge_attn_fwd(one, one, one, one, one, one, None, one, one, one, None, 1, 1, 128, 48, 1, 0, 0.125, None) \
        == _cabi.ERR_INVALID_ARG
    assert L.sparge_attn_fwd(one, one, one, None, one, one, None, one, one, one, None, 1, 1, 128, 64, 1, 0, 0.125, None) \
        == _cabi.ERR_NULL
    gran = lambda g, mode, thr: L.sparge_attn_fwd_gran(one, one, one, one, one, one, thr, one, one, one, None, 1, 1, 128, 64, 1, 0,
                                                       0.125, 8192, 8192, 64, None, None, 0, g, mode, None)
    assert gran(0, 0, None) == _cabi.ERR_INVALID_ARG and gran(4, 0, None) == _cabi.ERR_INVALID_ARG   # unknown granularity
    assert gran(1, 3, None) == _cabi.ERR_INVALID_ARG                                                   # unknown skip mode
    assert gran(2, 2, None) == _cabi.ERR_NULL                                                          # a mode without thresholds
    assert L.sparge_attn_fwd_gran(one, one, one, one, one, one, None, one, ctypes.c_void_p(20), one, None, 1, 1, 128, 64, 1, 0,
                                  0.125, 8192, 8192, 64, None, None, 0, 3, 0, None) == _cabi.ERR_INVALID_ARG   # K scales not 16-byte aligned
    assert L.sparge_k_mean_scratch_bytes(1, 12, 32760, 128) == 12 * 64 * 128 * 8
    with pytest.raises(ValueError):
        _cabi.check(_cabi.ERR_INVALID_ARG, "x")
    with pytest.raises(RuntimeError):
        _cabi.check(_cabi.ERR_CUDA, "x")


def test_public_signatures_match_reference():
    """Names, parameter order and defaults of spas_sage_attn/core.py:39,105,171,235,278."""
    import spas_sage_attn as A
    import spargeattn_b200 as S
    common = ["q", "k", "v", "attn_mask", "dropout_p", "is_causal", "scale", "smooth_k", "simthreshd1", "cdfthreshd"]
    tail = ["pvthreshd", "attention_sink", "tensor_layout", "output_dtype", "return_sparsity"]
    sig = inspect.signature(S.spas_sage2_attn_meansim_topk_cuda)
    assert list(sig.parameters) == common + ["topk"] + tail
    d = {k: v.default for k, v in sig.parameters.items()}
    assert d["simthreshd1"] == -0.1 and d["cdfthreshd"] is None and d["topk"] == 0.5 and d["pvthreshd"] == 50
    assert d["tensor_layout"] == "HND" and d["smooth_k"] is True and d["is_causal"] is False
    sig = inspect.signature(S.spas_sage2_attn_meansim_cuda)
    assert list(sig.parameters) == common + tail
    assert sig.parameters["simthreshd1"].default == 0.6 and sig.parameters["cdfthreshd"].default == 0.98
    sig = inspect.signature(S.block_sparse_sage2_attn_cuda)
    assert list(sig.parameters) == ["q", "k", "v", "mask_id", "dropout_p", "scale", "smooth_k", "pvthreshd",
                                    "attention_sink", "tensor_layout", "output_dtype", "return_sparsity"]
    for name in ("spas_sage2_attn_meansim_cuda", "spas_sage2_attn_meansim_topk_cuda", "block_sparse_sage2_attn_cuda",
                 "spas_sage_attn_meansim_cuda", "spas_sage_attn_meansim_topk_cuda"):
        assert getattr(A, name) is getattr(S, name)


def test_cpu_tensors_are_rejected_not_silently_computed():
    import spargeattn_b200 as S
    q = torch.randn(1, 2, 256, 64).bfloat16()
    with pytest.raises((RuntimeError, AssertionError, ValueError)):   # torch.cuda.set_device(cpu) raises first
        S.spas_sage2_attn_meansim_topk_cuda(q, q, q)


def test_api_assertions_match_reference():
    import spargeattn_b200 as S
    q = torch.randn(1, 2, 64, 64).bfloat16()
    with pytest.raises(AssertionError, match="seq_len should be not less than 128"):
        S.spas_sage2_attn_meansim_topk_cuda(q, q, q)
    with pytest.raises(AssertionError):
        S.spas_sage2_attn_meansim_topk_cuda(q, q, q, tensor_layout="BAD")
    from spargeattn_b200.core import hyperparameter_check
    with pytest.raises(ValueError):
        hyperparameter_check("x", 2, "cpu")
    with pytest.raises(AssertionError):
        hyperparameter_check(torch.ones(3), 2, "cpu")
    assert hyperparameter_check(0.5, 3, "cpu").tolist() == [0.5] * 3
    assert hyperparameter_check(torch.tensor(0.25), 2, "cpu").tolist() == [0.25] * 2


def test_product_does_not_import_the_oracle():
    import pathlib
    for p in pathlib.Path(ROOT, "spargeattn_b200").rglob("*.py"):
        assert "oracle" not in p.read_text().replace("the oracle", ""), p


def test_integration_stub_compiles_against_the_header(tmp_path):
    """The reference-side binding shown in INTEGRATION.md is compiled (syntax and types only) against the real header
    with a minimal stand-in for torch::Tensor: every call in the document matches the declared signatures."""
    import shutil
    import subprocess
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    blocks = re.findall(r"```cpp\n(.*?)```", text, flags=re.S)
    stub = [b for b in blocks if "sparge_topk_forward" in b]
    assert len(stub) == 1
    prelude = """
#include <cstdint>
namespace at { enum ScalarType { kHalf, kBFloat16 };
  struct Tensor { long size(int) const; void* data_ptr() const; template <class T> T* data_ptr() const; ScalarType scalar_type() const; };
  namespace cuda { struct Stream { void* stream() const; }; Stream getCurrentCUDAStream(); } }
namespace torch { using Tensor = at::Tensor; }
"""
    src = tmp_path / "stub.cpp"
    src.write_text(prelude + stub[0])
    r = subprocess.run([gxx, "-std=c++17", "-fsyntax-only", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
