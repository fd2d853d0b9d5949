"""GPU test of the allocation-free K-mean entry point (collected last on purpose).

`sparge_k_mean_static` serves hosts that cannot allocate device memory when they call in (their
framework owns the whole GPU, or an allocation would stall a latency-critical loop): its scratch is a
fixed array inside the library instead of a caller buffer.  The test drives it through the C ABI twice
in a row, with different shapes so that the second call reuses scratch the first one dirtied, and
expects exactly the bytes that `sparge_k_mean` (caller-provided scratch) produces.  It also checks the
size limit.  It must pass both alone in a fresh process and after every other test."""
import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_MAX_BYTES = 8 << 20


def _both(k):
    from spargeattn_b200 import _cabi, ops
    B, H, N, D = k.shape
    dt = _cabi.BF16 if k.dtype == torch.bfloat16 else _cabi.F16
    stream = torch.cuda.current_stream().cuda_stream
    ref = ops.k_mean(k)                                     # existing entry point, torch-allocated scratch
    out = torch.full_like(ref, float("nan"))
    before = torch.cuda.memory_allocated()
    status = _cabi.lib.sparge_k_mean_static(k.data_ptr(), out.data_ptr(), B, H, N, D, dt, stream)
    assert status == _cabi.OK, _cabi.strerror(status)
    assert torch.cuda.memory_allocated() == before          # nothing came from torch's allocator either
    torch.cuda.synchronize()
    return out, ref


def test_static_scratch_matches_regular_entry_point_twice():
    g = torch.Generator().manual_seed(21)
    k1 = (torch.randn(2, 3, 5000, 128, generator=g) + 2.0).to(torch.bfloat16).cuda()
    k2 = (torch.randn(1, 4, 777, 64, generator=g) * 3 - 1.0).to(torch.float16).cuda()
    for k in (k1, k2):                                      # two calls in a row share the same scratch array
        out, ref = _both(k)
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16))   # integer-exact, as in the other K-mean tests


def test_static_scratch_rejects_oversized_requests():
    from spargeattn_b200 import _cabi
    B, H, N, D = 4, 64, 40000, 128
    assert _cabi.lib.sparge_k_mean_scratch_bytes(B, H, N, D) > STATIC_MAX_BYTES
    dummy = torch.empty(16, device="cuda")
    status = _cabi.lib.sparge_k_mean_static(dummy.data_ptr(), dummy.data_ptr(), B, H, N, D, _cabi.BF16, None)
    assert status == _cabi.ERR_TOO_LARGE
    assert "exceeds" in _cabi.strerror(status)
