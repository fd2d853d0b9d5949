"""GPU parity of the preprocessing kernels against the CPU oracle: bit-exact for INT8 / FP8 /
index outputs.  Every call goes through the C ABI (spargeattn_b200.ops -> libsparge_b200.so)."""
import pytest
import torch

import sparge_oracle as O
from conftest import device_recip_scale

pytestmark = pytest.mark.gpu


def _ops():
    from spargeattn_b200 import ops
    return ops


def _rand_qk(B, H, N, D, dtype, seed, smooth=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, H, N, D, generator=g)
    if smooth:
        x = x + torch.cumsum(torch.randn(B, H, N, D, generator=g), dim=2) * 0.1
    k = torch.randn(B, H, N, D, generator=g) + torch.randn(D, generator=g) * 3
    if smooth:
        k = k + torch.cumsum(torch.randn(B, H, N, D, generator=g), dim=2) * 0.1
    return x.to(dtype), k.to(dtype)


SHAPES = [(1, 2, 128, 64), (1, 2, 200, 128), (2, 3, 640, 64), (1, 2, 1000, 128), (1, 4, 2048, 64), (1, 1, 130, 128)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_k_mean_bit_exact(shape, dtype):
    ops = _ops()
    B, H, N, D = shape
    _, k = _rand_qk(B, H, N, D, dtype, 1)
    km = ops.k_mean(k.cuda()).cpu()
    assert torch.equal(km.view(torch.int16), O.k_mean(k).view(torch.int16))


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("thr", [-0.1, 0.5])
def test_pool_sim_quant_bit_exact(shape, dtype, thr):
    ops = _ops()
    B, H, N, D = shape
    q, k = _rand_qk(B, H, N, D, dtype, 2)
    km = O.k_mean(k)
    thr_t = torch.full((H,), thr)
    for x, mean, bs in ((q, None, 128), (k, km, 64)):
        pool_o, sim_o, x8_o, sc_o = O.pool_sim_quant(x, mean, bs, thr_t)
        pool, sim, x8, sc = ops.pool_sim_quant(x.cuda(), None if mean is None else mean.cuda(), bs, thr_t.cuda())
        assert torch.equal(x8.cpu(), x8_o), f"int8 mismatch count {(x8.cpu() != x8_o).sum().item()}"
        assert torch.equal(sc.cpu(), sc_o)
        assert torch.equal(pool.cpu().view(torch.int16), pool_o.view(torch.int16))
        assert torch.equal(sim.cpu().bool(), sim_o)
        # quantiser-only entry (block-sparse API path, utils.py:89-159) gives the same int8 / scales
        _, _, x8b, scb = ops.pool_sim_quant(x.cuda(), None if mean is None else mean.cuda(), bs, None)
        assert torch.equal(x8b.cpu(), x8_o) and torch.equal(scb.cpu(), sc_o)


def test_pool_sim_zero_rows_and_partial_blocks():
    ops = _ops()
    B, H, N, D = 1, 2, 600, 64
    q, _ = _rand_qk(B, H, N, D, torch.bfloat16, 3)
    q[0, 0, 130] = 0          # an all-zero token makes its block non-self-similar
    thr = torch.full((H,), -0.1)
    pool_o, sim_o, x8_o, sc_o = O.pool_sim_quant(q, None, 128, thr)
    pool, sim, x8, sc = ops.pool_sim_quant(q.cuda(), None, 128, thr.cuda())
    assert not sim_o[0, 0, 1] and not sim_o[0, 0, -1] and sim_o[0, 1, 1]
    assert torch.equal(sim.cpu().bool(), sim_o) and torch.equal(x8.cpu(), x8_o)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_quant_v_bit_exact(shape, dtype):
    ops = _ops()
    B, H, N, D = shape
    g = torch.Generator().manual_seed(4)
    v = (torch.randn(B, H, N, D, generator=g) * torch.rand(D, generator=g) * 4).to(dtype)
    v[..., 3] = 0             # all-zero channel: zeros out, not NaN
    v8_o, vs_o = O.quant_v(v, device_recip_scale(v))
    v8, vs = ops.quant_v(v.cuda())
    assert torch.equal(vs.cpu(), vs_o)
    assert v8.shape == v8_o.shape
    assert torch.equal(v8.cpu(), O.e4m3_bits(v8_o)), f"{(v8.cpu() != O.e4m3_bits(v8_o)).sum().item()} fp8 bytes differ"


def test_quant_v_rounding_boundaries():
    """Products that sit just beside an e4m3 rounding tie (the instruction rounds through fp16)."""
    ops = _ops()
    B, H, N, D = 1, 1, 16384, 64
    g = torch.Generator().manual_seed(7)
    v = torch.randn(B, H, N, D, generator=g).to(torch.float16)
    v[0, 0, 0] = 2.25                                      # amax = 2.25 -> multiplier exactly 1
    ties = torch.tensor([1.0625, 1.1875, 0.40625, 0.0068359375, 1.6875, 0.84375])
    v[0, 0, 1:7, :] = ties.view(6, 1).to(torch.float16)
    v[0, 0, 7:13, :] = (ties * (1 + 2.0 ** -10)).view(6, 1).to(torch.float16)
    v[0, 0, 13:19, :] = (ties * (1 - 2.0 ** -11)).view(6, 1).to(torch.float16)
    v8_o, vs_o = O.quant_v(v, device_recip_scale(v))
    v8, vs = ops.quant_v(v.cuda())
    assert torch.equal(vs.cpu(), vs_o) and torch.equal(v8.cpu(), O.e4m3_bits(v8_o))


@pytest.mark.parametrize("shape", SHAPES + [(1, 2, 4096, 64)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal,sink,topk", [(False, False, 0.5), (True, False, 0.5), (False, True, 0.25), (True, True, 0.7)])
def test_select_mask_and_lut_bit_exact(shape, dtype, causal, sink, topk):
    ops = _ops()
    B, H, N, D = shape
    q, k = _rand_qk(B, H, N, D, dtype, 5)
    km = O.k_mean(k)
    thr = torch.full((H,), 0.2)
    topk_t = torch.full((H,), topk)
    pr = O.predictor(q, k, km, causal, thr, None, topk_t, sink)
    lut, valid, mask = ops.select_blocks(pr["pq"].cuda(), pr["pk"].cuda(), pr["sim_q"].to(torch.uint8).cuda(),
                                         pr["sim_k"].to(torch.uint8).cuda(), topk_t.cuda(), None, causal, sink,
                                         want_mask=True)
    assert torch.equal(mask.cpu().bool(), pr["map"]), f"{(mask.cpu().bool() != pr['map']).sum().item()} blocks differ"
    assert torch.equal(valid.cpu(), pr["valid"])
    assert torch.equal(lut.cpu(), pr["lut"])


@pytest.mark.parametrize("shape", [(1, 2, 640, 64), (2, 3, 1000, 128), (1, 2, 4096, 64), (1, 1, 8192, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal,cdf", [(False, 0.9), (True, 0.98), (False, 0.5), (False, 1.5), (False, 0.0)])
def test_select_cdf_mode_bit_exact(shape, dtype, causal, cdf):
    ops = _ops()
    B, H, N, D = shape
    q, k = _rand_qk(B, H, N, D, dtype, 8)
    km = O.k_mean(k)
    thr = torch.full((H,), 0.3)
    cdf_t = torch.full((H,), cdf)
    pr = O.predictor(q, k, km, causal, thr, cdf_t, None, False)
    lut, valid, mask = ops.select_blocks(pr["pq"].cuda(), pr["pk"].cuda(), pr["sim_q"].to(torch.uint8).cuda(),
                                         pr["sim_k"].to(torch.uint8).cuda(), None, cdf_t.cuda(), causal, False,
                                         want_mask=True)
    assert torch.equal(mask.cpu().bool(), pr["map"]), f"{(mask.cpu().bool() != pr['map']).sum().item()} blocks differ"
    assert torch.equal(valid.cpu(), pr["valid"]) and torch.equal(lut.cpu(), pr["lut"])


def test_select_best_first_order_is_a_permutation_of_the_reference_lut():
    ops = _ops()
    B, H, N, D = 2, 2, 3000, 64
    q, k = _rand_qk(B, H, N, D, torch.bfloat16, 9)
    pr = O.predictor(q, k, O.k_mean(k), False, torch.full((H,), 0.2), None, torch.full((H,), 0.4), False)
    args = (pr["pq"].cuda(), pr["pk"].cuda(), pr["sim_q"].to(torch.uint8).cuda(), pr["sim_k"].to(torch.uint8).cuda(),
            torch.full((H,), 0.4).cuda(), None, False, False)
    lut_a, valid_a, _ = ops.select_blocks(*args, best_first=False)
    lut_b, valid_b, _ = ops.select_blocks(*args, best_first=True)
    assert torch.equal(valid_a, valid_b) and torch.equal(lut_a.cpu(), pr["lut"])
    idx_a, idx_b = torch.cumsum(lut_a.cpu(), -1), torch.cumsum(lut_b.cpu(), -1)
    p = pr["p"].float()
    for b in range(B):
        for h in range(H):
            for r in range(idx_a.shape[2]):
                n = int(valid_a[b, h, r])
                a, bb = idx_a[b, h, r, :n], idx_b[b, h, r, :n]
                assert torch.equal(torch.sort(bb).values, a)                      # same set of blocks
                assert torch.equal(bb[1:], a[a != bb[0]])                          # the rest stays ascending
                best = p[b, h, r, a]
                assert bb[0] == a[torch.argmax(best)]                             # highest probability, lowest index on ties
                assert (lut_b[b, h, r, n:] == 0).all()


def test_select_ties_go_to_lower_index():
    """Identical pooled keys give identical probabilities: the stable order must keep the lowest indices."""
    ops = _ops()
    B, H, nq, nk, D = 1, 1, 2, 16, 64
    pq = torch.randn(B, H, nq, D).bfloat16()
    pk = torch.randn(1, 1, 1, D).bfloat16().expand(B, H, nk, D).contiguous()
    simq = torch.ones(B, H, nq, dtype=torch.uint8)
    simk = torch.ones(B, H, nk, dtype=torch.uint8)
    topk = torch.full((H,), 0.25)
    lut, valid, mask = ops.select_blocks(pq.cuda(), pk.cuda(), simq.cuda(), simk.cuda(), topk.cuda(), None, False, False, True)
    assert mask.cpu()[0, 0].tolist() == [[1] * 4 + [0] * 12] * 2
    assert valid.cpu().tolist() == [[[4, 4]]]


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64, torch.uint8, torch.bool, torch.float32])
def test_mask_to_lut_matches_oracle(dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(6)
    m = (torch.rand(2, 3, 9, 19, generator=g) < 0.4)
    m[0, 0, 0] = False        # empty row
    m[0, 0, 1] = True         # full row
    lut_o, valid_o = O.block_map_to_lut(m)
    lut, valid = ops.mask_to_lut(m.to(dtype).cuda())
    assert torch.equal(lut.cpu(), lut_o) and torch.equal(valid.cpu(), valid_o)
