"""Generate golden fixtures for the attention op's finer scale granularities from the compiled reference on a CUDA device.

Run once on a machine with a GPU and `oracle/_ref` (built by `oracle/build_ref.py`):

    python tests/golden/make_ref_gpu_gran_golden.py [out_dir]        # default: tests/golden

Per case (seeded inputs of `make_ref_gpu_golden.ref_gpu_inputs`, Q scaled by 3 so that the skip test fires):
  * the reference's Triton `per_warp_int8` (quant_per_block.py:102-148) on Q and the mean-smoothed K: INT8 bytes and
    scales (qk_quant_gran = 2 operands);
  * the reference op qk_int8_sv_f8_accum_f16_block_sparse_attn_inst_buf_fuse_v_scale_with_pv_threshold with
    qk_quant_gran = 2 on those operands and with qk_quant_gran = 3 on per-thread operands (the reference has no
    per-thread quantiser: they come from the CPU oracle's `per_thread_int8` and are not stored, tests rebuild them),
    both with pvthreshd = 4 and return_pv_count: outputs and counts.
Block map, LUT and FP8 V are the reference's own (stable sort); the map and the V quotient 2.25 / amax are stored.
"""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

CASES = [
    # name, B, H, N, D, topk, pvthreshd, seed
    ("n1000_d128", 1, 2, 1000, 128, 0.5, 4.0, 31),
    ("n1500_d64", 1, 2, 1500, 64, 0.6, 4.0, 32),
]


def main(out_dir):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    sys.path.insert(0, HERE)
    import ref_runner as RR
    RR.load()
    sys.path.insert(0, ROOT)
    from spargeattn_b200 import ops
    import sparge_oracle as O
    from make_ref_gpu_golden import ref_gpu_inputs
    dev = torch.device("cuda", 0)
    os.makedirs(out_dir, exist_ok=True)
    for name, B, H, N, D, topk, pv, seed in CASES:
        for dtype, tag in ((torch.bfloat16, "bf16"), (torch.float16, "fp16")):
            q, k, v = ref_gpu_inputs(B, H, N, D, dtype, seed)
            q = q * 3
            qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
            rq, rk, rv16, km = RR.prologue(qd, kd, vd)
            pr = RR.predictor(rq, rk, km, False, -0.1, None, topk, False, stable=True)
            v8_perm, vs, _ = RR.quant_v(rv16)
            amax = rv16.float().abs().amax(dim=-2)
            recip = ops.div_approx(torch.full_like(amax, 2.25), amax)
            ksm = (rk - km).to(rk.dtype).contiguous()
            q8, qs, k8, ks = RR.per_warp_int8(rq, ksm)
            pv_t = torch.full((H,), pv, dtype=torch.float32, device=dev)
            sm = D ** -0.5
            o2, c2 = RR.attention(q8, k8, v8_perm, pr["lut"], pr["valid"], pv_t, qs, ks, vs, sm, dtype, qk_quant_gran=2,
                                  return_pv_count=True)
            q8t, qst, k8t, kst = (t.to(dev) for t in O.per_thread_int8(rq.cpu(), ksm.cpu()))
            o3, c3 = RR.attention(q8t, k8t, v8_perm, pr["lut"], pr["valid"], pv_t, qst, kst, vs, sm, dtype, qk_quant_gran=3,
                                  return_pv_count=True)
            torch.cuda.synchronize()
            fix = dict(case=(B, H, N, D, topk, pv, seed), dtype=tag,
                       input_sum=float(q.double().sum() + k.double().sum() + v.double().sum()),
                       km=km.cpu(), map=pr["map"].cpu(), recip_scale=recip.cpu(),
                       q_int8=q8.cpu(), q_scale=qs.cpu(), k_int8=k8.cpu(), k_scale=ks.cpu(),
                       o_gran2=o2.cpu(), pv_count_gran2=c2.cpu(), o_gran3=o3.cpu(), pv_count_gran3=c3.cpu())
            path = os.path.join(out_dir, f"ref_gpu_gran_{name}_{tag}.pt")
            torch.save(fix, path)
            print(path, os.path.getsize(path), "bytes; kept products", int(c2.sum()), "of", int(pr["valid"].sum()) * 4, flush=True)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
