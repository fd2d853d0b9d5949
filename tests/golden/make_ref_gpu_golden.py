"""Generate golden fixtures from the compiled reference running on a CUDA device.

Run once on a machine with a GPU and `oracle/_ref` (built by `oracle/build_ref.py`):

    python tests/golden/make_ref_gpu_golden.py [out_dir]        # default: tests/golden

Each case runs the reference's own code path of spas_sage2_attn_meansim_topk_cuda on seeded inputs
(bf16 and fp16; the Triton CPU interpreter used by make_golden.py cannot do bf16 faithfully) and stores
what the reference produced: the torch K mean, pooled values and self-similarity flags, INT8 Q/K and
scales, the block map (with `torch.sort(stable=True)`, ties to the lower index), LUT and counts, the FP8
bytes of V (un-permuted to token-major) with its scales, and the attention output.  `recip_scale` is the
GPU's approximate quotient 2.25 / amax per V channel (evaluated by this library's sparge_div_approx with the
instruction the reference's fast-math build uses): the one input of the V quantiser that has no CPU definition.  `tie_flips` counts the
blocks of the map that change when the reference's sort is left unstable.  Inputs are not stored: tests
regenerate them with `ref_gpu_inputs` from the stored seed and check `input_sum`.
"""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

CASES = [
    # name, B, H, N, D, causal, topk, simthreshd1, sink, seed
    ("n128_d64", 1, 2, 128, 64, False, 0.5, 0.2, False, 21),
    ("n200_d128", 1, 2, 200, 128, False, 0.5, 0.2, False, 22),
    ("n640_d64_causal", 1, 2, 640, 64, True, 0.5, 0.2, False, 23),
    ("n1000_d128_sink", 1, 1, 1000, 128, False, 0.3, 0.5, True, 24),
    ("n2048_d64", 1, 1, 2048, 64, False, 0.5, -0.1, False, 25),
]


def ref_gpu_inputs(B, H, N, D, dtype, seed):
    """q, k, v = N(0,1) + a slow random walk (so that pooled blocks carry signal); K gets a channel bias."""
    g = torch.Generator().manual_seed(seed)
    walk = lambda: torch.cumsum(torch.randn(B, H, N, D, generator=g), dim=2) * 0.1
    q = (torch.randn(B, H, N, D, generator=g) + walk()).to(dtype)
    k = (torch.randn(B, H, N, D, generator=g) + walk() + torch.randn(D, generator=g) * 3).to(dtype)
    v = (torch.randn(B, H, N, D, generator=g) + walk()).to(dtype)
    return q, k, v


def main(out_dir):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_runner as RR
    RR.load()
    sys.path.insert(0, ROOT)
    from spargeattn_b200 import ops
    os.makedirs(out_dir, exist_ok=True)
    dev = torch.device("cuda", 0)
    for name, B, H, N, D, causal, topk, sim1, sink, seed in CASES:
        for dtype, tag in ((torch.bfloat16, "bf16"), (torch.float16, "fp16")):
            q, k, v = ref_gpu_inputs(B, H, N, D, dtype, seed)
            qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
            rq, rk, rv16, km = RR.prologue(qd, kd, vd)
            pr = RR.predictor(rq, rk, km, causal, sim1, None, topk, sink, stable=True)
            pu = RR.predictor(rq, rk, km, causal, sim1, None, topk, sink, stable=False)
            _, vs, v8_tok = RR.quant_v(rv16)
            amax = rv16.float().abs().amax(dim=-2)
            recip = ops.div_approx(torch.full_like(amax, 2.25), amax)
            o = RR.api_topk(qd, kd, vd, stable=True, topk=topk, is_causal=causal, simthreshd1=sim1, attention_sink=sink)
            torch.cuda.synchronize()
            fix = dict(case=(B, H, N, D, causal, topk, sim1, sink, seed), dtype=tag,
                       input_sum=float(q.double().sum() + k.double().sum() + v.double().sum()),
                       km=km.cpu(), pq=pr["pq"].cpu(), pk=pr["pk"].cpu(), sim_q=pr["sim_q"].cpu(), sim_k=pr["sim_k"].cpu(),
                       q_int8=pr["q_int8"].cpu(), q_scale=pr["q_scale"].cpu(), k_int8=pr["k_int8"].cpu(),
                       k_scale=pr["k_scale"].cpu(), map=pr["map"].cpu(), lut=pr["lut"].cpu(), valid=pr["valid"].cpu(),
                       v8=v8_tok.cpu(), v_scale=vs.cpu(), recip_scale=recip.cpu(), o=o.cpu(),
                       tie_flips=int((pr["map"] != pu["map"]).sum().item()))
            path = os.path.join(out_dir, f"ref_gpu_{name}_{tag}.pt")
            torch.save(fix, path)
            print(path, os.path.getsize(path), "bytes; tie flips", fix["tie_flips"], flush=True)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
