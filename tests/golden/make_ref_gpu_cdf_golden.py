"""Record what the compiled reference's cdf-threshold selection does on a CUDA device (bf16 and fp16).

    python tests/golden/make_ref_gpu_cdf_golden.py [out_dir]        # needs a GPU and oracle/_ref

The cdf mode of get_block_map_meansim_fuse_quant (spas_sage_attn/utils.py:396-403) sorts the pooled
probabilities, runs torch.cumsum on them *in the 16-bit type* and takes torch.searchsorted(cdf, threshold,
right=True). On the device torch's cumsum is a chunked parallel scan that rounds to the 16-bit type at every
combine, so the counts depend on that scan's order. This script hooks torch.cumsum / torch.searchsorted while
the reference runs and stores their inputs and outputs together with the final block map, so that the CPU
restatement of the scan can be checked bit for bit without a GPU.
"""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

CASES = [
    # name, B, H, N, D, causal, cdfthreshd, simthreshd1, seed
    ("cdf_n8192_d128", 1, 2, 8192, 128, False, 0.9, -0.1, 31),
    ("cdf_n32760_d128", 1, 1, 32760, 128, False, 0.98, -0.1, 32),
    ("cdf_n4000_d64_causal", 2, 3, 4000, 64, True, 0.95, -0.1, 33),
]


def main(out_dir):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    sys.path.insert(0, HERE)
    import ref_runner as RR
    from make_ref_gpu_golden import ref_gpu_inputs
    RR.load()
    os.makedirs(out_dir, exist_ok=True)
    dev = torch.device("cuda", 0)
    for name, B, H, N, D, causal, cdf, sim1, seed in CASES:
        for dtype, tag in ((torch.bfloat16, "bf16"), (torch.float16, "fp16")):
            q, k, v = ref_gpu_inputs(B, H, N, D, dtype, seed)
            qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
            rq, rk, _, km = RR.prologue(qd, kd, vd)
            seen = {}
            orig_cumsum, orig_search = torch.cumsum, torch.searchsorted

            def cumsum(x, *a, **kw):
                out = orig_cumsum(x, *a, **kw)
                seen["sorted"], seen["cdf"] = x.detach().cpu(), out.detach().cpu()
                return out

            def searchsorted(bounds, vals, *a, **kw):
                out = orig_search(bounds, vals, *a, **kw)
                seen["thr"], seen["n_sel"] = vals.detach().cpu(), out.detach().cpu()
                return out

            torch.cumsum, torch.searchsorted = cumsum, searchsorted
            try:
                pr = RR.predictor(rq, rk, km, causal, sim1, cdf, None, False, stable=True)
            finally:
                torch.cumsum, torch.searchsorted = orig_cumsum, orig_search
            torch.cuda.synchronize()
            fix = dict(case=(B, H, N, D, causal, cdf, sim1, seed), dtype=tag,
                       input_sum=float(q.double().sum() + k.double().sum() + v.double().sum()), km=km.cpu(),
                       sorted=seen["sorted"], cdf=seen["cdf"], thr=seen["thr"], n_sel=seen["n_sel"].to(torch.int32),
                       map=pr["map"].cpu(), valid=pr["valid"].cpu(), sim_q=pr["sim_q"].cpu(), sim_k=pr["sim_k"].cpu())
            path = os.path.join(out_dir, f"ref_gpu_{name}_{tag}.pt")
            torch.save(fix, path)
            print(path, os.path.getsize(path), "bytes", "thr dtype", seen["thr"].dtype, "cdf dtype", seen["cdf"].dtype, flush=True)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
