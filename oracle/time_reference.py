"""Times the compiled reference (oracle/_ref) on the current CUDA device.  TEST / BENCHMARK INFRASTRUCTURE.

    python oracle/time_reference.py --workloads 2 [--topk 0.5] [--steps 10] [--warmup 3]

Prints one JSON object per line: the reference's own public entry point spas_sage2_attn_meansim_topk_cuda
(spas_sage_attn/core.py:105-169, unmodified, its sm89 mma.sync kernel compiled for sm_100) on the synthetic inputs
of the named workload, CUDA-event time per call. Runs in a process of its own: it never imports this library's
package, whose shared object must not be mapped into a process that measures the reference.
"""
import argparse
import importlib.util
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, HERE)


def load_synthetic():
    spec = importlib.util.spec_from_file_location("sparge_synthetic", os.path.join(ROOT, "spargeattn_b200", "synthetic.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workloads", default="2")
    ap.add_argument("--topk", type=float, default=None)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--block-sparse", action="store_true", help="also time block_sparse_sage2_attn_cuda (workload 1 mask)")
    a = ap.parse_args()
    import ref_runner as RR
    if not RR.available():
        print(json.dumps({"unavailable": "oracle/_ref has not been built (python oracle/build_ref.py)"}))
        return
    RR.load()
    syn = load_synthetic()
    dev = torch.device("cuda", 0)
    for idx in [int(x) for x in a.workloads.split(",")]:
        w = syn.WORKLOADS[idx]
        B, H, N, D = syn.workload_shape(idx)
        heads = [(b, h) for b in range(B) for h in range(H)]
        q, k, v = syn.workload_heads_qkv(idx, heads, dev)
        q, k, v = (t.view(B, H, N, D) for t in (q, k, v))
        topk = a.topk if a.topk is not None else w["topk"]
        ms = RR.time_ms(lambda: RR.api_topk(q, k, v, stable=False, topk=topk, is_causal=w["causal"]), a.warmup, a.steps)
        ops = 4.0 * B * H * N * N * D * (0.5 if w["causal"] else 1.0)
        row = {"workload": idx, "shape": [B, H, N, D], "topk": topk, "ms": ms, "dense_equiv_TOPS": ops / ms / 1e9,
               "what": "reference spas_sage2_attn_meansim_topk_cuda (sm89 mma.sync kernel built for sm_100)"}
        if a.block_sparse and idx == 1:
            mask = syn.bernoulli_block_mask(B, H, N, 0.4, 1, dev)
            row["block_sparse_ms"] = RR.time_ms(lambda: RR.api_block_sparse(q, k, v, mask), a.warmup, a.steps)
        print(json.dumps(row), flush=True)
        del q, k, v
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
