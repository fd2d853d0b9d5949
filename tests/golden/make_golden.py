"""Generate golden fixtures for the oracle from the reference's own preprocessing code.

Run once, in a container that has the reference checkout (not needed at test time):

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference

It loads the reference's `spas_sage_attn/utils.py` by file path (its package `__init__`
needs compiled CUDA modules) and executes its Triton kernels under the Triton CPU
interpreter on seeded fp16 inputs.  bf16 inputs are not used: the interpreter truncates
bf16 stores, which the GPU does not.  `torch.sort` is called with `stable=True` (the
contract of this build: ties go to the lower block index).

Outputs: tests/golden/ref_predictor_*.pt  with the reference's block map, LUT, INT8 tensors
and scales; the inputs are regenerated from the stored seed by `golden_inputs`.
"""
import importlib.util
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = [
    # name, B, H, N, D, causal, topk, cdfthreshd, simthreshd1, sink, seed
    ("n600_d64_topk", 1, 2, 600, 64, False, 0.5, None, -0.1, False, 11),
    ("n1024_d128_causal", 1, 2, 1024, 128, True, 0.5, None, -0.1, False, 12),
    ("n1000_d64_sim06", 2, 2, 1000, 64, False, 0.3, None, 0.6, True, 13),
    ("n640_d128_cdf", 1, 3, 640, 128, False, None, 0.9, 0.3, False, 14),
]


def golden_inputs(B, H, N, D, seed):
    """fp16 q, k with a smooth component so that pooled blocks are informative, plus a K bias."""
    g = torch.Generator().manual_seed(seed)
    base = torch.randn(B, H, N, D, generator=g)
    walk = torch.cumsum(torch.randn(B, H, N, D, generator=g), dim=2) * 0.15
    q = (base + walk).to(torch.float16)
    base = torch.randn(B, H, N, D, generator=g)
    walk = torch.cumsum(torch.randn(B, H, N, D, generator=g), dim=2) * 0.15
    bias = torch.randn(D, generator=g) * 3.0
    k = (base + walk + bias).to(torch.float16)
    return q, k


def main(ref_root):
    assert os.environ.get("TRITON_INTERPRET") == "1", "run with TRITON_INTERPRET=1"
    spec = importlib.util.spec_from_file_location("ref_utils", os.path.join(ref_root, "spas_sage_attn", "utils.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    orig_sort = torch.sort

    def stable_sort(x, dim=-1, descending=False, stable=False):
        return orig_sort(x, dim=dim, descending=descending, stable=True)

    for name, B, H, N, D, causal, topk, cdf, sim1, sink, seed in CASES:
        q, k = golden_inputs(B, H, N, D, seed)
        km = k.mean(dim=-2, keepdim=True)
        torch.sort = stable_sort
        try:
            fmap, q8, qs, k8, ks = ref.get_block_map_meansim_fuse_quant(
                q, k, km, is_causal=causal, simthreshd1=sim1, cdfthreshd=cdf, topk=topk, return_lut=False,
                attention_sink=sink)
            lut, valid = ref.block_map_lut_triton(fmap.contiguous())
            q8v, qsv, k8v, ksv = ref.get_vanilla_qk_quant(q, k, km)
        finally:
            torch.sort = orig_sort
        out = dict(case=(B, H, N, D, causal, topk, cdf, sim1, sink, seed), km=km, map=fmap.bool(), lut=lut,
                   valid=valid, q_int8=q8, q_scale=qs, k_int8=k8, k_scale=ks,
                   vanilla_equal=bool((q8v == q8).all() and (k8v == k8).all() and (qsv == qs).all()
                                      and (ksv == ks).all()))
        path = os.path.join(HERE, f"ref_predictor_{name}.pt")
        torch.save(out, path)
        print(name, "map density", fmap.float().mean().item(), "->", path)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: TRITON_INTERPRET=1 python tests/golden/make_golden.py <path to the reference checkout>")
    main(sys.argv[1])
