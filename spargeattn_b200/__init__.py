"""B200 (sm_100a) implementation of SpargeAttn's training-free sparse attention hot path.

Same public names as the reference package (spas_sage_attn/__init__.py:1-7)."""
from .core import (
    spas_sage2_attn_meansim_cuda,
    spas_sage2_attn_meansim_topk_cuda,
    block_sparse_sage2_attn_cuda,
    spas_sage_attn_meansim_cuda,
    spas_sage_attn_meansim_topk_cuda,
)

__all__ = [
    "spas_sage2_attn_meansim_cuda",
    "spas_sage2_attn_meansim_topk_cuda",
    "block_sparse_sage2_attn_cuda",
    "spas_sage_attn_meansim_cuda",
    "spas_sage_attn_meansim_topk_cuda",
]
