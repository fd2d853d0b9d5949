"""Drop-in alias: `from spas_sage_attn import spas_sage2_attn_meansim_topk_cuda` keeps working in
model patches written for the reference package (spas_sage_attn/__init__.py:1-7)."""
from spargeattn_b200 import (  # noqa: F401
    spas_sage2_attn_meansim_cuda,
    spas_sage2_attn_meansim_topk_cuda,
    block_sparse_sage2_attn_cuda,
    spas_sage_attn_meansim_cuda,
    spas_sage_attn_meansim_topk_cuda,
)
