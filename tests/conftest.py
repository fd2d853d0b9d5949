import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def device_recip_scale(v):
    """2.25 / amax per (batch, head, channel) of V as the GPU's approximate division returns it: the one input
    of the oracle's V quantiser that has no CPU definition (see sparge_oracle.quant_v). Returns a CPU tensor."""
    import torch
    from spargeattn_b200 import ops
    amax = v.to(torch.float16).float().abs().amax(dim=-2).cuda()
    return ops.div_approx(torch.full_like(amax, 2.25), amax).cpu()
