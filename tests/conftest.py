import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str) -> dict:
    with np.load(GOLDEN / name) as z:
        return {k: torch.from_numpy(z[k]) if z[k].ndim else z[k].item() for k in z.files}


@pytest.fixture(scope="session")
def golden():
    return load_golden


def bf16_allowance(inp, grad_out, out_ref, grads_ref, floor: float = 2e-2) -> dict:
    """Relative tolerance per tensor for a bf16 kernel checked against the fp32-core oracle: ``floor`` (2e-2 of the
    oracle's largest value), or the error that the reference's own bf16 torch path -- matmuls in bf16, logits rounded
    to bf16 before the fp32 softmax (src/matterformer/models/simplicial_attention.py:161-180, 251-297) -- makes
    against the fp32 core on the same bf16-rounded inputs, whichever is larger.  Sharp softmaxes push the latter
    above 2e-2; near-uniform ones leave it around 5e-3."""
    from dataclasses import replace

    from oracle.simplicial_ref import simplicial_forward_backward

    names = ("q", "k1", "v1", "k2", "v2")
    low = replace(inp, **{n: getattr(inp, n).bfloat16() for n in names})
    out_bf, g_bf = simplicial_forward_backward(low, grad_out.bfloat16(), fp32_core=False)

    def rel(a, b):
        return (a.float() - b).abs().max().item() / max(b.abs().max().item(), 1e-30)

    allow = {"out": max(floor, rel(out_bf, out_ref))}
    for n in names:
        allow[n] = max(floor, rel(g_bf[n], grads_ref[n]))
    return allow
