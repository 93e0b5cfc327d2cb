import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_golden(name):
    return dict(np.load(GOLDEN / f"{name}.npz"))


def rebuild_module_case(g, dtype=torch.float32):
    """Re-create the seeded weights and inputs a module fixture was recorded on
    (same order of RNG draws as tests/golden/make_golden.py:module_case)."""
    dim, heads, dim_head, prenorm, b, n, split, seed, stride = (int(v) for v in g["meta"])
    torch.manual_seed(seed)
    inner = heads * dim_head
    lin1 = torch.nn.Linear(dim, inner * 6, bias=False)
    lin2 = torch.nn.Linear(inner, dim, bias=False)
    norm_w = None
    if prenorm:
        norm_w = torch.empty(dim).uniform_(0.5, 1.5)
    x = torch.randn(b, n, dim)
    gout = torch.randn(b, n, dim)
    cfg = dict(dim=dim, heads=heads, dim_head=dim_head, prenorm=bool(prenorm), b=b, n=n, split=split, stride=stride)
    return cfg, lin1.weight.detach().to(dtype), lin2.weight.detach().to(dtype), norm_w, x.to(dtype), gout.to(dtype)


def rebuild_core_case(g):
    b, h, n, d, seed = (int(v) for v in g["meta"])
    torch.manual_seed(seed)
    torch.nn.Linear(6 * h * d, 6 * h * d, bias=False)  # consumes the same RNG draws as the reference ctor
    torch.nn.Linear(h * d, 6 * h * d, bias=False)
    packed = torch.randn(b, n, 6 * h * d, dtype=torch.double)
    gout = torch.randn(b, n, h * d, dtype=torch.double)
    return (b, h, n, d), packed, gout


@pytest.fixture
def golden():
    return load_golden
