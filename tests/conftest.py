import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """Golden vectors produced by running the reference (tests/golden/make_golden.py)."""
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        return {k: torch.from_numpy(np.asarray(z[k])) for k in z.files if np.asarray(z[k]).dtype.kind in "fiubc"}


def rel_err(out, ref):
    """max|out - ref| / max|ref|: the parity metric of the path (<=1e-4 fp32, <=1e-10 fp64)."""
    wide = torch.complex128 if (out.is_complex() or ref.is_complex()) else torch.float64
    out = out.detach().resolve_conj().to(wide).cpu()
    ref = ref.detach().resolve_conj().to(wide).cpu()
    assert out.shape == ref.shape, (out.shape, ref.shape)
    if ref.numel() == 0:
        return 0.0
    denom = ref.abs().max().item()
    return (out - ref).abs().max().item() / (denom if denom > 0 else 1.0)


def tol(dtype):
    return 1e-4 if dtype in (torch.float32, torch.complex64) else 1e-10
