"""CPU-side checks: the C-ABI library loads and exports every symbol include/philtorch_b200.h
declares (no compute calls), argument errors are reported, and the product refuses CPU tensors."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "philtorch_b200.h")


def _declared():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(ptb_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_exported():
    from philtorch_b200 import _lib

    names = _declared()
    assert len(names) >= 15, names
    for n in names:
        assert hasattr(_lib.lib, n), f"{n} declared in the header but not exported"
    assert b"sm_100a" in _lib.lib.ptb_version()


def test_argument_errors_without_gpu():
    from philtorch_b200 import _lib

    lib = _lib.lib
    assert lib.ptb_workspace_bytes(0, 0) > 0
    assert lib.ptb_workspace_bytes(256, 1 << 20) >= 256 * 2048 * 16
    # negative sizes / null pointers are rejected before anything touches a device
    assert lib.ptb_lpv_recur_fwd(0, -1, 4, None, 1, None, 1, None, None, None, None, 0, None, None) == 1
    assert lib.ptb_lpv_recur_fwd(0, 2, 4, None, 1, None, 1, None, None, None, None, 0, None, None) == 1
    assert lib.ptb_lti_recur2_fwd(7, 0, 0, None, 1, None, None, 0, None, None, None, 0, None, None) == 0  # empty: ok
    buf = (ctypes.c_float * 64)()
    p = ctypes.addressof(buf)
    assert lib.ptb_lpv_recur_fwd(9, 2, 4, p, 1, p, 1, p, p, None, None, 0, None, None) == 1   # unknown dtype
    assert b"workspace" in lib.ptb_error_string(2)


def test_no_cpu_path():
    import philtorch_b200 as ptb

    a, zi, x = torch.rand(3), torch.zeros(3), torch.randn(3, 16)
    with pytest.raises(RuntimeError, match="CUDA"):
        ptb.lti.linear_recurrence(a, zi, x)
    with pytest.raises(RuntimeError, match="CUDA"):
        ptb.lpv.linear_recurrence(torch.rand(3, 16), zi, x)
    with pytest.raises(RuntimeError, match="CUDA"):
        ptb.lti.lfilter(torch.ones(3), torch.zeros(2), x)
    with pytest.raises(RuntimeError, match="CUDA"):
        ptb.lpv.state_space_recursion(torch.rand(3, 16, 2, 2), torch.zeros(3, 2), x)


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "philtorch_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                txt = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in txt and "from oracle" not in txt, f


def test_fake_impls_shapes():
    """Shape contracts of the ops, evaluated on meta tensors (no device needed)."""
    import philtorch_b200  # noqa: F401
    ops = torch.ops.philtorch_b200
    m = lambda *s: torch.empty(*s, device="meta")
    assert ops.lti_recur(m(3), m(3), m(3, 10)).shape == (3, 10)
    assert ops.lpv_recur(m(10), m(3), m(3, 10)).shape == (3, 10)
    assert ops.recur2(m(3, 10, 2, 2), m(3, 2), m(3, 10, 2)).shape == (3, 10, 2)
    assert ops.lti_recur2_sx(m(2, 2), m(3, 2), m(3, 10)).shape == (3, 10, 2)
    y, zf = ops.biquad_tdf2(m(3), m(2), None, m(4, 10))
    assert y.shape == (4, 10) and zf.shape == (4, 2)
    with pytest.raises(RuntimeError):
        ops.lti_recur(m(4), m(3), m(3, 10))
    with pytest.raises(RuntimeError):
        ops.recur2(m(3, 9, 2, 2), m(3, 2), m(3, 10, 2))
