"""GPU parity of the complex first-order recurrences (complex64 / complex128), which the reference
dispatches on its compiled ops as well (philtorch/csrc/lti_recur.cu:135-156) and which
``diag_state_space`` runs on complex poles (philtorch/lti/ssm.py:794-804).  Checked against the
CPU oracle, the golden vectors made by the reference, and torch's complex gradcheck.
Tolerance: max|out-ref|/max|ref| <= 1e-4 (complex64), <= 1e-10 (complex128)."""
import numpy as np
import pytest
import torch

import philtorch_b200 as ptb
from philtorch_b200.autograd import LPVRecurrence, LTIRecurrence
from conftest import load_golden, rel_err, tol
from oracle import cport

pytestmark = pytest.mark.gpu
DEV = "cuda"
CDT = {"c64": torch.complex64, "c128": torch.complex128}

# tiles hold 16-byte units: complex64 tiles are half, complex128 tiles a quarter of the fp32 sample
# counts (e.g. 6656 / 3328 time-invariant forward, 4608 / 2304 per-sample forward, 2560 / 1280 adjoint)
LENGTHS = [1, 2, 3, 5, 33, 101, 1279, 1280, 1281, 2303, 2304, 2305, 2560, 2561, 3328, 3329, 4608, 4609, 6656,
           6657, 13313, 30001]


def _poles(shape, g):
    r = 0.2 + 0.79 * torch.rand(*shape, generator=g, dtype=torch.float64)
    return torch.polar(r, 2 * np.pi * torch.rand(*shape, generator=g, dtype=torch.float64))


def _randc(shape, g):
    return torch.complex(torch.randn(*shape, generator=g, dtype=torch.float64),
                         torch.randn(*shape, generator=g, dtype=torch.float64))


def _run(kind, a, zi, x, gy):
    fn = LTIRecurrence if kind == "lti" else LPVRecurrence
    a_, zi_, x_ = (t.to(DEV).requires_grad_() for t in (a, zi, x))
    y = fn.apply(a_, zi_, x_)
    ga, gzi, gx = torch.autograd.grad(y, (a_, zi_, x_), gy.to(DEV))
    ptb.check_errors()
    return y, ga, gzi, gx


def _check(kind, a, zi, x, gy, dtype):
    t = tol(dtype)
    y, ga, gzi, gx = _run(kind, a, zi, x, gy)
    assert y.dtype == dtype and gx.dtype == dtype and ga.dtype == dtype
    if kind == "lti":
        y_ref = cport.lti_recur(a, zi, x)
        ga_ref, gzi_ref, gx_ref = cport.lti_recur_bwd(a, zi, y_ref, gy)
    else:
        y_ref = cport.recur1(a, zi, x)
        ga_ref, gzi_ref, gx_ref = cport.recur1_bwd(a, zi, y_ref, gy)
    assert rel_err(y, y_ref) <= t
    assert rel_err(gx, gx_ref) <= t
    assert rel_err(gzi, gzi_ref) <= t
    assert rel_err(ga, ga_ref.reshape(ga.shape)) <= t


@pytest.mark.parametrize("dtype", [torch.complex64, torch.complex128])
@pytest.mark.parametrize("T", LENGTHS)
@pytest.mark.parametrize("mode", ["batched", "shared1", "scalar"])
def test_lti_lengths(dtype, T, mode):
    B = 3
    g = torch.Generator().manual_seed(T * 13 + len(mode))
    a = _poles((B if mode == "batched" else 1,), g).to(dtype)
    if mode == "scalar":
        a = a[0]
    zi, x, gy = _randc((B,), g).to(dtype), _randc((B, T), g).to(dtype), _randc((B, T), g).to(dtype)
    _check("lti", a, zi, x, gy, dtype)


@pytest.mark.parametrize("dtype", [torch.complex64, torch.complex128])
@pytest.mark.parametrize("T", LENGTHS)
@pytest.mark.parametrize("batched", [True, False])
def test_lpv_lengths(dtype, T, batched):
    B = 3
    g = torch.Generator().manual_seed(T * 17 + int(batched))
    a = _poles((B, T) if batched else (T,), g).to(dtype)
    zi, x, gy = _randc((B,), g).to(dtype), _randc((B, T), g).to(dtype), _randc((B, T), g).to(dtype)
    _check("lpv", a, zi, x, gy, dtype)


@pytest.mark.parametrize("dtype", [torch.complex64, torch.complex128])
def test_many_rows(dtype):
    """More tiles than resident CTAs, several tiles per row."""
    B, T = 300, 20000
    g = torch.Generator().manual_seed(5)
    a = _poles((B,), g).to(dtype)
    zi, x, gy = _randc((B,), g).to(dtype), _randc((B, T), g).to(dtype), _randc((B, T), g).to(dtype)
    _check("lti", a, zi, x, gy, dtype)
    _check("lpv", _poles((B, T), g).to(dtype), zi, x, gy, dtype)


@pytest.mark.parametrize("tag", ["c64", "c128"])
def test_golden(tag):
    t = tol(CDT[tag])
    for mode in ("batched", "shared1", "scalar"):
        g = load_golden(f"lti_recur_{mode}_{tag}")
        y, ga, gzi, gx = _run("lti", g["a"], g["zi"], g["x"], g["gy"])
        assert rel_err(y, g["y"]) <= t and rel_err(ga, g["grad_a"]) <= t
        assert rel_err(gzi, g["grad_zi"]) <= t and rel_err(gx, g["grad_x"]) <= t
    for mode in ("batched", "shared"):
        g = load_golden(f"lpv_recur1_{mode}_{tag}")
        y, ga, gzi, gx = _run("lpv", g["a"], g["zi"], g["x"], g["gy"])
        assert rel_err(y, g["y"]) <= t and rel_err(y, g["y_python_loop"]) <= t
        assert rel_err(ga, g["grad_a"]) <= t and rel_err(gzi, g["grad_zi"]) <= t and rel_err(gx, g["grad_x"]) <= t


def test_lazy_conjugate_inputs():
    """A conjugated view carries a flag, not conjugated memory: the ops must see its values."""
    g = torch.Generator().manual_seed(9)
    B, T = 4, 3000
    a, zi, x = _poles((B,), g), _randc((B,), g), _randc((B, T), g)
    y = torch.ops.philtorch_b200.lti_recur(a.to(DEV).conj(), zi.to(DEV).conj(), x.to(DEV).conj())
    assert rel_err(y, cport.lti_recur(a.conj(), zi.conj(), x.conj())) <= 1e-10


@pytest.mark.parametrize("kind", ["lti", "lpv"])
def test_gradcheck(kind):
    g = torch.Generator().manual_seed(11)
    B, T = 2, 24
    a = _poles((B,) if kind == "lti" else (B, T), g).to(DEV).requires_grad_()
    zi = _randc((B,), g).to(DEV).requires_grad_()
    x = _randc((B, T), g).to(DEV).requires_grad_()
    fn = LTIRecurrence if kind == "lti" else LPVRecurrence
    assert torch.autograd.gradcheck(fn.apply, (a, zi, x), eps=1e-6, atol=1e-6)
    assert torch.autograd.gradgradcheck(fn.apply, (a, zi, x), eps=1e-6, atol=1e-5)


def test_real_only_ops_reject_complex():
    A = torch.zeros(2, 2, 2, dtype=torch.complex64, device=DEV)
    with pytest.raises(RuntimeError, match="float32 and float64"):
        torch.ops.philtorch_b200.lti_recur2(A, torch.zeros(2, 2, dtype=torch.complex64, device=DEV),
                                            torch.zeros(2, 8, 2, dtype=torch.complex64, device=DEV))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.complex64, torch.complex128])
@pytest.mark.parametrize("T", [1, 2, 37, 2561, 9300])
@pytest.mark.parametrize("mode", ["batched", "scalar"])
def test_reverse_time_recurrence(dtype, T, mode):
    """``ReverseLTIRecurrence`` (the adjoint kernel as a forward operator) against the oracle run on
    the reversed signal, values and all gradients."""
    from philtorch_b200.autograd import ReverseLTIRecurrence
    B = 3
    g = torch.Generator().manual_seed(T + len(mode))
    cplx = dtype.is_complex
    a = _poles((B,), g) if cplx else torch.rand(B, generator=g, dtype=torch.float64) * 1.9 - 0.95
    a = (a if mode == "batched" else a[0]).to(dtype)
    mk = (lambda s: _randc(s, g)) if cplx else (lambda s: torch.randn(*s, generator=g, dtype=torch.float64))
    end, x, gy = mk((B,)).to(dtype), mk((B, T)).to(dtype), mk((B, T)).to(dtype)
    a_, end_, x_ = (t.to(DEV).requires_grad_() for t in (a, end, x))
    out = ReverseLTIRecurrence.apply(a_, end_, x_)
    ga, gend, gx = torch.autograd.grad(out, (a_, end_, x_), gy.to(DEV))
    ptb.check_errors()
    ref = cport.lti_recur(a, end, x.flip(1)).flip(1)
    ga_ref, gend_ref, gx_ref = cport.lti_recur_bwd(a, end, ref.flip(1).contiguous(), gy.flip(1).contiguous())
    t = tol(dtype)
    assert rel_err(out, ref) <= t
    assert rel_err(gx, gx_ref.flip(1)) <= t
    assert rel_err(gend, gend_ref) <= t
    assert rel_err(ga, ga_ref.reshape(ga.shape)) <= 10 * t


def test_reverse_time_gradcheck():
    from philtorch_b200.autograd import ReverseLTIRecurrence
    g = torch.Generator().manual_seed(4)
    a = _poles((2,), g).to(DEV).requires_grad_()
    end = _randc((2,), g).to(DEV).requires_grad_()
    x = _randc((2, 19), g).to(DEV).requires_grad_()
    assert torch.autograd.gradcheck(ReverseLTIRecurrence.apply, (a, end, x), eps=1e-6, atol=1e-6)
    assert torch.autograd.gradgradcheck(ReverseLTIRecurrence.apply, (a, end, x), eps=1e-6, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("T", [1, 5, 2560, 2561, 30000])
def test_reverse_fused_op(dtype, T):
    """out = scale * (g + second - x) with g the reverse-time recurrence of x; first state a * g[0]."""
    B = 4
    g = torch.Generator().manual_seed(T)
    a = (torch.rand(B, generator=g, dtype=torch.float64) * 1.9 - 0.95).to(dtype)
    x, second = (torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype) for _ in range(2))
    g_in = torch.randn(B, generator=g, dtype=torch.float64).to(dtype)
    out, first = torch.ops.philtorch_b200.lti_recur_reverse_fused(a.to(DEV), x.to(DEV), second.to(DEV),
                                                                  g_in.to(DEV), 0.75, True)
    ptb.check_errors()
    xr = x.flip(1).contiguous()
    xr[:, 0] += g_in                       # the state entering from the right adds to the last sample
    rev = cport.lti_recur(a, torch.zeros(B, dtype=dtype), xr).flip(1)
    assert rel_err(out, 0.75 * (rev + second - x)) <= tol(dtype)
    assert rel_err(first, a * rev[:, 0]) <= tol(dtype)
