"""Autograd contracts of the Functions and ops, mirroring the reference's tests/test_grad.py
(gradcheck with forward-mode AD, gradgradcheck, every requires_grad combination, shared and
batched coefficients, fp64, T = 11, B = 3) and tests/test_pt2_comp.py (torch.library.opcheck)."""
import itertools

import pytest
import torch
from torch.autograd import gradcheck, gradgradcheck

import philtorch_b200 as ptb
from philtorch_b200.autograd import (BiquadTDF2, LPVRecurrence, LTIMatrixRecurrence, LTIRecurrence,
                                     MatrixRecurrence)

pytestmark = pytest.mark.gpu
DEV = "cuda"
B, T = 3, 11
COMBOS = [c for c in itertools.product([True, False], repeat=3) if any(c)]


def _t(*shape, scale=1.0, req=False):
    return (scale * torch.randn(*shape, dtype=torch.float64, device=DEV)).requires_grad_(req)


@pytest.mark.parametrize("req", COMBOS)
@pytest.mark.parametrize("a_shape", [(), (1,), (B,)])
def test_lti_recurrence_grad(req, a_shape):
    torch.manual_seed(0)
    a = (torch.rand(a_shape, dtype=torch.float64, device=DEV) * 1.6 - 0.8).requires_grad_(req[0])
    zi, x = _t(B, req=req[1]), _t(B, T, req=req[2])
    assert gradcheck(LTIRecurrence.apply, (a, zi, x), check_forward_ad=True)
    assert gradgradcheck(LTIRecurrence.apply, (a, zi, x))


@pytest.mark.parametrize("req", COMBOS)
@pytest.mark.parametrize("batched", [True, False])
def test_lpv_recurrence_grad(req, batched):
    torch.manual_seed(1)
    a = (torch.rand(*((B, T) if batched else (T,)), dtype=torch.float64, device=DEV) * 1.6 - 0.8).requires_grad_(req[0])
    zi, x = _t(B, req=req[1]), _t(B, T, req=req[2])
    assert gradcheck(LPVRecurrence.apply, (a, zi, x), check_forward_ad=True)
    assert gradgradcheck(LPVRecurrence.apply, (a, zi, x))


@pytest.mark.parametrize("req", COMBOS)
@pytest.mark.parametrize("batched", [True, False])
def test_lti_matrix_recurrence_grad(req, batched):
    torch.manual_seed(2)
    A = _t(*((B, 2, 2) if batched else (2, 2)), scale=0.4, req=req[0])
    zi, x = _t(B, 2, req=req[1]), _t(B, T, 2, req=req[2])
    assert gradcheck(LTIMatrixRecurrence.apply, (A, zi, x), check_forward_ad=True)
    assert gradgradcheck(LTIMatrixRecurrence.apply, (A, zi, x))


@pytest.mark.parametrize("req", COMBOS)
@pytest.mark.parametrize("batched", [True, False])
def test_matrix_recurrence_grad(req, batched):
    torch.manual_seed(3)
    A = _t(*((B, T, 2, 2) if batched else (T, 2, 2)), scale=0.4, req=req[0])
    zi, x = _t(B, 2, req=req[1]), _t(B, T, 2, req=req[2])
    assert gradcheck(MatrixRecurrence.apply, (A, zi, x), check_forward_ad=True)
    assert gradgradcheck(MatrixRecurrence.apply, (A, zi, x))


@pytest.mark.parametrize("batched", [True, False])
@pytest.mark.parametrize("with_zi", [True, False])
def test_biquad_grad(batched, with_zi):
    torch.manual_seed(4)
    b = _t(*((B, 3) if batched else (3,)), req=True)
    a = _t(*((B, 2) if batched else (2,)), scale=0.3, req=True)
    x = _t(B, T, req=True)
    zi = _t(B, 2, req=True) if with_zi else None
    fn = (lambda b_, a_, zi_, x_: BiquadTDF2.apply(b_, a_, zi_, x_)) if with_zi else \
        (lambda b_, a_, x_: BiquadTDF2.apply(b_, a_, None, x_)[0])
    args = (b, a, zi, x) if with_zi else (b, a, x)
    assert gradcheck(fn, args)
    assert gradgradcheck(fn, args)


def test_lfilter_scalar_input_state_space_grad():
    torch.manual_seed(5)
    A = _t(B, T, 2, 2, scale=0.4, req=True)
    zi, x = _t(B, 2, req=True), _t(B, T, req=True)
    assert gradcheck(lambda A_, z_, x_: ptb.lpv.state_space_recursion(A_, z_, x_), (A, zi, x))
    A2 = _t(B, 2, 2, scale=0.4, req=True)
    assert gradcheck(lambda A_, z_, x_: ptb.lti.state_space_recursion(A_, z_, x_, out_idx=1), (A2, zi, x))


def test_opcheck():
    ops = torch.ops.philtorch_b200
    f = lambda *s: torch.randn(*s, device=DEV)
    tests = ("test_schema", "test_faketensor")
    torch.library.opcheck(ops.lti_recur, (f(B) * 0.5, f(B), f(B, T)), test_utils=tests)
    torch.library.opcheck(ops.lpv_recur, (f(B, T) * 0.5, f(B), f(B, T)), test_utils=tests)
    torch.library.opcheck(ops.lti_recur2, (f(B, 2, 2) * 0.4, f(B, 2), f(B, T, 2)), test_utils=tests)
    torch.library.opcheck(ops.recur2, (f(T, 2, 2) * 0.4, f(B, 2), f(B, T, 2)), test_utils=tests)
    torch.library.opcheck(ops.recur2_sx, (f(B, T, 2, 2) * 0.4, f(B, 2), f(B, T)), test_utils=tests)
    torch.library.opcheck(ops.biquad_tdf2, (f(3), f(2) * 0.3, None, f(B, T)), test_utils=tests)
    torch.library.opcheck(ops.lpv_recur_bwd, (f(B, T) * 0.5, f(B), f(B, T), f(B, T), None, True, True),
                          test_utils=tests)
    ptb.check_errors()
