"""Dense N x N recurrences, 2 < N <= 8 (the reference's recurN / lti_recurN ops and the autograd
Functions on top of them), and time-invariant filters of order 3 and 5 through lti.lfilter: against
golden vectors made by running the reference's CPU extension, plus longer rows (many tiles, ragged
and unaligned lengths) against a sequential float64 loop."""
import os

import numpy as np
import pytest
import torch

import philtorch_b200 as ptb
from philtorch_b200.autograd import LTIMatrixRecurrence, MatrixRecurrence
from conftest import GOLDEN, rel_err, tol

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _load(tag):
    z = np.load(os.path.join(GOLDEN, f"dense_recurrence_{tag}.npz"))
    cases = {}
    for key in z.files:
        case, name = key.split("/", 1)
        cases.setdefault(case, {})[name] = torch.from_numpy(np.asarray(z[key]))
    return cases


@pytest.fixture(autouse=True, params=[0, 1], ids=["power-tables", "general"])
def constant_matrix_policy(request):
    """Constant matrices run on one of two kernel families (a table of matrix powers per row, or the
    general per-sample kernels): every case here runs on both."""
    from philtorch_b200 import _lib
    assert _lib.lib.ptb_recur_n_set_policy(request.param) == 0
    yield request.param
    assert _lib.lib.ptb_recur_n_set_policy(0) == 0


G = {"f32": _load("f32"), "f64": _load("f64")}
REC = sorted(k for k in G["f64"] if k.startswith("n"))
FIL = sorted(k for k in G["f64"] if k.startswith("lfilter"))


@pytest.mark.parametrize("tag", ["f32", "f64"])
@pytest.mark.parametrize("case", REC)
def test_recurrence_golden(tag, case):
    c = G[tag][case]
    t = tol(c["x"].dtype)
    A, zi, x = (c[k].to(DEV).requires_grad_() for k in ("A", "zi", "x"))
    fn = MatrixRecurrence if "_lpv_" in case else LTIMatrixRecurrence
    y = fn.apply(A, zi, x)
    gA, gzi, gx = torch.autograd.grad(y, (A, zi, x), c["gy"].to(DEV))
    assert rel_err(y, c["y"]) <= t and rel_err(gx, c["grad_x"]) <= t
    assert rel_err(gzi, c["grad_zi"]) <= t and rel_err(gA, c["grad_A"]) <= t * 10
    ptb.check_errors()


@pytest.mark.parametrize("tag", ["f32", "f64"])
@pytest.mark.parametrize("case", FIL)
def test_higher_order_lfilter_golden(tag, case):
    c = G[tag][case]
    t = tol(c["x"].dtype) * 10
    b, a, x = (c[k].to(DEV).requires_grad_() for k in ("b", "a", "x"))
    y = ptb.lti.lfilter(b, a, x, form=case.split("_")[1])
    gb, ga, gx = torch.autograd.grad(y, (b, a, x), c["gy"].to(DEV))
    assert rel_err(y, c["y"]) <= t and rel_err(gx, c["grad_x"]) <= t
    assert rel_err(gb, c["grad_b"]) <= t and rel_err(ga, c["grad_a"]) <= t
    ptb.check_errors()


def _loop(A, zi, x, lpv):
    h, out = zi, []
    for t in range(x.shape[1]):
        At = (A[:, t] if A.dim() == 4 else A[t]) if lpv else A
        h = (At @ h.unsqueeze(-1)).squeeze(-1) + x[:, t]
        out.append(h)
    return torch.stack(out, 1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("n,T", [(3, 1537), (4, 4096), (5, 1000), (7, 517), (8, 2050), (4, 20011), (8, 9001), (6, 1)])
@pytest.mark.parametrize("lpv", [True, False])
def test_many_tiles_against_loop(dtype, n, T, lpv):
    """Rows of several tiles, lengths that are not multiples of the tile or of 16 bytes: forward and
    gradients against a float64 loop differentiated by autograd."""
    B = 3
    g = torch.Generator().manual_seed(n * 1000 + T)
    lead = (B, T) if lpv else (B,)
    A = torch.randn(lead + (n, n), generator=g, dtype=torch.float64) * (0.5 / n ** 0.5)
    zi = torch.randn(B, n, generator=g, dtype=torch.float64)
    x = torch.randn(B, T, n, generator=g, dtype=torch.float64)
    gy = torch.randn(B, T, n, generator=g, dtype=torch.float64)
    ref_in = [t.clone().requires_grad_() for t in (A, zi, x)]
    y_r = _loop(*ref_in, lpv)
    g_r = torch.autograd.grad(y_r, ref_in, gy)
    ins = [t.to(dtype).to(DEV).requires_grad_() for t in (A, zi, x)]
    y = (MatrixRecurrence if lpv else LTIMatrixRecurrence).apply(*ins)
    gs = torch.autograd.grad(y, ins, gy.to(dtype).to(DEV))
    t_ = tol(dtype)
    assert rel_err(y, y_r) <= t_
    for got, ref in zip(gs, g_r):
        assert rel_err(got, ref) <= t_ * 10
    ptb.check_errors()


def test_state_space_recursion_scalar_input_order3():
    """A scalar sequence into state 0 of a three-state model (zero-padded like the reference's
    _ext_ss_recur), both front-ends, and the explicit error above eight states."""
    B, T, n = 2, 300, 3
    g = torch.Generator().manual_seed(1)
    A = (torch.randn(B, T, n, n, generator=g, dtype=torch.float64) * 0.3).to(DEV)
    zi = torch.randn(B, n, generator=g, dtype=torch.float64).to(DEV)
    x = torch.randn(B, T, generator=g, dtype=torch.float64).to(DEV)
    xp = torch.cat([x.unsqueeze(-1), x.new_zeros(B, T, n - 1)], -1)
    y = ptb.lpv.state_space_recursion(A, zi, x)
    assert rel_err(y, _loop(A.cpu(), zi.cpu(), xp.cpu(), True)) <= 1e-10
    y0 = ptb.lti.state_space_recursion(A[:, 0].contiguous(), zi, x, out_idx=1)
    assert rel_err(y0, _loop(A[:, 0].cpu(), zi.cpu(), xp.cpu(), False)[..., 1]) <= 1e-10
    with pytest.raises(NotImplementedError):
        ptb.lpv.state_space_recursion(torch.zeros(5, 9, 9, device=DEV), torch.zeros(2, 9, device=DEV),
                                      torch.zeros(2, 5, 9, device=DEV))
    ptb.check_errors()


def test_gradcheck_and_opcheck():
    g = torch.Generator().manual_seed(2)
    B, T, n = 2, 20, 3
    A = (torch.randn(B, T, n, n, generator=g, dtype=torch.float64) * 0.3).to(DEV).requires_grad_()
    Ai = (torch.randn(n, n, generator=g, dtype=torch.float64) * 0.3).to(DEV).requires_grad_()
    zi = torch.randn(B, n, generator=g, dtype=torch.float64).to(DEV).requires_grad_()
    x = torch.randn(B, T, n, generator=g, dtype=torch.float64).to(DEV).requires_grad_()
    assert torch.autograd.gradcheck(MatrixRecurrence.apply, (A, zi, x))
    assert torch.autograd.gradgradcheck(MatrixRecurrence.apply, (A, zi, x))
    assert torch.autograd.gradcheck(LTIMatrixRecurrence.apply, (Ai, zi, x))
    assert torch.autograd.gradgradcheck(LTIMatrixRecurrence.apply, (Ai, zi, x))
    torch.library.opcheck(torch.ops.philtorch_b200.recur_n.default, (A.detach(), zi.detach(), x.detach()))
    torch.library.opcheck(torch.ops.philtorch_b200.lti_recur_n.default, (Ai.detach(), zi.detach(), x.detach()))
    torch.library.opcheck(torch.ops.philtorch_b200.recur_n_adj.default, (A.detach(), x.detach(), None, True))
