"""``prototype.newton_solve`` (a nonlinear recurrence solved by Newton steps that are time-varying
linear recurrences on the GPU kernels) against the reference's result and iteration count
(tests/golden/newton_solve_f64.npz, made by running philtorch.prototype.nl.newton_solve) and against
the sequential evaluation of the recurrence, as the reference's tests/test_nl.py does."""
import pytest
import torch

import philtorch_b200 as ptb
from philtorch_b200.prototype import newton_solve
from conftest import load_golden, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("use_fprime", [True, False])
def test_first_order_smoother(use_fprime):
    g = load_golden("newton_solve_f64")
    x, at, rt, init = (g[k].to(DEV) for k in ("g", "at", "rt", "init"))

    def smoother(prev, inp):
        coeff = torch.where(inp < prev, at, rt)
        return coeff * inp + (1 - coeff) * prev

    def jac(prev, inp):
        return (1 - torch.where(inp < prev, at, rt)).unsqueeze(-2)

    y, iters = newton_solve(smoother, x, torch.ones_like(x), init=init, max_iter=10, atol=1e-8, rtol=1e-6,
                            fprime=jac if use_fprime else None)
    ptb.check_errors()
    assert iters == int(g["iters"])
    assert rel_err(y, g["y"]) <= 1e-10
    assert rel_err(y, g["y_sequential"]) <= 1e-6


def test_two_state_cell():
    g = load_golden("newton_solve_f64")
    W, x, init = (g[k].to(DEV) for k in ("W", "x2", "init2"))

    def cell(prev, inp):
        return torch.tanh(prev @ W.T + inp)

    def jac(prev, inp):
        return (1 - torch.tanh(prev @ W.T + inp) ** 2).unsqueeze(-1) * W

    y, iters, hist = newton_solve(cell, x, torch.zeros_like(x), init=init, max_iter=12, atol=1e-10, rtol=1e-8,
                                  fprime=jac, return_intermediate=True)
    ptb.check_errors()
    assert iters == int(g["iters2"])
    assert rel_err(y, g["y2"]) <= 1e-10
    assert rel_err(y, g["y2_sequential"]) <= 1e-8
    # each entry: the prefix solved so far (one more sample per iteration) and the squared residuals
    assert len(hist) == iters - 1 and all(h[0].shape[1] == k + 2 for k, h in enumerate(hist))
    res = [float(h[1].max()) for h in hist]
    assert res[-1] < res[0]                      # residuals shrink


def test_long_sequence_fp32():
    """A sequence of several tiles in fp32 against the time loop."""
    gen = torch.Generator().manual_seed(0)
    rows, n = 4, 20000
    x = torch.rand(rows, n, 1, generator=gen).to(DEV)
    at, rt = torch.rand(rows, 1, 1, generator=gen).to(DEV) * 0.5 + 0.3, torch.rand(rows, 1, 1, generator=gen).to(DEV) * 0.5 + 0.3
    init = torch.ones(rows, 1, device=DEV)

    def smoother(prev, inp):
        coeff = torch.where(inp < prev, at, rt)
        return coeff * inp + (1 - coeff) * prev

    y, iters = newton_solve(smoother, x, torch.ones_like(x), init=init, max_iter=30, atol=1e-6, rtol=1e-5,
                            fprime=lambda p, i: (1 - torch.where(i < p, at, rt)).unsqueeze(-2))
    ptb.check_errors()
    h, seq = init.cpu().double(), []
    xc, atc, rtc = x.cpu().double(), at.cpu().double().squeeze(1), rt.cpu().double().squeeze(1)
    for t in range(n):
        c = torch.where(xc[:, t] < h, atc, rtc)
        h = c * xc[:, t] + (1 - c) * h
        seq.append(h)
    assert iters < 30
    assert rel_err(y, torch.stack(seq, 1)) <= 1e-4
