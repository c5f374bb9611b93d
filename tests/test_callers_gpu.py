"""GPU parity of the callers that are pure first-order passes: ``lti.comb_filter`` and
``lti.interp.cspline`` / ``cubic_spline``, against the golden vectors made by running the reference
(outputs and gradients), the numpy restatements in oracle/callers.py at larger sizes, and scipy
(the reference's own check, tests/test_interp.py).  Tolerance: max|out-ref|/max|ref| <= 1e-4 (fp32),
<= 1e-10 (fp64)."""
import numpy as np
import pytest
import torch

import philtorch_b200 as ptb
from philtorch_b200.lti import comb_filter
from philtorch_b200.lti.interp import cspline, cubic_spline
from conftest import load_golden, rel_err, tol
from oracle import callers

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = {"f32": torch.float32, "f64": torch.float64}
COMB_CASES = [(1, "none"), (5, "none"), (13, "shared"), (5, "batched"), (32, "none")]


@pytest.fixture(params=["folded_scan", "comb_kernels", "comb_slabs_256", "comb_slabs_128", "comb_slabs_64"], autouse=True)
def comb_route(request, monkeypatch):
    """Every test runs on every route of comb_filter: the folded first-order scan, the lane-per-phase
    comb kernels, and the slab kernels with bands of 256, 128 and 64 phases (which hand layouts they
    cannot take -- delay or length not a multiple of 16 bytes -- to the lane-per-phase kernels)."""
    from philtorch_b200 import _lib
    from philtorch_b200.lti import filtering
    monkeypatch.setattr(filtering, "COMB_KERNEL_MIN_LANES", 10 ** 12 if request.param == "folded_scan" else 1)
    policy = {"folded_scan": 0, "comb_kernels": 1, "comb_slabs_256": 2, "comb_slabs_128": 3, "comb_slabs_64": 4}[request.param]
    assert _lib.lib.ptb_comb_set_policy(policy) == 0
    yield request.param
    assert _lib.lib.ptb_comb_set_policy(0) == 0


@pytest.mark.parametrize("tag", ["f32", "f64"])
@pytest.mark.parametrize("delay,zs", COMB_CASES)
@pytest.mark.parametrize("mode", ["batched", "scalar"])
def test_comb_golden(tag, delay, zs, mode):
    g = load_golden(f"comb_d{delay}_zi{zs}_{mode}_{tag}")
    t = tol(DT[tag])
    a = g["a"].to(DEV).requires_grad_()
    x = g["x"].to(DEV).requires_grad_()
    zi = g["zi"].to(DEV) if "zi" in g else None
    res = comb_filter(a, delay, x, zi=zi)
    if zi is not None and delay > 1:
        y, zf = res
        assert rel_err(zf, g["zf"]) <= t
    else:
        y = res
    ga, gx = torch.autograd.grad(y, (a, x), g["gy"].to(DEV))
    ptb.check_errors()
    assert rel_err(y, g["y"]) <= t
    assert rel_err(ga, g["grad_a"]) <= t
    assert rel_err(gx, g["grad_x"]) <= t


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("delay,n", [(2, 50001), (7, 30000), (100, 100000), (1000, 65536), (4096, 10000)])
def test_comb_sizes(dtype, delay, n):
    g = torch.Generator().manual_seed(delay)
    rows = 6
    a = (torch.rand(rows, generator=g, dtype=torch.float64) * 1.9 - 0.95).to(dtype)
    x = torch.randn(rows, n, generator=g, dtype=torch.float64).to(dtype)
    zi = torch.randn(rows, delay, generator=g, dtype=torch.float64).to(dtype)
    y, zf = comb_filter(a.to(DEV), delay, x.to(DEV), zi=zi.to(DEV))
    ptb.check_errors()
    ref = torch.from_numpy(callers.comb_filter(a.numpy(), delay, x.numpy(), zi.numpy()))
    assert rel_err(y, ref) <= tol(dtype)
    assert rel_err(zf, ref[:, -delay:].flip(1)) <= tol(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("delay,n,zi_kind", [(3, 1000, "batched"), (129, 5000, "shared"), (1000, 30011, "batched"),
                                              (500, 300, "batched"), (64, 64 * 40, None), (1000, 68000, "batched"),
                                              (300, 300 * 131 + 152, "shared"), (260, 260 * 16, "batched"),
                                              (4, 4096, None)])
@pytest.mark.parametrize("a_batched", [True, False])
def test_comb_routes_agree(dtype, delay, n, zi_kind, a_batched, comb_route, monkeypatch):
    """Outputs and all gradients (a, zi, x) of the comb kernels against the folded scan."""
    if comb_route == "folded_scan":
        pytest.skip("compares the two routes once")
    from philtorch_b200.lti import filtering
    gen = torch.Generator().manual_seed(delay + n)
    rows = 5
    a0 = (torch.rand(rows if a_batched else (), generator=gen, dtype=torch.float64) * 1.9 - 0.95).to(dtype).to(DEV)
    x0 = torch.randn(rows, n, generator=gen, dtype=torch.float64).to(dtype).to(DEV)
    gy = torch.randn(rows, n, generator=gen, dtype=torch.float64).to(dtype).to(DEV)
    zi0 = None if zi_kind is None else torch.randn(*((rows, delay) if zi_kind == "batched" else (delay,)),
                                                   generator=gen, dtype=torch.float64).to(dtype).to(DEV)
    out = {}
    for route, lanes in (("kernels", 1), ("fold", 10 ** 12)):
        monkeypatch.setattr(filtering, "COMB_KERNEL_MIN_LANES", lanes)
        a, x = a0.clone().requires_grad_(), x0.clone().requires_grad_()
        zi = None if zi0 is None else zi0.clone().requires_grad_()
        res = comb_filter(a, delay, x, zi=zi)
        y = res[0] if isinstance(res, tuple) else res
        ins = [a, x] + ([zi] if zi is not None else [])
        out[route] = [y] + list(torch.autograd.grad(y, ins, gy))
    ptb.check_errors()
    t = tol(dtype)
    for got, ref in zip(out["kernels"], out["fold"]):
        assert rel_err(got, ref) <= (10 * t if got.dim() < 2 else t)


def test_comb_argument_checks():
    x = torch.zeros(4, 100, device=DEV)
    with pytest.raises(AssertionError, match="at most 1D"):
        comb_filter(torch.zeros(4, 1, device=DEV), 3, x)
    with pytest.raises(AssertionError, match="must be 2D"):
        comb_filter(torch.zeros(4, device=DEV), 3, x[0])
    with pytest.raises(AssertionError, match="batch size"):
        comb_filter(torch.zeros(3, device=DEV), 3, x)


@pytest.mark.parametrize("tag", ["f32", "f64"])
def test_cspline_golden(tag):
    g = load_golden(f"cspline_{tag}")
    t = tol(DT[tag])
    x = g["x"].to(DEV).requires_grad_()
    gy = g["gy"].to(DEV)
    for form, pfe in (("parallel", True), ("cascade", False)):
        for pad, sp in (("scipy", True), ("reflect", False)):
            c = cspline(x, parallel_form=pfe, scipy_padding=sp)
            (gx,) = torch.autograd.grad(c, x, gy)
            assert rel_err(c, g[f"c_{form}_{pad}"]) <= t
            assert rel_err(gx, g[f"grad_x_{form}_{pad}"]) <= t
    for m in (2, 3, 7):
        for pad, sp in (("scipy", True), ("reflect", False)):
            y = cubic_spline(x, m, scipy_padding=sp)
            gu = torch.linspace(-1, 1, y.shape[1], dtype=y.dtype, device=DEV).expand_as(y)
            (gx,) = torch.autograd.grad(y, x, gu)
            assert rel_err(y, g[f"up_m{m}_{pad}"]) <= t
            assert rel_err(gx, g[f"up_grad_x_m{m}_{pad}"]) <= t
    ptb.check_errors()
    assert cubic_spline(x, 1) is x
    with pytest.raises(NotImplementedError):
        cspline(x, lamb=0.1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("n", [20, 100, 20000])
@pytest.mark.parametrize("pfe", [True, False])
def test_cspline_scipy(dtype, n, pfe):
    """As tests/test_interp.py:60-70 of the reference: the coefficients of scipy.signal.cspline1d."""
    from scipy.signal import cspline1d
    x = torch.randn(3, n, dtype=torch.float64, generator=torch.Generator().manual_seed(n))
    c = cspline(x.to(dtype).to(DEV), parallel_form=pfe, scipy_padding=True)
    ref = torch.from_numpy(np.stack([cspline1d(row) for row in x.to(dtype).double().numpy()]))
    assert rel_err(c, ref) <= tol(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("m", [2, 5])
@pytest.mark.parametrize("scipy_padding", [True, False])
def test_cubic_spline_sizes(dtype, m, scipy_padding):
    x = torch.randn(5, 30000, dtype=torch.float64, generator=torch.Generator().manual_seed(m)).to(dtype)
    y = cubic_spline(x.to(DEV), m, scipy_padding=scipy_padding)
    ptb.check_errors()
    ref = torch.from_numpy(callers.cubic_spline(x.double().numpy(), m, scipy_padding))
    assert rel_err(y, ref) <= tol(dtype)
    assert rel_err(y[:, ::m], x) <= tol(dtype)        # the spline interpolates the samples


@pytest.mark.parametrize("scipy_padding", [True, False])
def test_cubic_spline_long_rows(scipy_padding):
    """Two rows of 2^17 samples (the prefilter cuts them into pieces), upsampled by 3, with the gradient
    checked through the adjoint identity <gy, S u> = <S^T gy, u> of the linear map S."""
    n, m = 1 << 17, 3
    gen = torch.Generator().manual_seed(23)
    x0 = torch.randn(2, n, generator=gen, dtype=torch.float64)
    x = x0.to(DEV).requires_grad_()
    y = cubic_spline(x, m, scipy_padding=scipy_padding)
    ref = torch.from_numpy(callers.cubic_spline(x0.numpy(), m, scipy_padding))
    assert rel_err(y.detach(), ref) <= tol(torch.float64)
    gy = torch.randn(y.shape, generator=gen, dtype=torch.float64).to(DEV)
    (gx,) = torch.autograd.grad(y, x, gy)
    u = torch.randn(2, n, generator=gen, dtype=torch.float64)
    lhs = (gy.cpu() * torch.from_numpy(callers.cubic_spline(u.numpy(), m, scipy_padding))).sum()
    rhs = (gx.cpu() * u).sum()
    ptb.check_errors()
    assert abs(lhs - rhs) <= 1e-9 * float(gy.norm() * u.norm())


@pytest.mark.parametrize("scipy_padding", [True, False])
@pytest.mark.parametrize("pfe", [True, False])
def test_cspline_gradcheck(scipy_padding, pfe, comb_route):
    if comb_route != "folded_scan":
        pytest.skip("independent of the comb route")
    x = torch.randn(2, 40, dtype=torch.float64, device=DEV, generator=torch.Generator(DEV).manual_seed(3))
    x.requires_grad_()
    fn = lambda v: cspline(v, parallel_form=pfe, scipy_padding=scipy_padding)   # noqa: E731
    assert torch.autograd.gradcheck(fn, (x,), eps=1e-6, atol=1e-7)
    assert torch.autograd.gradgradcheck(fn, (x,), eps=1e-6, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("n", [2, 3, 7, 1500, 40000])
@pytest.mark.parametrize("scipy_padding", [True, False])
def test_cspline_forms_agree(dtype, n, scipy_padding, comb_route):
    """The fused two-pass evaluation against the cascaded one (different kernels), values and gradients."""
    if comb_route != "folded_scan":
        pytest.skip("independent of the comb route")
    gen = torch.Generator().manual_seed(n)
    x0 = torch.randn(4, n, generator=gen, dtype=torch.float64).to(dtype).to(DEV)
    gy = torch.randn(4, n, generator=gen, dtype=torch.float64).to(dtype).to(DEV)
    res = []
    for pfe in (True, False):
        x = x0.clone().requires_grad_()
        c = cspline(x, parallel_form=pfe, scipy_padding=scipy_padding)
        res.append((c, torch.autograd.grad(c, x, gy)[0]))
    ptb.check_errors()
    assert rel_err(res[0][0], res[1][0]) <= 10 * tol(dtype)
    assert rel_err(res[0][1], res[1][1]) <= 10 * tol(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("scipy_padding", [True, False])
def test_cspline_row_pieces(dtype, scipy_padding, comb_route):
    """Few long rows (3 x 2^18) run as 16 pieces per row whose entering states are power sums over the
    neighbouring samples: against the oracle's whole-row evaluation, and values and gradients against
    the cascaded form, which runs whole rows on other kernels."""
    if comb_route != "folded_scan":
        pytest.skip("independent of the comb route")
    from philtorch_b200.lti import interp
    rows, n = 3, 1 << 18
    assert interp._segments(rows, n, torch.empty((), dtype=dtype).element_size()) == 16
    gen = torch.Generator().manual_seed(17)
    x0 = torch.randn(rows, n, generator=gen, dtype=torch.float64).to(dtype)
    gy = torch.randn(rows, n, generator=gen, dtype=torch.float64).to(dtype).to(DEV)
    res = []
    for pfe in (True, False):
        x = x0.to(DEV).requires_grad_()
        c = cspline(x, parallel_form=pfe, scipy_padding=scipy_padding)
        res.append((c.detach(), torch.autograd.grad(c, x, gy)[0]))
    ptb.check_errors()
    ref = torch.from_numpy(callers.cspline(x0.double().numpy(), scipy_padding))
    assert rel_err(res[0][0], ref) <= tol(dtype)
    assert rel_err(res[0][0], res[1][0]) <= 10 * tol(dtype)
    assert rel_err(res[0][1], res[1][1]) <= 10 * tol(dtype)


def test_comb_large_signal_routes_agree(comb_route, monkeypatch):
    """A signal of benchmark proportions (16 rows x 2^20 samples, delay 1000: 1048 steps of 1000
    phases, a ragged tail of 576 samples): the default kernel choice against the folded scan, outputs
    and all gradients."""
    if comb_route != "folded_scan":
        pytest.skip("compares the default choice with the folded scan once")
    from philtorch_b200.lti import filtering
    rows, n, delay = 16, 1 << 20, 1000
    gen = torch.Generator(device=DEV).manual_seed(3)
    a0 = torch.rand(rows, device=DEV, generator=gen) * 1.8 - 0.9
    x0 = torch.randn(rows, n, device=DEV, generator=gen)
    zi0 = torch.randn(rows, delay, device=DEV, generator=gen)
    gy = torch.randn(rows, n, device=DEV, generator=gen)
    out = {}
    for route, lanes in (("kernels", 1), ("fold", 10 ** 12)):
        monkeypatch.setattr(filtering, "COMB_KERNEL_MIN_LANES", lanes)
        a, x, zi = a0.clone().requires_grad_(), x0.clone().requires_grad_(), zi0.clone().requires_grad_()
        y, zf = comb_filter(a, delay, x, zi=zi)
        out[route] = [y, zf] + list(torch.autograd.grad(y, (a, x, zi), gy))
    ptb.check_errors()
    for got, ref in zip(out["kernels"], out["fold"]):
        assert rel_err(got, ref.cpu()) <= (1e-3 if got.dim() < 2 else 1e-4)
