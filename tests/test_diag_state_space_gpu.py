"""GPU parity of ``lti.diag_state_space`` (state-space model in its eigenbasis: batch * M complex
first-order recurrences) against the golden vectors made by running the reference's
``philtorch.lti.diag_state_space`` (outputs, final states, gradients) and, at larger sizes, the
sequential state-space restatement in oracle/callers.py.
Tolerance: max|out-ref|/max|ref| <= 1e-4 (fp32), <= 1e-10 (fp64); gradients that pass through the
eigen-decomposition of a matrix are compared at 1e-3 / 1e-8 (two different, equally valid
eigenvector normalisations are differentiated)."""
import pytest
import torch

import philtorch_b200 as ptb
from philtorch_b200.lti import diag_state_space
from conftest import load_golden, rel_err, tol
from oracle import callers

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = {"f32": torch.float32, "f64": torch.float64}


@pytest.fixture(autouse=True, params=[True, False], ids=["fused-bank", "mode-signals"])
def modal_route(request, monkeypatch):
    """Scalar-in / real-scalar-out models run on the fused bank-of-modes kernels, everything else
    (and every higher-order derivative) on the route that keeps the mode signals in memory: every
    case here runs with the fused kernels enabled and disabled."""
    from philtorch_b200.lti import ssm
    monkeypatch.setattr(ssm, "FUSED_MODAL_BANK", request.param)
    return request.param


def _dev(g, *names):
    return [g[n].to(DEV) for n in names]


@pytest.mark.parametrize("tag", ["f32", "f64"])
def test_matrix_system_golden(tag):
    g = load_golden(f"diag_ssm_matrix_{tag}")
    t = tol(DT[tag])
    A, x, Bm, Cm = (v.requires_grad_() for v in _dev(g, "A", "x", "B", "C"))
    D, zi, gy = _dev(g, "D", "zi", "gy")
    y, zf = diag_state_space(x, A=A, B=Bm, C=Cm, D=D, zi=zi)
    gA, gx, gB, gC = torch.autograd.grad(y, (A, x, Bm, Cm), gy)
    ptb.check_errors()
    assert y.dtype == DT[tag] and zf.dtype == DT[tag]
    assert rel_err(y, g["y"]) <= t and rel_err(zf, g["zf"]) <= t
    assert rel_err(gx, g["grad_x"]) <= t and rel_err(gB, g["grad_B"]) <= t and rel_err(gC, g["grad_C"]) <= t
    assert rel_err(gA, g["grad_A"]) <= (1e-3 if tag == "f32" else 1e-8)


@pytest.mark.parametrize("tag", ["f32", "f64"])
def test_given_eigenbasis_golden(tag):
    g = load_golden(f"diag_ssm_eig_batched_{tag}")
    t = tol(DT[tag])
    L, x = (v.requires_grad_() for v in _dev(g, "L", "x"))
    V, Bm, Cm, gy = _dev(g, "V", "B", "C", "gy")
    y = diag_state_space(x, L=L, V=V, B=Bm, C=Cm)
    gL, gx = torch.autograd.grad(y, (L, x), gy)
    ptb.check_errors()
    assert rel_err(y, g["y"]) <= t
    assert rel_err(gL, g["grad_L"]) <= t and rel_err(gx, g["grad_x"]) <= t
    # the inverse given instead of the eigenvectors
    y2 = diag_state_space(x, L=L, Vinv=torch.linalg.inv(V), B=Bm, C=Cm)
    assert rel_err(y2, g["y"]) <= 10 * t


@pytest.mark.parametrize("tag", ["f32", "f64"])
def test_modes_and_selected_state_golden(tag):
    g = load_golden(f"diag_ssm_modes_{tag}")
    t = tol(DT[tag])
    L = g["L"].to(DEV).requires_grad_()
    y = diag_state_space(g["x"].to(DEV), L=L)
    (gL,) = torch.autograd.grad(y, L, g["gy"].to(DEV))
    assert y.is_complex()
    assert rel_err(y, g["y"]) <= t and rel_err(gL, g["grad_L"]) <= t
    A2, x2 = _dev(g, "A2", "x2")
    y_idx = diag_state_space(x2, A=A2, out_idx=1)
    assert rel_err(y_idx, g["y_idx"]) <= t
    # eigenvalues AND the matrix given: eigenvectors are solved for
    y_la = diag_state_space(x2, L=torch.linalg.eigvals(A2), A=A2, out_idx=1)
    assert rel_err(y_la, g["y_idx"]) <= 10 * t
    ptb.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("M,batched", [(2, False), (4, True), (6, False)])
def test_against_sequential_state_space(dtype, M, batched):
    """Orders above two run as M first-order modes; compared with the time loop in the original basis."""
    gen = torch.Generator().manual_seed(M)
    rows, n = 7, 20000
    A = torch.randn(*((rows,) if batched else ()), M, M, generator=gen, dtype=torch.float64)
    A = A / (1.05 * torch.linalg.eigvals(A).abs().amax(-1)[..., None, None])
    x = torch.randn(rows, n, generator=gen, dtype=torch.float64)
    Bm, Cm = torch.randn(M, generator=gen, dtype=torch.float64), torch.randn(M, generator=gen, dtype=torch.float64)
    zi = torch.randn(rows, M, generator=gen, dtype=torch.float64)
    D = torch.tensor([0.3], dtype=torch.float64)
    y, zf = diag_state_space(x.to(dtype).to(DEV), A=A.to(dtype).to(DEV), B=Bm.to(dtype).to(DEV),
                             C=Cm.to(dtype).to(DEV), D=D.to(dtype).to(DEV), zi=zi.to(dtype).to(DEV))
    ptb.check_errors()
    y_ref, zf_ref = callers.state_space(A.to(dtype).double().numpy(), x.to(dtype).double().numpy(),
                                        Bm.to(dtype).double().numpy(), Cm.to(dtype).double().numpy(), D.numpy(),
                                        zi.to(dtype).double().numpy())
    t = 2e-3 if dtype == torch.float32 else 1e-9      # the eigenbasis change costs a few digits (cond(V))
    assert rel_err(y, torch.from_numpy(y_ref)) <= t
    assert rel_err(zf, torch.from_numpy(zf_ref)) <= t


def test_argument_checks():
    x = torch.zeros(4, 50, device=DEV)
    with pytest.raises(ValueError, match="C and out_idx"):
        diag_state_space(x, A=torch.eye(2, device=DEV), C=torch.ones(2, device=DEV), out_idx=0)
    with pytest.raises(AssertionError, match="Either L or A"):
        diag_state_space(x)
    with pytest.raises(AssertionError, match="cannot both be None"):
        diag_state_space(x, L=torch.zeros(4, 2, device=DEV))
    with pytest.raises(ValueError, match="Input matrix B"):
        diag_state_space(x, A=torch.eye(2, device=DEV), B=torch.ones(5, device=DEV))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("num_order,den_order", [(1, 1), (2, 2), (3, 3), (4, 5), (4, 6), (0, 8)])
@pytest.mark.parametrize("form", ["df2", "tdf2"])
@pytest.mark.parametrize("batched", [True, False])
def test_lfilter_diag_backend_scipy(dtype, num_order, den_order, form, batched):
    """``lfilter(..., backend='diag_ssm')`` of any order against scipy.signal.lfilter, the check of the
    reference's tests/test_lti_lfilter.py:355-422."""
    import numpy as np
    from scipy import signal
    from philtorch_b200.lti import lfilter
    rng = np.random.default_rng(num_order * 10 + den_order)
    rows, n = 6, 4000
    nb = rows if batched else 1
    # stable denominators from random poles inside the unit circle (conjugate pairs + real poles)
    a_rows = []
    for _ in range(nb):
        pairs = den_order // 2
        p = 0.3 + 0.65 * rng.random(pairs)
        ph = np.pi * rng.random(pairs)
        roots = np.concatenate([p * np.exp(1j * ph), p * np.exp(-1j * ph), rng.uniform(-0.9, 0.9, den_order % 2)])
        a_rows.append(np.real(np.poly(roots))[1:])
    a = np.stack(a_rows)
    b = rng.standard_normal((nb, num_order + 1))
    x = rng.standard_normal((rows, n))
    to = lambda v: torch.from_numpy(v if batched else v[0]).to(dtype).to(DEV)   # noqa: E731
    y = lfilter(to(b), to(a), torch.from_numpy(x).to(dtype).to(DEV), form=form, backend="diag_ssm")
    ptb.check_errors()
    bq, aq = to(b).double().cpu().numpy().reshape(nb, -1), to(a).double().cpu().numpy().reshape(nb, -1)
    xq = torch.from_numpy(x).to(dtype).double().numpy()
    ref = np.stack([signal.lfilter(bq[i % nb], np.concatenate([[1.0], aq[i % nb]]), xq[i]) for i in range(rows)])
    if y.is_complex():
        assert y.imag.abs().max().item() <= (1e-3 if dtype == torch.float32 else 1e-9) * max(1.0, np.abs(ref).max())
        y = y.real
    assert rel_err(y, torch.from_numpy(ref)) <= (2e-3 if dtype == torch.float32 else 1e-9)


@pytest.mark.parametrize("form", ["df2", "tdf2"])
def test_lfilter_diag_backend_matches_ssm_backend(form):
    """Second order with an initial state: both backends return the same (y, zf)."""
    from philtorch_b200.lti import lfilter
    gen = torch.Generator().manual_seed(2)
    rows, n = 5, 3000
    r, th = 0.5 + 0.4 * torch.rand(rows, generator=gen, dtype=torch.float64), 3.0 * torch.rand(rows, generator=gen, dtype=torch.float64)
    a = torch.stack([-2 * r * torch.cos(th), r * r], -1).to(DEV)
    b = torch.randn(rows, 3, generator=gen, dtype=torch.float64).to(DEV)
    x = torch.randn(rows, n, generator=gen, dtype=torch.float64).to(DEV)
    zi = torch.randn(rows, 2, generator=gen, dtype=torch.float64).to(DEV)
    y1, zf1 = lfilter(b, a, x, zi=zi, form=form, backend="ssm")
    y2, zf2 = lfilter(b, a, x, zi=zi, form=form, backend="diag_ssm")
    assert rel_err(y2.real if y2.is_complex() else y2, y1) <= 1e-9
    assert rel_err(zf2.real if zf2.is_complex() else zf2, zf1) <= 1e-9


@pytest.mark.parametrize("dtype", [torch.complex64, torch.complex128])
@pytest.mark.parametrize("real_out", [True, False])
@pytest.mark.parametrize("coef_batched", [True, False])
@pytest.mark.parametrize("rows,M,N", [(1, 1, 1), (3, 4, 2), (5, 3, 255), (2, 6, 256), (4, 2, 257), (3, 5, 5000)])
def test_modal_mix_kernels(dtype, real_out, coef_batched, rows, M, N):
    """The fused output map (mode sum, one-sample shift, real part) and its adjoint against plain torch."""
    from philtorch_b200.autograd import ModalMix, modal_mix_reference
    gen = torch.Generator().manual_seed(rows * 100 + M * 10 + N)
    mk = lambda *s: torch.complex(torch.randn(*s, generator=gen, dtype=torch.float64),   # noqa: E731
                                  torch.randn(*s, generator=gen, dtype=torch.float64)).to(dtype).to(DEV)
    w, w0, coef = mk(rows, M, N), mk(rows, M), mk(*((rows, M) if coef_batched else (M,)))
    gy = mk(rows, N)
    gy = gy.real.contiguous() if real_out else gy
    outs = []
    for fn in (lambda *a: ModalMix.apply(*a), modal_mix_reference):
        ins = [t.clone().requires_grad_() for t in (w, w0, coef)]
        y = fn(*ins, real_out)
        outs.append([y] + list(torch.autograd.grad(y, ins, gy)))
    ptb.check_errors()
    t = 1e-5 if dtype == torch.complex64 else 1e-12
    for got, ref in zip(outs[0], outs[1]):
        assert got.dtype == ref.dtype and rel_err(got, ref) <= t


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("gain_batched", [True, False])
def test_modal_drive(dtype, gain_batched):
    """Real input broadcast into complex modes: values and both gradients against plain torch."""
    from philtorch_b200.autograd import ModalDrive
    gen = torch.Generator().manual_seed(8)
    rows, M, N = 4, 3, 3000
    cdt = torch.complex64 if dtype == torch.float32 else torch.complex128
    x = torch.randn(rows, N, generator=gen, dtype=torch.float64).to(dtype).to(DEV)
    gain = torch.complex(torch.randn(*((rows, M) if gain_batched else (M,)), generator=gen, dtype=torch.float64),
                         torch.randn(*((rows, M) if gain_batched else (M,)), generator=gen, dtype=torch.float64))
    gain = gain.to(cdt).to(DEV)
    gu = torch.complex(torch.randn(rows, M, N, generator=gen, dtype=torch.float64),
                       torch.randn(rows, M, N, generator=gen, dtype=torch.float64)).to(cdt).to(DEV)
    outs = []
    for fn in (ModalDrive.apply, lambda a, b: b.unsqueeze(-1) * a.unsqueeze(1)):
        a, b = x.clone().requires_grad_(), gain.clone().requires_grad_()
        u = fn(a, b)
        outs.append([u] + list(torch.autograd.grad(u, (a, b), gu)))
    ptb.check_errors()
    for got, ref in zip(outs[0], outs[1]):
        assert got.dtype == ref.dtype and rel_err(got, ref) <= (1e-5 if dtype == torch.float32 else 1e-12)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("M,N,batch", [(1, 300, 3), (2, 2048, 2), (4, 5000, 5), (5, 1023, 3), (8, 4097, 2), (4, 70001, 4)])
def test_fused_bank_matches_mode_signal_route(dtype, M, N, batch, modal_route):
    """The fused kernels against the route that materialises the modes (itself pinned to the
    reference's golden vectors above): outputs, final states and every gradient, with initial
    states, a feed-through term and row lengths that end inside a tile and inside a thread."""
    from philtorch_b200.lti import ssm
    if not modal_route:
        pytest.skip("compares the two routes itself")
    import math
    g = torch.Generator().manual_seed(M * 100 + N)
    cdt = torch.complex64 if dtype == torch.float32 else torch.complex128
    r = 0.6 + 0.39 * torch.rand(batch, M, generator=g, dtype=torch.float64)
    th = 2 * math.pi * torch.rand(batch, M, generator=g, dtype=torch.float64)
    L = torch.polar(r, th).to(cdt).to(DEV)
    V = torch.view_as_complex(torch.randn(batch, M, M, 2, generator=g, dtype=torch.float64)).to(cdt).to(DEV)
    V = V + 2 * torch.eye(M, device=DEV, dtype=cdt)
    Bm = torch.randn(batch, M, generator=g, dtype=torch.float64).to(dtype).to(DEV)
    Cm = torch.randn(batch, M, generator=g, dtype=torch.float64).to(dtype).to(DEV)
    D = torch.randn(batch, generator=g, dtype=torch.float64).to(dtype).to(DEV)
    zi = torch.randn(batch, M, generator=g, dtype=torch.float64).to(dtype).to(DEV)
    x = torch.randn(batch, N, generator=g, dtype=torch.float64).to(dtype).to(DEV)
    gy = torch.randn(batch, N, generator=g, dtype=torch.float64).to(dtype).to(DEV)
    gzf = torch.randn(batch, M, generator=g, dtype=torch.float64).to(dtype).to(DEV)
    res = []
    for fused in (True, False):
        ssm.FUSED_MODAL_BANK = fused
        ins = [t.clone().requires_grad_() for t in (x, L, Bm, Cm, D, zi)]
        y, zf = diag_state_space(ins[0], L=ins[1], V=V, B=ins[2], C=ins[3], D=ins[4], zi=ins[5])
        res.append((y, zf) + torch.autograd.grad([y, zf], ins, [gy, gzf]))
        if fused:
            assert type(y.grad_fn).__name__ != "AddBackward0"    # the feed-through term is inside the kernel
    t = tol(dtype) * 10
    for name, a, b in zip(("y", "zf", "gx", "gL", "gB", "gC", "gD", "gzi"), *res):
        assert a.shape == b.shape and rel_err(a, b) <= t, name
    ptb.check_errors()
