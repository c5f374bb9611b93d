"""Host-side logic of the callers built on the first-order recurrence (``comb_filter`` folding,
spline prefilter boundary terms, ``diag_state_space`` basis changes) on CPU: the CUDA autograd
Functions are replaced by stand-ins that run the CPU oracle, and the results are compared with the
golden vectors made by running the reference."""
import pytest
import torch

from conftest import load_golden, rel_err
from oracle import cport


class _Forward:
    """Stand-in for ``LTIRecurrence`` (forward only)."""

    @staticmethod
    def apply(a, zi, x):
        return cport.lti_recur(a, zi.contiguous(), x)


class _Reverse:
    """Stand-in for ``ReverseLTIRecurrence``: g[t] = a g[t+1] + x[t], g[T] = end."""

    @staticmethod
    def apply(a, end, x):
        return cport.lti_recur(a, end.contiguous(), x.flip(1)).flip(1)


class _Mix:
    """Stand-in for ``ModalMix``: its plain-torch form."""

    @staticmethod
    def apply(w, w0, coef, real_out):
        from philtorch_b200.autograd import modal_mix_reference
        return modal_mix_reference(w, w0, coef, real_out)


@pytest.fixture
def cpu_kernels(monkeypatch):
    import philtorch_b200.lti.filtering as filtering
    import philtorch_b200.lti.interp as interp
    import philtorch_b200.lti.recur as recur
    import philtorch_b200.lti.ssm as ssm
    for mod in (recur, interp, ssm):
        monkeypatch.setattr(mod, "LTIRecurrence", _Forward)
    monkeypatch.setattr(interp, "ReverseLTIRecurrence", _Reverse)
    monkeypatch.setattr(ssm, "ModalMix", _Mix)
    monkeypatch.setattr(filtering, "COMB_KERNEL_MIN_LANES", 10 ** 12)   # the folded route is the host logic


@pytest.mark.parametrize("delay,zs", [(1, "none"), (5, "none"), (13, "shared"), (5, "batched"), (32, "none")])
@pytest.mark.parametrize("mode", ["batched", "scalar"])
def test_comb_fold(cpu_kernels, delay, zs, mode):
    from philtorch_b200.lti import comb_filter
    g = load_golden(f"comb_d{delay}_zi{zs}_{mode}_f64")
    res = comb_filter(g["a"], delay, g["x"], zi=g.get("zi"))
    if isinstance(res, tuple):
        assert rel_err(res[1], g["zf"]) <= 1e-12
        res = res[0]
    assert rel_err(res, g["y"]) <= 1e-12


@pytest.mark.parametrize("parallel_form", [True, False])
@pytest.mark.parametrize("scipy_padding", [True, False])
def test_spline_boundaries(cpu_kernels, parallel_form, scipy_padding):
    from philtorch_b200.lti import interp
    g = load_golden("cspline_f64")
    key = f"{'parallel' if parallel_form else 'cascade'}_{'scipy' if scipy_padding else 'reflect'}"
    c = interp._coefficients(g["x"], parallel_form, scipy_padding, fused=False)
    assert rel_err(c, g["c_" + key]) <= 1e-12


@pytest.mark.parametrize("scipy_padding", [True, False])
def test_spline_row_pieces(cpu_kernels, monkeypatch, scipy_padding):
    """Few long rows are cut into pieces whose entering states are power sums over the neighbouring
    samples: with the two kernel passes replaced by the oracle, values equal the whole-row
    composite evaluation and the gradient is the transposed map (float64, so the truncated sums are exact)."""
    from philtorch_b200.lti import interp

    def causal(a, start, x):
        return cport.lti_recur(a.expand(x.shape[0]).contiguous(), start.contiguous(), x.contiguous())

    def reverse_fused(a, x, second, g_in, need_first):
        rows = x.shape[0]
        a_rows = a.expand(rows).contiguous()
        # g[t] = x[t] + a g[t+1], g[T-1] = x[T-1] + g_in: the forward oracle over the flipped signal
        g = cport.lti_recur(a_rows, (g_in / a_rows).contiguous(), x.flip(1).contiguous()).flip(1)
        return interp.GAIN * (g + second - x), (a_rows * g[:, 0] if need_first else x.new_empty(0))

    monkeypatch.setattr(interp, "_causal_kernel", causal)
    monkeypatch.setattr(interp, "_reverse_fused_kernel", reverse_fused)
    monkeypatch.setattr(interp, "SEGMENT_MIN_LENGTH", 2048)
    gen = torch.Generator().manual_seed(11)
    x0 = torch.randn(3, 1 << 14, generator=gen, dtype=torch.float64)
    gy = torch.randn(3, 1 << 14, generator=gen, dtype=torch.float64)
    assert interp._segments(3, 1 << 14, 8) == 8
    assert interp._segments(3, (1 << 14) + 2, 8) == 1 and interp._segments(300, 1 << 14, 8) == 1
    x = x0.clone().requires_grad_()
    c = interp._coefficients(x, True, scipy_padding, fused=True)
    (gx,) = torch.autograd.grad(c, x, gy)
    assert rel_err(c.detach(), interp._coefficients(x0, True, scipy_padding, fused=False)) <= 1e-12
    # the map is linear, c = M x, so the gradient M^T gy satisfies <gy, M u> = <M^T gy, u> for any u
    # (the stand-ins are not differentiable, the composite form gives no gradient to compare with)
    for seed in (1, 2):
        u = torch.randn(3, 1 << 14, generator=torch.Generator().manual_seed(seed), dtype=torch.float64)
        lhs = (gy * interp._coefficients(u, True, scipy_padding, fused=False)).sum()
        rhs = (gx * u).sum()
        assert abs(lhs - rhs) <= 1e-10 * (gy.norm() * u.norm())


def test_diag_state_space_basis(cpu_kernels):
    from philtorch_b200.lti import diag_state_space
    g = load_golden("diag_ssm_matrix_f64")
    y, zf = diag_state_space(g["x"], A=g["A"], B=g["B"], C=g["C"], D=g["D"], zi=g["zi"])
    assert not y.is_complex() and rel_err(y, g["y"]) <= 1e-10 and rel_err(zf, g["zf"]) <= 1e-10
    g = load_golden("diag_ssm_eig_batched_f64")
    assert rel_err(diag_state_space(g["x"], L=g["L"], V=g["V"], B=g["B"], C=g["C"]), g["y"]) <= 1e-10
    g = load_golden("diag_ssm_modes_f64")
    assert rel_err(diag_state_space(g["x"], L=g["L"]), g["y"]) <= 1e-10
    assert rel_err(diag_state_space(g["x2"], A=g["A2"], out_idx=1), g["y_idx"]) <= 1e-10
    y_la = diag_state_space(g["x2"], L=torch.linalg.eigvals(g["A2"]), A=g["A2"], out_idx=1)
    assert rel_err(y_la, g["y_idx"]) <= 1e-9


def test_lfilter_diag_backend_high_order(cpu_kernels):
    """Order 5 through the eigenbasis against scipy.signal.lfilter."""
    import numpy as np
    from scipy import signal
    from philtorch_b200.lti import lfilter
    rng = np.random.default_rng(5)
    p, ph = 0.3 + 0.6 * rng.random(2), np.pi * rng.random(2)
    roots = np.concatenate([p * np.exp(1j * ph), p * np.exp(-1j * ph), [0.5]])
    a = np.real(np.poly(roots))[1:]
    b = rng.standard_normal(4)
    x = rng.standard_normal((3, 500))
    for form in ("df2", "tdf2"):
        y = lfilter(torch.from_numpy(b), torch.from_numpy(a), torch.from_numpy(x), form=form, backend="diag_ssm")
        ref = np.stack([signal.lfilter(b, np.concatenate([[1.0], a]), row) for row in x])
        assert rel_err(y.real if y.is_complex() else y, torch.from_numpy(ref)) <= 1e-9
