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
