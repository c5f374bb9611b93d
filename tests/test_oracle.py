"""Pins the CPU oracle (oracle/recur_oracle.c) against the reference: the golden vectors
made by running the reference, and -- when it was compiled into oracle/_ref -- the
reference CPU extension itself on fresh seeded inputs."""
import pytest
import torch

from conftest import load_golden, rel_err, tol
from oracle import cport, refext

DT = {"f32": torch.float32, "f64": torch.float64}


@pytest.mark.parametrize("tag", ["f32", "f64"])
@pytest.mark.parametrize("mode", ["batched", "shared1", "scalar"])
def test_lti_recur_golden(tag, mode):
    g = load_golden(f"lti_recur_{mode}_{tag}")
    t = tol(DT[tag])
    y = cport.lti_recur(g["a"], g["zi"], g["x"])
    assert rel_err(y, g["y"]) <= t
    ga, gzi, gx = cport.lti_recur_bwd(g["a"], g["zi"], g["y"], g["gy"])
    assert rel_err(ga, g["grad_a"]) <= t
    assert rel_err(gzi, g["grad_zi"]) <= t
    assert rel_err(gx, g["grad_x"]) <= t


@pytest.mark.parametrize("tag", ["f32", "f64"])
@pytest.mark.parametrize("mode", ["batched", "shared"])
def test_recur1_golden(tag, mode):
    g = load_golden(f"lpv_recur1_{mode}_{tag}")
    t = tol(DT[tag])
    y = cport.recur1(g["a"], g["zi"], g["x"])
    assert rel_err(y, g["y"]) <= t
    assert rel_err(y, g["y_python_loop"]) <= t
    assert rel_err(y, g["y_python_unrolled"]) <= (1e-4 if tag == "f32" else 1e-9)
    ga, gzi, gx = cport.recur1_bwd(g["a"], g["zi"], g["y"], g["gy"])
    assert rel_err(ga, g["grad_a"]) <= t
    assert rel_err(gzi, g["grad_zi"]) <= t
    assert rel_err(gx, g["grad_x"]) <= t


@pytest.mark.parametrize("tag,dtype", [("c64", torch.complex64), ("c128", torch.complex128)])
def test_complex_first_order_golden(tag, dtype):
    """The complex restatement (conjugating adjoint) against vectors made by the reference's
    ``LTIRecurrence`` / 1x1 ``MatrixRecurrence`` on complex data."""
    t = tol(dtype)
    for mode in ("batched", "shared1", "scalar"):
        g = load_golden(f"lti_recur_{mode}_{tag}")
        assert g["y"].dtype == dtype
        assert rel_err(cport.lti_recur(g["a"], g["zi"], g["x"]), g["y"]) <= t
        ga, gzi, gx = cport.lti_recur_bwd(g["a"], g["zi"], g["y"], g["gy"])
        assert rel_err(ga, g["grad_a"]) <= t and rel_err(gzi, g["grad_zi"]) <= t and rel_err(gx, g["grad_x"]) <= t
    for mode in ("batched", "shared"):
        g = load_golden(f"lpv_recur1_{mode}_{tag}")
        y = cport.recur1(g["a"], g["zi"], g["x"])
        assert rel_err(y, g["y"]) <= t and rel_err(y, g["y_python_loop"]) <= t
        ga, gzi, gx = cport.recur1_bwd(g["a"], g["zi"], g["y"], g["gy"])
        assert rel_err(ga, g["grad_a"]) <= t and rel_err(gzi, g["grad_zi"]) <= t and rel_err(gx, g["grad_x"]) <= t


@pytest.mark.parametrize("tag", ["f32", "f64"])
@pytest.mark.parametrize("mode", ["batched", "shared"])
@pytest.mark.parametrize("kind", ["lti", "lpv"])
def test_recur2_golden(tag, mode, kind):
    g = load_golden(f"{kind}_recur2_{mode}_{tag}")
    t = tol(DT[tag])
    fwd = cport.lti_recur2 if kind == "lti" else cport.recur2
    bwd = cport.lti_recur2_bwd if kind == "lti" else cport.recur2_bwd
    y = fwd(g["A"], g["zi"], g["x"])
    assert rel_err(y, g["y"]) <= t
    if kind == "lpv":
        assert rel_err(y, g["y_python_loop"]) <= t
    gA, gzi, gx = bwd(g["A"], g["zi"], g["y"], g["gy"])
    assert rel_err(gA, g["grad_A"]) <= t
    assert rel_err(gzi, g["grad_zi"]) <= t
    assert rel_err(gx, g["grad_x"]) <= t


@pytest.mark.parametrize("tag", ["f32", "f64"])
@pytest.mark.parametrize("mode", ["batched", "shared"])
def test_biquad_golden(tag, mode):
    g = load_golden(f"lfilter_order2_{mode}_{tag}")
    t = tol(DT[tag])
    y, _ = cport.biquad_tdf2(g["b"], g["a"], None, g["x"])
    assert rel_err(y, g["tdf2_y"]) <= t
    y, zf = cport.biquad_tdf2(g["b"], g["a"], g["zi"], g["x"])
    assert rel_err(y, g["tdf2_y_zi"]) <= t
    assert rel_err(zf, g["tdf2_zf"]) <= t


@pytest.mark.parametrize("tag", ["f32", "f64"])
@pytest.mark.parametrize("mode", ["batched", "shared"])
def test_biquad_adjoint_golden(tag, mode):
    """The section's adjoint against gradients the reference's autograd produced."""
    g = load_golden(f"lfilter_order2_{mode}_{tag}")
    t = tol(DT[tag])
    gb, ga, _, gx = cport.biquad_tdf2_bwd(g["b"], g["a"], None, g["x"], g["gy"])
    assert rel_err(gb, g["tdf2_grad_b"]) <= t and rel_err(ga, g["tdf2_grad_a"]) <= t
    assert rel_err(gx, g["tdf2_grad_x"]) <= t
    gb, ga, gzi, gx = cport.biquad_tdf2_bwd(g["b"], g["a"], g["zi"], g["x"], g["gy"], g["gzf"])
    assert rel_err(gb, g["tdf2_zi_grad_b"]) <= t and rel_err(ga, g["tdf2_zi_grad_a"]) <= t
    assert rel_err(gx, g["tdf2_zi_grad_x"]) <= t and rel_err(gzi, g["tdf2_zi_grad_zi"]) <= t


def test_sos_chain_golden():
    """Six chained sections (the reduced third benchmark configuration) against the reference's run."""
    from philtorch_b200.workloads import sos_cascade

    g = load_golden("config3_small")
    w = sos_cascade(B=4, T=4096, sections=6)
    ins, y = cport.sos_chain(w["b"], w["a"], w["x"])
    gb, ga, gx = cport.sos_chain_bwd(w["b"], w["a"], ins, w["gy"])
    assert rel_err(y, g["y"]) <= 1e-4 and rel_err(gx, g["grad_x"]) <= 1e-4
    assert rel_err(gb, g["grad_b"]) <= 1e-4 and rel_err(ga, g["grad_a"]) <= 1e-4


def test_g_in_chains_adjoint():
    """An adjoint state entering from the right equals running the adjoint on the
    concatenated sequence (used when a long sequence is split along time)."""
    torch.manual_seed(0)
    B, T = 3, 64
    a = torch.rand(B, T, dtype=torch.float64) * 1.9 - 0.95
    zi = torch.randn(B, dtype=torch.float64)
    x = torch.randn(B, T, dtype=torch.float64)
    gy = torch.randn(B, T, dtype=torch.float64)
    y = cport.recur1(a, zi, x)
    ga, gzi, gx = cport.recur1_bwd(a, zi, y, gy)
    h = T // 2
    ga2, gzi2, gx2 = cport.recur1_bwd(a[:, h:], y[:, h - 1], y[:, h:], gy[:, h:])
    ga1, gzi1, gx1 = cport.recur1_bwd(a[:, :h], zi, y[:, :h], gy[:, :h], g_in=gzi2)
    assert rel_err(torch.cat([gx1, gx2], 1), gx) <= 1e-12
    assert rel_err(torch.cat([ga1, ga2], 1), ga) <= 1e-12
    assert rel_err(gzi1, gzi) <= 1e-12


needs_ref = pytest.mark.skipif(not refext.available(), reason="reference extension not built")


@needs_ref
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_against_reference_extension(dtype):
    torch.manual_seed(1)
    B, T = 5, 333
    t = tol(dtype)
    zi = torch.randn(B, dtype=dtype)
    x = torch.randn(B, T, dtype=dtype)
    gy = torch.randn(B, T, dtype=dtype)
    for a in (torch.rand(B, dtype=dtype) * 1.8 - 0.9, torch.rand(1, dtype=dtype) * 1.8 - 0.9):
        y = cport.lti_recur(a, zi, x)
        assert rel_err(y, refext.lti_recur(a, zi, x)) <= t
        for o, r in zip(cport.lti_recur_bwd(a, zi, y, gy), refext.lti_recur_bwd(a, zi, y, gy)):
            assert rel_err(o, r) <= t
    for a in (torch.rand(B, T, dtype=dtype) * 1.9 - 0.95, torch.rand(T, dtype=dtype) * 1.9 - 0.95):
        y = cport.recur1(a, zi, x)
        assert rel_err(y, refext.recur1(a, zi, x)) <= t
        for o, r in zip(cport.recur1_bwd(a, zi, y, gy), refext.recur1_bwd(a, zi, y, gy)):
            assert rel_err(o, r) <= t
    zi2 = torch.randn(B, 2, dtype=dtype)
    x2 = torch.randn(B, T, 2, dtype=dtype)
    gy2 = torch.randn(B, T, 2, dtype=dtype)
    for A in (torch.randn(B, 2, 2, dtype=dtype) * 0.4, torch.randn(2, 2, dtype=dtype) * 0.4):
        y = cport.lti_recur2(A, zi2, x2)
        assert rel_err(y, refext.lti_recur2(A, zi2, x2)) <= t
        for o, r in zip(cport.lti_recur2_bwd(A, zi2, y, gy2), refext.lti_recur2_bwd(A, zi2, y, gy2)):
            assert rel_err(o, r) <= t
    for A in (torch.randn(B, T, 2, 2, dtype=dtype) * 0.4, torch.randn(T, 2, 2, dtype=dtype) * 0.4):
        y = cport.recur2(A, zi2, x2)
        assert rel_err(y, refext.recur2(A, zi2, x2)) <= t
        for o, r in zip(cport.recur2_bwd(A, zi2, y, gy2), refext.recur2_bwd(A, zi2, y, gy2)):
            assert rel_err(o, r) <= t


# ---- callers that are pure first-order passes (numpy restatements in oracle/callers.py) ----------
COMB_CASES = [(1, "none"), (5, "none"), (13, "shared"), (5, "batched"), (32, "none")]


@pytest.mark.parametrize("delay,zs", COMB_CASES)
@pytest.mark.parametrize("mode", ["batched", "scalar"])
def test_comb_oracle_golden(delay, zs, mode):
    from oracle import callers
    g = load_golden(f"comb_d{delay}_zi{zs}_{mode}_f64")
    zi = g.get("zi")
    y = callers.comb_filter(g["a"].numpy(), delay, g["x"].numpy(), None if zi is None else zi.numpy())
    assert rel_err(torch.from_numpy(y), g["y"]) <= 1e-12


@pytest.mark.parametrize("scipy_padding", [True, False])
def test_cspline_oracle_golden(scipy_padding):
    from oracle import callers
    g = load_golden("cspline_f64")
    pad = "scipy" if scipy_padding else "reflect"
    c = torch.from_numpy(callers.cspline(g["x"].numpy(), scipy_padding))
    assert rel_err(c, g[f"c_parallel_{pad}"]) <= 1e-12
    assert rel_err(c, g[f"c_cascade_{pad}"]) <= 1e-12     # the reference's two evaluations agree
    for m in (2, 3, 7):
        y = torch.from_numpy(callers.cubic_spline(g["x"].numpy(), m, scipy_padding))
        assert rel_err(y, g[f"up_m{m}_{pad}"]) <= 1e-12


def test_cspline_oracle_scipy():
    """The check the reference's own test makes (tests/test_interp.py:60-70)."""
    from scipy.signal import cspline1d
    from oracle import callers
    x = torch.randn(4, 200, dtype=torch.float64, generator=torch.Generator().manual_seed(1)).numpy()
    c = callers.cspline(x, True)
    for row in range(4):
        assert abs(c[row] - cspline1d(x[row])).max() <= 1e-10


def test_state_space_oracle_golden():
    """The sequential state-space restatement against ``diag_state_space`` run by the reference."""
    from oracle import callers
    g = load_golden("diag_ssm_matrix_f64")
    y, zf = callers.state_space(g["A"].numpy(), g["x"].numpy(), g["B"].numpy(), g["C"].numpy(), g["D"].numpy(),
                                g["zi"].numpy())
    assert rel_err(torch.from_numpy(y), g["y"]) <= 1e-10
    assert rel_err(torch.from_numpy(zf), g["zf"]) <= 1e-10
