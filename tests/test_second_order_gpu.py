"""GPU parity of the 2x2 kernels (torch ops -> ctypes -> C ABI) against the CPU oracle and the
golden vectors made by the reference.  Tolerance: max|out-ref|/max|ref| <= 1e-4 (fp32),
<= 1e-10 (fp64)."""
import math

import pytest
import torch

import philtorch_b200 as ptb
from philtorch_b200 import workloads
from philtorch_b200.autograd import LTIMatrixRecurrence, MatrixRecurrence
from conftest import load_golden, rel_err, tol
from oracle import cport

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=[10**9, 1], ids=["large-cta", "small-cta"])
def lpv_forward_kernel(request):
    """The time-varying 2x2 forward runs on one of two kernels, normally picked by the batch size:
    every case here runs on both."""
    from philtorch_b200 import _lib
    assert _lib.lib.ptb_lpv_recur2_set_small_cta_min_rows(request.param) == 0
    yield request.param
    assert _lib.lib.ptb_lpv_recur2_set_small_cta_min_rows(48) == 0
DEV = "cuda"
DT = {"f32": torch.float32, "f64": torch.float64}
# tiles are a few thousand samples (e.g. 3840 forward / 2816 backward in fp32, 1792 / 1280 in fp64)
LENGTHS = [1, 2, 3, 7, 33, 101, 768, 769, 1279, 1280, 1281, 1792, 1793, 2816, 2817, 3839, 3840, 3841, 9001, 16000]


def _stable_A(shape, g, dtype):
    """Random 2x2 matrices with spectral radius < 1 (rotation-scaling plus a small perturbation)."""
    r = 0.5 + 0.45 * torch.rand(shape, generator=g, dtype=torch.float64)
    th = math.pi * torch.rand(shape, generator=g, dtype=torch.float64)
    A = torch.stack([torch.stack([r * torch.cos(th), -r * torch.sin(th)], -1),
                     torch.stack([r * torch.sin(th), r * torch.cos(th)], -1)], -2)
    return (A + 0.02 * torch.randn(A.shape, generator=g, dtype=torch.float64)).to(dtype)


def _run(kind, A, zi, x, gy):
    fn = LTIMatrixRecurrence if kind == "lti" else MatrixRecurrence
    A_, zi_, x_ = (t.to(DEV).requires_grad_() for t in (A, zi, x))
    y = fn.apply(A_, zi_, x_)
    gA, gzi, gx = torch.autograd.grad(y, (A_, zi_, x_), gy.to(DEV))
    ptb.check_errors()
    return y, gA, gzi, gx


def _check(kind, A, zi, x, gy, dtype):
    t = tol(dtype)
    y, gA, gzi, gx = _run(kind, A, zi, x, gy)
    fwd = cport.lti_recur2 if kind == "lti" else cport.recur2
    bwd = cport.lti_recur2_bwd if kind == "lti" else cport.recur2_bwd
    y_ref = fwd(A, zi, x)
    gA_ref, gzi_ref, gx_ref = bwd(A, zi, y_ref, gy)
    assert rel_err(y, y_ref) <= t
    assert rel_err(gx, gx_ref) <= t
    assert rel_err(gzi, gzi_ref) <= t
    assert rel_err(gA, gA_ref) <= t


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("T", LENGTHS)
@pytest.mark.parametrize("batched", [True, False])
def test_lpv_lengths(dtype, T, batched):
    B = 3
    g = torch.Generator().manual_seed(T * 3 + batched)
    A = _stable_A((B, T) if batched else (T,), g, dtype)
    zi = torch.randn(B, 2, generator=g, dtype=torch.float64).to(dtype)
    x = torch.randn(B, T, 2, generator=g, dtype=torch.float64).to(dtype)
    gy = torch.randn(B, T, 2, generator=g, dtype=torch.float64).to(dtype)
    _check("lpv", A, zi, x, gy, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("T", LENGTHS)
@pytest.mark.parametrize("batched", [True, False])
def test_lti_lengths(dtype, T, batched):
    B = 3
    g = torch.Generator().manual_seed(T * 5 + batched)
    A = _stable_A((B,) if batched else (), g, dtype)
    zi = torch.randn(B, 2, generator=g, dtype=torch.float64).to(dtype)
    x = torch.randn(B, T, 2, generator=g, dtype=torch.float64).to(dtype)
    gy = torch.randn(B, T, 2, generator=g, dtype=torch.float64).to(dtype)
    _check("lti", A, zi, x, gy, dtype)


@pytest.mark.parametrize("tag", ["f32", "f64"])
@pytest.mark.parametrize("mode", ["batched", "shared"])
@pytest.mark.parametrize("kind", ["lti", "lpv"])
def test_golden(tag, mode, kind):
    g = load_golden(f"{kind}_recur2_{mode}_{tag}")
    t = tol(DT[tag])
    y, gA, gzi, gx = _run(kind, g["A"], g["zi"], g["x"], g["gy"])
    assert rel_err(y, g["y"]) <= t
    assert rel_err(gA, g["grad_A"]) <= t
    assert rel_err(gzi, g["grad_zi"]) <= t
    assert rel_err(gx, g["grad_x"]) <= t
    if kind == "lpv":   # public API, scalar input into state 0, one state returned
        A, zi, x = (g[k].to(DEV) for k in ("A", "zi", "x"))
        assert rel_err(ptb.lpv.state_space_recursion(A, zi, x), g["y_python_loop"]) <= t
        assert rel_err(ptb.lpv.state_space_recursion(A, zi, x[..., 0], out_idx=1), g["y_python_loop_x2d_idx1"]) <= t


def test_lti_state_space_recursion_golden():
    g = load_golden("lti_state_space_recursion_f64")
    A, zi, x = (g[k].to(DEV) for k in ("A", "zi", "x"))
    assert rel_err(ptb.lti.state_space_recursion(A, zi, x), g["y"]) <= 1e-10
    assert rel_err(ptb.lti.state_space_recursion(A[0], zi, x), g["y_shared"]) <= 1e-10
    assert rel_err(ptb.lti.state_space_recursion(A, zi, x[..., 0], out_idx=0), g["y_x2d_idx0"]) <= 1e-10
    assert rel_err(ptb.lti.state_space_recursion(A, zi, x, unroll_factor=5), g["y_unrolled"]) <= 1e-9
    with pytest.raises(ValueError):
        ptb.lti.state_space_recursion(A, zi, x, unroll_factor=0)
    with pytest.raises(AssertionError):
        ptb.lti.state_space_recursion(A, zi[:2], x)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("lpv", [True, False])
def test_scalar_input_path(dtype, lpv):
    """x of shape (B,T) feeds state 0 only; gradients w.r.t. x are (B,T)."""
    B, T = 4, 5000
    g = torch.Generator().manual_seed(17)
    A = _stable_A((B, T) if lpv else (B,), g, dtype)
    zi = torch.randn(B, 2, generator=g, dtype=torch.float64).to(dtype)
    x = torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype)
    gy = torch.randn(B, T, 2, generator=g, dtype=torch.float64).to(dtype)
    A_, zi_, x_ = (t.to(DEV).requires_grad_() for t in (A, zi, x))
    fn = ptb.lpv.state_space_recursion if lpv else ptb.lti.state_space_recursion
    y = fn(A_, zi_, x_)
    gA, gzi, gx = torch.autograd.grad(y, (A_, zi_, x_), gy.to(DEV))
    xp = torch.stack([x, torch.zeros_like(x)], -1)
    y_ref = (cport.recur2 if lpv else cport.lti_recur2)(A, zi, xp)
    gA_ref, gzi_ref, gx_ref = (cport.recur2_bwd if lpv else cport.lti_recur2_bwd)(A, zi, y_ref, gy)
    t = tol(dtype)
    assert rel_err(y, y_ref) <= t and rel_err(gA, gA_ref) <= t
    assert rel_err(gzi, gzi_ref) <= t and rel_err(gx, gx_ref[..., 0]) <= t
    ptb.check_errors()


@pytest.mark.parametrize("tag", ["f32", "f64"])
def test_config4_golden(tag):
    dtype = DT[tag]
    g = load_golden(f"config4_small_{tag}")
    w = workloads.lpv_second_order(B=2, T=4096, dtype=dtype)
    A_, x_ = (w[k].to(DEV).requires_grad_() for k in ("A", "x"))
    y = ptb.lpv.state_space_recursion(A_, w["zi"].to(DEV), x_)
    gA, gx = torch.autograd.grad(y, (A_, x_), w["gy"].to(DEV))
    t = tol(dtype)
    assert rel_err(y, g["y"]) <= t and rel_err(gA, g["grad_A"]) <= t and rel_err(gx, g["grad_x"]) <= t
    ptb.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_many_tiles(dtype):
    B, T = 24, 1 << 16
    w = workloads.lpv_second_order(B=B, T=T, dtype=dtype)
    xp = torch.stack([w["x"], torch.zeros_like(w["x"])], -1)
    _check("lpv", w["A"], torch.randn(B, 2, dtype=dtype), xp, w["gy"], dtype)
    _check("lti", w["A"][:, 0].contiguous(), torch.randn(B, 2, dtype=dtype), xp, w["gy"], dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("scalar_x", [False, True])
def test_shared_matrix_gradient_sum(dtype, scalar_x):
    """Matrices shared by the rows, (T,2,2): the kernels add every row's outer products into the one
    gradient array; compared with the per-row gradients of the same matrices expanded over the rows,
    summed afterwards, and with the oracle."""
    B, T = 40, 6000
    g = torch.Generator().manual_seed(23)
    A = _stable_A((T,), g, dtype)
    zi = torch.randn(B, 2, generator=g, dtype=torch.float64).to(dtype)
    x = torch.randn((B, T) if scalar_x else (B, T, 2), generator=g, dtype=torch.float64).to(dtype)
    gy = torch.randn(B, T, 2, generator=g, dtype=torch.float64).to(dtype)
    A_, zi_, x_ = (t.to(DEV).requires_grad_() for t in (A, zi, x))
    y = ptb.lpv.state_space_recursion(A_, zi_, x_)
    gA, gzi, gx = torch.autograd.grad(y, (A_, zi_, x_), gy.to(DEV))
    assert gA.shape == A.shape
    Ab = A.to(DEV).expand(B, T, 2, 2).contiguous().requires_grad_()
    yb = ptb.lpv.state_space_recursion(Ab, zi_, x_)
    gAb, gzib, gxb = torch.autograd.grad(yb, (Ab, zi_, x_), gy.to(DEV))
    t = tol(dtype)
    assert rel_err(y, yb.cpu()) == 0
    assert rel_err(gx, gxb.cpu()) == 0 and rel_err(gzi, gzib.cpu()) == 0
    assert rel_err(gA, gAb.sum(0).cpu()) <= t
    xp = torch.stack([x, torch.zeros_like(x)], -1) if scalar_x else x
    y_ref = cport.recur2(A, zi, xp)
    gA_ref, _, _ = cport.recur2_bwd(A, zi, y_ref, gy)
    assert rel_err(gA, gA_ref) <= t
