"""Time-varying 2x2 recurrence with the rows cut into segments (fold + fix-up kernels of
csrc/shard_fixup2.cuh) against the sequential C oracle and against the unsegmented kernels."""
import math

import pytest
import torch

import philtorch_b200 as ptb
from philtorch_b200 import sharded
from oracle import cport
from conftest import rel_err, tol

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _matrices(kind, shape, g, dtype):
    """(…,2,2) matrices: contracting, orthogonal (products never vanish) or zero."""
    th = 2 * math.pi * torch.rand(shape, generator=g, dtype=torch.float64)
    if kind == "zero":
        return torch.zeros(shape + (2, 2), dtype=dtype)
    r = torch.ones(shape, dtype=torch.float64) if kind == "rotation" else \
        0.3 + 0.65 * torch.rand(shape, generator=g, dtype=torch.float64)
    A = torch.stack([torch.stack([r * th.cos(), -r * th.sin()], -1), torch.stack([r * th.sin(), r * th.cos()], -1)], -2)
    if kind == "contracting":
        A = A + 0.02 * torch.randn(shape + (2, 2), generator=g, dtype=torch.float64)
    return A.to(dtype)


def _case(B, T, kind, scalar_x, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    A = _matrices(kind, (B, T), g, dtype)
    zi = torch.randn(B, 2, generator=g, dtype=torch.float64).to(dtype)
    scale = 1.0 / math.sqrt(T) if kind == "rotation" else 1.0   # a random walk otherwise
    x = (scale * torch.randn((B, T) if scalar_x else (B, T, 2), generator=g, dtype=torch.float64)).to(dtype)
    gy = (scale * torch.randn(B, T, 2, generator=g, dtype=torch.float64)).to(dtype)
    return A, zi, x, gy


def _oracle(A, zi, x, gy):
    xp = torch.stack([x, torch.zeros_like(x)], -1) if x.dim() == 2 else x
    y = cport.recur2(A, zi, xp)
    gA, gzi, gx = cport.recur2_bwd(A, zi, y, gy)
    return y, gA, gzi, (gx[..., 0] if x.dim() == 2 else gx)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("scalar_x", [False, True])
@pytest.mark.parametrize("kind", ["contracting", "rotation", "zero"])
@pytest.mark.parametrize("B,T,S", [(3, 8192, 2), (2, 6000, 4), (1, 24576, 8), (5, 4 * 1027, 4), (2, 64, 16)])
def test_segments_against_oracle(dtype, scalar_x, kind, B, T, S):
    A, zi, x, gy = _case(B, T, kind, scalar_x, dtype, seed=T + S)
    A_, zi_, x_ = (t.to(DEV).requires_grad_() for t in (A, zi, x))
    y = sharded.SegmentedMatrixRecurrence.apply(A_, zi_, x_, S)
    gA, gzi, gx = torch.autograd.grad(y, (A_, zi_, x_), gy.to(DEV))
    y_r, gA_r, gzi_r, gx_r = _oracle(A, zi, x, gy)
    t = tol(dtype) if kind != "rotation" else (2e-4 if dtype == torch.float32 else 1e-9)
    assert gx.shape == x.shape and gA.shape == A.shape
    assert rel_err(y, y_r) <= t
    assert rel_err(gx, gx_r) <= t
    assert rel_err(gzi, gzi_r) <= t
    assert rel_err(gA, gA_r) <= t
    ptb.check_errors()


@pytest.mark.parametrize("scalar_x", [False, True])
def test_few_long_rows_take_the_segmented_path(scalar_x):
    B, T = 4, 1 << 21
    S = sharded.auto_segments2(B, T)
    assert S == 32
    A, zi, x, gy = _case(B, T, "contracting", scalar_x, torch.float32, seed=5)
    A_, zi_, x_ = (t.to(DEV).requires_grad_() for t in (A, zi, x))
    y = ptb.lpv.state_space_recursion(A_, zi_, x_)
    assert type(y.grad_fn).__name__.startswith("SegmentedMatrixRecurrence")
    gA, gzi, gx = torch.autograd.grad(y, (A_, zi_, x_), gy.to(DEV))
    # the unsegmented kernels on the same data
    from philtorch_b200.autograd import MatrixRecurrence, matrix_recurrence_scalar_input
    y1 = matrix_recurrence_scalar_input(A_, zi_, x_, True) if scalar_x else MatrixRecurrence.apply(A_, zi_, x_)
    gA1, gzi1, gx1 = torch.autograd.grad(y1, (A_, zi_, x_), gy.to(DEV))
    for a, b in ((y, y1), (gA, gA1), (gzi, gzi1), (gx, gx1)):
        assert rel_err(a, b.cpu()) <= 2e-5
    # and the oracle on the first and last rows
    y_r, gA_r, gzi_r, gx_r = _oracle(A[[0, B - 1]], zi[[0, B - 1]], x[[0, B - 1]], gy[[0, B - 1]])
    assert rel_err(y[[0, B - 1]], y_r) <= 1e-4 and rel_err(gA[[0, B - 1]], gA_r) <= 1e-4
    assert rel_err(gx[[0, B - 1]], gx_r) <= 1e-4 and rel_err(gzi[[0, B - 1]], gzi_r) <= 1e-4
    ptb.check_errors()


def test_large_batches_and_short_rows_are_not_segmented():
    assert sharded.auto_segments2(128, 1 << 20) == 1
    assert sharded.auto_segments2(64, 1 << 20) == 4
    assert sharded.auto_segments2(16, 1 << 20) == 16
    assert sharded.auto_segments2(8, 1 << 16) == 1      # too small to pay for the extra launches
    assert sharded.auto_segments2(2, (1 << 22) + 2) == 2   # odd halves cannot be cut further


def test_segmented_double_backward():
    torch.manual_seed(0)
    B, T, S = 2, 8, 2
    A = (0.4 * torch.randn(B, T, 2, 2, dtype=torch.float64, device=DEV)).requires_grad_()
    zi = torch.randn(B, 2, dtype=torch.float64, device=DEV).requires_grad_()
    x = torch.randn(B, T, 2, dtype=torch.float64, device=DEV).requires_grad_()
    fn = lambda A_, z_, x_: sharded.SegmentedMatrixRecurrence.apply(A_, z_, x_, S)   # noqa: E731
    assert torch.autograd.gradcheck(fn, (A, zi, x))
    assert torch.autograd.gradgradcheck(fn, (A, zi, x))


@pytest.mark.parametrize("which", ["x", "A", "zi"])
def test_segments_partial_gradients(which):
    """Only one of the inputs requires a gradient: against the unsegmented kernels."""
    from philtorch_b200.autograd import MatrixRecurrence
    B, T, S = 3, 8192, 4
    A, zi, x, gy = _case(B, T, "contracting", False, torch.float32, seed=9)
    ins = {"A": A.to(DEV), "zi": zi.to(DEV), "x": x.to(DEV)}
    ins[which] = ins[which].requires_grad_()
    y = sharded.SegmentedMatrixRecurrence.apply(ins["A"], ins["zi"], ins["x"], S)
    g, = torch.autograd.grad(y, (ins[which],), gy.to(DEV))
    y1 = MatrixRecurrence.apply(ins["A"], ins["zi"], ins["x"])
    g1, = torch.autograd.grad(y1, (ins[which],), gy.to(DEV))
    assert rel_err(y, y1.cpu()) <= 1e-5 and rel_err(g, g1.cpu()) <= 1e-5
    ptb.check_errors()
