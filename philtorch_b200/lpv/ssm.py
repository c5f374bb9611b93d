"""Parameter-varying state-space front-end on the GPU kernels (state dimensions 1 to 8).

Public names follow philtorch/lpv/ssm.py of the reference (``state_space_recursion`` :208-334,
pure PyTorch there; ``MatrixRecurrence`` :34-115).  First-order inputs run the native
per-sample-coefficient kernel, where the reference relies on the third-party ``torchlpc``
(philtorch/lpv/ssm.py:188-195).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from .. import sharded
from ..autograd import LPVRecurrence, MatrixRecurrence, matrix_recurrence_scalar_input
from .recur import _has_tangent

__all__ = ["MatrixRecurrence", "state_space_recursion", "state_space", "extension_backend_indicator"]


def extension_backend_indicator(x: Tensor, M: int) -> bool:
    """True when the compiled kernels handle this input (CUDA, fp32/fp64, state dimension <= 8)."""
    return x.is_cuda and 1 <= M <= 8 and x.dtype in (torch.float32, torch.float64)


def _ext_ss_recur(A: Tensor, zi: Tensor, x: Tensor, *, out_idx: Optional[int] = None, **_) -> Tensor:
    """Counterpart of philtorch/lpv/ssm.py:167-205: run the recurrence on the kernels."""
    M = A.size(-1)
    if M == 1:
        xs = x if x.dim() == 2 else x.squeeze(-1)
        y = LPVRecurrence.apply(A[..., 0, 0], zi.squeeze(-1), xs).unsqueeze(-1)
    elif M == 2:
        S = 1
        if (A.dim() == 4 and x.is_cuda and x.dtype in (torch.float32, torch.float64)
                and not torch.compiler.is_compiling()):   # the segmented Function drives the library directly
            # a handful of long rows: cut into segments the kernels see as independent rows (the tiles of
            # one row wait on one another, so few rows leave most of the memory bandwidth unused)
            S = sharded.auto_segments2(x.size(0), x.size(1))
        if S > 1 and not _has_tangent(A, zi, x):
            y = sharded.SegmentedMatrixRecurrence.apply(A, zi, x, S)
        elif x.dim() == 2:
            y = matrix_recurrence_scalar_input(A, zi, x, True)
        else:
            y = MatrixRecurrence.apply(A, zi, x)
    else:
        if x.dim() == 2:   # the sequence feeds state 0 (zero-padded, as the reference does before its op)
            x = torch.cat([x.unsqueeze(-1), x.new_zeros(x.shape + (M - 1,))], dim=-1)
        y = MatrixRecurrence.apply(A, zi, x)   # dense N x N kernels, M <= 8
    if out_idx is not None and y.dim() == 3:
        y = y[:, :, out_idx]
    return y


def state_space_recursion(A: Tensor, zi: Tensor, x: Tensor, *, unroll_factor: int = 1,
                          out_idx: Optional[int] = None) -> Tensor:
    """State evolution ``h[t] = A[t] h[t-1] + x[t]`` of a time-varying model.

    Args:
        A: (N, M, M) or (B, N, M, M), M in {1, 2}.
        zi: (B, M) initial states.
        x: (B, N, M), or (B, N) feeding state 0 only.
        unroll_factor: validated (>= 1), otherwise unused.
        out_idx: return only this state.

    Returns:
        (B, N, M), or (B, N) with ``out_idx``.
    """
    assert x.dim() in (2, 3), f"Input signal must be 2D or 3D (batch, time, [features]), got {x.shape}"
    assert A.dim() in (3, 4), f"State matrix A must be 3D or 4D, got {A.shape}"
    assert A.size(-2) == A.size(-1), f"State matrix A must be square, got {A.shape}"
    assert A.size(-3) == x.size(1), \
        f"State matrix A must have the same time dimension as x, got A: {A.size(-3)}, x: {x.size(1)}"
    if A.dim() == 4:
        assert x.size(0) == A.size(0), \
            f"Batch size of A must match batch size of x, got A: {A.size(0)}, x: {x.size(0)}"
    if x.dim() == 3:
        assert A.size(-1) == x.size(-1), \
            f"Last dimension of A must match last dimension of x, got A: {A.size(-1)}, x: {x.size(-1)}"
    batch_size, M = x.size(0), A.size(-1)
    assert zi.dim() == 2, f"Initial conditions zi must be 2D, got {zi.shape}"
    assert zi.size(0) == batch_size, \
        f"Batch size of zi must match batch size of x, got zi: {zi.size(0)}, x: {batch_size}"
    assert zi.size(1) == M, f"Last dimension of zi must match last dimension of A, got zi: {zi.size(1)}, A: {M}"
    if unroll_factor < 1:
        raise ValueError("Unroll factor must be >= 1")
    return _ext_ss_recur(A, zi, x, out_idx=out_idx)


# ---------------------------------------------------------------------------------------------------
# state_space: per-sample input / output / feed-through maps around the recurrence.
# Every accepted shape of B, C and D is first brought to the common layout
#     (batch | 1, N | 1, rows, cols)
# and then applied with ONE broadcasting matrix-vector product; the tables below list the shapes in
# the order the reference tries them (philtorch/lpv/ssm.py:413-577), which decides how an ambiguous
# shape (e.g. batch == N) is read.  `_` stands for a free output dimension.
def _as_map(W: Tensor, shape_rules, what: str, hint: str):
    """shape_rules: (pattern, needs_2d_x, layout) triples; pattern entries are ints or None (free).
    layout: for every dim of W its role 'b', 'n', 'r' (rows) or 'c' (cols).  Returns (W4, has_rows, index
    of the rule that matched)."""
    shp = tuple(W.shape)
    for idx, (pattern, ok, layout) in enumerate(shape_rules):
        if len(pattern) != len(shp) or not all(p is None or p == d for p, d in zip(pattern, shp)):
            continue
        assert ok, f"Input signal x must be 2D when {what} is of shape {shp}"
        view = [1, 1, 1, 1]
        for role, d in zip(layout, shp):
            view["bnrc".index(role)] = d
        return W.reshape(view), "r" in layout, idx
    raise ValueError(f"{what} of shape {shp} is not one of the accepted shapes: {hint}")


def _apply_map(W4: Tensor, has_rows: bool, v: Tensor) -> Tensor:
    """(batch, N, rows) = W4 (b?, n?, rows, cols) times v (batch, N, cols); the rows axis is dropped
    for maps that produce a scalar per sample."""
    if W4.shape[-1] == 1:                      # outer product with a scalar sequence
        out = W4[..., 0] * v
    elif W4.shape[-2] == 1:                    # inner product per sample
        out = (W4[..., 0, :] * v).sum(-1, keepdim=True)
    else:
        out = torch.matmul(W4, v.unsqueeze(-1)).squeeze(-1)
    return out if has_rows else out[..., 0]


def state_space(A: Tensor, x: Tensor, B: Optional[Tensor] = None, C: Optional[Tensor] = None,
                D: Optional[Tensor] = None, zi: Optional[Tensor] = None, unroll_factor: Optional[int] = None,
                out_idx: Optional[int] = None):
    """Discrete parameter-varying state-space model

        h[t+1] = A[t] h[t] + B[t] x[t],   y[t] = C[t] h[t] + D[t] x[t]

    with the calling convention and the accepted shapes of philtorch/lpv/ssm.py:337-581: A (N, M, M)
    or (batch, N, M, M); x (batch, N) or (batch, N, F); B, C, D constant, per sample, per batch row or
    both; returns ``y``, or ``(y, zf)`` when ``zi`` is given.  The recurrence runs on the kernels
    (M <= 8); ``unroll_factor`` is accepted and ignored.
    """
    assert x.dim() in (2, 3), f"Input signal must be 2D or 3D (batch, time, [features]), got {x.shape}"
    assert A.dim() in (3, 4), f"State matrix A must be 3D or 4D, got {A.shape}"
    assert A.size(-2) == A.size(-1), f"State matrix A must be square, got {A.shape}"
    assert A.size(-3) == x.size(1), \
        f"State matrix A must have the same time dimension as x, got A: {A.size(-3)}, x: {x.size(1)}"
    if not (C is None or out_idx is None):
        raise ValueError("C and out_idx cannot be used together. Use either C or out_idx.")
    batch, N = x.shape[0], x.shape[1]
    M = A.size(-1)
    x2d = x.dim() == 2
    F_ = -1 if x2d else x.size(-1)          # -1 never equals a dimension: feature patterns need a 3-D x
    xv = x.unsqueeze(-1) if x2d else x      # (batch, N, cols)
    return_zf = zi is not None
    if zi is None:
        zi = x.new_zeros(batch, M)
    elif zi.dim() == 1:
        zi = zi.unsqueeze(0).expand(batch, -1)

    if B is None:
        Bx = x
    else:
        rules = (((M,), x2d, "r"), ((M, F_), True, "rc"), ((N, M), x2d, "nr"), ((batch, M), x2d, "br"),
                 ((N, M, F_), True, "nrc"), ((batch, N, M), x2d, "bnr"), ((batch, M, F_), True, "brc"),
                 ((batch, N, M, F_), True, "bnrc"))
        W4, _, _ = _as_map(B, rules, "B", "(M,), (M, F), (N, M), (batch, M), (N, M, F), (batch, N, M), "
                                        "(batch, M, F) or (batch, N, M, F)")
        Bx = _apply_map(W4, True, xv)

    if return_zf or out_idx is None:
        h = _ext_ss_recur(A, zi, Bx)
        zf = h[:, -1, :] if return_zf else None
        if out_idx is None:
            h = torch.cat([zi.unsqueeze(1), h[:, :-1]], dim=1)
        else:
            h = torch.cat([zi[:, None, out_idx], h[:, :-1, out_idx]], dim=1)
    else:
        zf = None
        h = _ext_ss_recur(A, zi, Bx, out_idx=out_idx)
        h = torch.cat([zi[:, None, out_idx], h[:, :-1]], dim=1)

    Dx = None
    if D is not None:
        if D.dim() == 0:
            D = D.reshape(1)
        rules = (((F_,), True, "c"), ((N,), x2d, "n"), ((batch,), x2d, "b"), ((1,), True, "n"), ((None,), x2d, "r"),
                 ((N, F_), True, "nc"), ((batch, F_), True, "bc"), ((N, None), x2d, "nr"), ((batch, N), x2d, "bn"),
                 ((batch, None), x2d, "br"), ((None, F_), not x2d, "rc"),
                 ((batch, N, F_), True, "bnc"), ((batch, N, None), x2d, "bnr"), ((N, None, F_), True, "nrc"),
                 ((batch, None, F_), True, "brc"), ((batch, N, None, F_), True, "bnrc"))
        W4, rows, which = _as_map(D, rules, "D", "a scalar, (N,), (batch,), (F,), (P,), (N, F), (batch, F), (N, P), "
                                          "(batch, N), (batch, P), (P, F), (batch, N, F), (batch, N, P), (N, P, F), "
                                          "(batch, P, F) or (batch, N, P, F)")
        if which == 3 and not x2d:   # a scalar gain on a feature signal keeps the features
            Dx = x * D
        else:
            Dx = _apply_map(W4, rows, xv)

    if C is None:
        Ch = h
    else:
        rules = (((M,), True, "c"), ((N, M), True, "nc"), ((batch, M), True, "bc"), ((None, M), True, "rc"),
                 ((N, None, M), True, "nrc"), ((batch, N, M), True, "bnc"), ((batch, None, M), True, "brc"),
                 ((batch, N, None, M), True, "bnrc"))
        W4, rows, _ = _as_map(C, rules, "C", "(M,), (N, M), (batch, M), (P, M), (N, P, M), (batch, N, M), "
                                          "(batch, P, M) or (batch, N, P, M)")
        Ch = _apply_map(W4, rows, h)

    y = Ch if Dx is None else Ch + Dx
    return (y, zf) if return_zf else y
