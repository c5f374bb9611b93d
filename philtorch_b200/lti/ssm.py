"""Time-invariant state-space front-end on the GPU kernels (orders 1 and 2).

Public names and argument conventions follow philtorch/lti/ssm.py of the reference:
``state_space_recursion`` (:198-383 there, pure PyTorch) and ``state_space`` (:386-510).  Every
call runs the compiled kernels; ``unroll_factor`` is accepted for compatibility (the reference
only reaches its extension when it is 1) and ignored.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from ..autograd import LTIMatrixRecurrence, LTIRecurrence, matrix_recurrence_scalar_input

__all__ = ["LTIMatrixRecurrence", "state_space_recursion", "state_space", "extension_backend_indicator"]


def extension_backend_indicator(x: Tensor, M: int) -> bool:
    """True when the compiled kernels handle this input (CUDA, fp32/fp64, state dimension <= 2)."""
    return x.is_cuda and M in (1, 2) and x.dtype in (torch.float32, torch.float64)


def _ext_ss_recur(A: Tensor, zi: Tensor, x: Tensor, *, out_idx: Optional[int] = None, **_) -> Tensor:
    """Counterpart of philtorch/lti/ssm.py:162-195: run the recurrence on the kernels."""
    M = A.size(-1)
    if M == 1:
        xs = x if x.dim() == 2 else x.squeeze(-1)
        y = LTIRecurrence.apply(A[..., 0, 0], zi.squeeze(-1), xs).unsqueeze(-1)
    elif M == 2:
        if x.dim() == 2:
            y = matrix_recurrence_scalar_input(A, zi, x, False)
        else:
            y = LTIMatrixRecurrence.apply(A, zi, x)
    else:
        raise NotImplementedError(f"state dimension {M}: philtorch_b200 implements orders 1 and 2 only")
    if out_idx is not None and y.dim() == 3:
        y = y[:, :, out_idx]
    return y


def state_space_recursion(A: Tensor, zi: Tensor, x: Tensor, *, unroll_factor: int = 1,
                          out_idx: Optional[int] = None) -> Tensor:
    """State evolution ``h[t] = A h[t-1] + x[t]`` of a time-invariant model.

    Args:
        A: (M, M) or (B, M, M), M in {1, 2}.
        zi: (B, M) initial states.
        x: (B, T, M), or (B, T) feeding state 0 only.
        unroll_factor: validated (>= 1), otherwise unused.
        out_idx: return only this state.

    Returns:
        (B, T, M), or (B, T) with ``out_idx``.
    """
    assert x.dim() in (2, 3), f"Input signal must be 2D or 3D (batch, time, [features]), got {x.shape}"
    assert A.dim() in (2, 3), f"State matrix A must be 2D or 3D, got {A.shape}"
    assert A.size(-2) == A.size(-1), f"State matrix A must be square, got {A.shape}"
    if A.dim() == 3:
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


def _input_map(x: Tensor, Bm: Optional[Tensor], batch_size: int, M: int) -> Tensor:
    """B x for the shapes the filter front-ends use (philtorch/lti/ssm.py:466-485)."""
    if Bm is None:
        return x
    features = -1 if x.dim() == 2 else x.size(-1)
    shp = tuple(Bm.shape)
    if shp == (M,):
        assert x.dim() == 2, f"Input signal x must be 2D when B is of shape {(M,)}, got {x.shape}"
        return x.unsqueeze(-1) * Bm
    if shp == (batch_size, M):
        assert x.dim() == 2, f"Input signal x must be 2D when B is of shape {(batch_size, M)}, got {x.shape}"
        return x.unsqueeze(-1) * Bm.unsqueeze(1)
    if shp == (M, features):
        return x @ Bm.T
    if shp == (batch_size, M, features):
        return torch.linalg.vecdot(Bm.unsqueeze(1).conj(), x.unsqueeze(-2))
    raise ValueError(f"Input matrix B must be of shape ({M},), ({batch_size}, {M}), ({M}, {features}) or "
                     f"({batch_size}, {M}, {features}), got {shp}")


def _output_map(h: Tensor, x: Tensor, C: Optional[Tensor], D: Optional[Tensor], batch_size: int, M: int) -> Tensor:
    """C h + D x for the shapes the filter front-ends use (philtorch/lti/ssm.py:513-589)."""
    Dx = None
    if D is not None:
        shp = tuple(D.shape)
        if shp in ((), (1,)):
            Dx = x * D
        elif shp == (batch_size,):
            assert x.dim() == 2, f"Input signal x must be 2D when D is of shape ({batch_size},), got {x.shape}"
            Dx = D.unsqueeze(1) * x
        elif x.dim() == 3 and shp == (x.size(-1),):
            Dx = x @ D
        else:
            raise ValueError(f"Feedthrough D must be a scalar, ({batch_size},) or (features,), got {shp}")
    if C is not None:
        shp = tuple(C.shape)
        if shp == (M,):
            Ch = h @ C
        elif shp == (batch_size, M):
            Ch = torch.linalg.vecdot(C.unsqueeze(1).conj(), h)
        elif len(shp) == 2 and shp[1] == M:
            Ch = h @ C.T
        elif len(shp) == 3 and shp[0] == batch_size and shp[2] == M:
            Ch = h @ C.mT
        else:
            raise ValueError(f"Output matrix C must be of shape ({M},), ({batch_size}, {M}), (_, {M}) or "
                             f"({batch_size}, _, {M}), got {shp}")
    else:
        Ch = h
    return Ch if Dx is None else Ch + Dx


def state_space(A: Tensor, x: Tensor, B: Optional[Tensor] = None, C: Optional[Tensor] = None,
                D: Optional[Tensor] = None, zi: Optional[Tensor] = None, unroll_factor: Optional[int] = None,
                out_idx: Optional[int] = None):
    """Discrete time-invariant state-space model

        h[t+1] = A h[t] + B x[t],   y[t] = C h[t] + D x[t]

    with the calling convention of philtorch/lti/ssm.py:386-510: returns ``y``, or ``(y, zf)``
    when ``zi`` is given.  ``unroll_factor`` is accepted and ignored.
    """
    assert x.dim() in (2, 3), f"Input signal must be 2D or 3D (batch, time, [features]), got {x.shape}"
    assert A.dim() in (2, 3), f"State matrix A must be 2D or 3D, got {A.shape}"
    assert A.size(-2) == A.size(-1), f"State matrix A must be square, got {A.shape}"
    if A.dim() == 3:
        assert x.size(0) == A.size(0), \
            f"Batch size of A must match batch size of x, got A: {A.size(0)}, x: {x.size(0)}"
    if not (C is None or out_idx is None):
        raise ValueError("C and out_idx cannot be used together. Use either C or out_idx.")
    batch_size, M = x.shape[0], A.size(-1)
    return_zf = zi is not None
    if zi is None:
        zi = x.new_zeros(batch_size, M)
    elif zi.dim() == 1:
        zi = zi.unsqueeze(0).expand(batch_size, -1)
    Bx = _input_map(x, B, batch_size, M)
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
    y = _output_map(h, x, C, D, batch_size, M)
    return (y, zf) if return_zf else y
