"""Parameter-varying state-space front-end on the GPU kernels (orders 1 and 2).

Public names follow philtorch/lpv/ssm.py of the reference (``state_space_recursion`` :208-334,
pure PyTorch there; ``MatrixRecurrence`` :34-115).  First-order inputs run the native
per-sample-coefficient kernel, where the reference relies on the third-party ``torchlpc``
(philtorch/lpv/ssm.py:188-195).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from ..autograd import LPVRecurrence, MatrixRecurrence, matrix_recurrence_scalar_input

__all__ = ["MatrixRecurrence", "state_space_recursion", "extension_backend_indicator"]


def extension_backend_indicator(x: Tensor, M: int) -> bool:
    """True when the compiled kernels handle this input (CUDA, fp32/fp64, state dimension <= 2)."""
    return x.is_cuda and M in (1, 2) and x.dtype in (torch.float32, torch.float64)


def _ext_ss_recur(A: Tensor, zi: Tensor, x: Tensor, *, out_idx: Optional[int] = None, **_) -> Tensor:
    """Counterpart of philtorch/lpv/ssm.py:167-205: run the recurrence on the kernels."""
    M = A.size(-1)
    if M == 1:
        xs = x if x.dim() == 2 else x.squeeze(-1)
        y = LPVRecurrence.apply(A[..., 0, 0], zi.squeeze(-1), xs).unsqueeze(-1)
    elif M == 2:
        if x.dim() == 2:
            y = matrix_recurrence_scalar_input(A, zi, x, True)
        else:
            y = MatrixRecurrence.apply(A, zi, x)
    else:
        raise NotImplementedError(f"state dimension {M}: philtorch_b200 implements orders 1 and 2 only")
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
