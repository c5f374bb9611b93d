"""First-order recurrence with per-sample coefficients: public API of philtorch/lpv/recur.py."""
from __future__ import annotations

import torch
import torch.autograd.forward_ad as fwAD
from torch import Tensor

from ..autograd import LPVRecurrence

__all__ = ["LPVRecurrence", "linear_recurrence"]


def linear_recurrence(a: Tensor, init: Tensor, x: Tensor, *, unroll_factor: int = 1) -> Tensor:
    """Recurrence ``h[t] = a[t] * h[t-1] + x[t]`` with time-varying ``a`` on the GPU kernels.

    Same signature and argument checks as the reference's pure-PyTorch
    ``philtorch.lpv.linear_recurrence`` (philtorch/lpv/recur.py:20-61).

    Args:
        a: coefficients, shape (N,) (shared by the batch) or (B, N).
        init: initial state, shape () or (1,) or (B,).
        x: input, shape (B, N), CUDA, float32 or float64.
        unroll_factor: accepted for compatibility and validated (>= 1); unused.

    Returns:
        Tensor of shape (B, N).
    """
    assert x.dim() == 2, f"Input x must be 2D, got {x.shape}"
    assert a.dim() in (1, 2), f"State matrix a must be 1D or 2D, got {a.shape}"
    if a.dim() == 1 and a.size(0) != x.size(1):
        raise ValueError(
            f"State matrix a must be 1D with the same length as x, got a: {a.size(0)}, x: {x.size(1)}")
    batch_size = x.size(0)
    assert init.dim() in (0, 1), f"Initial state init must be 1D or 0D, got {init.shape}"
    if init.dim() == 1 and init.size(0) > 1 and init.size(0) != batch_size:
        raise ValueError(
            f"Initial state init must be 1D with the same batch size as x, got init: {init.size(0)}, x: {batch_size}")
    if unroll_factor < 1:
        raise ValueError("Unroll factor must be >= 1")
    if init.dim() == 0 or init.size(0) != batch_size:
        init = init.expand(batch_size)
    if x.is_cuda and a.dim() == 2 and not x.is_complex() and not torch.compiler.is_compiling():
        # a handful of long rows: cut into segments the kernels see as independent rows (the tiles of
        # one row wait on one another, so few rows leave most of the memory bandwidth unused); the
        # segmented Function drives the library directly, so a traced graph keeps the plain op
        from .. import sharded

        S = sharded.auto_segments(batch_size, x.size(1), True)
        if S > 1 and x.dtype in (torch.float32, torch.float64) and not _has_tangent(a, init, x):
            return sharded.TimeShardedLPVRecurrence.apply(a, init, x, sharded.LOCAL, None, S)
    return LPVRecurrence.apply(a, init, x)


def _has_tangent(*tensors: Tensor) -> bool:
    """True inside forward-mode AD (the segmented path has no jvp rule; LPVRecurrence has)."""
    return any(fwAD.unpack_dual(t).tangent is not None for t in tensors)
