"""First-order time-invariant recurrence: public API of philtorch/lti/recur.py."""
from __future__ import annotations

from torch import Tensor

from ..autograd import LTIRecurrence

__all__ = ["LTIRecurrence", "linear_recurrence"]


def linear_recurrence(a: Tensor, init: Tensor, x: Tensor, *, unroll_factor: int = 1) -> Tensor:
    """Batched scalar recurrence ``h[t] = a * h[t-1] + x[t]`` on the GPU kernels.

    Same signature and argument checks as the reference's pure-PyTorch
    ``philtorch.lti.linear_recurrence`` (philtorch/lti/recur.py:94-134).

    Args:
        a: coefficient, shape () or (1,) (shared) or (B,).
        init: initial state, shape () or (1,) or (B,).
        x: input, shape (B, N), CUDA, float32 or float64.
        unroll_factor: accepted for compatibility and validated (>= 1); the block size of
            the reference's Python scan has no meaning for the single-pass kernel.

    Returns:
        Tensor of shape (B, N).
    """
    assert x.dim() == 2, f"Input x must be 2D, got {x.shape}"
    assert a.dim() in (0, 1), f"State matrix a must be 1D or 0D, got {a.shape}"
    if a.dim() == 1 and a.size(0) > 1 and a.size(0) != x.size(0):
        raise ValueError(
            f"State matrix a must be 1D with the same batch size as x, got a: {a.size(0)}, x: {x.size(0)}")
    batch_size = x.size(0)
    assert init.dim() in (0, 1), f"Initial state init must be 1D or 0D, got {init.shape}"
    if init.dim() == 1 and init.size(0) > 1 and init.size(0) != batch_size:
        raise ValueError(
            f"Initial state init must be 1D with the same batch size as x, got init: {init.size(0)}, x: {batch_size}")
    if unroll_factor < 1:
        raise ValueError("Unroll factor must be >= 1")
    if init.dim() == 0 or init.size(0) != batch_size:
        init = init.expand(batch_size)
    return LTIRecurrence.apply(a, init, x)
