"""Small matrix helpers used by the filter front-ends."""
from __future__ import annotations

import torch
from torch import Tensor


def companion(a: Tensor) -> Tensor:
    """Companion matrix of all-pole coefficients ``a`` (a0 = 1 implicit), shape (..., M, M):
    first row ``-a``, ones on the sub-diagonal (same convention as philtorch/mat.py:42-62)."""
    assert a.dim() >= 1, "All-pole coefficients must be at least 1D."
    M = a.size(-1)
    top = (-a).unsqueeze(-2)
    if M == 1:
        return top
    shift = torch.eye(M, dtype=a.dtype, device=a.device)[:-1].expand(a.shape[:-1] + (M - 1, M))
    return torch.cat([top, shift], dim=-2)
