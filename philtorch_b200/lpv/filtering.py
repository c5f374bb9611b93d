"""Parameter-varying IIR filtering (orders 1 and 2) on the GPU kernels.

``lfilter`` keeps the signature of philtorch/lpv/filtering.py:138-194 for the state-space backend
and the forms 'df2' and 'tdf2'.  Batches of a few dozen rows and more run on one fused kernel per
direction (csrc/lpv_biquad.cuh); smaller ones on the 2x2 scan kernels (``state_space_recursion``)
driven by the per-sample companion matrices, with the input and output maps around them (B_t x_t,
the one-sample delay, C_t h_{t-1} + D_t x_t; philtorch/lpv/filtering.py:288-325,
philtorch/lpv/ssm.py:413-500) as a few elementwise passes.  The FIR-based forms 'df1' / 'tdf1', orders above two and the 'torchlpc'
backend are outside this package.
"""
from __future__ import annotations

from typing import Optional, Union

import torch
import torch.nn.functional as F
from torch import Tensor

from ..autograd import LPVBiquad
from .ssm import state_space_recursion

# From this many rows on, the filter runs on the fused kernels (one pass per direction, first
# derivatives only); below it on the 2x2 scan kernels with elementwise passes around them
# (differentiable to any order).  Set to a huge value to switch the fused path off.
FUSED_MIN_ROWS = 32

__all__ = ["lfilter"]


def _ssm_lfilter(b: Tensor, a: Tensor, x: Tensor, zi: Optional[Tensor], form: str):
    B, N = x.shape
    # equal orders, as philtorch/lpv/filtering.py:297-300
    if b.size(-1) < a.size(-1) + 1:
        b = F.pad(b, (0, a.size(-1) + 1 - b.size(-1)))
    elif b.size(-1) > a.size(-1) + 1:
        a = F.pad(a, (0, b.size(-1) - a.size(-1) - 1))
    order = a.size(-1)
    if order > 2:
        raise NotImplementedError(f"filter order {order}: philtorch_b200 implements first- and second-order "
                                  "sections only")
    if order < 1:
        raise ValueError("the filter needs at least one recursive or delayed coefficient")
    if order == 1:   # run as a second-order section with a zero second coefficient
        a, b = F.pad(a, (0, 1)), F.pad(b, (0, 1))
    for name, t in (("b", b), ("a", a)):
        if t.size(-2) != N or (t.dim() == 3 and t.size(0) != B):
            raise ValueError(f"{name} must be (B, N, .) or (N, .) with B, N matching x.")
    return_zf = zi is not None
    if zi is None:
        zi2 = x.new_zeros(B, 2)
    else:
        if zi.dim() == 1:
            zi = zi.unsqueeze(0).expand(B, -1)
        zi2 = F.pad(zi, (0, 2 - zi.size(-1))) if zi.size(-1) < 2 else zi
    if form in ("df2", "tdf2") and B >= FUSED_MIN_ROWS:   # one fused kernel per direction
        if b.dim() != a.dim():
            # one tensor shared by the rows, the other per row (the reference broadcasts them,
            # philtorch/lpv/filtering.py:297-320): give the shared one a batch axis; autograd's expand
            # rule then sums its gradient over the rows
            if b.dim() == 2:
                b = b.unsqueeze(0).expand(B, -1, -1)
            else:
                a = a.unsqueeze(0).expand(B, -1, -1)
        y, zf = LPVBiquad.apply(b, a, zi2 if return_zf else None, x, form)
        return (y, zf[:, :order]) if return_zf else y
    a1, a2 = a[..., 0], a[..., 1]
    zero, one = torch.zeros_like(a1), torch.ones_like(a1)
    b0 = b[..., :1]
    Bv = b[..., 1:] - b0 * a          # (.., N, 2): C of the df2 form, B of the tdf2 form
    D = b[..., 0]
    if form == "df2":
        # h_t = companion(a_t) h_{t-1} + [x_t, 0];  y_t = C_t . h_{t-1} + D_t x_t
        A = torch.stack([torch.stack([-a1, -a2], -1), torch.stack([one, zero], -1)], -2)
        h = state_space_recursion(A, zi2, x)
        h_prev = torch.cat([zi2.unsqueeze(1), h[:, :-1]], dim=1)
        y = (Bv * h_prev).sum(-1) + D * x
    elif form == "tdf2":
        # h_t = companion(a_t)^T h_{t-1} + B_t x_t;  y_t = h0_{t-1} + D_t x_t
        A = torch.stack([torch.stack([-a1, one], -1), torch.stack([-a2, zero], -1)], -2)
        h = state_space_recursion(A, zi2, x.unsqueeze(-1) * Bv)
        h0_prev = torch.cat([zi2[:, None, 0], h[:, :-1, 0]], dim=1)
        y = h0_prev + D * x
    elif form in ("df1", "tdf1"):
        raise NotImplementedError(f"form={form!r} is built on an FIR convolution, which is outside this package; "
                                  "use 'df2' or 'tdf2'")
    else:
        raise ValueError(f"Unknown filter form: {form}")
    if return_zf:
        return y, h[:, -1, :order]
    return y


def lfilter(b: Tensor, a: Tensor, x: Tensor, zi: Optional[Tensor] = None, form: str = "df2",
            backend: str = "ssm", **kwargs) -> Union[Tensor, tuple[Tensor, Tensor]]:
    """Apply a batch of parameter-varying IIR filters (``a0 = 1`` implicit, ``a`` excludes it).

    Args:
        b: numerator per sample, (B, N, Mb+1) or (N, Mb+1).
        a: denominator per sample without a0, (B, N, Ma) or (N, Ma); max(Mb, Ma) <= 2.
        x: input, (B, N) or (N,), CUDA, float32 or float64.
        zi: initial state, (B, max(Mb, Ma)) or (max(Mb, Ma),); when given, ``(y, zf)`` is returned.
        form: 'df2' (default) or 'tdf2'.
        backend: only 'ssm'.
        **kwargs: ``unroll_factor`` is accepted for compatibility and ignored.
    """
    squeeze_first = (x.dim() == 1) & (b.dim() == 2) & (a.dim() == 2) & ((zi is None) or (zi.dim() == 1))
    if x.dim() == 1:
        x = x.unsqueeze(0)
    elif x.dim() > 2:
        raise ValueError("Input signal x must be 1D or 2D.")
    assert b.dim() in (2, 3), "Numerator coefficients b must be 2D or 3D."
    assert a.dim() in (2, 3), "Denominator coefficients a must be 2D or 3D."
    kwargs.pop("unroll_factor", None)
    if kwargs:
        raise TypeError(f"unexpected keyword arguments: {sorted(kwargs)}")
    if backend != "ssm":
        if backend == "torchlpc":
            raise NotImplementedError("backend='torchlpc' is outside this package; use backend='ssm'")
        raise ValueError(f"Unknown backend: {backend}")
    y = _ssm_lfilter(b, a, x, zi, form)
    if isinstance(y, tuple):
        y, zf = y
        if squeeze_first:
            y, zf = y.squeeze(0), zf.squeeze(0)
        return y, zf
    return y.squeeze(0) if squeeze_first else y
