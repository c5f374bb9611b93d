"""Cubic B-spline coefficients and integer-factor upsampling (philtorch/lti/interp.py).

The spline coefficients are the input filtered by the symmetric all-pole filter with the pole
``r = sqrt(3) - 2`` (Unser, "B-Spline Signal Processing: Part II"): a causal and an anticausal
first-order time-invariant recurrence, both of which run on the first-order kernel.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import Tensor

from ..autograd import LTIRecurrence

__all__ = ["cspline", "cubic_spline"]

POLE = math.sqrt(3.0) - 2.0


def _recur(x: Tensor, pole: Tensor, init: Tensor, gain=None) -> Tensor:
    """h[t] = pole * h[t-1] + gain * x[t] per row, h[-1] = init (philtorch/lti/interp.py:10-20)."""
    rows = x.shape[0]
    return LTIRecurrence.apply(pole.expand(rows), init.expand(rows).contiguous(), x if gain is None else x * gain)


def _coefficients(x: Tensor, parallel_form: bool, scipy_padding: bool) -> Tensor:
    """philtorch/lti/interp.py:23-57.  The signal is continued by mirroring: with the sample at the
    border repeated (scipy's cspline1d) or not (torch's 'reflect' padding)."""
    length = x.shape[-1]
    r = torch.tensor(POLE, device=x.device, dtype=x.dtype)
    # state of the causal recurrence at t = -1: the geometric sum over the mirrored past
    if scipy_padding:
        start = x @ r.pow(torch.arange(length, device=x.device, dtype=x.dtype))
    else:
        start = x[..., 1:] @ r.pow(torch.arange(length - 1, device=x.device, dtype=x.dtype))

    if parallel_form:
        # partial fractions: causal + anticausal part, the second being the same recurrence continued
        # over the mirrored signal
        back = x.flip(-1) if scipy_padding else x[..., :-1].flip(-1)
        h = _recur(torch.cat([x, back], dim=-1), r, start)
        causal, anticausal = h[..., :length], h[..., -length:].flip(-1)
        return (causal + anticausal - x) * (-6.0 * POLE / (1.0 - POLE * POLE))

    # cascade: causal pass, then the anticausal pass over its output
    h = _recur(x, r, start)
    if scipy_padding:
        last = h[..., -1] * (POLE / (POLE - 1.0))
    else:
        last = (2.0 * h[..., -1] - x[..., -1]) * (-POLE / (1.0 - POLE * POLE))
    rest = _recur(h[..., :-1].flip(-1), r, last, gain=-r).flip(-1)
    return torch.cat([rest, last.unsqueeze(-1)], dim=-1) * 6.0


def cspline(x: Tensor, parallel_form: bool = True, scipy_padding: bool = False, lamb: float = 0.0,
            **kwargs) -> Tensor:
    """Cubic B-spline coefficients of ``x`` (B, L) -> (B, L); signature of philtorch/lti/interp.py:75-98.

    ``parallel_form`` selects the partial-fraction (one recurrence over the mirrored signal) or the
    cascaded (two recurrences) evaluation; ``scipy_padding`` the mirror convention of
    ``scipy.signal.cspline1d``.  Smoothing (``lamb != 0``) is not implemented, as in the reference.
    ``**kwargs`` (``unroll_factor``) are accepted for compatibility.
    """
    if lamb != 0.0:
        raise NotImplementedError("Regularization for cubic spline interpolation is not implemented.")
    return _coefficients(x, parallel_form, scipy_padding)


def _bspline3(t: Tensor) -> Tensor:
    """The cubic B-spline basis function (philtorch/lti/interp.py:60-72)."""
    u = t.abs()
    inner = (4.0 - 6.0 * u * u + 3.0 * u * u * u) / 6.0
    outer = (2.0 - u).clamp_min(0.0).pow(3) / 6.0
    return torch.where(u <= 1, inner, outer)


def cubic_spline(x: Tensor, m: int, scipy_padding: bool = False, **kwargs) -> Tensor:
    """Upsample ``x`` (B, L) by the integer factor ``m`` with cubic splines -> (B, (L-1)*m + 1)
    (philtorch/lti/interp.py:101-139): spline coefficients, then an m-phase FIR of 4 taps."""
    assert m >= 1 and isinstance(m, int), "Interpolation factor m must be an integer >= 1."
    if m == 1:
        return x
    c = cspline(x, scipy_padding=scipy_padding, **kwargs)
    # tap k of phase p weighs the coefficient at distance (k - 2 + p/m) from the output sample
    offsets = torch.arange(-2, 2, 1 / m, device=x.device, dtype=x.dtype).reshape(4, m)
    taps = _bspline3(offsets).flip(0).T.unsqueeze(1)                      # (m, 1, 4)
    if scipy_padding:
        padded = torch.cat([c[:, :1], c, c[:, -2:].flip(-1)], dim=1).unsqueeze(1)
    else:
        padded = F.pad(c.unsqueeze(1), (1, 2), mode="reflect")
    y = F.conv1d(padded, taps).transpose(1, 2).reshape(x.shape[0], -1)   # phases interleaved in time
    return y[..., : -(m - 1)]
