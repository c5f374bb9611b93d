"""Cubic B-spline coefficients and integer-factor upsampling (philtorch/lti/interp.py).

The spline coefficients are the input filtered by the symmetric all-pole filter with the pole
``r = sqrt(3) - 2`` (Unser, "B-Spline Signal Processing: Part II"): a causal and an anticausal
first-order time-invariant recurrence.  The causal pass is the forward kernel of the first-order
recurrence and the anticausal pass its adjoint kernel, which runs from the last sample to the
first: the signal is never mirrored, concatenated or reversed in memory (the reference filters
the mirrored signal and flips the halves back).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import Tensor

from ..autograd import LTIRecurrence, ReverseLTIRecurrence

__all__ = ["cspline", "cubic_spline"]

POLE = math.sqrt(3.0) - 2.0
GAIN = -6.0 * POLE / (1.0 - POLE * POLE)   # of the partial-fraction form
MIRROR_TERMS = 1024   # POLE**k is exactly zero (also as a denormal float64) long before k = 1024


def _causal(x: Tensor, pole: Tensor, init: Tensor) -> Tensor:
    """h[t] = pole * h[t-1] + x[t] per row, h[-1] = init (philtorch/lti/interp.py:10-20)."""
    rows = x.shape[0]
    return LTIRecurrence.apply(pole.expand(rows), init.expand(rows).contiguous(), x)


def _anticausal(x: Tensor, pole: Tensor, end: Tensor) -> Tensor:
    """g[t] = pole * g[t+1] + x[t] per row, g[L] = end."""
    rows = x.shape[0]
    return ReverseLTIRecurrence.apply(pole.expand(rows), end.expand(rows).contiguous(), x)


class _ParallelFormCoefficients(torch.autograd.Function):
    """The partial-fraction evaluation as two kernel passes per direction: the causal recurrence,
    then the reverse-time recurrence that also forms ``k (h + g - x)`` on its way out (20 B per
    sample in fp32).  The operator is linear in x, so the backward pass is the transposed pair of
    passes and needs nothing saved; boundary terms (mirror sum, end state) are rank-one corrections."""

    @staticmethod
    def forward(ctx, x: Tensor, scipy_padding: bool) -> Tensor:
        ops = torch.ops.philtorch_b200
        r = torch.full((1,), POLE, device=x.device, dtype=x.dtype)
        off = 0 if scipy_padding else 1
        terms = min(x.shape[-1] - off, MIRROR_TERMS)
        pw = r.pow(torch.arange(terms, device=x.device, dtype=x.dtype))
        start = x[:, off:off + terms] @ pw
        h = ops.lti_recur(r, start, x)
        end = h[:, -1] if scipy_padding else (h[:, -1] - x[:, -1]) / POLE
        out, _ = ops.lti_recur_reverse_fused(r, x, h, end * POLE, GAIN, False)
        ctx.scipy_padding = scipy_padding
        ctx.save_for_backward(x)
        return out

    @staticmethod
    def backward(ctx, grad_out: Tensor):
        (x,) = ctx.saved_tensors
        sp = ctx.scipy_padding
        if torch.is_grad_enabled():       # higher-order graph: differentiate the composite evaluation
            with torch.enable_grad():
                xr = x.detach().requires_grad_()
                (gx,) = torch.autograd.grad(_coefficients(xr, True, sp, fused=False), xr, grad_out,
                                            create_graph=True)
            return gx, None
        ops = torch.ops.philtorch_b200
        G = grad_out.contiguous()
        r = torch.full((1,), POLE, device=G.device, dtype=G.dtype)
        off = 0 if sp else 1
        terms = min(G.shape[-1] - off, MIRROR_TERMS)
        pw = r.pow(torch.arange(terms, device=G.device, dtype=G.dtype))
        q = ops.lti_recur(r, torch.zeros_like(G[:, 0]), G)          # transpose of the reverse-time pass
        e_bar = q[:, -1] * POLE                                      # gradient of its end state
        g_in = e_bar if sp else e_bar / POLE                         # ... which enters the causal pass at its last sample
        gx, s_bar = ops.lti_recur_reverse_fused(r, G, q, g_in, GAIN, True)   # transpose of the causal pass + combine
        gx[:, off:off + terms] += (GAIN * s_bar).unsqueeze(1) * pw   # the mirror sum that starts the causal pass
        if not sp:
            gx[:, -1] -= GAIN * e_bar / POLE
        return gx, None


def _coefficients(x: Tensor, parallel_form: bool, scipy_padding: bool, fused: bool = True) -> Tensor:
    """philtorch/lti/interp.py:23-57.  The signal is continued by mirroring: with the sample at the
    border repeated (scipy's cspline1d) or not (torch's 'reflect' padding)."""
    r = torch.tensor(POLE, device=x.device, dtype=x.dtype)
    # state of the causal recurrence at t = -1: the geometric sum over the mirrored past, of which
    # only the first terms are non-zero in floating point
    if parallel_form and fused and x.dim() == 2 and x.shape[-1] >= 2:
        return _ParallelFormCoefficients.apply(x, scipy_padding)
    past = x if scipy_padding else x[..., 1:]
    terms = min(past.shape[-1], MIRROR_TERMS)
    start = past[..., :terms] @ r.pow(torch.arange(terms, device=x.device, dtype=x.dtype))
    h = _causal(x, r, start)

    if parallel_form:
        # partial fractions: causal + anticausal part.  The anticausal part continues the causal
        # recurrence over the mirrored signal, i.e. it runs backwards over x from the causal end state
        end = h[..., -1] if scipy_padding else (h[..., -1] - x[..., -1]) / POLE
        g = _anticausal(x, r, end)
        return (h + g).sub_(x).mul_(GAIN)

    # cascade: the anticausal pass runs over the output of the causal one, from its own last value
    if scipy_padding:
        last = h[..., -1] * (POLE / (POLE - 1.0))
    else:
        last = (2.0 * h[..., -1] - x[..., -1]) * (-POLE / (1.0 - POLE * POLE))
    drive = h * (-POLE)
    drive[..., -1] = last                  # so that c[L-1] = last with a zero state beyond the end
    return _anticausal(drive, r, torch.zeros_like(last)) * 6.0


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
