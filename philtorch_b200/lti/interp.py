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


SEGMENT_TARGET_ROWS = 256    # rows from which the scan kernels run at full rate (fewer, longer rows: -15 % at 64)
SEGMENT_MIN_LENGTH = 1 << 14

_CONSTANTS: dict = {}


def _constants(device, dtype, terms: int):
    """(pole as a 1-element tensor, POLE**k for k < terms, the same reversed, POLE**(k+1)), made once
    per device, dtype and length (never kept when made while a CUDA graph is being captured)."""
    key = (device, dtype, terms)
    hit = _CONSTANTS.get(key)
    if hit is not None:
        return hit
    r = torch.full((1,), POLE, device=device, dtype=dtype)
    pw = r.pow(torch.arange(terms, device=device, dtype=dtype))
    made = (r, pw, pw.flip(0).contiguous(), pw * POLE)
    if not (device.type == "cuda" and torch.cuda.is_current_stream_capturing()):
        _CONSTANTS[key] = made
    return made


def _segments(rows: int, length: int, itemsize: int) -> int:
    """Pieces each row is cut into so that the kernels see about SEGMENT_TARGET_ROWS rows: a power of
    two that divides the length into pieces of whole 16-byte units, none shorter than
    SEGMENT_MIN_LENGTH.  1 = rows stay whole."""
    S = 1
    unit = 16 // itemsize
    while (rows * S < SEGMENT_TARGET_ROWS and length % (2 * S) == 0
           and (length // (2 * S)) % unit == 0 and length // (2 * S) >= max(SEGMENT_MIN_LENGTH, MIRROR_TERMS)):
        S *= 2
    return S


def _causal_kernel(a: Tensor, start: Tensor, x: Tensor) -> Tensor:
    return torch.ops.philtorch_b200.lti_recur(a, start, x)


def _reverse_fused_kernel(a: Tensor, x: Tensor, second: Tensor, g_in: Tensor, need_first: bool):
    return torch.ops.philtorch_b200.lti_recur_reverse_fused(a, x, second, g_in, GAIN, need_first)


def _two_pass(x: Tensor, start: Tensor, end_of, transposed: bool):
    """The causal recurrence over x, then the reverse-time recurrence fused with the combination
    ``GAIN (h + g - x)``; returns the combination and the state that leaves the reverse pass at t = 0.

    ``start`` (B,) is the causal state before the first sample; ``end_of(h_last)`` gives the state of
    the reverse pass beyond the last sample, times the pole, from the causal pass's last output.
    Few long rows are cut into pieces that the kernels treat as rows of their own: the pole is a
    constant whose powers vanish (exactly, in floating point) within MIRROR_TERMS samples, so the state
    entering a piece is the power sum over the MIRROR_TERMS samples next to it, in the causal pass
    those before it and in the reverse pass those after it.  No sample is read or written twice."""
    B, T = x.shape
    terms = min(T, MIRROR_TERMS)
    r, _, pw_rev, pw_pole = _constants(x.device, x.dtype, terms)
    S = _segments(B, T, x.element_size())
    if S == 1:
        h = _causal_kernel(r, start, x)
        out, first = _reverse_fused_kernel(r, x, h, end_of(h[:, -1]), transposed)
        return out, (first if transposed else None)
    L = T // S
    rows = x.view(B * S, L)
    # two matrix-vector products over strided views (no copies): every piece's last samples give the
    # causal state entering the next piece, its first samples the reverse state entering the previous one
    tails = (rows[:, L - terms:] @ pw_rev).view(B, S)
    heads = (rows[:, :terms] @ pw_pole).view(B, S)
    starts = torch.cat([start.unsqueeze(1), tails[:, :-1]], 1)
    h = _causal_kernel(r, starts.view(-1), rows)
    ends = torch.cat([heads[:, 1:], end_of(h.view(B, T)[:, -1]).unsqueeze(1)], 1)
    out, first = _reverse_fused_kernel(r, rows, h, ends.view(-1), transposed)
    return out.view(B, T), (first.view(B, S)[:, 0] if transposed else None)


class _ParallelFormCoefficients(torch.autograd.Function):
    """The partial-fraction evaluation as two kernel passes per direction: the causal recurrence,
    then the reverse-time recurrence that also forms ``k (h + g - x)`` on its way out (20 B per
    sample in fp32).  The operator is linear in x, so the backward pass is the transposed pair of
    passes and needs nothing saved; boundary terms (mirror sum, end state) are rank-one corrections."""

    @staticmethod
    def forward(ctx, x: Tensor, scipy_padding: bool) -> Tensor:
        off = 0 if scipy_padding else 1
        terms = min(x.shape[-1] - off, MIRROR_TERMS)
        x = x.contiguous()
        pw = _constants(x.device, x.dtype, terms)[1]
        start = x[:, off:off + terms] @ pw
        if scipy_padding:
            end_of = lambda h_last: h_last * POLE
        else:
            x_last = x[:, -1]
            end_of = lambda h_last: h_last - x_last          # ((h - x) / POLE) * POLE
        out, _ = _two_pass(x, start, end_of, False)
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
        G = grad_out.contiguous()
        off = 0 if sp else 1
        terms = min(G.shape[-1] - off, MIRROR_TERMS)
        pw = _constants(G.device, G.dtype, terms)[1]
        # transpose of the reverse-time pass (a causal pass from zero), whose last value times the pole
        # is the gradient of the forward end state; that enters the transposed causal pass at its last
        # sample (scaled by 1 / POLE without scipy's padding)
        last = []
        def end_of(q_last):
            last.append(q_last)
            return q_last * POLE if sp else q_last
        gx, s_bar = _two_pass(G, torch.zeros_like(G[:, 0]), end_of, True)
        # the mirror sum that starts the causal pass, and (reflect padding) the last sample's part in the end state
        gx[:, off:off + terms].addcmul_(s_bar.unsqueeze(1), pw, value=GAIN)
        if not sp:
            gx[:, -1].sub_(last[0], alpha=GAIN)
        return gx, None


def _coefficients(x: Tensor, parallel_form: bool, scipy_padding: bool, fused: bool = True) -> Tensor:
    """philtorch/lti/interp.py:23-57.  The signal is continued by mirroring: with the sample at the
    border repeated (scipy's cspline1d) or not (torch's 'reflect' padding)."""
    if parallel_form and fused and x.dim() == 2 and x.shape[-1] >= 2:
        return _ParallelFormCoefficients.apply(x, scipy_padding)
    # state of the causal recurrence at t = -1: the geometric sum over the mirrored past, of which
    # only the first terms are non-zero in floating point
    past = x if scipy_padding else x[..., 1:]
    terms = min(past.shape[-1], MIRROR_TERMS)
    r, pw = _constants(x.device, x.dtype, terms)[:2]   # filled on the device: no host-to-device copy
    r = r[0]
    start = past[..., :terms] @ pw
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
