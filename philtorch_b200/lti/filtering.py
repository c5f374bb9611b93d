"""Time-invariant IIR filtering (orders 1 and 2) on the GPU kernels.

``lfilter`` / ``filtfilt`` / ``lfilter_zi`` keep the signatures of philtorch/lti/filtering.py.
The default transposed-direct-form-II path runs ONE fused kernel per direction for a section
(scalar in, scalar out); ``form="df2"`` goes through the 2x2 state-space kernels.  The FIR-based
forms (``df1`` / ``tdf1``) are outside this package; orders above two run through
``backend="diag_ssm"`` (complex first-order modes) or, factored into sections, through ``sosfilt``.
"""
from __future__ import annotations

from typing import Optional, Union

import torch
import torch.nn.functional as F
from torch import Tensor

from ..autograd import BiquadTDF2, CombFilter, SOSCascade
from ..ops import SOS_CASCADE_SIZES
from ..mat import companion
from .recur import linear_recurrence
from .ssm import diag_state_space, state_space

MAX_ORDER = 8   # largest state dimension of the dense recurrence kernels

__all__ = ["lfilter", "filtfilt", "lfilter_zi", "sosfilt", "comb_filter"]


COMB_KERNEL_MIN_LANES = 8192   # (row, phase) pairs from which the comb kernels replace the folded scan


def comb_filter(a: Tensor, delay: int, x: Tensor, zi: Optional[Tensor] = None, **kwargs):
    """Feedback comb filter ``y[t] = x[t] - a * y[t - delay]`` (philtorch/lti/filtering.py:15-71).

    The ``delay`` interleaved phases of a row are independent first-order recurrences with the
    coefficient ``-a``.  With at least ``COMB_KERNEL_MIN_LANES`` (row, phase) pairs the comb kernels
    run on the signal as it lies in memory, one thread per pair (no fold, no transposes; once
    differentiable).  Smaller problems are folded to ``B * delay`` rows of ``ceil(N / delay)``
    samples and run through the first-order time-invariant scan, as the reference does.

    Args:
        a: feedback coefficient, shape () (shared) or (B,).
        delay: the delay in samples, >= 1.
        x: input, shape (B, N).
        zi: the last ``delay`` outputs before the signal, oldest last, shape (delay,) or (B, delay).
        **kwargs: accepted for compatibility (``unroll_factor``).

    Returns:
        y of shape (B, N); for ``delay > 1`` and a given ``zi`` the pair ``(y, zf)`` with
        ``zf = y[:, -delay:]`` reversed, as the reference does (with ``delay == 1`` it returns y
        alone, also with a ``zi``).
    """
    assert a.dim() <= 1, "Denominator coefficients a must be at most 1D."
    assert x.dim() == 2, "Input signal x must be 2D."
    assert delay >= 0, "Delay must be non-negative."
    if a.dim() == 1:
        assert a.size(0) == x.size(0), "The first dimension of a must match the batch size of x."
    if delay == 1:
        return linear_recurrence(-a, torch.zeros_like(a) if zi is None else zi.squeeze(-1), x, **kwargs)

    batch, n = x.shape
    if batch * delay >= COMB_KERNEL_MIN_LANES and not (a.dim() == 1 and a.size(0) == 1 and batch > 1):
        y = CombFilter.apply(a, zi, x, delay)
        return (y, y[:, -delay:].flip(1)) if zi is not None else y
    tail = (-n) % delay
    if tail:
        x = F.pad(x, (0, tail))
    phases = x.view(batch, -1, delay).transpose(1, 2).reshape(batch * delay, -1)   # row b*delay + d: phase d of row b
    if a.dim() == 1:
        a = a.repeat_interleave(delay)
    return_zf = zi is not None
    if zi is None:
        zi = torch.zeros_like(a)
    elif zi.dim() == 1:
        zi = zi.flip(0).repeat(batch)
    else:
        zi = zi.flip(1).flatten()
    y = linear_recurrence(-a, zi, phases, **kwargs)
    y = y.view(batch, delay, -1).transpose(1, 2).reshape(batch, -1)
    if tail:
        y = y[:, :-tail]
    if return_zf:
        return y, y[:, -delay:].flip(1)
    return y


def _pad_to_order2(b: Tensor, a: Tensor):
    """Coefficient vectors of a section of order <= 2 padded to b: (...,3), a: (...,2)."""
    order = max(b.size(-1) - 1, a.size(-1))
    if order > 2:
        raise NotImplementedError(f"filter order {order}: philtorch_b200 implements first- and second-order "
                                  "sections only (cascade them for higher orders)")
    if order < 1:
        raise ValueError("the filter needs at least one recursive or delayed coefficient")
    if b.size(-1) < 3:
        b = F.pad(b, (0, 3 - b.size(-1)))
    if a.size(-1) < 2:
        a = F.pad(a, (0, 2 - a.size(-1)))
    return b, a, order


def _tdf2_section(b: Tensor, a: Tensor, x: Tensor, zi: Optional[Tensor]):
    b2, a2, order = _pad_to_order2(b, a)
    if b2.dim() != a2.dim():   # one batched, one shared
        B = x.size(0)
        b2 = b2.expand(B, -1) if b2.dim() == 1 else b2
        a2 = a2.expand(B, -1) if a2.dim() == 1 else a2
    zi2 = None
    if zi is not None:
        if zi.dim() == 1:
            zi = zi.unsqueeze(0).expand(x.size(0), -1)
        zi2 = F.pad(zi, (0, 2 - zi.size(-1))) if zi.size(-1) < 2 else zi
    y, zf = BiquadTDF2.apply(b2, a2, zi2, x)
    if zi is None:
        return y
    return y, zf[:, :order]


def _ssm_lfilter(b: Tensor, a: Tensor, x: Tensor, zi: Optional[Tensor] = None, form: str = "tdf2", **kwargs):
    kwargs.pop("unroll_factor", None)   # block size of the reference's Python scan; meaningless here
    if kwargs:
        raise TypeError(f"unexpected keyword arguments: {sorted(kwargs)}")
    order = max(b.size(-1) - 1, a.size(-1))
    if form == "tdf2" and order <= 2:
        return _tdf2_section(b, a, x, zi)     # the fused section kernel
    if form in ("tdf2", "df2"):
        # the filter's companion system on the recurrence kernels (orders up to 8 on the dense N x N
        # kernels), with the input / output maps of philtorch/lti/filtering.py:288-313
        if order > MAX_ORDER:
            raise NotImplementedError(f"filter order {order}: the 'ssm' backend covers orders up to {MAX_ORDER}; "
                                      "cascade second-order sections (sosfilt) or use backend='diag_ssm'")
        if b.size(-1) < a.size(-1) + 1:
            b = F.pad(b, (0, a.size(-1) + 1 - b.size(-1)))
        elif b.size(-1) > a.size(-1) + 1:
            a = F.pad(a, (0, b.size(-1) - a.size(-1) - 1))
        b0 = b[..., :1]
        mix = b[..., 1:] - b0 * a
        if form == "df2":
            return state_space(companion(a), x, B=None, C=mix, D=b[..., 0], zi=zi, out_idx=None)
        return state_space(companion(a).mT, x, B=mix, C=None, D=b[..., 0], zi=zi, out_idx=0)
    if form in ("df1", "tdf1"):
        raise NotImplementedError(f"form={form!r} is built on an FIR convolution, which is outside this package; "
                                  "use 'tdf2' or 'df2'")
    raise ValueError(f"Unknown filter form: {form}")


def _diag_ssm_lfilter(b: Tensor, a: Tensor, x: Tensor, zi: Optional[Tensor] = None, form: str = "df2",
                      delayed_form: bool = False, **kwargs):
    """The filter as a state-space model evaluated in its eigenbasis (philtorch/lti/filtering.py:336-410)
    for numerators no longer than the denominator (longer ones need the FIR quotient of a
    polynomial division, which is outside this package)."""
    if b.size(-1) > a.size(-1) + 1:
        raise NotImplementedError("backend='diag_ssm' with more numerator than denominator coefficients needs an FIR "
                                  "stage, which is outside this package")
    if b.size(-1) < a.size(-1) + 1:
        b = F.pad(b, (0, a.size(-1) + 1 - b.size(-1)))
    A = companion(a)
    b0 = b[..., :1]
    mix = b[..., 1:] - b0 * a
    if form == "df2":
        return diag_state_space(x, A=A, B=None, C=mix, D=b[..., 0], zi=zi, **kwargs)
    if form == "tdf2":
        return diag_state_space(x, A=A.mT.conj(), B=mix.conj(), C=None, D=b[..., 0].conj(), zi=zi, out_idx=0,
                                **kwargs)
    raise ValueError(f"Unknown filter form: {form}")


def lfilter(b: Tensor, a: Tensor, x: Tensor, zi: Optional[Tensor] = None, form: str = "tdf2",
            backend: str = "ssm", **kwargs) -> Union[Tensor, tuple[Tensor, Tensor]]:
    """Apply a batch of time-invariant IIR filters (``a0 = 1`` implicit, ``a`` excludes it).

    Args:
        b: numerator, (B, Mb+1) or (Mb+1,).
        a: denominator without a0, (B, Ma) or (Ma,); max(Mb, Ma) <= 2.
        x: input, (B, N) or (N,), CUDA, float32 or float64.
        zi: initial state, (B, max(Mb, Ma)) or (max(Mb, Ma),); when given, ``(y, zf)`` is returned.
        form: 'tdf2' (default, fused kernel) or 'df2'.
        backend: 'ssm' (orders 1-2, real kernels) or 'diag_ssm': the filter's companion system in its
            eigenbasis, ANY order, as Ma complex first-order recurrences (``diag_state_space``); it
            takes ``L`` / ``V`` / ``Vinv`` (poles and eigenvectors, when known) through ``**kwargs``
            and returns a complex tensor with a vanishing imaginary part for form 'tdf2', as the
            reference does.
        **kwargs: ``unroll_factor`` is accepted for compatibility and ignored.
    """
    squeeze_first = (x.dim() == 1) & (b.dim() == 1) & (a.dim() == 1) & ((zi is None) or (zi.dim() == 1))
    if x.dim() == 1:
        x = x.unsqueeze(0)
    elif x.dim() > 2:
        raise ValueError("Input signal x must be 1D or 2D.")
    assert b.dim() in (1, 2), "Numerator coefficients b must be 1D or 2D."
    assert a.dim() in (1, 2), "Denominator coefficients a must be 1D or 2D."
    if backend == "diag_ssm":
        y = _diag_ssm_lfilter(b, a, x, zi, form=form, **kwargs)
    elif backend == "ssm":
        y = _ssm_lfilter(b, a, x, zi, form=form, **kwargs)
    else:
        raise ValueError(f"Unknown backend: {backend}")
    if isinstance(y, tuple):
        y, zf = y
        if squeeze_first:
            y, zf = y.squeeze(0), zf.squeeze(0)
        return y, zf
    return y.squeeze(0) if squeeze_first else y


def sosfilt(b: Tensor, a: Tensor, x: Tensor, zi: Optional[Tensor] = None) -> Union[Tensor, tuple[Tensor, Tensor]]:
    """A cascade of K second-order sections, the result of
    ``for k in range(K): x = lfilter(b[k], a[k], x, form="tdf2")`` (the way a cascade is run with
    philtorch/lti/filtering.py:211-333), computed by fused kernels: up to eight sections per pass
    over the signal, forward and backward.

    Args:
        b: numerators, (K, 3) or (K, B, 3).
        a: denominators without a0 = 1, (K, 2) or (K, B, 2).
        x: input, (B, N), CUDA, float32 or float64.
        zi: initial states of all sections, (K, B, 2); when given, ``(y, zf)`` is returned.
    """
    if x.dim() != 2:
        raise ValueError("Input signal x must be 2D (batch, time).")
    if b.dim() not in (2, 3) or a.dim() not in (2, 3) or b.size(0) != a.size(0):
        raise ValueError("b must be (K,3) or (K,B,3) and a (K,2) or (K,B,2) with the same K.")
    if b.dim() != a.dim():   # one batched, one shared
        B = x.size(0)
        b = b.unsqueeze(1).expand(-1, B, -1) if b.dim() == 2 else b
        a = a.unsqueeze(1).expand(-1, B, -1) if a.dim() == 2 else a
    K = b.size(0)
    kmax = max(SOS_CASCADE_SIZES)
    y, zfs, k0 = x, [], 0
    while k0 < K:
        n = min(kmax, K - k0)
        bg, ag = b[k0:k0 + n], a[k0:k0 + n]
        zg = None if zi is None else zi[k0:k0 + n]
        if n == 1:
            y, zf = BiquadTDF2.apply(bg[0], ag[0], None if zg is None else zg[0], y)
            zf = zf.unsqueeze(0)
        else:
            m = min(q for q in SOS_CASCADE_SIZES if q >= n)
            if m > n:   # pad with identity sections: y = x, no state
                eye_b = torch.zeros_like(bg[:1]).index_fill(-1, torch.zeros(1, dtype=torch.long, device=b.device), 1.0)
                bg = torch.cat([bg] + [eye_b] * (m - n))
                ag = torch.cat([ag] + [torch.zeros_like(ag[:1])] * (m - n))
                if zg is not None:
                    zg = torch.cat([zg] + [torch.zeros_like(zg[:1])] * (m - n))
            y, zf = SOSCascade.apply(bg, ag, zg, y)
            zf = zf[:n]
        zfs.append(zf)
        k0 += n
    if zi is None:
        return y
    return y, torch.cat(zfs)


def lfilter_zi(a: Tensor, b: Optional[Tensor] = None, transpose: bool = True) -> Tensor:
    """Initial state for which a constant unit input gives a constant output (step steady state),
    as philtorch/lti/filtering.py:107-142: solves (I - A) zi = B for the chosen structure."""
    assert a.dim() >= 1, "Denominator coefficients a must be at least 1D."
    if not transpose:
        n = a.size(-1) + 1
        A = companion(a)
        Bv = a.new_zeros(n - 1)
        Bv[0] = 1.0
    elif b is not None:
        assert b.dim() >= 1, "Numerator coefficients b must be at least 1D."
        n = max(b.size(-1), a.size(-1) + 1)
        if b.size(-1) < n:
            b = F.pad(b, (0, n - b.size(-1)))
        if a.size(-1) < n - 1:
            a = F.pad(a, (0, n - 1 - a.size(-1)))
        A = companion(a).mT
        Bv = b[..., 1:] - b[..., :1] * a
    else:
        raise ValueError("Numerator coefficients b must be provided for transpose=True.")
    IminusA = torch.eye(n - 1, device=a.device, dtype=a.dtype) - A
    if IminusA.dim() == 2 and Bv.dim() > 1:
        IminusA = IminusA.expand(*Bv.shape[:-1], -1, -1)
    return torch.linalg.solve(IminusA, Bv)


def filtfilt(b: Tensor, a: Tensor, x: Tensor, padmode: Optional[str] = "replicate", padlen: Optional[int] = None,
             method: str = "pad", irlen: Optional[int] = None, form: str = "tdf2", **kwargs) -> Tensor:
    """Zero-phase filtering: forward pass, time reversal, second pass (philtorch/lti/filtering.py:413-484).
    Edges are padded by ``padlen`` (default 3 x taps) samples in ``padmode`` and both passes start
    from the step steady state scaled by the first sample."""
    assert method in ("pad", "gust"), "Method must be either 'pad' or 'gust'."
    if method == "gust":
        raise NotImplementedError("Gustafsson's method is not implemented yet.")
    if padmode is None:
        padlen = 0
    ntaps = max(b.size(-1), a.size(-1) + 1)
    edge = 3 * ntaps if padlen is None else padlen
    assert x.size(-1) > edge, f"Input signal length {x.size(-1)} must be greater than pad length {edge}."
    if edge > 0 and padmode is not None:
        ext = F.pad(x.view(-1, x.size(-1)), (edge, edge), mode=padmode)
        if x.dim() == 1:
            ext = ext.squeeze(0)
    else:
        ext = x
    zi = lfilter_zi(a, b, transpose=(form == "tdf2"))
    y, _ = lfilter(b, a, ext, zi=zi * ext[..., :1], form=form, **kwargs)
    y, _ = lfilter(b, a, y.flip(-1), zi=zi * y[..., -1:], form=form, **kwargs)
    if edge > 0:
        y = y[..., edge:-edge]
    return y.flip(-1)
