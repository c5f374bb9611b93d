"""ctypes front-end of ``recur_oracle.c``.  TEST INFRASTRUCTURE ONLY.

All functions take and return CPU ``torch`` tensors (fp32 or fp64; the first-order
routines also complex64 / complex128; made contiguous here) with the shapes of the reference ops:

* ``lti_recur(a, zi, x)``     a: () | (1,) | (B,), zi: (B,), x: (B,T)
  -- philtorch/csrc/host_lti_recur.cpp:42-80
* ``recur1(a, zi, x)``        a: (T,) | (B,T)  -- first-order LPV, the N = 1 case of
  philtorch/csrc/host_recurN.cpp:236-281 / philtorch/lpv/recur.py:20-101
* ``lti_recur2(A, zi, x)``    A: (2,2) | (B,2,2), zi: (B,2), x: (B,T,2)
  -- philtorch/csrc/host_lti_recurN.cpp:63-108
* ``recur2(A, zi, x)``        A: (T,2,2) | (B,T,2,2)
  -- philtorch/csrc/host_recurN.cpp:236-281
* ``*_bwd(coef, zi, y, gy, g_in=None)`` -> (grad_coef, grad_zi, grad_x): the adjoint
  rules of philtorch/__init__.py:34-148.
* ``biquad_tdf2(b, a, zi, x)`` -> (y, zf): philtorch/lti/filtering.py:304-317.
"""
from __future__ import annotations

import ctypes

import torch

from . import build_ref

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build_ref.build_c_oracle())  # no-op when up to date
    return _lib


def _suf(t: torch.Tensor) -> str:
    if t.dtype == torch.float32:
        return "f32"
    if t.dtype == torch.float64:
        return "f64"
    if t.dtype == torch.complex64:
        return "c64"
    if t.dtype == torch.complex128:
        return "c128"
    raise TypeError(f"oracle handles fp32/fp64 (first order: also complex64/128), got {t.dtype}")


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _c(t: torch.Tensor) -> torch.Tensor:
    assert t.device.type == "cpu"
    return t.detach().resolve_conj().contiguous()


def _i64(v):
    return ctypes.c_int64(int(v))


def lti_recur(a, zi, x):
    a, zi, x = _c(a), _c(zi), _c(x)
    B, T = x.shape
    batched = int(a.dim() == 1 and a.numel() == B)
    y = torch.empty_like(x)
    getattr(lib(), "oracle_lti_recur_" + _suf(x))(_i64(B), _i64(T), _p(a), batched, _p(zi), _p(x), _p(y))
    return y


def lti_recur_bwd(a, zi, y, gy, g_in=None):
    a, zi, y, gy = _c(a), _c(zi), _c(y), _c(gy)
    g_in = _c(g_in) if g_in is not None else None
    B, T = y.shape
    batched = int(a.dim() == 1 and a.numel() == B)
    gx = torch.empty_like(y)
    ga = torch.empty_like(a)
    gzi = torch.empty_like(zi)
    getattr(lib(), "oracle_lti_recur_bwd_" + _suf(y))(
        _i64(B), _i64(T), _p(a), batched, _p(zi), _p(y), _p(gy), _p(g_in), _p(gx), _p(ga), _p(gzi))
    return ga, gzi, gx


def recur1(a, zi, x):
    a, zi, x = _c(a), _c(zi), _c(x)
    B, T = x.shape
    batched = int(a.dim() == 2)
    y = torch.empty_like(x)
    getattr(lib(), "oracle_recur1_" + _suf(x))(_i64(B), _i64(T), _p(a), batched, _p(zi), _p(x), _p(y))
    return y


def recur1_bwd(a, zi, y, gy, g_in=None):
    a, zi, y, gy = _c(a), _c(zi), _c(y), _c(gy)
    g_in = _c(g_in) if g_in is not None else None
    B, T = y.shape
    batched = int(a.dim() == 2)
    gx = torch.empty_like(y)
    ga = torch.empty_like(a)
    gzi = torch.empty_like(zi)
    getattr(lib(), "oracle_recur1_bwd_" + _suf(y))(
        _i64(B), _i64(T), _p(a), batched, _p(zi), _p(y), _p(gy), _p(g_in), _p(gx), _p(ga), _p(gzi))
    return ga, gzi, gx


def _recur2(A, zi, x, timevar):
    A, zi, x = _c(A), _c(zi), _c(x)
    B, T, _ = x.shape
    batched = int(A.dim() == (4 if timevar else 3))
    y = torch.empty_like(x)
    getattr(lib(), "oracle_recur2_" + _suf(x))(
        _i64(B), _i64(T), _p(A), batched, int(timevar), _p(zi), _p(x), _p(y))
    return y


def _recur2_bwd(A, zi, y, gy, timevar, g_in=None):
    A, zi, y, gy = _c(A), _c(zi), _c(y), _c(gy)
    g_in = _c(g_in) if g_in is not None else None
    B, T, _ = y.shape
    batched = int(A.dim() == (4 if timevar else 3))
    gx = torch.empty_like(y)
    gA = torch.empty_like(A)
    gzi = torch.empty_like(zi)
    getattr(lib(), "oracle_recur2_bwd_" + _suf(y))(
        _i64(B), _i64(T), _p(A), batched, int(timevar), _p(zi), _p(y), _p(gy), _p(g_in),
        _p(gx), _p(gA), _p(gzi))
    return gA, gzi, gx


def lti_recur2(A, zi, x):
    return _recur2(A, zi, x, False)


def recur2(A, zi, x):
    return _recur2(A, zi, x, True)


def lti_recur2_bwd(A, zi, y, gy, g_in=None):
    return _recur2_bwd(A, zi, y, gy, False, g_in)


def recur2_bwd(A, zi, y, gy, g_in=None):
    return _recur2_bwd(A, zi, y, gy, True, g_in)


def biquad_tdf2(b, a, zi, x):
    b, a, x = _c(b), _c(a), _c(x)
    zi = _c(zi) if zi is not None else None
    B, T = x.shape
    batched = int(b.dim() == 2)
    y = torch.empty_like(x)
    zf = x.new_empty(B, 2)
    getattr(lib(), "oracle_biquad_tdf2_" + _suf(x))(
        _i64(B), _i64(T), _p(b), _p(a), batched, _p(zi), _p(x), _p(y), _p(zf))
    return y, zf


def biquad_tdf2_bwd(b, a, zi, x, gy, gzf=None):
    """Adjoint of ``biquad_tdf2``: (grad_b, grad_a, grad_zi, grad_x)."""
    b, a, x, gy = _c(b), _c(a), _c(x), _c(gy)
    zi = _c(zi) if zi is not None else None
    gzf = _c(gzf) if gzf is not None else None
    B, T = x.shape
    gx = torch.empty_like(x)
    gb, ga = torch.empty_like(b), torch.empty_like(a)
    gzi = x.new_empty(B, 2)
    getattr(lib(), "oracle_biquad_tdf2_bwd_" + _suf(x))(
        _i64(B), _i64(T), _p(b), _p(a), int(b.dim() == 2), _p(zi), _p(x), _p(gy), _p(gzf),
        _p(gx), _p(gb), _p(ga), _p(gzi))
    return gb, ga, gzi, gx


def sos_chain(b, a, x):
    """K chained TDF-II sections (b (K,3)|(K,B,3), a (K,2)|(K,B,2)), the way the reference runs a
    cascade (K ``lfilter`` calls, philtorch/lti/filtering.py:304-317): returns the inputs of every
    section and the final output."""
    u, ins = x, []
    for k in range(b.shape[0]):
        ins.append(u)
        u, _ = biquad_tdf2(b[k], a[k], None, u)
    return ins, u


def sos_chain_bwd(b, a, ins, gy):
    """Adjoint of ``sos_chain``: (grad_b, grad_a, grad_x), sections taken in reverse order."""
    gb, ga = torch.empty_like(b), torch.empty_like(a)
    g = gy
    for k in range(b.shape[0] - 1, -1, -1):
        gb[k], ga[k], _, g = biquad_tdf2_bwd(b[k], a[k], None, ins[k], g)
    return gb, ga, g
