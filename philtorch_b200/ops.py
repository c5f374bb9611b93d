"""Torch custom ops of the recurrence path (namespace ``philtorch_b200``).

They mirror the reference's dispatcher ops (philtorch/csrc/host_recur2.cpp:162-171: functional,
schema ``(Tensor A, Tensor zi, Tensor x) -> Tensor``, shape contracts of the fake impls in
philtorch/__init__.py:159-244) and add what the reference lacks: a native first-order
per-sample-coefficient op and fused adjoint ops, so a backward pass is one kernel instead of
flip/roll/cat copies around a second forward call.

Every op runs the hand-written sm_100a kernels through the C ABI (``_lib``); CPU tensors and
dtypes other than float32/float64 (and, for the first-order recurrences, complex64/complex128 and
float16/bfloat16 with float32 arithmetic) raise.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from . import _lib
from ._lib import lib, ptr

_LIB = torch.library.Library("philtorch_b200", "DEF")
_TAGS = (torch.Tag.pt2_compliant_tag,)


def _same_dtype(a: Tensor, zi: Tensor, x: Tensor) -> None:
    if zi.dtype != x.dtype:
        raise RuntimeError("zi must have the same scalar type as input")
    if a.dtype != x.dtype:
        raise RuntimeError("A must have the same scalar type as input")


def _dense(t: Tensor) -> Tensor:
    """Dense memory holding the tensor's VALUES (a lazily conjugated complex view is materialised)."""
    if t.is_contiguous() and not t.is_conj():
        return t
    return t.resolve_conj().contiguous()


_LOW_PRECISION = (torch.float16, torch.bfloat16)
# Coefficients shared by the rows: from this many samples on, the adjoint kernels add every row's
# tile of the coefficient gradient into the one shared array while they write it out (the order of
# the additions, and so the last bits of the sums, varies from run to run); smaller problems write
# per-row gradients and sum them afterwards, which is bit-reproducible (what gradcheck expects)
SHARED_ACCUMULATE_MIN_SAMPLES = 1 << 16


def _two_byte_kernels_apply(args) -> bool:
    """The first-order kernels read and write float16 / bfloat16 arrays directly (float32 arithmetic in
    registers, 2 bytes per sample of traffic) when every array qualifies for bulk copies: one common
    2-byte dtype, rows of a multiple of 8 samples, 16-byte aligned data."""
    tensors = [a for a in args if isinstance(a, Tensor)]
    if len({t.dtype for t in tensors}) != 1:
        return False
    for t in tensors:
        if t.dim() >= 1 and t.shape[-1] % 8 != 0 and t.dim() == 2:
            return False
        if t.is_contiguous() and t.data_ptr() % 16 != 0:
            return False
    return True


def _fp32_arithmetic(fn):
    """float16 / bfloat16 tensors (which the reference's first-order ops also dispatch,
    philtorch/csrc/lti_recur.cu:135-156): the recurrence is evaluated in float32 and every result is
    rounded once to the storage type, instead of rounding after every step as a 16-bit scan does.
    Arrays that qualify (see ``_two_byte_kernels_apply``) go to the kernels as they are; others are
    converted to float32 and back around the float32 kernels."""
    def wrapped(*args):
        low = next((a.dtype for a in args if isinstance(a, Tensor) and a.dtype in _LOW_PRECISION), None)
        if low is None:
            return fn(*args)
        if _two_byte_kernels_apply(args):
            return fn(*args)
        up = [a.float() if isinstance(a, Tensor) and a.dtype in _LOW_PRECISION else a for a in args]
        out = fn(*up)
        if isinstance(out, tuple):
            return tuple(o.to(low) for o in out)
        return out.to(low)
    wrapped.__name__ = fn.__name__
    wrapped.__doc__ = fn.__doc__
    return wrapped


def _opt(t: Optional[Tensor]) -> Optional[Tensor]:
    return None if t is None else _dense(t)


# =============================================================================== first order, LTI
_LIB.define("lti_recur(Tensor a, Tensor zi, Tensor x) -> Tensor", tags=_TAGS)
_LIB.define("lti_recur_bwd(Tensor a, Tensor zi, Tensor y, Tensor gy, Tensor? g_in, bool need_a, bool need_zi, "
            "bool need_x=True) -> (Tensor, Tensor, Tensor)", tags=_TAGS)


def _check_lti_recur(a: Tensor, zi: Tensor, x: Tensor) -> None:
    torch._check(x.dim() == 2, lambda: f"x must be 2D (batch, time), got {tuple(x.shape)}")
    torch._check(a.dim() <= 1, lambda: "A must be 1D or scalar.")
    torch._check(zi.dim() == 1, lambda: "zi must be a vector")
    torch._check(zi.shape[0] == x.shape[0], lambda: "x and zi must have the same batch size.")
    if a.dim() == 1 and a.shape[0] != 1:
        torch._check(a.shape[0] == x.shape[0], lambda: "If A is 1D, its length must match x's batch size.")


@_fp32_arithmetic
def _lti_recur(a: Tensor, zi: Tensor, x: Tensor) -> Tensor:
    _check_lti_recur(a, zi, x)
    dev = _lib.require_cuda(a, zi, x)
    _same_dtype(a, zi, x)
    B, T = x.shape
    a_c, zi_c, x_c = _dense(a), _dense(zi), _dense(x)
    y = torch.empty_like(x_c)
    if B and T:
        _lib.call(lib.ptb_lti_recur_fwd, dev, B, T, _lib.dtype_code(x, True), B, T, ptr(a_c),
                  int(a.dim() == 1 and a.shape[0] == B), ptr(zi_c), 1, ptr(x_c), ptr(y), None)
    return y


@_fp32_arithmetic
def _lti_recur_bwd(a, zi, y, gy, g_in, need_a, need_zi, need_x=True):
    dev = _lib.require_cuda(a, zi, y, gy, g_in)
    B, T = y.shape
    a_c, zi_c, y_c, gy_c, gin_c = _dense(a), _dense(zi), _dense(y), _dense(gy), _opt(g_in)
    gx = torch.empty_like(y_c) if need_x else y.new_empty(0)   # not wanted: the kernel skips the store
    ga = torch.empty_like(a_c) if need_a else a.new_empty(0)   # every entry is written by the reduction
    gzi = torch.empty_like(zi_c) if need_zi else zi.new_empty(0)
    if B and T:
        _lib.call(lib.ptb_lti_recur_bwd, dev, B, T, _lib.dtype_code(y, True), B, T, ptr(a_c),
                  int(a.dim() == 1 and a.shape[0] == B), ptr(zi_c), 1, ptr(y_c), ptr(gy_c), ptr(gin_c),
                  ptr(gx) if need_x else None, ptr(ga) if need_a else None, ptr(gzi) if need_zi else None)
    else:
        ga.zero_()
        gzi.zero_()
    return ga, gzi, gx


_LIB.impl("lti_recur", _lti_recur, "CUDA")
_LIB.impl("lti_recur_bwd", _lti_recur_bwd, "CUDA")


@torch.library.register_fake("philtorch_b200::lti_recur")
def _(a, zi, x):
    _check_lti_recur(a, zi, x)
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@torch.library.register_fake("philtorch_b200::lti_recur_bwd")
def _(a, zi, y, gy, g_in, need_a, need_zi, need_x=True):
    return (torch.empty_like(a) if need_a else a.new_empty(0),
            torch.empty_like(zi) if need_zi else zi.new_empty(0),
            torch.empty_like(y, memory_format=torch.contiguous_format) if need_x else y.new_empty(0))


# =============================================================================== first order, LPV
_LIB.define("lpv_recur(Tensor a, Tensor zi, Tensor x) -> Tensor", tags=_TAGS)
_LIB.define("lpv_recur_bwd(Tensor a, Tensor zi, Tensor y, Tensor gy, Tensor? g_in, bool need_a, bool need_zi, "
            "bool need_x=True) -> (Tensor, Tensor, Tensor)", tags=_TAGS)


def _check_lpv_recur(a: Tensor, zi: Tensor, x: Tensor) -> None:
    torch._check(x.dim() == 2, lambda: f"x must be 2D (batch, time), got {tuple(x.shape)}")
    torch._check(a.dim() in (1, 2), lambda: "a must be 1D (time) or 2D (batch, time).")
    torch._check(zi.dim() == 1, lambda: "zi must be a vector")
    torch._check(zi.shape[0] == x.shape[0], lambda: "x and zi must have the same batch size.")
    torch._check(a.shape[-1] == x.shape[1], lambda: "a's last dimension must match x's time dimension.")
    if a.dim() == 2:
        torch._check(a.shape[0] == x.shape[0], lambda: "If a is 2D, its first dimension must match x's batch size.")


@_fp32_arithmetic
def _lpv_recur(a: Tensor, zi: Tensor, x: Tensor) -> Tensor:
    _check_lpv_recur(a, zi, x)
    dev = _lib.require_cuda(a, zi, x)
    _same_dtype(a, zi, x)
    B, T = x.shape
    a_c, zi_c, x_c = _dense(a), _dense(zi), _dense(x)
    y = torch.empty_like(x_c)
    if B and T:
        _lib.call(lib.ptb_lpv_recur_fwd, dev, B, T, _lib.dtype_code(x, True), B, T, ptr(a_c), int(a.dim() == 2),
                  ptr(zi_c), 1, ptr(x_c), ptr(y), None)
    return y


@_fp32_arithmetic
def _lpv_recur_bwd(a, zi, y, gy, g_in, need_a, need_zi, need_x=True):
    dev = _lib.require_cuda(a, zi, y, gy, g_in)
    B, T = y.shape
    a_c, zi_c, y_c, gy_c, gin_c = _dense(a), _dense(zi), _dense(y), _dense(gy), _opt(g_in)
    gx = torch.empty_like(y_c) if need_x else y.new_empty(0)   # not wanted: the kernel skips the store
    gzi = torch.empty_like(zi_c) if need_zi else zi.new_empty(0)
    if (need_a and a.dim() == 1 and B * T >= SHARED_ACCUMULATE_MIN_SAMPLES and y.dtype not in _LOW_PRECISION
            and (T * y.element_size()) % 16 == 0 and all(t.data_ptr() % 16 == 0 for t in (a_c, y_c, gy_c))):
        # coefficients shared by the rows: the kernel adds every row's tile into the one (T,) gradient
        ga = torch.zeros_like(a_c)
        _lib.call(lib.ptb_lpv_recur_bwd_shared, dev, B, T, _lib.dtype_code(y, True), B, T, ptr(a_c), ptr(zi_c), 1,
                  ptr(y_c), ptr(gy_c), ptr(gin_c), ptr(gx) if need_x else None, ptr(ga), ptr(gzi) if need_zi else None)
        return ga, gzi, gx
    ga_rows = torch.empty_like(y_c) if need_a else a.new_empty(0)   # per-row, (B,T)
    if B and T:
        _lib.call(lib.ptb_lpv_recur_bwd, dev, B, T, _lib.dtype_code(y, True), B, T, ptr(a_c), int(a.dim() == 2),
                  ptr(zi_c), 1, ptr(y_c), ptr(gy_c), ptr(gin_c), ptr(gx) if need_x else None,
                  ptr(ga_rows) if need_a else None, ptr(gzi) if need_zi else None)
    elif need_zi:
        gzi.zero_()
    if need_a and a.dim() == 1:
        ga_rows = ga_rows.sum(0)   # coefficients shared by the batch: philtorch/__init__.py:62-65
    return ga_rows, gzi, gx


_LIB.impl("lpv_recur", _lpv_recur, "CUDA")
_LIB.impl("lpv_recur_bwd", _lpv_recur_bwd, "CUDA")


@torch.library.register_fake("philtorch_b200::lpv_recur")
def _(a, zi, x):
    _check_lpv_recur(a, zi, x)
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@torch.library.register_fake("philtorch_b200::lpv_recur_bwd")
def _(a, zi, y, gy, g_in, need_a, need_zi, need_x=True):
    return (torch.empty_like(a) if need_a else a.new_empty(0),
            torch.empty_like(zi) if need_zi else zi.new_empty(0),
            torch.empty_like(y, memory_format=torch.contiguous_format) if need_x else y.new_empty(0))


# carry pass of a time-sharded first-order scan: (product of a, end state from zero) per row
_LIB.define("lpv_recur_carry(Tensor a, Tensor x, bool reverse) -> Tensor", tags=_TAGS)


def _lpv_recur_carry(a: Tensor, x: Tensor, reverse: bool) -> Tensor:
    torch._check(x.dim() == 2 and a.dim() in (1, 2) and a.shape[-1] == x.shape[1],
                 lambda: "a must be (T,) or (B,T) and x (B,T)")
    dev = _lib.require_cuda(a, x)
    if a.dtype != x.dtype:
        raise RuntimeError("a must have the same scalar type as input")
    B, T = x.shape
    a_c, x_c = a.contiguous(), x.contiguous()
    carry = x.new_empty(B, 2)
    if B and T:
        _lib.call(lib.ptb_lpv_recur_carry, dev, B, T, _lib.dtype_code(x), B, T, ptr(a_c), int(a.dim() == 2),
                  ptr(x_c), int(reverse), ptr(carry))
    elif B:
        carry[:, 0] = 1
        carry[:, 1] = 0
    return carry


_LIB.impl("lpv_recur_carry", _lpv_recur_carry, "CUDA")

# local scan of a time shard from a zero state, plus the shard's total map, in one pass
_LIB.define("lpv_recur_zero_carry(Tensor a, Tensor x) -> (Tensor, Tensor)", tags=_TAGS)


def _lpv_recur_zero_carry(a: Tensor, x: Tensor):
    torch._check(x.dim() == 2 and a.dim() in (1, 2) and a.shape[-1] == x.shape[1] and x.shape[1] > 0,
                 lambda: "a must be (T,) or (B,T) and x (B,T), T > 0")
    dev = _lib.require_cuda(a, x)
    if a.dtype != x.dtype:
        raise RuntimeError("a must have the same scalar type as input")
    B, T = x.shape
    a_c, x_c = a.contiguous(), x.contiguous()
    y = torch.empty_like(x_c)
    carry = x.new_empty(B, 2)
    if B:
        _lib.call(lib.ptb_lpv_recur_fwd_carry, dev, B, T, _lib.dtype_code(x), B, T, ptr(a_c), int(a.dim() == 2),
                  ptr(x_c), ptr(y), ptr(carry))
    return y, carry


_LIB.impl("lpv_recur_zero_carry", _lpv_recur_zero_carry, "CUDA")


@torch.library.register_fake("philtorch_b200::lpv_recur_zero_carry")
def _(a, x):
    return torch.empty_like(x, memory_format=torch.contiguous_format), x.new_empty(x.shape[0], 2)



@torch.library.register_fake("philtorch_b200::lpv_recur_carry")
def _(a, x, reverse):
    return x.new_empty(x.shape[0], 2)


# =============================================================================== 2x2
# x is (B,T,2), or (B,T) for the *_sx ops (scalar sequence feeding state 0 only).
for _n in ("lti_recur2", "lti_recur2_sx", "recur2", "recur2_sx"):
    _LIB.define(f"{_n}(Tensor A, Tensor zi, Tensor x) -> Tensor", tags=_TAGS)
for _n in ("lti_recur2_bwd", "recur2_bwd"):
    _LIB.define(f"{_n}(Tensor A, Tensor zi, Tensor y, Tensor gy, Tensor? g_in, bool x_scalar, bool need_A, "
                "bool need_zi) -> (Tensor, Tensor, Tensor)", tags=_TAGS)


def _check_recur2(A: Tensor, zi: Tensor, x: Tensor, lpv: bool, sx: bool) -> None:
    torch._check(A.dim() >= 2 and A.shape[-1] == 2 and A.shape[-2] == 2, lambda: "A must be square.")
    if lpv:
        torch._check(A.dim() in (3, 4), lambda: "A must be 3D or 4D.")
    else:
        torch._check(A.dim() in (2, 3), lambda: "A must be 2D or 3D.")
    torch._check(zi.dim() == 2 and zi.shape[1] == 2, lambda: "zi must have last dimension of size 2.")
    if sx:
        torch._check(x.dim() == 2, lambda: "x must be 2D (batch, time).")
    else:
        torch._check(x.dim() == 3 and x.shape[2] == 2, lambda: "x must have last dimension of size 2.")
    torch._check(x.shape[0] == zi.shape[0], lambda: "x and zi must have the same batch size.")
    if lpv:
        torch._check(x.shape[1] == A.shape[-3], lambda: "x's second dimension must match A's last-3 dimension.")
    if A.dim() == (4 if lpv else 3):
        torch._check(A.shape[0] == x.shape[0], lambda: "A's first dimension must match x's batch size.")


def _make_recur2(lpv: bool, sx: bool):
    fn = lib.ptb_lpv_recur2_fwd if lpv else lib.ptb_lti_recur2_fwd

    def impl(A: Tensor, zi: Tensor, x: Tensor) -> Tensor:
        _check_recur2(A, zi, x, lpv, sx)
        dev = _lib.require_cuda(A, zi, x)
        _same_dtype(A, zi, x)
        B, T = x.shape[0], x.shape[1]
        A_c, zi_c, x_c = A.contiguous(), zi.contiguous(), x.contiguous()
        y = x.new_empty(B, T, 2)
        if B and T:
            _lib.call(fn, dev, B, T, _lib.dtype_code(x), B, T, ptr(A_c), int(A.dim() == (4 if lpv else 3)),
                      ptr(zi_c), ptr(x_c), int(sx), ptr(y), None)
        return y

    def fake(A, zi, x):
        _check_recur2(A, zi, x, lpv, sx)
        return x.new_empty(x.shape[0], x.shape[1], 2)

    return impl, fake


def _make_recur2_bwd(lpv: bool):
    fn = lib.ptb_lpv_recur2_bwd if lpv else lib.ptb_lti_recur2_bwd

    def impl(A, zi, y, gy, g_in, x_scalar, need_A, need_zi):
        dev = _lib.require_cuda(A, zi, y, gy, g_in)
        B, T = y.shape[0], y.shape[1]
        A_c, zi_c, y_c, gy_c, gin_c = A.contiguous(), zi.contiguous(), y.contiguous(), gy.contiguous(), _opt(g_in)
        gx = y.new_empty((B, T) if x_scalar else (B, T, 2))
        batched = A.dim() == (4 if lpv else 3)
        gzi = torch.empty_like(zi_c) if need_zi else zi.new_empty(0)
        if (lpv and need_A and not batched and B * T >= SHARED_ACCUMULATE_MIN_SAMPLES
                and (T * (1 if x_scalar else 2) * y.element_size()) % 16 == 0
                and all(t.data_ptr() % 16 == 0 for t in (A_c, y_c, gy_c, gx))):
            # matrices shared by the rows: the kernel adds every row's tile into the one (T,2,2) gradient
            gA = torch.zeros_like(A_c)
            _lib.call(lib.ptb_lpv_recur2_bwd_shared, dev, B, T, _lib.dtype_code(y), B, T, ptr(A_c), ptr(zi_c), ptr(y_c),
                      ptr(gy_c), ptr(gin_c), int(x_scalar), ptr(gx), ptr(gA), ptr(gzi) if need_zi else None)
            return gA, gzi, gx
        if not need_A:
            gA = A.new_empty(0)
        elif lpv:
            gA = y.new_empty(B, T, 2, 2)            # per row
        else:
            gA = torch.zeros_like(A_c)
        if B and T:
            _lib.call(fn, dev, B, T, _lib.dtype_code(y), B, T, ptr(A_c), int(batched), ptr(zi_c), ptr(y_c),
                      ptr(gy_c), ptr(gin_c), int(x_scalar), ptr(gx), ptr(gA) if need_A else None,
                      ptr(gzi) if need_zi else None)
        elif need_zi:
            gzi.zero_()
        if need_A and lpv and not batched:
            gA = gA.sum(0)   # coefficients shared by the batch: philtorch/__init__.py:62-65
        return gA, gzi, gx

    def fake(A, zi, y, gy, g_in, x_scalar, need_A, need_zi):
        B, T = y.shape[0], y.shape[1]
        return (torch.empty_like(A) if need_A else A.new_empty(0),
                torch.empty_like(zi) if need_zi else zi.new_empty(0),
                y.new_empty((B, T) if x_scalar else (B, T, 2)))

    return impl, fake


for _n, _lpv, _sx in (("lti_recur2", False, False), ("lti_recur2_sx", False, True),
                      ("recur2", True, False), ("recur2_sx", True, True)):
    _impl, _fake = _make_recur2(_lpv, _sx)
    _LIB.impl(_n, _impl, "CUDA")
    torch.library.register_fake(f"philtorch_b200::{_n}")(_fake)
for _n, _lpv in (("lti_recur2_bwd", False), ("recur2_bwd", True)):
    _impl, _fake = _make_recur2_bwd(_lpv)
    _LIB.impl(_n, _impl, "CUDA")
    torch.library.register_fake(f"philtorch_b200::{_n}")(_fake)


# =============================================================================== N x N, 2 < N <= 8
# Dense state matrices above 2x2: the reference's recurN / lti_recurN ops (CPU only there,
# philtorch/csrc/host_recurN.cpp:236-281, philtorch/csrc/host_lti_recurN.cpp:63-108).
MAX_STATE_DIM = 8
_LIB.define("recur_n(Tensor A, Tensor zi, Tensor x) -> Tensor", tags=_TAGS)
_LIB.define("lti_recur_n(Tensor A, Tensor zi, Tensor x) -> Tensor", tags=_TAGS)
_LIB.define("recur_n_adj(Tensor A, Tensor gy, Tensor? g_in, bool timevar) -> (Tensor, Tensor)", tags=_TAGS)


def _check_recur_n(A: Tensor, zi: Optional[Tensor], x: Tensor, lpv: bool) -> None:
    torch._check(x.dim() == 3, lambda: "x must be 3D (batch, time, state).")
    n = x.shape[2]
    torch._check(A.dim() >= 2 and A.shape[-1] == n and A.shape[-2] == n, lambda: "A must be square.")
    torch._check(1 <= n <= MAX_STATE_DIM, lambda: f"state dimension {n}: the kernels cover 1..{MAX_STATE_DIM}.")
    if lpv:
        torch._check(A.dim() in (3, 4), lambda: "A must be 3D or 4D.")
        torch._check(x.shape[1] == A.shape[-3], lambda: "x's second dimension must match A's last-3 dimension.")
    else:
        torch._check(A.dim() in (2, 3), lambda: "A must be 2D or 3D.")
    if zi is not None:
        torch._check(zi.dim() == 2 and zi.shape[1] == n, lambda: "zi must have the state dimension of x.")
        torch._check(x.shape[0] == zi.shape[0], lambda: "x and zi must have the same batch size.")
    if A.dim() == (4 if lpv else 3):
        torch._check(A.shape[0] == x.shape[0], lambda: "A's first dimension must match x's batch size.")


def _make_recur_n(lpv: bool):
    def impl(A: Tensor, zi: Tensor, x: Tensor) -> Tensor:
        _check_recur_n(A, zi, x, lpv)
        dev = _lib.require_cuda(A, zi, x)
        _same_dtype(A, zi, x)
        B, T, n = x.shape
        A_c, zi_c, x_c = A.contiguous(), zi.contiguous(), x.contiguous()
        y = torch.empty_like(x_c)
        if B and T:
            code = _lib.dtype_code(x)
            _lib.call(lib.ptb_recur_n_fwd, dev, B, T, code, n, B, T, ptr(A_c), int(A.dim() == (4 if lpv else 3)),
                      int(lpv), ptr(zi_c), ptr(x_c), ptr(y), None,
                      ws_bytes=lib.ptb_recur_n_workspace_bytes(code, n, B, T))
        return y

    def fake(A, zi, x):
        _check_recur_n(A, zi, x, lpv)
        return torch.empty_like(x, memory_format=torch.contiguous_format)

    return impl, fake


def _recur_n_adj(A: Tensor, gy: Tensor, g_in: Optional[Tensor], timevar: bool):
    """g[t] = gy[t] + c[t+1], c[t] = A[t]^T g[t], c[T] = g_in: returns (g, c[0])."""
    _check_recur_n(A, g_in, gy, timevar)
    dev = _lib.require_cuda(A, gy, g_in)
    if A.dtype != gy.dtype or (g_in is not None and g_in.dtype != gy.dtype):
        raise RuntimeError("A and g_in must have the same scalar type as gy")
    B, T, n = gy.shape
    A_c, gy_c, gin_c = A.contiguous(), gy.contiguous(), _opt(g_in)
    g = torch.empty_like(gy_c)
    c0 = gy.new_zeros(B, n) if g_in is None else gin_c.clone()
    if B and T:
        code = _lib.dtype_code(gy)
        _lib.call(lib.ptb_recur_n_adj, dev, B, T, code, n, B, T, ptr(A_c), int(A.dim() == (4 if timevar else 3)),
                  int(timevar), ptr(gy_c), ptr(gin_c), ptr(g), ptr(c0),
                  ws_bytes=lib.ptb_recur_n_workspace_bytes(code, n, B, T))
    return g, c0


for _n, _lpv in (("recur_n", True), ("lti_recur_n", False)):
    _impl, _fake = _make_recur_n(_lpv)
    _LIB.impl(_n, _impl, "CUDA")
    torch.library.register_fake(f"philtorch_b200::{_n}")(_fake)
_LIB.impl("recur_n_adj", _recur_n_adj, "CUDA")


@torch.library.register_fake("philtorch_b200::recur_n_adj")
def _(A, gy, g_in, timevar):
    return torch.empty_like(gy, memory_format=torch.contiguous_format), gy.new_empty(gy.shape[0], gy.shape[2])


_LIB.define("outer_prev_sum(Tensor g, Tensor h, Tensor zi) -> Tensor", tags=_TAGS)


def _outer_prev_sum(g: Tensor, h: Tensor, zi: Tensor) -> Tensor:
    """(B,n,n): sum over t of g[b,t] (x) h[b,t-1] with h[b,-1] = zi[b] (grad_A of a constant matrix)."""
    dev = _lib.require_cuda(g, h, zi)
    torch._check(g.dim() == 3 and h.shape == g.shape and zi.shape == (g.shape[0], g.shape[2]),
                 lambda: "g, h must be (B,T,n) and zi (B,n).")
    torch._check(1 <= g.shape[2] <= MAX_STATE_DIM, lambda: f"state dimension above {MAX_STATE_DIM}")
    if h.dtype != g.dtype or zi.dtype != g.dtype:
        raise RuntimeError("g, h and zi must have the same scalar type")
    B, T, n = g.shape
    if not (B and T):
        return g.new_zeros(B, n, n)
    g_c, h_c, zi_c = g.contiguous(), h.contiguous(), zi.contiguous()
    chunks = lib.ptb_outer_prev_sum_chunks(B, T)
    part = g.new_empty(B, chunks, n, n)
    with torch.cuda.device(dev):
        _lib.check(lib.ptb_outer_prev_sum(_lib.dtype_code(g), n, B, T, ptr(g_c), ptr(h_c), ptr(zi_c), ptr(part),
                                          torch.cuda.current_stream(dev).cuda_stream), "ptb_outer_prev_sum")
    return part.sum(1)


_LIB.impl("outer_prev_sum", _outer_prev_sum, "CUDA")


@torch.library.register_fake("philtorch_b200::outer_prev_sum")
def _(g, h, zi):
    return g.new_empty(g.shape[0], g.shape[2], g.shape[2])


# =============================================================================== TDF-II section
_LIB.define("biquad_tdf2(Tensor b, Tensor a, Tensor? zi, Tensor x) -> (Tensor, Tensor)", tags=_TAGS)
_LIB.define("biquad_tdf2_bwd(Tensor b, Tensor a, Tensor x, Tensor y, Tensor gy, Tensor? gzf, bool need_coef, "
            "bool need_zi) -> (Tensor, Tensor, Tensor, Tensor)", tags=_TAGS)


def _check_biquad(b: Tensor, a: Tensor, zi: Optional[Tensor], x: Tensor) -> None:
    torch._check(x.dim() == 2, lambda: "x must be 2D (batch, time).")
    torch._check(b.dim() in (1, 2) and b.shape[-1] == 3, lambda: "b must be (3,) or (B,3).")
    torch._check(a.dim() == b.dim() and a.shape[-1] == 2, lambda: "a must be (2,) or (B,2), like b.")
    if b.dim() == 2:
        torch._check(b.shape[0] == x.shape[0] and a.shape[0] == x.shape[0],
                     lambda: "batched coefficients must match x's batch size.")
    if zi is not None:
        torch._check(zi.dim() == 2 and zi.shape[0] == x.shape[0] and zi.shape[1] == 2, lambda: "zi must be (B,2).")


def _biquad_tdf2(b, a, zi, x):
    _check_biquad(b, a, zi, x)
    dev = _lib.require_cuda(b, a, zi, x)
    if b.dtype != x.dtype or a.dtype != x.dtype or (zi is not None and zi.dtype != x.dtype):
        raise RuntimeError("b, a and zi must have the same scalar type as input")
    B, T = x.shape
    b_c, a_c, zi_c, x_c = b.contiguous(), a.contiguous(), _opt(zi), x.contiguous()
    y = torch.empty_like(x_c)
    zf = x.new_empty(B, 2)
    if B and T:
        _lib.call(lib.ptb_biquad_tdf2_fwd, dev, B, T, _lib.dtype_code(x), B, T, ptr(b_c), ptr(a_c),
                  int(b.dim() == 2), ptr(zi_c), ptr(x_c), ptr(y), ptr(zf))
    elif B:
        zf.copy_(zi_c) if zi_c is not None else zf.zero_()
    return y, zf


def _biquad_tdf2_bwd(b, a, x, y, gy, gzf, need_coef, need_zi):
    dev = _lib.require_cuda(b, a, x, y, gy, gzf)
    B, T = x.shape
    b_c, a_c, x_c, y_c, gy_c, gzf_c = b.contiguous(), a.contiguous(), x.contiguous(), y.contiguous(), \
        gy.contiguous(), _opt(gzf)
    gx = torch.empty_like(x_c)
    # the reduction that ends the launch writes every entry: zeros only when nothing is launched
    fresh = torch.empty_like if (B and T) else torch.zeros_like
    gb = fresh(b_c) if need_coef else b.new_empty(0)
    ga = fresh(a_c) if need_coef else a.new_empty(0)
    gzi = x.new_empty(B, 2) if need_zi else x.new_empty(0)
    if B and T:
        _lib.call(lib.ptb_biquad_tdf2_bwd, dev, B, T, _lib.dtype_code(x), B, T, ptr(b_c), ptr(a_c),
                  int(b.dim() == 2), ptr(x_c), ptr(y_c), ptr(gy_c), ptr(gzf_c), ptr(gx),
                  ptr(gb) if need_coef else None, ptr(ga) if need_coef else None,
                  ptr(gzi) if need_zi else None)
    elif need_zi:
        gzi.copy_(gzf_c) if gzf_c is not None else gzi.zero_()
    return gb, ga, gzi, gx


_LIB.impl("biquad_tdf2", _biquad_tdf2, "CUDA")
_LIB.impl("biquad_tdf2_bwd", _biquad_tdf2_bwd, "CUDA")


@torch.library.register_fake("philtorch_b200::biquad_tdf2")
def _(b, a, zi, x):
    _check_biquad(b, a, zi, x)
    return torch.empty_like(x, memory_format=torch.contiguous_format), x.new_empty(x.shape[0], 2)


@torch.library.register_fake("philtorch_b200::biquad_tdf2_bwd")
def _(b, a, x, y, gy, gzf, need_coef, need_zi):
    return (torch.empty_like(b) if need_coef else b.new_empty(0),
            torch.empty_like(a) if need_coef else a.new_empty(0),
            x.new_empty(x.shape[0], 2) if need_zi else x.new_empty(0),
            torch.empty_like(x, memory_format=torch.contiguous_format))


# =============================================================================== reverse-time pass, fused combine
_LIB.define("lti_recur_reverse_fused(Tensor a, Tensor x, Tensor second, Tensor? g_in, float scale, bool need_first)"
            " -> (Tensor, Tensor)", tags=_TAGS)


def _lti_recur_reverse_fused(a, x, second, g_in, scale, need_first):
    """out = scale * (g + second - x), g[t] = x[t] + a g[t+1], g[T-1] = x[T-1] + g_in; (out, a g[0])."""
    torch._check(x.dim() == 2 and second.shape == x.shape, lambda: "x and second must be (B, T) alike.")
    torch._check(a.dim() <= 1 and a.numel() in (1, x.shape[0]), lambda: "a must hold one value or one per row.")
    dev = _lib.require_cuda(a, x, second, g_in)
    if a.dtype != x.dtype or second.dtype != x.dtype or (g_in is not None and g_in.dtype != x.dtype):
        raise RuntimeError("a, second and g_in must have the same scalar type as input")
    B, T = x.shape
    a_c, x_c, s_c, gin_c = a.contiguous(), x.contiguous(), second.contiguous(), _opt(g_in)
    out = torch.empty_like(x_c)
    first = x.new_zeros(B) if need_first else x.new_empty(0)
    if B and T:
        _lib.call(lib.ptb_lti_recur_reverse_fused, dev, B, T, _lib.dtype_code(x), B, T, ptr(a_c),
                  int(a.dim() == 1 and a.shape[0] == B and B > 1), ptr(x_c), ptr(s_c), ptr(gin_c), float(scale),
                  ptr(out), ptr(first) if need_first else None)
    return out, first


_LIB.impl("lti_recur_reverse_fused", _lti_recur_reverse_fused, "CUDA")


@torch.library.register_fake("philtorch_b200::lti_recur_reverse_fused")
def _(a, x, second, g_in, scale, need_first):
    return (torch.empty_like(x, memory_format=torch.contiguous_format),
            x.new_empty(x.shape[0]) if need_first else x.new_empty(0))


# =============================================================================== eigenbasis output map
_LIB.define("modal_mix(Tensor w, Tensor? w0, Tensor coef, bool real_out) -> Tensor", tags=_TAGS)
_LIB.define("modal_mix_bwd(Tensor w, Tensor w0, Tensor coef, Tensor gy, bool real_out, bool need_coef)"
            " -> (Tensor, Tensor, Tensor)", tags=_TAGS)


def _check_modal(w: Tensor, w0: Tensor, coef: Tensor) -> None:
    torch._check(w.dim() == 3 and w.is_complex(), lambda: "w must be complex (rows, M, N).")
    torch._check(w0 is None or tuple(w0.shape) == tuple(w.shape[:2]), lambda: "w0 must be (rows, M).")
    torch._check(tuple(coef.shape) in ((w.shape[1],), tuple(w.shape[:2])), lambda: "coef must be (M,) or (rows, M).")
    torch._check((w0 is None or w0.dtype == w.dtype) and coef.dtype == w.dtype,
                 lambda: "w, w0 and coef must share a complex dtype.")


def _real_of(dtype):
    return torch.float32 if dtype == torch.complex64 else torch.float64


def _modal_mix(w, w0, coef, real_out):
    """y[r,t] = sum_m coef[r,m] w[r,m,t-1] (w[r,m,-1] = w0[r,m]); the real part when real_out.
    Without w0 there is no delay: y[r,t] = sum_m coef[r,m] w[r,m,t]."""
    _check_modal(w, w0, coef)
    dev = _lib.require_cuda(w, w0, coef)
    R, M, N = w.shape
    w_c, w0_c, c_c = _dense(w), _opt(w0), _dense(coef)
    y = torch.empty(R, N, dtype=_real_of(w.dtype) if real_out else w.dtype, device=w.device)
    if R and N:
        _lib.call(lib.ptb_modal_mix_fwd, dev, R, N, _lib.dtype_code(w, True), R, M, N, ptr(w_c), ptr(w0_c), ptr(c_c),
                  int(coef.dim() == 2), int(real_out), ptr(y), ws_bytes=0)
    return y


def _modal_mix_bwd(w, w0, coef, gy, real_out, need_coef):
    dev = _lib.require_cuda(w, w0, coef, gy)
    R, M, N = w.shape
    w_c, w0_c, c_c, gy_c = _dense(w), _dense(w0), _dense(coef), _dense(gy)
    gw = torch.empty_like(w_c)
    gw0 = torch.zeros_like(w0_c)
    nblk = lib.ptb_modal_mix_partial_blocks(N)
    part = torch.zeros(R, nblk, M, dtype=w.dtype, device=w.device) if need_coef else None
    if R and N:
        _lib.call(lib.ptb_modal_mix_bwd, dev, R, N, _lib.dtype_code(w, True), R, M, N, ptr(w_c), ptr(w0_c), ptr(c_c),
                  int(coef.dim() == 2), int(real_out), ptr(gy_c), ptr(gw), ptr(gw0), ptr(part), ws_bytes=0)
    if need_coef:
        gc = part.sum(1) if coef.dim() == 2 else part.sum((0, 1))
    else:
        gc = coef.new_empty(0)
    return gw, gw0, gc


_LIB.define("modal_drive(Tensor x, Tensor gain) -> Tensor", tags=_TAGS)


def _check_modal_drive(x: Tensor, gain: Tensor) -> None:
    torch._check(x.dim() == 2 and not x.is_complex(), lambda: "x must be real (rows, N).")
    torch._check(gain.is_complex() and (gain.dim() == 1 or (gain.dim() == 2 and gain.shape[0] == x.shape[0])),
                 lambda: "gain must be complex (M,) or (rows, M).")
    torch._check(_real_of(gain.dtype) == x.dtype, lambda: "x must have the precision of gain.")


def _modal_drive(x, gain):
    """u[r,m,t] = gain[(r,)m] * x[r,t]."""
    _check_modal_drive(x, gain)
    dev = _lib.require_cuda(x, gain)
    R, N = x.shape
    M = gain.shape[-1]
    x_c, g_c = x.contiguous(), _dense(gain)
    u = torch.empty(R, M, N, dtype=gain.dtype, device=x.device)
    if R and N:
        _lib.call(lib.ptb_modal_drive_fwd, dev, R, N, _lib.dtype_code(gain, True), R, M, N, ptr(x_c), ptr(g_c),
                  int(gain.dim() == 2), ptr(u), ws_bytes=0)
    return u


_LIB.impl("modal_drive", _modal_drive, "CUDA")


@torch.library.register_fake("philtorch_b200::modal_drive")
def _(x, gain):
    _check_modal_drive(x, gain)
    return torch.empty(x.shape[0], gain.shape[-1], x.shape[1], dtype=gain.dtype, device=x.device)


_LIB.impl("modal_mix", _modal_mix, "CUDA")
_LIB.impl("modal_mix_bwd", _modal_mix_bwd, "CUDA")


@torch.library.register_fake("philtorch_b200::modal_mix")
def _(w, w0, coef, real_out):
    _check_modal(w, w0, coef)
    return torch.empty(w.shape[0], w.shape[2], dtype=_real_of(w.dtype) if real_out else w.dtype, device=w.device)


@torch.library.register_fake("philtorch_b200::modal_mix_bwd")
def _(w, w0, coef, gy, real_out, need_coef):
    return (torch.empty_like(w, memory_format=torch.contiguous_format), torch.empty_like(w0),
            torch.empty_like(coef) if need_coef else coef.new_empty(0))


# =============================================================================== fused bank of modes
_LIB.define("modal_bank(Tensor x, Tensor lam, Tensor gain, Tensor coef, Tensor? d, Tensor w0)"
            " -> (Tensor, Tensor, Tensor)", tags=_TAGS)
_LIB.define("modal_bank_bwd(Tensor x, Tensor lam, Tensor gain, Tensor coef, Tensor? d, Tensor chk, Tensor gy, "
            "Tensor? g_wf, int need) -> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)", tags=_TAGS)
MODAL_BANK_MAX_MODES = 8


def _cplx_of(dtype):
    return torch.complex64 if dtype == torch.float32 else torch.complex128


def _check_modal_bank(x, lam, gain, coef, d, w0) -> None:
    torch._check(x.dim() == 2 and x.dtype in (torch.float32, torch.float64), lambda: "x must be real (rows, N).")
    R, M = x.shape[0], lam.shape[-1]
    torch._check(1 <= M <= MODAL_BANK_MAX_MODES, lambda: f"1..{MODAL_BANK_MAX_MODES} modes, got {M}.")
    for name, t in (("lam", lam), ("gain", gain), ("coef", coef), ("w0", w0)):
        torch._check(tuple(t.shape) == (R, M) and t.dtype == _cplx_of(x.dtype),
                     lambda: f"{name} must be complex (rows, M) of x's precision.")
    torch._check(d is None or (tuple(d.shape) == (R,) and d.dtype == x.dtype), lambda: "d must be real (rows,).")


def _modal_bank(x, lam, gain, coef, d, w0):
    """y[r,t] = Re(sum_m coef w_m[t-1]) + d x[t], w_m[t] = lam w_m[t-1] + gain x[t]; returns
    (y, final modes, the modes entering every tile -- needed by the backward op)."""
    _check_modal_bank(x, lam, gain, coef, d, w0)
    dev = _lib.require_cuda(x, lam, gain, coef, d, w0)
    R, N = x.shape
    M = lam.shape[1]
    x_c, lam_c, gain_c, coef_c, d_c, w0_c = x.contiguous(), _dense(lam), _dense(gain), _dense(coef), _opt(d), _dense(w0)
    y = torch.empty_like(x_c)
    wf = w0_c.clone()
    chk = w0.new_empty(R, lib.ptb_modal_bank_tiles(M, max(N, 1)), M)
    if R and N:
        with torch.cuda.device(dev):
            _lib.check(lib.ptb_modal_bank_fwd(_lib.dtype_code(x), R, M, N, ptr(x_c), ptr(lam_c), ptr(gain_c),
                                              ptr(coef_c), ptr(d_c), ptr(w0_c), ptr(y), ptr(wf), ptr(chk),
                                              torch.cuda.current_stream(dev).cuda_stream), "ptb_modal_bank_fwd")
    return y, wf, chk


def _modal_bank_bwd(x, lam, gain, coef, d, chk, gy, g_wf, need):
    dev = _lib.require_cuda(x, lam, gain, coef, d, chk, gy, g_wf)
    R, N = x.shape
    M = lam.shape[1]
    x_c, lam_c, gain_c, coef_c, d_c = x.contiguous(), _dense(lam), _dense(gain), _dense(coef), _opt(d)
    gy_c, gwf_c, chk_c = gy.contiguous(), _opt(g_wf), chk.contiguous()
    gx = torch.empty_like(x_c)
    gw0 = torch.zeros_like(lam_c) if g_wf is None else gwf_c.clone()
    nt = chk.shape[1]
    part = x.new_zeros(R, nt, 6 * M + 1)
    if R and N:
        scratch = torch.empty_like(chk_c)
        with torch.cuda.device(dev):
            _lib.check(lib.ptb_modal_bank_bwd(_lib.dtype_code(x), R, M, N, ptr(x_c), ptr(lam_c), ptr(gain_c),
                                              ptr(coef_c), ptr(d_c), ptr(chk_c), ptr(gy_c), ptr(gwf_c), int(need), ptr(gx),
                                              ptr(gw0), ptr(part), ptr(scratch),
                                              torch.cuda.current_stream(dev).cuda_stream), "ptb_modal_bank_bwd")
    sums = part.sum(1)                                                    # (R, 6M + 1)
    cz = torch.view_as_complex(sums[:, :6 * M].reshape(R, 3, M, 2).contiguous())
    return gx, cz[:, 1].contiguous(), cz[:, 0].contiguous(), cz[:, 2].contiguous(), sums[:, 6 * M].contiguous(), gw0


_LIB.impl("modal_bank", _modal_bank, "CUDA")
_LIB.impl("modal_bank_bwd", _modal_bank_bwd, "CUDA")


@torch.library.register_fake("philtorch_b200::modal_bank")
def _(x, lam, gain, coef, d, w0):
    _check_modal_bank(x, lam, gain, coef, d, w0)
    nt = (x.shape[1] + (2048 if lam.shape[1] <= 4 else 1024) - 1) // (2048 if lam.shape[1] <= 4 else 1024)
    return (torch.empty_like(x, memory_format=torch.contiguous_format), torch.empty_like(w0),
            w0.new_empty(x.shape[0], max(nt, 1), lam.shape[1]))


@torch.library.register_fake("philtorch_b200::modal_bank_bwd")
def _(x, lam, gain, coef, d, chk, gy, g_wf, need):
    return (torch.empty_like(x, memory_format=torch.contiguous_format), torch.empty_like(lam), torch.empty_like(lam),
            torch.empty_like(lam), x.new_empty(x.shape[0]), torch.empty_like(lam))


# =============================================================================== comb filter
_LIB.define("comb(Tensor a, Tensor? zi, Tensor x, int delay) -> Tensor", tags=_TAGS)
_LIB.define("comb_bwd(Tensor a, Tensor? zi, Tensor y, Tensor gy, int delay, bool need_a, bool need_zi)"
            " -> (Tensor, Tensor, Tensor)", tags=_TAGS)


def _check_comb(a: Tensor, zi: Optional[Tensor], x: Tensor, delay: int) -> None:
    torch._check(x.dim() == 2, lambda: "x must be 2D (batch, time).")
    torch._check(delay >= 1, lambda: "delay must be at least 1.")
    torch._check(a.dim() == 0 or (a.dim() == 1 and a.shape[0] in (1, x.shape[0])),
                 lambda: "a must be a scalar or (B,).")
    if zi is not None:
        torch._check(tuple(zi.shape) in ((delay,), (x.shape[0], delay)), lambda: "zi must be (delay,) or (B, delay).")


def _comb_args(a, zi, x):
    B = x.shape[0]
    a_batched = int(a.dim() == 1 and a.shape[0] == B and B > 1)
    zi_mode = 0 if zi is None else (1 if zi.dim() == 1 else 2)
    return a_batched, zi_mode


def _comb(a, zi, x, delay):
    _check_comb(a, zi, x, delay)
    dev = _lib.require_cuda(a, zi, x)
    if a.dtype != x.dtype or (zi is not None and zi.dtype != x.dtype):
        raise RuntimeError("a and zi must have the same scalar type as input")
    B, N = x.shape
    a_c, zi_c, x_c = a.contiguous(), _opt(zi), x.contiguous()
    a_batched, zi_mode = _comb_args(a, zi, x)
    y = torch.empty_like(x_c)
    if B and N:
        _lib.call(lib.ptb_comb_fwd, dev, B, N, _lib.dtype_code(x), B, N, delay, ptr(a_c), a_batched, ptr(zi_c),
                  zi_mode, ptr(x_c), ptr(y), ws_bytes=0)
    return y


def _comb_bwd(a, zi, y, gy, delay, need_a, need_zi):
    dev = _lib.require_cuda(a, zi, y, gy)
    B, N = y.shape
    a_c, zi_c, y_c, gy_c = a.contiguous(), _opt(zi), y.contiguous(), gy.contiguous()
    a_batched, zi_mode = _comb_args(a, zi, y)
    gx = torch.empty_like(y_c)
    nblk = lib.ptb_comb_partial_blocks(delay)
    part = y.new_zeros(B, nblk) if need_a else None
    gst = y.new_zeros(B, delay) if need_zi else None
    if B and N:
        _lib.call(lib.ptb_comb_bwd, dev, B, N, _lib.dtype_code(y), B, N, delay, ptr(a_c), a_batched, ptr(zi_c),
                  zi_mode, ptr(y_c), ptr(gy_c), ptr(gx), ptr(part), ptr(gst), ws_bytes=0)
    if need_a:
        ga = part.sum(1) if a_batched else part.sum().reshape(a.shape)
    else:
        ga = a.new_empty(0)
    if need_zi:
        gzi = gst if zi.dim() == 2 else gst.sum(0)
    else:
        gzi = y.new_empty(0)
    return ga, gzi, gx


_LIB.impl("comb", _comb, "CUDA")
_LIB.impl("comb_bwd", _comb_bwd, "CUDA")


@torch.library.register_fake("philtorch_b200::comb")
def _(a, zi, x, delay):
    _check_comb(a, zi, x, delay)
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@torch.library.register_fake("philtorch_b200::comb_bwd")
def _(a, zi, y, gy, delay, need_a, need_zi):
    return (torch.empty_like(a) if need_a else a.new_empty(0),
            torch.empty_like(zi) if need_zi else y.new_empty(0),
            torch.empty_like(y, memory_format=torch.contiguous_format))


# =============================================================================== fused SOS cascade
_LIB.define("sos_cascade(Tensor b, Tensor a, Tensor? zi, Tensor x, bool keep_mid) -> (Tensor, Tensor, Tensor)",
            tags=_TAGS)
_LIB.define("sos_cascade_bwd(Tensor b, Tensor a, Tensor x, Tensor mid, Tensor y, Tensor gy, Tensor? gzf, "
            "bool need_coef, bool need_zi) -> (Tensor, Tensor, Tensor, Tensor)", tags=_TAGS)

SOS_CASCADE_SIZES = (2, 4, 6, 8)   # numbers of sections the fused kernels are built for


def _check_sos(b: Tensor, a: Tensor, zi: Optional[Tensor], x: Tensor) -> None:
    torch._check(x.dim() == 2, lambda: "x must be 2D (batch, time).")
    torch._check(b.dim() in (2, 3) and b.shape[-1] == 3, lambda: "b must be (K,3) or (K,B,3).")
    torch._check(a.dim() == b.dim() and a.shape[-1] == 2 and a.shape[0] == b.shape[0],
                 lambda: "a must be (K,2) or (K,B,2), like b.")
    torch._check(b.shape[0] in SOS_CASCADE_SIZES, lambda: f"the number of sections must be one of {SOS_CASCADE_SIZES}.")
    if b.dim() == 3:
        torch._check(b.shape[1] == x.shape[0] and a.shape[1] == x.shape[0],
                     lambda: "batched coefficients must match x's batch size.")
    if zi is not None:
        torch._check(zi.dim() == 3 and zi.shape[0] == b.shape[0] and zi.shape[1] == x.shape[0] and zi.shape[2] == 2,
                     lambda: "zi must be (K,B,2).")


def _sos_cascade(b, a, zi, x, keep_mid):
    _check_sos(b, a, zi, x)
    dev = _lib.require_cuda(b, a, zi, x)
    if b.dtype != x.dtype or a.dtype != x.dtype or (zi is not None and zi.dtype != x.dtype):
        raise RuntimeError("b, a and zi must have the same scalar type as input")
    K = b.shape[0]
    B, T = x.shape
    b_c, a_c, zi_c, x_c = b.contiguous(), a.contiguous(), _opt(zi), x.contiguous()
    y = torch.empty_like(x_c)
    mid = x.new_empty((K - 1, B, T) if keep_mid else (0,))
    zf = x.new_empty(K, B, 2)
    if B and T:
        code = _lib.dtype_code(x)
        _lib.call(lib.ptb_sos_cascade_fwd, dev, B, T, code, K, B, T, ptr(b_c), ptr(a_c), int(b.dim() == 3),
                  ptr(zi_c), ptr(x_c), ptr(y), ptr(mid) if keep_mid else None, ptr(zf),
                  ws_bytes=lib.ptb_sos_cascade_workspace_bytes(code, K, B, T))
    elif B:
        zf.copy_(zi_c) if zi_c is not None else zf.zero_()
    return y, mid, zf


def _sos_cascade_bwd(b, a, x, mid, y, gy, gzf, need_coef, need_zi):
    dev = _lib.require_cuda(b, a, x, mid, y, gy, gzf)
    K = b.shape[0]
    B, T = x.shape
    b_c, a_c, x_c, mid_c, y_c, gy_c, gzf_c = b.contiguous(), a.contiguous(), x.contiguous(), mid.contiguous(), \
        y.contiguous(), gy.contiguous(), _opt(gzf)
    if need_coef and mid.numel() != (K - 1) * B * T:
        raise RuntimeError("coefficient gradients need the intermediate section outputs (keep_mid=True)")
    gx = torch.empty_like(x_c)
    # the reduction that ends the launch writes every entry: zeros only when nothing is launched
    fresh = torch.empty_like if (B and T) else torch.zeros_like
    gb = fresh(b_c) if need_coef else b.new_empty(0)
    ga = fresh(a_c) if need_coef else a.new_empty(0)
    gzi = x.new_empty(K, B, 2) if need_zi else x.new_empty(0)
    if B and T:
        code = _lib.dtype_code(x)
        _lib.call(lib.ptb_sos_cascade_bwd, dev, B, T, code, K, B, T, ptr(b_c), ptr(a_c), int(b.dim() == 3),
                  ptr(x_c), ptr(mid_c) if need_coef else None, ptr(y_c), ptr(gy_c), ptr(gzf_c), ptr(gx),
                  ptr(gb) if need_coef else None, ptr(ga) if need_coef else None, ptr(gzi) if need_zi else None,
                  ws_bytes=lib.ptb_sos_cascade_workspace_bytes(code, K, B, T))
    elif need_zi:
        gzi.copy_(gzf_c) if gzf_c is not None else gzi.zero_()
    return gb, ga, gzi, gx


_LIB.impl("sos_cascade", _sos_cascade, "CUDA")
_LIB.impl("sos_cascade_bwd", _sos_cascade_bwd, "CUDA")


@torch.library.register_fake("philtorch_b200::sos_cascade")
def _(b, a, zi, x, keep_mid):
    _check_sos(b, a, zi, x)
    K = b.shape[0]
    return (torch.empty_like(x, memory_format=torch.contiguous_format),
            x.new_empty((K - 1, x.shape[0], x.shape[1]) if keep_mid else (0,)), x.new_empty(K, x.shape[0], 2))


@torch.library.register_fake("philtorch_b200::sos_cascade_bwd")
def _(b, a, x, mid, y, gy, gzf, need_coef, need_zi):
    return (torch.empty_like(b) if need_coef else b.new_empty(0),
            torch.empty_like(a) if need_coef else a.new_empty(0),
            x.new_empty(b.shape[0], x.shape[0], 2) if need_zi else x.new_empty(0),
            torch.empty_like(x, memory_format=torch.contiguous_format))


# =============================================================================== fused LPV biquad (df2)
for _form in ("df2", "tdf2"):
    _LIB.define(f"lpv_biquad_{_form}(Tensor b, Tensor a, Tensor? zi, Tensor x, bool keep_states) "
                "-> (Tensor, Tensor, Tensor)", tags=_TAGS)
    _LIB.define(f"lpv_biquad_{_form}_bwd(Tensor b, Tensor a, Tensor x, Tensor hp, Tensor gy, Tensor? gzf, "
                "bool need_zi) -> (Tensor, Tensor, Tensor, Tensor)", tags=_TAGS)


def _check_lpv_biquad(b: Tensor, a: Tensor, zi: Optional[Tensor], x: Tensor) -> None:
    torch._check(x.dim() == 2, lambda: "x must be 2D (batch, time).")
    torch._check(b.dim() in (2, 3) and b.shape[-1] == 3 and b.shape[-2] == x.shape[1],
                 lambda: "b must be (N,3) or (B,N,3).")
    torch._check(a.dim() == b.dim() and a.shape[-1] == 2 and a.shape[-2] == x.shape[1],
                 lambda: "a must be (N,2) or (B,N,2), like b.")
    if b.dim() == 3:
        torch._check(b.shape[0] == x.shape[0] and a.shape[0] == x.shape[0],
                     lambda: "batched coefficients must match x's batch size.")
    if zi is not None:
        torch._check(zi.dim() == 2 and zi.shape[0] == x.shape[0] and zi.shape[1] == 2, lambda: "zi must be (B,2).")


def _lpv_biquad_fwd(fn, b, a, zi, x, keep_states):
    _check_lpv_biquad(b, a, zi, x)
    dev = _lib.require_cuda(b, a, zi, x)
    if b.dtype != x.dtype or a.dtype != x.dtype or (zi is not None and zi.dtype != x.dtype):
        raise RuntimeError("b, a and zi must have the same scalar type as input")
    B, T = x.shape
    b_c, a_c, zi_c, x_c = b.contiguous(), a.contiguous(), _opt(zi), x.contiguous()
    y = torch.empty_like(x_c)
    hp = x.new_empty((B, T, 2) if keep_states else (0,))
    zf = x.new_empty(B, 2)
    if B and T:
        code = _lib.dtype_code(x)
        _lib.call(fn, dev, B, T, code, B, T, ptr(b_c), ptr(a_c), int(b.dim() == 3), ptr(zi_c),
                  ptr(x_c), ptr(y), ptr(hp) if keep_states else None, ptr(zf),
                  ws_bytes=lib.ptb_lpv_biquad_workspace_bytes(code, B, T))
    elif B:
        zf.copy_(zi_c) if zi_c is not None else zf.zero_()
    return y, hp, zf


def _lpv_biquad_bwd(fn, b, a, x, hp, gy, gzf, need_zi):
    dev = _lib.require_cuda(b, a, x, hp, gy, gzf)
    B, T = x.shape
    b_c, a_c, x_c, hp_c, gy_c, gzf_c = b.contiguous(), a.contiguous(), x.contiguous(), hp.contiguous(), \
        gy.contiguous(), _opt(gzf)
    if hp.numel() != B * T * 2:
        raise RuntimeError("the backward pass needs the states kept by the forward pass (keep_states=True)")
    gx = torch.empty_like(x_c)
    gb = x.new_empty(B, T, 3)
    ga = x.new_empty(B, T, 2)
    gzi = x.new_empty(B, 2) if need_zi else x.new_empty(0)
    if B and T:
        code = _lib.dtype_code(x)
        _lib.call(fn, dev, B, T, code, B, T, ptr(b_c), ptr(a_c), int(b.dim() == 3), ptr(x_c),
                  ptr(hp_c), ptr(gy_c), ptr(gzf_c), ptr(gx), ptr(gb), ptr(ga), ptr(gzi) if need_zi else None,
                  ws_bytes=lib.ptb_lpv_biquad_workspace_bytes(code, B, T))
    elif need_zi:
        gzi.copy_(gzf_c) if gzf_c is not None else gzi.zero_()
    return gb, ga, gzi, gx


def _lpv_fake_fwd(b, a, zi, x, keep_states):
    _check_lpv_biquad(b, a, zi, x)
    return (torch.empty_like(x, memory_format=torch.contiguous_format),
            x.new_empty((x.shape[0], x.shape[1], 2) if keep_states else (0,)), x.new_empty(x.shape[0], 2))


def _lpv_fake_bwd(b, a, x, hp, gy, gzf, need_zi):
    return (x.new_empty(x.shape[0], x.shape[1], 3), x.new_empty(x.shape[0], x.shape[1], 2),
            x.new_empty(x.shape[0], 2) if need_zi else x.new_empty(0),
            torch.empty_like(x, memory_format=torch.contiguous_format))


for _form, _ffn, _bfn in (("df2", lib.ptb_lpv_biquad_df2_fwd, lib.ptb_lpv_biquad_df2_bwd),
                          ("tdf2", lib.ptb_lpv_biquad_tdf2_fwd, lib.ptb_lpv_biquad_tdf2_bwd)):
    _LIB.impl(f"lpv_biquad_{_form}",
              (lambda fn: lambda b, a, zi, x, keep: _lpv_biquad_fwd(fn, b, a, zi, x, keep))(_ffn), "CUDA")
    _LIB.impl(f"lpv_biquad_{_form}_bwd",
              (lambda fn: lambda b, a, x, hp, gy, gzf, nz: _lpv_biquad_bwd(fn, b, a, x, hp, gy, gzf, nz))(_bfn), "CUDA")
    torch.library.register_fake(f"philtorch_b200::lpv_biquad_{_form}")(_lpv_fake_fwd)
    torch.library.register_fake(f"philtorch_b200::lpv_biquad_{_form}_bwd")(_lpv_fake_bwd)


# CPU (and any other backend) tensors: fail loudly instead of "no kernel registered" noise.
def _no_backend(name):
    def fn(*args, **kwargs):
        raise RuntimeError(f"philtorch_b200::{name} runs on CUDA tensors only (there is no CPU path)")
    return fn


for _name in ("lti_recur", "lti_recur_bwd", "lpv_recur", "lpv_recur_bwd", "lti_recur2", "lti_recur2_sx", "recur2",
              "recur2_sx", "lti_recur2_bwd", "recur2_bwd", "biquad_tdf2", "biquad_tdf2_bwd", "lpv_recur_carry", "lpv_recur_zero_carry",
              "sos_cascade", "sos_cascade_bwd", "lpv_biquad_df2", "lpv_biquad_df2_bwd",
              "lpv_biquad_tdf2", "lpv_biquad_tdf2_bwd", "comb", "comb_bwd", "lti_recur_reverse_fused",
              "modal_mix", "modal_mix_bwd", "modal_drive", "recur_n", "lti_recur_n", "recur_n_adj", "modal_bank",
              "modal_bank_bwd", "outer_prev_sum"):
    _LIB.impl(_name, _no_backend(_name), "CPU")
