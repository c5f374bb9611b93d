"""Torch custom ops of the recurrence path (namespace ``philtorch_b200``).

They mirror the reference's dispatcher ops (philtorch/csrc/host_recur2.cpp:162-171: functional,
schema ``(Tensor A, Tensor zi, Tensor x) -> Tensor``, shape contracts of the fake impls in
philtorch/__init__.py:159-244) and add what the reference lacks: a native first-order
per-sample-coefficient op and fused adjoint ops, so a backward pass is one kernel instead of
flip/roll/cat copies around a second forward call.

Every op runs the hand-written sm_100a kernels through the C ABI (``_lib``); CPU tensors and
dtypes other than float32/float64 raise.
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


def _opt(t: Optional[Tensor]) -> Optional[Tensor]:
    return None if t is None else t.contiguous()


# =============================================================================== first order, LTI
_LIB.define("lti_recur(Tensor a, Tensor zi, Tensor x) -> Tensor", tags=_TAGS)
_LIB.define("lti_recur_bwd(Tensor a, Tensor zi, Tensor y, Tensor gy, Tensor? g_in, bool need_a, bool need_zi)"
            " -> (Tensor, Tensor, Tensor)", tags=_TAGS)


def _check_lti_recur(a: Tensor, zi: Tensor, x: Tensor) -> None:
    torch._check(x.dim() == 2, lambda: f"x must be 2D (batch, time), got {tuple(x.shape)}")
    torch._check(a.dim() <= 1, lambda: "A must be 1D or scalar.")
    torch._check(zi.dim() == 1, lambda: "zi must be a vector")
    torch._check(zi.shape[0] == x.shape[0], lambda: "x and zi must have the same batch size.")
    if a.dim() == 1 and a.shape[0] != 1:
        torch._check(a.shape[0] == x.shape[0], lambda: "If A is 1D, its length must match x's batch size.")


def _lti_recur(a: Tensor, zi: Tensor, x: Tensor) -> Tensor:
    _check_lti_recur(a, zi, x)
    dev = _lib.require_cuda(a, zi, x)
    _same_dtype(a, zi, x)
    B, T = x.shape
    a_c, zi_c, x_c = a.contiguous(), zi.contiguous(), x.contiguous()
    y = torch.empty_like(x_c)
    if B and T:
        _lib.call(lib.ptb_lti_recur_fwd, dev, B, T, _lib.dtype_code(x), B, T, ptr(a_c),
                  int(a.dim() == 1 and a.shape[0] == B), ptr(zi_c), 1, ptr(x_c), ptr(y), None)
    return y


def _lti_recur_bwd(a, zi, y, gy, g_in, need_a, need_zi):
    dev = _lib.require_cuda(a, zi, y, gy, g_in)
    B, T = y.shape
    a_c, zi_c, y_c, gy_c, gin_c = a.contiguous(), zi.contiguous(), y.contiguous(), gy.contiguous(), _opt(g_in)
    gx = torch.empty_like(y_c)
    ga = torch.zeros_like(a_c) if need_a else a.new_empty(0)
    gzi = torch.empty_like(zi_c) if need_zi else zi.new_empty(0)
    if B and T:
        _lib.call(lib.ptb_lti_recur_bwd, dev, B, T, _lib.dtype_code(y), B, T, ptr(a_c),
                  int(a.dim() == 1 and a.shape[0] == B), ptr(zi_c), 1, ptr(y_c), ptr(gy_c), ptr(gin_c),
                  ptr(gx), ptr(ga) if need_a else None, ptr(gzi) if need_zi else None)
    elif need_zi:
        gzi.zero_()
    return ga, gzi, gx


_LIB.impl("lti_recur", _lti_recur, "CUDA")
_LIB.impl("lti_recur_bwd", _lti_recur_bwd, "CUDA")


@torch.library.register_fake("philtorch_b200::lti_recur")
def _(a, zi, x):
    _check_lti_recur(a, zi, x)
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@torch.library.register_fake("philtorch_b200::lti_recur_bwd")
def _(a, zi, y, gy, g_in, need_a, need_zi):
    return (torch.empty_like(a) if need_a else a.new_empty(0),
            torch.empty_like(zi) if need_zi else zi.new_empty(0),
            torch.empty_like(y, memory_format=torch.contiguous_format))


# =============================================================================== first order, LPV
_LIB.define("lpv_recur(Tensor a, Tensor zi, Tensor x) -> Tensor", tags=_TAGS)
_LIB.define("lpv_recur_bwd(Tensor a, Tensor zi, Tensor y, Tensor gy, Tensor? g_in, bool need_a, bool need_zi)"
            " -> (Tensor, Tensor, Tensor)", tags=_TAGS)


def _check_lpv_recur(a: Tensor, zi: Tensor, x: Tensor) -> None:
    torch._check(x.dim() == 2, lambda: f"x must be 2D (batch, time), got {tuple(x.shape)}")
    torch._check(a.dim() in (1, 2), lambda: "a must be 1D (time) or 2D (batch, time).")
    torch._check(zi.dim() == 1, lambda: "zi must be a vector")
    torch._check(zi.shape[0] == x.shape[0], lambda: "x and zi must have the same batch size.")
    torch._check(a.shape[-1] == x.shape[1], lambda: "a's last dimension must match x's time dimension.")
    if a.dim() == 2:
        torch._check(a.shape[0] == x.shape[0], lambda: "If a is 2D, its first dimension must match x's batch size.")


def _lpv_recur(a: Tensor, zi: Tensor, x: Tensor) -> Tensor:
    _check_lpv_recur(a, zi, x)
    dev = _lib.require_cuda(a, zi, x)
    _same_dtype(a, zi, x)
    B, T = x.shape
    a_c, zi_c, x_c = a.contiguous(), zi.contiguous(), x.contiguous()
    y = torch.empty_like(x_c)
    if B and T:
        _lib.call(lib.ptb_lpv_recur_fwd, dev, B, T, _lib.dtype_code(x), B, T, ptr(a_c), int(a.dim() == 2),
                  ptr(zi_c), 1, ptr(x_c), ptr(y), None)
    return y


def _lpv_recur_bwd(a, zi, y, gy, g_in, need_a, need_zi):
    dev = _lib.require_cuda(a, zi, y, gy, g_in)
    B, T = y.shape
    a_c, zi_c, y_c, gy_c, gin_c = a.contiguous(), zi.contiguous(), y.contiguous(), gy.contiguous(), _opt(g_in)
    gx = torch.empty_like(y_c)
    ga_rows = torch.empty_like(y_c) if need_a else a.new_empty(0)   # per-row, (B,T)
    gzi = torch.empty_like(zi_c) if need_zi else zi.new_empty(0)
    if B and T:
        _lib.call(lib.ptb_lpv_recur_bwd, dev, B, T, _lib.dtype_code(y), B, T, ptr(a_c), int(a.dim() == 2),
                  ptr(zi_c), 1, ptr(y_c), ptr(gy_c), ptr(gin_c), ptr(gx),
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
def _(a, zi, y, gy, g_in, need_a, need_zi):
    return (torch.empty_like(a) if need_a else a.new_empty(0),
            torch.empty_like(zi) if need_zi else zi.new_empty(0),
            torch.empty_like(y, memory_format=torch.contiguous_format))


# CPU (and any other backend) tensors: fail loudly instead of "no kernel registered" noise.
def _no_backend(name):
    def fn(*args, **kwargs):
        raise RuntimeError(f"philtorch_b200::{name} runs on CUDA tensors only (there is no CPU path)")
    return fn


for _name in ("lti_recur", "lti_recur_bwd", "lpv_recur", "lpv_recur_bwd"):
    _LIB.impl(_name, _no_backend(_name), "CPU")
