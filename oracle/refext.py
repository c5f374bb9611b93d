"""The reference project's own CPU extension as a checker.  TEST INFRASTRUCTURE ONLY.

``oracle/_ref/philtorch_ref_C.so`` is compiled by ``build_ref.py`` from the reference
checkout's ``philtorch/csrc/host_*.cpp``.  Loading it registers the five dispatcher
ops ``torch.ops.philtorch.{lti_recur,lti_recur2,lti_recurN,recur2,recurN}`` for CPU
tensors (philtorch/csrc/host_recur2.cpp:162-171).

The reference keeps its adjoint rules in Python (philtorch/__init__.py:34-148,
philtorch/lti/recur.py:25-59, philtorch/lti/ssm.py:67-96, philtorch/lpv/ssm.py:64-99).
They are restated here on top of the reference forward ops so that a forward+backward
of the reference path can be evaluated (and timed as the CPU baseline) on a machine
that only has the compiled extension.
"""
from __future__ import annotations

import os

import torch

from . import build_ref

_loaded = False


def available() -> bool:
    return os.path.exists(build_ref.REF_SO) or hasattr(torch.ops.philtorch, "lti_recur")


def load() -> None:
    global _loaded
    if _loaded:
        return
    if hasattr(torch.ops.philtorch, "lti_recur"):
        # the ops are defined already (an installed copy of the reference package was imported and
        # brought its own build of the same extension): defining the library twice would fail
        _loaded = True
        return
    if not available():
        raise RuntimeError("reference CPU extension not built: run oracle/build_ref.py "
                           "on a machine that has the reference checkout")
    torch.ops.load_library(build_ref.REF_SO)
    _loaded = True


def ops():
    load()
    return torch.ops.philtorch


# ---------------------------------------------------------------- forward
def lti_recur(a, zi, x):
    return ops().lti_recur(a, zi, x)


def recur1(a, zi, x):
    """First-order LPV through the reference's generic-order op with N = 1
    (philtorch/csrc/host_recurN.cpp:236-281)."""
    return ops().recurN(a[..., None, None], zi[:, None], x[..., None])[..., 0]


def lti_recur2(A, zi, x):
    return ops().lti_recur2(A, zi, x)


def recur2(A, zi, x):
    return ops().recur2(A, zi, x)


# ---------------------------------------------------------------- adjoints
def lti_recur_bwd(a, zi, y, gy):
    """philtorch/lti/recur.py:25-59."""
    bp_init = gy[:, -1]
    flipped = torch.cat(
        [bp_init.unsqueeze(1), ops().lti_recur(a, bp_init, gy[:, :-1].flip(1))], dim=1)
    grad_zi = flipped[:, -1] * a
    grad_x = flipped.flip(1)
    padded = torch.cat([zi.unsqueeze(1), y[:, :-1]], dim=1)
    if a.dim() == 1 and a.numel() == y.shape[0] and a.numel() > 1:
        grad_a = torch.linalg.vecdot(padded, grad_x)
    else:
        grad_a = (padded.flatten() @ grad_x.flatten()).reshape(a.shape)
    return grad_a, grad_zi, grad_x


def _matrix_bwd(op, A, zi, y, gy, timevar):
    """philtorch/__init__.py:34-112 (LPV: coefficients transposed, rolled by -1 along
    time and flipped; LTI: transposed)."""
    AmT = A.mT
    if timevar:
        run_A = torch.roll(AmT, shifts=-1, dims=-3).flip(-3)
    else:
        run_A = AmT
    flipped = op(run_A.contiguous(), torch.zeros_like(zi), gy.flip(1).contiguous())
    A0T = AmT[..., 0, :, :] if timevar else AmT
    grad_zi = (A0T @ flipped[:, -1, :, None]).squeeze(-1)
    grad_x = flipped.flip(1)
    padded = torch.cat([zi.unsqueeze(1), y[:, :-1]], dim=1)
    if timevar:
        if A.dim() == 3:
            grad_A = grad_x.permute(1, 2, 0) @ padded.transpose(0, 1)
        else:
            grad_A = padded.unsqueeze(-2) * grad_x.unsqueeze(-1)
    else:
        if A.dim() == 2:
            grad_A = grad_x.flatten(0, 1).T @ padded.flatten(0, 1)
        else:
            grad_A = grad_x.mT @ padded
    return grad_A, grad_zi, grad_x


def lti_recur2_bwd(A, zi, y, gy):
    return _matrix_bwd(ops().lti_recur2, A, zi, y, gy, False)


def recur2_bwd(A, zi, y, gy):
    return _matrix_bwd(ops().recur2, A, zi, y, gy, True)


def recur1_bwd(a, zi, y, gy):
    gA, gzi, gx = _matrix_bwd(ops().recurN, a[..., None, None], zi[:, None], y[..., None],
                              gy[..., None], True)
    return gA[..., 0, 0], gzi[:, 0], gx[..., 0]
