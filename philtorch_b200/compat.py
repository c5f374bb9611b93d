"""The B200 kernels behind the reference package's own dispatcher ops.

The reference (philtorch) reaches native code through five ops,
``torch.ops.philtorch.{lti_recur, lti_recur2, lti_recurN, recur2, recurN}``, all with the schema
``(Tensor A, Tensor zi, Tensor x) -> Tensor`` (philtorch/csrc/host_recur2.cpp:162-171); its CPU
extension implements them on the CPU dispatch key, its ``.cu`` files (Thrust scans,
philtorch/csrc/lti_recur.cu:160, lti_recur2.cu:115, recur2.cu:119) on the CUDA key.  ``register()``
installs the kernels of this package on the CUDA key of those very ops, so the UNMODIFIED reference
package -- its autograd Functions (philtorch/lti/recur.py:8-78, philtorch/lti/ssm.py:43-115,
philtorch/lpv/ssm.py:34-115), ``lfilter(..., unroll_factor=1)``, ``state_space_recursion`` -- runs
on them for CUDA tensors:

    import philtorch                  # the reference, with its CPU extension (it defines the ops)
    import philtorch_b200.compat
    philtorch_b200.compat.register()

Only the CUDA key is touched: CPU tensors keep running the reference's own kernels, and the
reference's fake implementations and autograd formulas (philtorch/__init__.py:159-268) stay in
charge.  The reference's backward passes re-enter these ops with flipped / rolled coefficient
copies; use the ``philtorch_b200`` functions directly to get the fused adjoint kernels instead.
"""
from __future__ import annotations

import torch
from torch import Tensor

from . import ops  # noqa: F401  (registers torch.ops.philtorch_b200.*)

_ops = torch.ops.philtorch_b200
_OPS = ("lti_recur", "lti_recur2", "lti_recurN", "recur2", "recurN")
_lib = None


def _lti_recur(A: Tensor, zi: Tensor, x: Tensor) -> Tensor:
    return _ops.lti_recur(A, zi, x)


def _lti_recur2(A: Tensor, zi: Tensor, x: Tensor) -> Tensor:
    return _ops.lti_recur2(A, zi, x)


def _recur2(A: Tensor, zi: Tensor, x: Tensor) -> Tensor:
    return _ops.recur2(A, zi, x)


def _state_dim(A: Tensor, zi: Tensor, x: Tensor) -> int:
    n = x.shape[-1]
    torch._check(A.shape[-1] == n and A.shape[-2] == n, lambda: "A must be square.")
    torch._check(zi.dim() == 2 and zi.shape[1] == n, lambda: "zi must have the state dimension of x.")
    return n


def _lti_recurN(A: Tensor, zi: Tensor, x: Tensor) -> Tensor:
    n = _state_dim(A, zi, x)
    if n == 1:   # (1,1) or (B,1,1) -> () or (B,)
        return _ops.lti_recur(A.reshape(A.shape[:-2]), zi[:, 0], x[..., 0]).unsqueeze(-1)
    if n == 2:
        return _ops.lti_recur2(A, zi, x)
    return _ops.lti_recur_n(A, zi, x)


def _recurN(A: Tensor, zi: Tensor, x: Tensor) -> Tensor:
    n = _state_dim(A, zi, x)
    if n == 1:   # (T,1,1) or (B,T,1,1) -> (T,) or (B,T)
        return _ops.lpv_recur(A[..., 0, 0], zi[:, 0], x[..., 0]).unsqueeze(-1)
    if n == 2:
        return _ops.recur2(A, zi, x)
    return _ops.recur_n(A, zi, x)


_IMPLS = {"lti_recur": _lti_recur, "lti_recur2": _lti_recur2, "lti_recurN": _lti_recurN, "recur2": _recur2,
          "recurN": _recurN}


def registered() -> bool:
    return _lib is not None


def register(allow_override: bool = False) -> None:
    """Installs the kernels as the CUDA implementation of ``torch.ops.philtorch.*``.

    The ops must exist already: import the reference package (or load its compiled extension with
    ``torch.ops.load_library``) first.  A reference build that carries its own CUDA kernels already
    occupies the CUDA key; pass ``allow_override=True`` to replace them.  Idempotent.
    """
    global _lib
    if _lib is not None:
        return
    missing = [n for n in _OPS if not hasattr(torch.ops.philtorch, n)]
    if missing:
        raise RuntimeError(
            "torch.ops.philtorch." + ", ".join(missing) + " not defined: import the reference package with its "
            "compiled extension (or torch.ops.load_library its _C library) before compat.register()")
    lib = torch.library.Library("philtorch", "IMPL")
    for name in _OPS:
        try:
            lib.impl(name, _IMPLS[name], "CUDA", allow_override=allow_override)
        except TypeError:   # older torch: no allow_override argument
            lib.impl(name, _IMPLS[name], "CUDA")
    _lib = lib
