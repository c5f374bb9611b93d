"""Autograd Functions of the recurrence path.

Same names, argument order and saved tensors as the reference's Functions
(``LTIRecurrence`` philtorch/lti/recur.py:8-78, ``LTIMatrixRecurrence``
philtorch/lti/ssm.py:43-115, ``MatrixRecurrence`` philtorch/lpv/ssm.py:34-115), plus
``LPVRecurrence`` for the first-order per-sample case the reference leaves to pure PyTorch.

First-order backward passes run ONE fused adjoint kernel.  When a higher-order graph is being
recorded (``create_graph=True``) the backward is instead expressed with differentiable
pieces -- the same Functions applied to the time-reversed gradient -- so double backward and
forward-mode (``jvp``) keep working, as pinned by the reference's gradcheck tests
(tests/test_grad.py of the reference).
"""
from __future__ import annotations

from typing import Any, Optional

import torch
from torch import Tensor
from torch.autograd import Function

from . import ops  # noqa: F401  (registers torch.ops.philtorch_b200.*)

_ops = torch.ops.philtorch_b200


def _prev_states(init: Tensor, out: Tensor) -> Tensor:
    """[y[-1], y[0], ..., y[T-2]] along time: the state each coefficient multiplies."""
    return torch.cat([init.unsqueeze(1), out[:, :-1]], dim=1)


def _none_if_empty(t: Tensor, needed: bool) -> Optional[Tensor]:
    return t if needed else None


class LTIRecurrence(Function):
    """y[t] = a*y[t-1] + x[t] with a of shape (), (1,) or (B,)."""

    @staticmethod
    def forward(a: Tensor, init: Tensor, x: Tensor) -> Tensor:
        return _ops.lti_recur(a, init, x)

    @staticmethod
    def setup_context(ctx: Any, inputs, output) -> None:
        a, init, _ = inputs
        ctx.save_for_backward(a, init, output)
        ctx.save_for_forward(a, init, output)

    @staticmethod
    def backward(ctx: Any, grad_out: Tensor):
        a, init, out = ctx.saved_tensors
        need_a, need_init, need_x = ctx.needs_input_grad
        if not torch.is_grad_enabled():
            ga, gi, gx = _ops.lti_recur_bwd(a, init, out, grad_out, None, need_a, need_init)
            return _none_if_empty(ga, need_a), _none_if_empty(gi, need_init), _none_if_empty(gx, need_x)
        # differentiable form: the adjoint is the same recurrence on the reversed sequence
        g = LTIRecurrence.apply(a, torch.zeros_like(init), grad_out.flip(1)).flip(1)
        grad_a = grad_init = grad_x = None
        if need_init:
            grad_init = g[:, 0] * a
        if need_x:
            grad_x = g
        if need_a:
            prod = _prev_states(init, out) * g
            grad_a = prod.sum(1) if (a.dim() == 1 and a.shape[0] == out.shape[0] and a.shape[0] > 1) \
                else prod.sum().reshape(a.shape)
        return grad_a, grad_init, grad_x

    @staticmethod
    def jvp(ctx: Any, grad_a: Optional[Tensor], grad_init: Optional[Tensor], grad_x: Optional[Tensor]) -> Tensor:
        a, init, out = ctx.saved_tensors
        fwd_init = grad_init if grad_init is not None else torch.zeros_like(init)
        fwd_x = grad_x if grad_x is not None else torch.zeros_like(out)
        if grad_a is not None:
            fwd_x = fwd_x + _prev_states(init, out) * grad_a.reshape(-1, 1)
        return LTIRecurrence.apply(a, fwd_init, fwd_x)


class LPVRecurrence(Function):
    """y[t] = a[t]*y[t-1] + x[t] with a of shape (T,) or (B,T)."""

    @staticmethod
    def forward(a: Tensor, init: Tensor, x: Tensor) -> Tensor:
        return _ops.lpv_recur(a, init, x)

    @staticmethod
    def setup_context(ctx: Any, inputs, output) -> None:
        a, init, _ = inputs
        ctx.save_for_backward(a, init, output)
        ctx.save_for_forward(a, init, output)

    @staticmethod
    def backward(ctx: Any, grad_out: Tensor):
        a, init, out = ctx.saved_tensors
        need_a, need_init, need_x = ctx.needs_input_grad
        if not torch.is_grad_enabled():
            ga, gi, gx = _ops.lpv_recur_bwd(a, init, out, grad_out, None, need_a, need_init)
            return _none_if_empty(ga, need_a), _none_if_empty(gi, need_init), _none_if_empty(gx, need_x)
        # g[t] = a[t+1] g[t+1] + gy[t]: coefficients shifted by one sample, then reversed
        a_rev = torch.roll(a, shifts=-1, dims=-1).flip(-1)
        g = LPVRecurrence.apply(a_rev, torch.zeros_like(init), grad_out.flip(1)).flip(1)
        grad_a = grad_init = grad_x = None
        if need_init:
            grad_init = g[:, 0] * a[..., 0]
        if need_x:
            grad_x = g
        if need_a:
            grad_a = _prev_states(init, out) * g
            if a.dim() == 1:
                grad_a = grad_a.sum(0)
        return grad_a, grad_init, grad_x

    @staticmethod
    def jvp(ctx: Any, grad_a: Optional[Tensor], grad_init: Optional[Tensor], grad_x: Optional[Tensor]) -> Tensor:
        a, init, out = ctx.saved_tensors
        fwd_init = grad_init if grad_init is not None else torch.zeros_like(init)
        fwd_x = grad_x if grad_x is not None else torch.zeros_like(out)
        if grad_a is not None:
            fwd_x = fwd_x + _prev_states(init, out) * grad_a
        return LPVRecurrence.apply(a, fwd_init, fwd_x)
