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

    # forward takes the context itself (no separate setup_context): Function.apply then skips binding
    # the arguments to forward's signature on every call, ~10 us of host time per application
    @staticmethod
    def forward(ctx: Any, a: Tensor, init: Tensor, x: Tensor) -> Tensor:
        output = _ops.lti_recur(a, init, x)
        ctx.save_for_backward(a, init, output)
        ctx.save_for_forward(a, init, output)
        return output

    @staticmethod
    def backward(ctx: Any, grad_out: Tensor):
        a, init, out = ctx.saved_tensors
        need_a, need_init, need_x = ctx.needs_input_grad
        if not torch.is_grad_enabled():
            ga, gi, gx = _ops.lti_recur_bwd(a, init, out, grad_out, None, need_a, need_init, need_x)
            return _none_if_empty(ga, need_a), _none_if_empty(gi, need_init), _none_if_empty(gx, need_x)
        # differentiable form: the adjoint is the same recurrence on the reversed sequence
        # (complex data: on conj(a), with conj(y[t-1]) in the coefficient gradient; .conj() of a real
        # tensor is the tensor itself)
        g = LTIRecurrence.apply(a.conj(), torch.zeros_like(init), grad_out.flip(1)).flip(1)
        grad_a = grad_init = grad_x = None
        if need_init:
            grad_init = g[:, 0] * a.conj()
        if need_x:
            grad_x = g
        if need_a:
            prod = _prev_states(init, out).conj() * g
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


class ReverseLTIRecurrence(Function):
    """g[t] = a*g[t+1] + x[t] with g[T] = end: the first-order recurrence running from the last
    sample to the first, (a, end, x) -> g, without reversing anything in memory: the forward pass
    is the adjoint kernel of ``LTIRecurrence`` and the backward pass its forward kernel.  The
    reference reaches the same result with flip -> recurrence -> flip
    (philtorch/lti/interp.py:41-56, philtorch/lti/filtering.py:413-484)."""

    @staticmethod
    def forward(a: Tensor, end: Tensor, x: Tensor) -> Tensor:
        # the adjoint kernel conjugates its coefficient and takes a*g[T] as the state entering from the right
        _, _, g = _ops.lti_recur_bwd(a.conj(), end, x, x, a * end, False, False)
        return g

    @staticmethod
    def setup_context(ctx: Any, inputs, output) -> None:
        a, end, _ = inputs
        ctx.save_for_backward(a, end, output)

    @staticmethod
    def backward(ctx: Any, grad_out: Tensor):
        a, end, out = ctx.saved_tensors
        need_a, need_end, need_x = ctx.needs_input_grad
        if torch.is_grad_enabled():   # higher-order graph: the same function through LTIRecurrence
            q = LTIRecurrence.apply(a.conj(), torch.zeros_like(end), grad_out)
        else:
            q = _ops.lti_recur(a.conj(), torch.zeros_like(end), grad_out)
        grad_a = grad_end = None
        if need_end:
            grad_end = q[:, -1] * a.conj()
        if need_a:
            prod = torch.cat([out[:, 1:], end.unsqueeze(1)], dim=1).conj() * q
            grad_a = prod.sum(1) if (a.dim() == 1 and a.shape[0] == out.shape[0] and a.shape[0] > 1) \
                else prod.sum().reshape(a.shape)
        return grad_a, grad_end, (q if need_x else None)


class LPVRecurrence(Function):
    """y[t] = a[t]*y[t-1] + x[t] with a of shape (T,) or (B,T)."""

    @staticmethod
    def forward(ctx: Any, a: Tensor, init: Tensor, x: Tensor) -> Tensor:   # context in forward: see LTIRecurrence
        output = _ops.lpv_recur(a, init, x)
        ctx.save_for_backward(a, init, output)
        ctx.save_for_forward(a, init, output)
        return output

    @staticmethod
    def backward(ctx: Any, grad_out: Tensor):
        a, init, out = ctx.saved_tensors
        need_a, need_init, need_x = ctx.needs_input_grad
        if not torch.is_grad_enabled():
            ga, gi, gx = _ops.lpv_recur_bwd(a, init, out, grad_out, None, need_a, need_init, need_x)
            return _none_if_empty(ga, need_a), _none_if_empty(gi, need_init), _none_if_empty(gx, need_x)
        # g[t] = a[t+1] g[t+1] + gy[t]: coefficients shifted by one sample, then reversed
        a_rev = torch.roll(a.conj(), shifts=-1, dims=-1).flip(-1)
        g = LPVRecurrence.apply(a_rev, torch.zeros_like(init), grad_out.flip(1)).flip(1)
        grad_a = grad_init = grad_x = None
        if need_init:
            grad_init = g[:, 0] * a[..., 0].conj()
        if need_x:
            grad_x = g
        if need_a:
            grad_a = _prev_states(init, out).conj() * g
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


def _prev_states2(zi: Tensor, y: Tensor) -> Tensor:
    return torch.cat([zi.unsqueeze(1), y[:, :-1]], dim=1)


def _pad_state0(x: Tensor) -> Tensor:
    """(B,T) -> (B,T,2) with the sequence in state 0 (philtorch/lti/ssm.py:187-191)."""
    return torch.stack([x, torch.zeros_like(x)], dim=-1)


class LTIMatrixRecurrence(Function):
    """h[t] = A h[t-1] + x[t] with A of shape (2,2) or (B,2,2), zi (B,2), x (B,T,2)."""

    @staticmethod
    def forward(A: Tensor, zi: Tensor, x: Tensor) -> Tensor:
        n = x.size(-1)
        if n == 2:
            return _ops.lti_recur2(A, zi, x)
        if n == 1:
            return _ops.lti_recur(A.reshape(A.shape[:-2]), zi[:, 0], x[..., 0]).unsqueeze(-1)
        if n > ops.MAX_STATE_DIM:
            raise NotImplementedError(f"state dimension {n}: the kernels cover 1..{ops.MAX_STATE_DIM}")
        return _ops.lti_recur_n(A, zi, x)

    @staticmethod
    def setup_context(ctx: Any, inputs, output) -> None:
        A, zi, _ = inputs
        ctx.save_for_backward(A, zi, output)
        ctx.save_for_forward(A, zi, output)

    @staticmethod
    def backward(ctx: Any, grad_y: Tensor):
        A, zi, y = ctx.saved_tensors
        need_A, need_zi, need_x = ctx.needs_input_grad
        if not torch.is_grad_enabled() and y.size(-1) == 2:
            gA, gzi, gx = _ops.lti_recur2_bwd(A, zi, y, grad_y, None, False, need_A, need_zi)
            return _none_if_empty(gA, need_A), _none_if_empty(gzi, need_zi), _none_if_empty(gx, need_x)
        if not torch.is_grad_enabled() and y.size(-1) > 2:
            # one reversed scan on the kernels; grad_A is an (n x T)(T x n) product per row
            g, c0 = _ops.recur_n_adj(A, grad_y, None, False)
            gA = None
            if need_A:   # sum_t g[t] (x) h[t-1], read once on the way (no shifted copy, no skinny GEMM)
                gA = _ops.outer_prev_sum(g, y, zi)
                if A.dim() == 2:
                    gA = gA.sum(0)
            return gA, (c0 if need_zi else None), (g if need_x else None)
        AmT = A.mT
        g = LTIMatrixRecurrence.apply(AmT, torch.zeros_like(zi), grad_y.flip(1)).flip(1)
        grad_A = grad_zi = grad_x = None
        if need_zi:
            grad_zi = (AmT @ g[:, 0, :, None]).squeeze(-1)
        if need_x:
            grad_x = g
        if need_A:
            prev = _prev_states2(zi, y)
            grad_A = g.flatten(0, 1).T @ prev.flatten(0, 1) if A.dim() == 2 else g.mT @ prev
        return grad_A, grad_zi, grad_x

    @staticmethod
    def jvp(ctx: Any, grad_A, grad_zi, grad_x) -> Tensor:
        A, zi, y = ctx.saved_tensors
        fwd_zi = grad_zi if grad_zi is not None else torch.zeros_like(zi)
        fwd_x = grad_x if grad_x is not None else torch.zeros_like(y)
        if grad_A is not None:
            prev = _prev_states2(zi, y)
            dA = grad_A if grad_A.dim() == 2 else grad_A.unsqueeze(-3)
            fwd_x = fwd_x + (dA @ prev.unsqueeze(-1)).squeeze(-1)
        return LTIMatrixRecurrence.apply(A, fwd_zi, fwd_x)


class MatrixRecurrence(Function):
    """h[t] = A[t] h[t-1] + x[t] with A of shape (T,2,2) or (B,T,2,2), zi (B,2), x (B,T,2)."""

    @staticmethod
    def forward(A: Tensor, zi: Tensor, x: Tensor) -> Tensor:
        n = x.size(-1)
        if n == 2:
            return _ops.recur2(A, zi, x)
        if n == 1:
            return _ops.lpv_recur(A[..., 0, 0], zi[:, 0], x[..., 0]).unsqueeze(-1)
        if n > ops.MAX_STATE_DIM:
            raise NotImplementedError(f"state dimension {n}: the kernels cover 1..{ops.MAX_STATE_DIM}")
        return _ops.recur_n(A, zi, x)

    @staticmethod
    def setup_context(ctx: Any, inputs, output) -> None:
        A, zi, _ = inputs
        ctx.save_for_backward(A, zi, output)
        ctx.save_for_forward(A, zi, output)

    @staticmethod
    def backward(ctx: Any, grad_y: Tensor):
        A, zi, y = ctx.saved_tensors
        need_A, need_zi, need_x = ctx.needs_input_grad
        if not torch.is_grad_enabled() and y.size(-1) == 2:
            gA, gzi, gx = _ops.recur2_bwd(A, zi, y, grad_y, None, False, need_A, need_zi)
            return _none_if_empty(gA, need_A), _none_if_empty(gzi, need_zi), _none_if_empty(gx, need_x)
        if not torch.is_grad_enabled() and y.size(-1) > 2:
            g, c0 = _ops.recur_n_adj(A, grad_y, None, True)
            gA = None
            if need_A:
                gA = g.unsqueeze(-1) * _prev_states2(zi, y).unsqueeze(-2)
                if A.dim() == 3:
                    gA = gA.sum(0)
            return gA, (c0 if need_zi else None), (g if need_x else None)
        AmT = A.mT
        A_rev = torch.roll(AmT, shifts=-1, dims=-3).flip(-3)
        g = MatrixRecurrence.apply(A_rev, torch.zeros_like(zi), grad_y.flip(1)).flip(1)
        grad_A = grad_zi = grad_x = None
        if need_zi:
            grad_zi = (AmT[..., 0, :, :] @ g[:, 0, :, None]).squeeze(-1)
        if need_x:
            grad_x = g
        if need_A:
            prev = _prev_states2(zi, y)
            grad_A = g.unsqueeze(-1) * prev.unsqueeze(-2)
            if A.dim() == 3:
                grad_A = grad_A.sum(0)
        return grad_A, grad_zi, grad_x

    @staticmethod
    def jvp(ctx: Any, grad_A, grad_zi, grad_x) -> Tensor:
        A, zi, y = ctx.saved_tensors
        fwd_zi = grad_zi if grad_zi is not None else torch.zeros_like(zi)
        fwd_x = grad_x if grad_x is not None else torch.zeros_like(y)
        if grad_A is not None:
            prev = _prev_states2(zi, y)
            fwd_x = fwd_x + (grad_A @ prev.unsqueeze(-1)).squeeze(-1)
        return MatrixRecurrence.apply(A, fwd_zi, fwd_x)


class _ScalarInputMatrixRecurrence(Function):
    """2x2 recurrence driven by a scalar sequence x (B,T) into state 0; ``lpv`` selects per-sample
    coefficients.  Same result as zero-padding x to (B,T,2) (philtorch/lti/ssm.py:187-191,
    philtorch/lpv/ssm.py:197-201) without materialising the padded tensor or its gradient."""

    @staticmethod
    def forward(A: Tensor, zi: Tensor, x: Tensor, lpv: bool) -> Tensor:
        return _ops.recur2_sx(A, zi, x) if lpv else _ops.lti_recur2_sx(A, zi, x)

    @staticmethod
    def setup_context(ctx: Any, inputs, output) -> None:
        A, zi, _, lpv = inputs
        ctx.lpv = lpv
        ctx.save_for_backward(A, zi, output)

    @staticmethod
    def backward(ctx: Any, grad_y: Tensor):
        A, zi, y = ctx.saved_tensors
        need_A, need_zi, need_x, _ = ctx.needs_input_grad
        if not torch.is_grad_enabled():
            op = _ops.recur2_bwd if ctx.lpv else _ops.lti_recur2_bwd
            gA, gzi, gx = op(A, zi, y, grad_y, None, True, need_A, need_zi)
            return _none_if_empty(gA, need_A), _none_if_empty(gzi, need_zi), _none_if_empty(gx, need_x), None
        raise RuntimeError("double backward through the scalar-input fast path is not supported; "
                           "pass x with shape (B, T, 2)")


def matrix_recurrence_scalar_input(A: Tensor, zi: Tensor, x: Tensor, lpv: bool) -> Tensor:
    """2x2 recurrence fed by a scalar sequence (B,T) through the fused scalar-input kernels."""
    return _ScalarInputMatrixRecurrence.apply(A, zi, x, lpv)


def _defined(*pairs):
    """(outputs, their gradients) without the pairs whose gradient is undefined."""
    kept = [(o, g) for o, g in pairs if g is not None]
    return [o for o, _ in kept], [g for _, g in kept]


class BiquadTDF2(Function):
    """One transposed-direct-form-II second-order section, (b, a, zi, x) -> (y, zf)."""

    @staticmethod
    def forward(b: Tensor, a: Tensor, zi: Optional[Tensor], x: Tensor):
        return _ops.biquad_tdf2(b, a, zi, x)

    @staticmethod
    def setup_context(ctx: Any, inputs, output) -> None:
        b, a, zi, x = inputs
        y, _ = output
        ctx.has_zi = zi is not None
        ctx.set_materialize_grads(False)   # an unused zf arrives as None, not as a zero tensor to fill and read
        ctx.save_for_backward(b, a, x, y, *([zi] if zi is not None else []))

    @staticmethod
    def backward(ctx: Any, grad_y: Tensor, grad_zf: Tensor):
        b, a, x, y, *rest = ctx.saved_tensors
        need_b, need_a, need_zi, need_x = ctx.needs_input_grad
        need_zi = need_zi and ctx.has_zi
        if torch.is_grad_enabled():
            # higher-order graph: recompute through the differentiable state-space form
            zi = rest[0] if rest else None
            with torch.enable_grad():
                y2, zf2 = _biquad_reference_form(b, a, zi, x)
                ins = [t for t, n in ((b, need_b), (a, need_a), (zi, need_zi), (x, need_x)) if n]
                outs, gouts = _defined((y2, grad_y), (zf2, grad_zf))
                gs = list(torch.autograd.grad(outs, ins, gouts, create_graph=True, allow_unused=True))
            out = []
            for n in (need_b, need_a, need_zi, need_x):
                out.append(gs.pop(0) if n else None)
            return tuple(out)
        if grad_y is None:
            grad_y = torch.zeros_like(x)
        gb, ga, gzi, gx = _ops.biquad_tdf2_bwd(b, a, x, y, grad_y, grad_zf, need_b or need_a, need_zi)
        return (_none_if_empty(gb, need_b), _none_if_empty(ga, need_a), _none_if_empty(gzi, need_zi),
                _none_if_empty(gx, need_x))


def modal_mix_reference(w: Tensor, w0: Tensor, coef: Tensor, real_out: bool) -> Tensor:
    """``ModalMix`` in plain torch operations (the differentiable form behind higher-order graphs)."""
    prev = torch.cat([w0.unsqueeze(-1), w[:, :, :-1]], dim=2)
    y = (coef.unsqueeze(-1) * prev).sum(1)
    return y.real if real_out else y


class ModalMix(Function):
    """y[r,t] = sum_m coef[(r,)m] * w[r,m,t-1] with w[r,m,-1] = w0[r,m], optionally its real part:
    the output map of ``diag_state_space`` (mode sum, one-sample shift, real part) in one pass."""

    @staticmethod
    def forward(ctx: Any, w: Tensor, w0: Tensor, coef: Tensor, real_out: bool) -> Tensor:
        ctx.real_out = real_out
        ctx.save_for_backward(w, w0, coef)
        return _ops.modal_mix(w, w0, coef, real_out)

    @staticmethod
    def backward(ctx: Any, grad_y: Tensor):
        w, w0, coef = ctx.saved_tensors
        need_w, need_w0, need_coef = ctx.needs_input_grad[:3]
        if torch.is_grad_enabled():
            with torch.enable_grad():
                ins = [t.detach().requires_grad_() for t in (w, w0, coef)]
                gs = torch.autograd.grad(modal_mix_reference(*ins, ctx.real_out), ins, grad_y, create_graph=True)
            return gs[0] if need_w else None, gs[1] if need_w0 else None, gs[2] if need_coef else None, None
        gw, gw0, gc = _ops.modal_mix_bwd(w, w0, coef, grad_y, ctx.real_out, need_coef)
        return gw if need_w else None, gw0 if need_w0 else None, _none_if_empty(gc, need_coef), None


class ModalDrive(Function):
    """u[r,m,t] = gain[(r,)m] * x[r,t]: a real signal broadcast into M complex modes (the input map
    of ``diag_state_space`` for a scalar input).  The backward pass is one ``modal_mix`` launch
    (the mode sum with conj(gain), no delay) instead of a complex product and a strided reduction."""

    @staticmethod
    def forward(ctx: Any, x: Tensor, gain: Tensor) -> Tensor:
        ctx.save_for_backward(x, gain)
        if x.is_cuda and not x.is_complex() and gain.is_complex() and gain.real.dtype == x.dtype:
            return _ops.modal_drive(x, gain)
        return gain.unsqueeze(-1) * x.unsqueeze(1)

    @staticmethod
    def backward(ctx: Any, grad_u: Tensor):
        x, gain = ctx.saved_tensors
        need_x, need_gain = ctx.needs_input_grad
        if torch.is_grad_enabled():
            with torch.enable_grad():
                ins = [x.detach().requires_grad_(), gain.detach().requires_grad_()]
                gs = torch.autograd.grad(ins[1].unsqueeze(-1) * ins[0].unsqueeze(1), ins, grad_u, create_graph=True)
            return gs[0] if need_x else None, gs[1] if need_gain else None
        gx = _ops.modal_mix(grad_u, None, gain.conj(), not x.is_complex()).to(x.dtype) if need_x else None
        ggain = None
        if need_gain:
            ggain = (grad_u * x.conj().unsqueeze(1)).sum(-1)
            if gain.dim() == 1:
                ggain = ggain.sum(0)
        return gx, ggain


class ModalBank(Function):
    """A real signal through M complex first-order modes and back into one real output, fused:
    ``(x, lam, gain, coef, d, w0) -> (y, wf)`` with x (rows, N) real, lam / gain / coef / w0 (rows, M)
    complex, d (rows,) real or None;  w_m[t] = lam_m w_m[t-1] + gain_m x[t],
    y[t] = Re(sum_m coef_m w_m[t-1]) + d x[t], wf = w[:, :, N-1].  The scalar-in / real-scalar-out case
    of ``diag_state_space`` without ever forming the (rows, M, N) mode signals.  First derivatives."""

    @staticmethod
    def forward(ctx: Any, x: Tensor, lam: Tensor, gain: Tensor, coef: Tensor, d: Optional[Tensor], w0: Tensor):
        y, wf, chk = _ops.modal_bank(x, lam, gain, coef, d, w0)
        ctx.has_d = d is not None
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(x, lam, gain, coef, chk, *([d] if d is not None else []))
        return y, wf

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx: Any, grad_y: Tensor, grad_wf: Tensor):
        x, lam, gain, coef, chk, *rest = ctx.saved_tensors
        d = rest[0] if rest else None
        if grad_y is None:
            grad_y = torch.zeros_like(x)
        need = ctx.needs_input_grad
        mask = (1 if need[2] else 0) | (2 if need[1] else 0) | (4 if need[3] else 0)
        gx, glam, ggain, gcoef, gd, gw0 = _ops.modal_bank_bwd(x, lam, gain, coef, d, chk, grad_y, grad_wf, mask)
        return (gx if need[0] else None, glam if need[1] else None, ggain if need[2] else None,
                gcoef if need[3] else None, gd if (ctx.has_d and need[4]) else None, gw0 if need[5] else None)


class CombFilter(Function):
    """y[t] = x[t] - a*y[t-delay] on the signal's own layout, (a, zi, x, delay) -> y; zi: None, (delay,)
    or (B, delay) in the reference's order (zi[..., k] = the output k+1 samples before the start)."""

    @staticmethod
    def forward(ctx: Any, a: Tensor, zi: Optional[Tensor], x: Tensor, delay: int) -> Tensor:
        y = _ops.comb(a, zi, x, delay)
        ctx.delay, ctx.has_zi = delay, zi is not None
        ctx.save_for_backward(a, y, *([zi] if zi is not None else []))
        return y

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx: Any, grad_y: Tensor):
        a, y, *rest = ctx.saved_tensors
        zi = rest[0] if rest else None
        need_a, need_zi, need_x = ctx.needs_input_grad[:3]
        need_zi = need_zi and ctx.has_zi
        ga, gzi, gx = _ops.comb_bwd(a, zi, y, grad_y, ctx.delay, need_a, need_zi)
        return _none_if_empty(ga, need_a), _none_if_empty(gzi, need_zi), _none_if_empty(gx, need_x), None


class SOSCascade(Function):
    """K second-order sections (TDF-II) in one fused pass, (b, a, zi, x) -> (y, zf) with b (K,3) or
    (K,B,3), a (K,2) or (K,B,2), zi/zf (K,B,2).  Same results as K chained ``BiquadTDF2`` calls
    (the reference chains ``lfilter`` calls, philtorch/lti/filtering.py:304-317)."""

    @staticmethod
    def forward(ctx: Any, b: Tensor, a: Tensor, zi: Optional[Tensor], x: Tensor):
        need_coef = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
        y, mid, zf = _ops.sos_cascade(b, a, zi, x, need_coef)
        ctx.has_zi = zi is not None
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(b, a, x, mid, y, *([zi] if zi is not None else []))
        return y, zf

    @staticmethod
    def backward(ctx: Any, grad_y: Tensor, grad_zf: Tensor):
        b, a, x, mid, y, *rest = ctx.saved_tensors
        need_b, need_a, need_zi, need_x = ctx.needs_input_grad
        need_zi = need_zi and ctx.has_zi
        if torch.is_grad_enabled():
            # higher-order graph: recompute as a chain of differentiable single sections
            zi = rest[0] if rest else None
            with torch.enable_grad():
                u, zfs = x, []
                for k in range(b.shape[0]):
                    u, zf_k = BiquadTDF2.apply(b[k], a[k], None if zi is None else zi[k], u)
                    zfs.append(zf_k)
                ins = [t for t, n in ((b, need_b), (a, need_a), (zi, need_zi), (x, need_x)) if n]
                outs, gouts = _defined((u, grad_y), (torch.stack(zfs), grad_zf))
                gs = list(torch.autograd.grad(outs, ins, gouts, create_graph=True, allow_unused=True))
            out = []
            for n in (need_b, need_a, need_zi, need_x):
                out.append(gs.pop(0) if n else None)
            return tuple(out)
        if grad_y is None:
            grad_y = torch.zeros_like(x)
        gb, ga, gzi, gx = _ops.sos_cascade_bwd(b, a, x, mid, y, grad_y, grad_zf, need_b or need_a, need_zi)
        return (_none_if_empty(gb, need_b), _none_if_empty(ga, need_a), _none_if_empty(gzi, need_zi),
                _none_if_empty(gx, need_x))


class LPVBiquad(Function):
    """Time-varying second-order filter, fused: (b, a, zi, x, form) -> (y, zf) with per-sample
    b (N,3) | (B,N,3) and a (N,2) | (B,N,2), form 'df2' or 'tdf2'; philtorch.lpv.lfilter for orders
    <= 2 (philtorch/lpv/filtering.py:288-326).  First derivatives only."""

    @staticmethod
    def forward(ctx: Any, b: Tensor, a: Tensor, zi: Optional[Tensor], x: Tensor, form: str):
        need = any(ctx.needs_input_grad)
        fwd = _ops.lpv_biquad_df2 if form == "df2" else _ops.lpv_biquad_tdf2
        y, hp, zf = fwd(b, a, zi, x, need)
        ctx.has_zi = zi is not None
        ctx.form = form
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(b, a, x, hp)
        return y, zf

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx: Any, grad_y: Tensor, grad_zf: Tensor):
        b, a, x, hp = ctx.saved_tensors
        need_b, need_a, need_zi, need_x = ctx.needs_input_grad[:4]
        need_zi = need_zi and ctx.has_zi
        if grad_y is None:
            grad_y = torch.zeros_like(x)
        bwd = _ops.lpv_biquad_df2_bwd if ctx.form == "df2" else _ops.lpv_biquad_tdf2_bwd
        gb, ga, gzi, gx = bwd(b, a, x, hp, grad_y, grad_zf, need_zi)
        if b.dim() == 2:   # coefficients shared by the rows
            gb, ga = gb.sum(0), ga.sum(0)
        return (gb if need_b else None, ga if need_a else None, _none_if_empty(gzi, need_zi),
                gx if need_x else None, None)


def _biquad_reference_form(b: Tensor, a: Tensor, zi: Optional[Tensor], x: Tensor):
    """The same section written with differentiable pieces (2x2 recurrence + elementwise glue),
    following philtorch/lti/filtering.py:304-317 and philtorch/lti/ssm.py:466-504."""
    B = x.shape[0]
    a1, a2 = a[..., 0], a[..., 1]
    zero, one = torch.zeros_like(a1), torch.ones_like(a1)
    At = torch.stack([torch.stack([-a1, one], -1), torch.stack([-a2, zero], -1)], -2)
    Bv = b[..., 1:] - b[..., :1] * a
    if zi is None:
        zi = x.new_zeros(B, 2)
    Bx = x.unsqueeze(-1) * (Bv if Bv.dim() == 1 else Bv.unsqueeze(1))
    h = LTIMatrixRecurrence.apply(At, zi, Bx)
    h0 = torch.cat([zi[:, None, 0], h[:, :-1, 0]], dim=1)
    b0 = b[..., 0]
    y = h0 + (b0 if b0.dim() == 0 else b0.unsqueeze(1)) * x
    return y, h[:, -1, :]
