"""Time-invariant state-space front-end on the GPU kernels (state dimensions 1 to 8).

Public names and argument conventions follow philtorch/lti/ssm.py of the reference:
``state_space_recursion`` (:198-383 there, pure PyTorch) and ``state_space`` (:386-510).  Every
call runs the compiled kernels; ``unroll_factor`` is accepted for compatibility (the reference
only reaches its extension when it is 1) and ignored.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from ..autograd import (LTIMatrixRecurrence, LTIRecurrence, ModalBank, ModalDrive, ModalMix,
                        matrix_recurrence_scalar_input)
from ..ops import MODAL_BANK_MAX_MODES

# scalar-input / real-scalar-output models of up to eight modes take the fused kernels (first
# derivatives only); False: always the composite route (mode signals in memory, any order of derivative)
FUSED_MODAL_BANK = True

__all__ = ["LTIMatrixRecurrence", "state_space_recursion", "state_space", "diag_state_space",
           "extension_backend_indicator"]


def extension_backend_indicator(x: Tensor, M: int) -> bool:
    """True when the compiled kernels handle this input (CUDA, fp32/fp64, state dimension <= 8)."""
    return x.is_cuda and 1 <= M <= 8 and x.dtype in (torch.float32, torch.float64)


def _ext_ss_recur(A: Tensor, zi: Tensor, x: Tensor, *, out_idx: Optional[int] = None, **_) -> Tensor:
    """Counterpart of philtorch/lti/ssm.py:162-195: run the recurrence on the kernels."""
    M = A.size(-1)
    if M == 1:
        xs = x if x.dim() == 2 else x.squeeze(-1)
        y = LTIRecurrence.apply(A[..., 0, 0], zi.squeeze(-1), xs).unsqueeze(-1)
    elif M == 2:
        if x.dim() == 2:
            y = matrix_recurrence_scalar_input(A, zi, x, False)
        else:
            y = LTIMatrixRecurrence.apply(A, zi, x)
    else:
        if x.dim() == 2:   # the sequence feeds state 0 (zero-padded, as the reference does before its op)
            x = torch.cat([x.unsqueeze(-1), x.new_zeros(x.shape + (M - 1,))], dim=-1)
        y = LTIMatrixRecurrence.apply(A, zi, x)   # dense N x N kernels, M <= 8
    if out_idx is not None and y.dim() == 3:
        y = y[:, :, out_idx]
    return y


def state_space_recursion(A: Tensor, zi: Tensor, x: Tensor, *, unroll_factor: int = 1,
                          out_idx: Optional[int] = None) -> Tensor:
    """State evolution ``h[t] = A h[t-1] + x[t]`` of a time-invariant model.

    Args:
        A: (M, M) or (B, M, M), M in {1, 2}.
        zi: (B, M) initial states.
        x: (B, T, M), or (B, T) feeding state 0 only.
        unroll_factor: validated (>= 1), otherwise unused.
        out_idx: return only this state.

    Returns:
        (B, T, M), or (B, T) with ``out_idx``.
    """
    assert x.dim() in (2, 3), f"Input signal must be 2D or 3D (batch, time, [features]), got {x.shape}"
    assert A.dim() in (2, 3), f"State matrix A must be 2D or 3D, got {A.shape}"
    assert A.size(-2) == A.size(-1), f"State matrix A must be square, got {A.shape}"
    if A.dim() == 3:
        assert x.size(0) == A.size(0), \
            f"Batch size of A must match batch size of x, got A: {A.size(0)}, x: {x.size(0)}"
    if x.dim() == 3:
        assert A.size(-1) == x.size(-1), \
            f"Last dimension of A must match last dimension of x, got A: {A.size(-1)}, x: {x.size(-1)}"
    batch_size, M = x.size(0), A.size(-1)
    assert zi.dim() == 2, f"Initial conditions zi must be 2D, got {zi.shape}"
    assert zi.size(0) == batch_size, \
        f"Batch size of zi must match batch size of x, got zi: {zi.size(0)}, x: {batch_size}"
    assert zi.size(1) == M, f"Last dimension of zi must match last dimension of A, got zi: {zi.size(1)}, A: {M}"
    if unroll_factor < 1:
        raise ValueError("Unroll factor must be >= 1")
    return _ext_ss_recur(A, zi, x, out_idx=out_idx)


def _input_map(x: Tensor, Bm: Optional[Tensor], batch_size: int, M: int) -> Tensor:
    """B x for the shapes the filter front-ends use (philtorch/lti/ssm.py:466-485)."""
    if Bm is None:
        return x
    features = -1 if x.dim() == 2 else x.size(-1)
    shp = tuple(Bm.shape)
    if shp == (M,):
        assert x.dim() == 2, f"Input signal x must be 2D when B is of shape {(M,)}, got {x.shape}"
        return x.unsqueeze(-1) * Bm
    if shp == (batch_size, M):
        assert x.dim() == 2, f"Input signal x must be 2D when B is of shape {(batch_size, M)}, got {x.shape}"
        return x.unsqueeze(-1) * Bm.unsqueeze(1)
    if shp == (M, features):
        return x @ Bm.T
    if shp == (batch_size, M, features):
        return torch.linalg.vecdot(Bm.unsqueeze(1).conj(), x.unsqueeze(-2))
    raise ValueError(f"Input matrix B must be of shape ({M},), ({batch_size}, {M}), ({M}, {features}) or "
                     f"({batch_size}, {M}, {features}), got {shp}")


def _output_map(h: Tensor, x: Tensor, C: Optional[Tensor], D: Optional[Tensor], batch_size: int, M: int) -> Tensor:
    """C h + D x for the shapes the filter front-ends use (philtorch/lti/ssm.py:513-589)."""
    Dx = None
    if D is not None:
        shp = tuple(D.shape)
        if shp in ((), (1,)):
            Dx = x * D
        elif shp == (batch_size,):
            assert x.dim() == 2, f"Input signal x must be 2D when D is of shape ({batch_size},), got {x.shape}"
            Dx = D.unsqueeze(1) * x
        elif x.dim() == 3 and shp == (x.size(-1),):
            Dx = x @ D
        else:
            raise ValueError(f"Feedthrough D must be a scalar, ({batch_size},) or (features,), got {shp}")
    if C is not None:
        shp = tuple(C.shape)
        if shp == (M,):
            Ch = h @ C
        elif shp == (batch_size, M):
            Ch = torch.linalg.vecdot(C.unsqueeze(1).conj(), h)
        elif len(shp) == 2 and shp[1] == M:
            Ch = h @ C.T
        elif len(shp) == 3 and shp[0] == batch_size and shp[2] == M:
            Ch = h @ C.mT
        else:
            raise ValueError(f"Output matrix C must be of shape ({M},), ({batch_size}, {M}), (_, {M}) or "
                             f"({batch_size}, _, {M}), got {shp}")
    else:
        Ch = h
    return Ch if Dx is None else Ch + Dx


def state_space(A: Tensor, x: Tensor, B: Optional[Tensor] = None, C: Optional[Tensor] = None,
                D: Optional[Tensor] = None, zi: Optional[Tensor] = None, unroll_factor: Optional[int] = None,
                out_idx: Optional[int] = None):
    """Discrete time-invariant state-space model

        h[t+1] = A h[t] + B x[t],   y[t] = C h[t] + D x[t]

    with the calling convention of philtorch/lti/ssm.py:386-510: returns ``y``, or ``(y, zf)``
    when ``zi`` is given.  ``unroll_factor`` is accepted and ignored.
    """
    assert x.dim() in (2, 3), f"Input signal must be 2D or 3D (batch, time, [features]), got {x.shape}"
    assert A.dim() in (2, 3), f"State matrix A must be 2D or 3D, got {A.shape}"
    assert A.size(-2) == A.size(-1), f"State matrix A must be square, got {A.shape}"
    if A.dim() == 3:
        assert x.size(0) == A.size(0), \
            f"Batch size of A must match batch size of x, got A: {A.size(0)}, x: {x.size(0)}"
    if not (C is None or out_idx is None):
        raise ValueError("C and out_idx cannot be used together. Use either C or out_idx.")
    batch_size, M = x.shape[0], A.size(-1)
    return_zf = zi is not None
    if zi is None:
        zi = x.new_zeros(batch_size, M)
    elif zi.dim() == 1:
        zi = zi.unsqueeze(0).expand(batch_size, -1)
    Bx = _input_map(x, B, batch_size, M)
    if return_zf or out_idx is None:
        h = _ext_ss_recur(A, zi, Bx)
        zf = h[:, -1, :] if return_zf else None
        if out_idx is None:
            h = torch.cat([zi.unsqueeze(1), h[:, :-1]], dim=1)
        else:
            h = torch.cat([zi[:, None, out_idx], h[:, :-1, out_idx]], dim=1)
    else:
        zf = None
        h = _ext_ss_recur(A, zi, Bx, out_idx=out_idx)
        h = torch.cat([zi[:, None, out_idx], h[:, :-1]], dim=1)
    y = _output_map(h, x, C, D, batch_size, M)
    return (y, zf) if return_zf else y


def _eigen_basis(L: Optional[Tensor], V: Optional[Tensor], Vinv: Optional[Tensor], A: Optional[Tensor],
                 x: Tensor, batch_size: int):
    """Eigenvalues (M,) | (batch, M), eigenvectors and their inverse, M -- with the argument
    contract of philtorch/lti/ssm.py:640-721."""
    if L is None:
        assert A is not None, "Either L or A must be provided"
        assert A.dim() in (2, 3), f"State matrix A must be 2D or 3D, got {A.shape}"
        assert A.size(-2) == A.size(-1), f"State matrix A must be square, got {A.shape}"
        if A.dim() == 3:
            assert x.size(0) == A.size(0), \
                f"Batch size of A must match batch size of x, got A: {A.size(0)}, x: {x.size(0)}"
        L, V = torch.linalg.eig(A)
        return L, V, torch.linalg.inv(V), A.size(-1)
    if L.dim() == 1:
        M, nd, lead = L.size(0), 2, ()
    elif L.dim() == 2 and L.size(0) == batch_size:
        M, nd, lead = L.size(1), 3, (batch_size,)
        assert not (V is None and Vinv is None), "P and Vinv cannot both be None when L is a batch of vectors"
    else:
        raise ValueError(f"L must be a vector or a batch of vectors, got {L.shape}")
    for name, mat in (("P", V), ("Vinv", Vinv), ("A", A)):
        if mat is not None:
            assert mat.dim() == nd, f"{name} must be {nd}D, got {mat.shape}"
            assert tuple(mat.shape) == lead + (M, M), f"{name} must be square with size {M}, got {mat.shape}"
    if V is None and Vinv is None:
        if A is None:      # scalar modes: the states are the modes themselves
            V = Vinv = torch.eye(M, device=x.device, dtype=x.dtype)
        elif M == 1:
            V = Vinv = torch.ones(lead + (1, 1), device=x.device, dtype=L.dtype)
        else:              # eigenvectors of A for the given eigenvalues: null vectors of A - l I
            # (columns scaled to a unit first entry; V V^-1 cancels any scaling)
            eye = torch.eye(M, device=A.device, dtype=L.dtype)
            shifted = A.to(L.dtype).unsqueeze(-3) - L[..., None, None] * eye          # (..., M, M, M)
            rest = torch.linalg.lstsq(shifted[..., 1:], -shifted[..., :1]).solution    # (..., M, M-1, 1)
            V = torch.cat([torch.ones_like(rest[..., :1, 0]), rest[..., 0]], dim=-1).mT
            Vinv = torch.linalg.inv(V)
    elif V is None:
        V = torch.linalg.inv_ex(Vinv).inverse
    elif Vinv is None:
        # inv_ex: no error check, hence no device synchronisation per call (a singular V gives
        # non-finite outputs where torch.linalg.inv, which the reference calls, raises)
        Vinv = torch.linalg.inv_ex(V).inverse
    return L, V, Vinv, M


def diag_state_space(x: Tensor, L: Optional[Tensor] = None, V: Optional[Tensor] = None,
                     Vinv: Optional[Tensor] = None, A: Optional[Tensor] = None, B: Optional[Tensor] = None,
                     C: Optional[Tensor] = None, D: Optional[Tensor] = None, zi: Optional[Tensor] = None,
                     out_idx: Optional[int] = None, unroll_factor: Optional[int] = None):
    """State-space model evaluated in the eigenbasis ``A = V diag(L) V^-1`` (signature and argument
    contract of philtorch/lti/ssm.py:590-850).

    In that basis the M states are independent first-order recurrences with the (in general
    complex) poles ``L``: ``batch * M`` rows of the first-order time-invariant kernel, complex64 /
    complex128 when the poles are.  Input and output maps are folded into the basis first
    (``V^-1 B`` before, ``C V`` after the recurrence), so nothing of size (batch, N, M) is formed
    unless the states themselves are the result.  Returns ``y``, or ``(y, zf)`` when ``zi`` is given.
    ``unroll_factor`` is accepted for compatibility and ignored.
    """
    assert x.dim() in (2, 3), f"Input signal must be 2D or 3D (batch, time, [features]), got {x.shape}"
    if not (C is None or out_idx is None):
        raise ValueError("C and out_idx cannot be used together. Use either C or out_idx.")
    batch_size, N = x.size(0), x.size(1)
    L, V, Vinv, M = _eigen_basis(L, V, Vinv, A, x, batch_size)
    return_zf = zi is not None
    if zi is None:
        zi = x.new_zeros(batch_size, M)
    elif zi.dim() == 1:
        zi = zi.unsqueeze(0).expand(batch_size, -1)
    cdt = torch.promote_types(torch.promote_types(L.dtype, Vinv.dtype), x.dtype)   # complex as soon as the basis is
    Lc, Vc, Vic, zc = L.to(cdt), V.to(cdt), Vinv.to(cdt), zi.to(cdt)

    # ---- into the eigenbasis: w0 = V^-1 zi, u[b, m, t] = (V^-1 B x[b, t])[m]
    w0 = (Vic @ zc.unsqueeze(-1)).squeeze(-1)                                   # (batch, M)
    if B is None:
        G = Vic[..., 0] if x.dim() == 2 else Vic        # the input enters state 0 / x carries M features
    else:
        Bc = B.to(cdt)
        shp = tuple(B.shape)
        if shp == (M,):
            G = Vic @ Bc                                 # (M,) | (batch, M)
        elif shp == (batch_size, M):
            assert x.dim() == 2, f"Input signal x must be 2D when B is of shape {(batch_size, M)}, got {x.shape}"
            G = (Vic @ Bc.unsqueeze(-1)).squeeze(-1)     # (batch, M)
        elif B.dim() in (2, 3) and shp[-2] == M:
            G = Vic @ Bc                                 # (M, features) | (batch, M, features)
        else:
            features = -1 if x.dim() == 2 else x.size(-1)
            raise ValueError(f"Input matrix B must be of shape ({M},), ({batch_size}, {M}), ({M}, {features}) or "
                             f"({batch_size}, {M}, {features}), got {shp}")
    if (FUSED_MODAL_BANK and x.dim() == 2 and x.is_cuda and x.dtype in (torch.float32, torch.float64)
            and M <= MODAL_BANK_MAX_MODES and cdt == (torch.complex64 if x.dtype == torch.float32 else torch.complex128)
            and tuple(G.shape) in ((M,), (batch_size, M)) and out_idx is None
            and C is not None and not C.is_complex() and tuple(C.shape) in ((M,), (batch_size, M))
            and (D is None or (not D.is_complex() and tuple(D.shape) in ((), (1,), (batch_size,))))):
        # scalar in, real scalar out: ONE fused pass per direction over x / y; the (batch, M, N) modes
        # are never formed (csrc/modal_bank.cuh)
        Cc = C.to(cdt)
        CV = Cc @ Vc if C.dim() == 1 else (Cc.unsqueeze(1) @ Vc).squeeze(1)
        d = None if D is None else D.to(x.dtype).reshape(-1).expand(batch_size)
        y, wf = ModalBank.apply(x, Lc.expand(batch_size, M), G.to(cdt).expand(batch_size, M),
                                CV.expand(batch_size, M), d, w0)
        if return_zf:
            return y, (Vc @ wf.unsqueeze(-1)).squeeze(-1).real
        return y
    if x.dim() == 2 and tuple(G.shape) in ((M,), (batch_size, M)) and G.is_complex():
        u = ModalDrive.apply(x, G)                       # (batch, M, N) without a transpose
    elif x.dim() == 2 and tuple(G.shape) in ((M,), (batch_size, M)):
        u = G.unsqueeze(-1) * x.to(cdt).unsqueeze(1)
    else:
        u = _input_map(x.to(cdt), G, batch_size, M).mT
    u = u.expand(batch_size, M, N).reshape(batch_size * M, N)
    poles = Lc.expand(batch_size, M).reshape(-1)
    w = LTIRecurrence.apply(poles, w0.reshape(-1).contiguous(), u).view(batch_size, M, N)

    # ---- back: the state BEFORE sample t is h[t] = V [w0, w[0], ..., w[N-2]][t].  An output map is
    # folded into the basis (C V) and applied to the modes directly; the one-sample shift then
    # happens on the (smaller) output instead of on the (batch, M, N) modes.
    real_out = C is not None and not C.is_complex()
    zf = None
    if return_zf:
        zf = (Vc @ w[:, :, -1:]).squeeze(-1)
        zf = zf.real if real_out else zf
    if C is None and out_idx is None:
        w_prev = torch.cat([w0.unsqueeze(-1), w[:, :, :-1]], dim=2)             # (batch, M, N)
        return_y = _output_map((Vc @ w_prev).mT, x, None, D, batch_size, M)     # all states, (batch, N, M)
        return (return_y, zf) if return_zf else return_y
    if out_idx is not None:
        CV = Vc[..., out_idx, :]                                                # (M,) | (batch, M)
    else:
        shp = tuple(C.shape)
        Cc = C.to(cdt)
        if shp == (M,):
            CV = Cc @ Vc
        elif shp == (batch_size, M):
            CV = (Cc.unsqueeze(1) @ Vc).squeeze(1)
        elif (len(shp) == 2 and shp[1] == M) or (len(shp) == 3 and shp[0] == batch_size and shp[2] == M):
            CV = Cc @ Vc                                                        # (K, M) | (batch, K, M)
        else:
            raise ValueError(f"Output matrix C must be of shape ({M},), ({batch_size}, {M}), (_, {M}) or "
                             f"({batch_size}, _, {M}), got {shp}")
    vector_out = out_idx is None and C.dim() >= 2 and tuple(C.shape) != (batch_size, M)
    if vector_out:
        after = (CV @ w).mT                                                     # (batch, N, K)
        first = (CV @ w0.unsqueeze(-1)).squeeze(-1).expand(batch_size, -1)      # (batch, K)
        h = torch.cat([first.unsqueeze(1), after[:, :-1]], dim=1)
        if real_out:
            h = h.real
    else:                                                                       # one pass: mode sum, shift, real part
        h = ModalMix.apply(w, w0, CV.contiguous(), real_out)
    y = _output_map(h, x, None, D, batch_size, M)
    return (y, zf) if return_zf else y
