"""First-order per-sample-coefficient recurrence with the TIME axis split across devices.

The reference has no multi-device code; this mode exists for rows too long for one GPU
(e.g. B = 8, T = 2^28).  Rank r of W owns the contiguous samples [r T/W, (r+1) T/W) of every row.

Forward, per rank
  (1) ONE pass over the shard: the scan started from a zero state, y0, together with the shard's
      total affine map (P_r, e_r) = (product of a, y0's last sample);
  (2) ONE all-gather of the (B, 2) maps; every rank folds the maps of the ranks before it into its
      true incoming state  s_r = P_{r-1} s_{r-1} + e_{r-1}  (s_0 = zi);
  (3) fix-up  y[t] = y0[t] + (prod_{u<=t} a[u]) s_r, ONE kernel launch (``ptb_lpv_recur_fixup_fwd``)
      that also does the fold of step (2) on the device.  The running correction normally
      underflows to exactly zero after a few thousand samples (|a| < 1) and stays zero from there
      on, so every row is corrected block by block from its start and the walk stops, per row, at
      the first block that the correction enters as exactly 0.0.  If the products never vanish the
      walk covers the whole shard: still exact.  No device->host read anywhere on the path.
Backward mirrors it from the right: the local adjoint scan with a zero incoming state, one
all-gather of (P_r, adjoint end state), and a fix-up of grad_x / grad_a over a suffix.

The collectives are tiny (W x B x 2 scalars) and latency-bound; everything else is local, so a
rank moves the same 12 + 20 bytes per sample as an unsharded run.

Segments.  A handful of long rows is the kernels' worst case: tiles of one row depend on one
another, so with B = 8 the single-pass scan runs at ~0.7 of the memory bandwidth.  The same
algebra fixes that inside a rank: the local shard is cut into S segments per row, which the
kernels see as B*S independent rows (a reshape, no copy); the segments' maps are folded exactly
like the ranks' maps, and the fix-up runs over all segments at once.  S is chosen so that
B*S >= 256 rows of at least 2^20 samples (``segments=None``) or given; S = 1 is the plain algorithm.  Without an
initialised process group the function runs as a single rank, so it also serves one GPU.
The fold over the segments happens inside the fix-up kernel (each (row, segment) CTA folds the at
most W-1 + S-1 maps before it from shared memory), so a direction is: scan, [fold_maps +
all-gather when W > 1], fix-up.
"""
from __future__ import annotations

from typing import Any, Optional

import torch
import torch.distributed as dist
from torch import Tensor
from torch.autograd import Function

from . import _lib
from ._lib import lib, ptr

class _GpuKernels:
    """The compiled kernels (default).  Tests substitute a CPU stand-in with the same methods to
    exercise the rank logic without a GPU."""

    @staticmethod
    def scan_zero(a: Tensor, x: Tensor):
        """(y from a zero state, maps (R,2) = {prod a, y[:, -1]})"""
        return torch.ops.philtorch_b200.lpv_recur_zero_carry(a, x)

    @staticmethod
    def forward(a: Tensor, zi: Tensor, x: Tensor) -> Tensor:
        return torch.ops.philtorch_b200.lpv_recur(a, zi, x)

    @staticmethod
    def backward(a, zi, y, gy, g_in, need_a: bool):
        return torch.ops.philtorch_b200.lpv_recur_bwd(a, zi, y, gy, g_in, need_a, True)

    @staticmethod
    def fold_maps(maps: Tensor, B: int, S: int, reverse: bool) -> Tensor:
        """(B*S,2) piece maps -> (B,2) total map of every row (one tiny launch)."""
        out = maps.new_empty(B, 2)
        _stream_call(lib.ptb_lpv_recur_fold_maps, maps.device, _lib.dtype_code(maps), B, S, ptr(maps), int(reverse),
                     ptr(out))
        return out

    @staticmethod
    def fixup_forward(a, y, maps, zi, rank_maps, rank: int, world: int, B: int, S: int) -> Tensor:
        """Corrects y (B*S, L) in place; returns the states (B*S,) entering the pieces."""
        states = y.new_empty(B * S)
        _stream_call(lib.ptb_lpv_recur_fixup_fwd, y.device, _lib.dtype_code(y), B, S, y.shape[1], ptr(a),
                     int(a.dim() == 2), ptr(y), ptr(maps), ptr(zi), ptr(rank_maps), rank, world, ptr(states))
        return states

    @staticmethod
    def fixup_backward(a, y, states, maps, rank_maps, rank: int, world: int, gx, ga, B: int, S: int) -> Tensor:
        """Corrects gx (and ga) in place; returns the adjoint state (B,) leaving the shard on its left."""
        gzi = y.new_empty(B)
        _stream_call(lib.ptb_lpv_recur_fixup_bwd, y.device, _lib.dtype_code(y), B, S, y.shape[1], ptr(a),
                     int(a.dim() == 2), ptr(y), ptr(states), ptr(maps), ptr(rank_maps), rank, world, ptr(gx), ptr(ga),
                     ptr(gzi))
        return gzi


def _stream_call(fn, device, *args) -> None:
    with torch.cuda.device(device):
        _lib.check(fn(*args, torch.cuda.current_stream(device).cuda_stream), fn.__name__)


def _all_gather(t: Tensor, group) -> Tensor:
    world = dist.get_world_size(group)
    out = t.new_empty((world * t.shape[0],) + tuple(t.shape[1:]))   # concatenated along dim 0
    dist.all_gather_into_tensor(out, t.contiguous(), group=group)
    return out.view((world,) + tuple(t.shape))


def fold_carries_forward(carries: Tensor, zi: Tensor, rank: int) -> Tensor:
    """State entering shard ``rank``: s_0 = zi, s_{q+1} = P_q s_q + e_q.  carries: (W, B, 2).
    (What the fix-up kernel computes on the device; kept as the readable statement of the rule.)"""
    s = zi
    for q in range(rank):
        s = carries[q, :, 0] * s + carries[q, :, 1]
    return s


def fold_carries_backward(carries: Tensor, rank: int) -> Tensor:
    """Adjoint state entering shard ``rank`` from the right: c_W = 0, c_q = P_q c_{q+1} + e_q."""
    world = carries.shape[0]
    c = torch.zeros_like(carries[0, :, 0])
    for q in range(world - 1, rank, -1):
        c = carries[q, :, 0] * c + carries[q, :, 1]
    return c


SEGMENT_MIN_ROWS = 256         # segments are added until the kernels see at least this many rows ...
SEGMENT_MIN_LENGTH = 1 << 17   # ... of at least this many samples (a dozen tiles: the ragged last tile stays small)
SEGMENT_MIN_SAMPLES = 1 << 24  # smaller problems are launch-bound: the extra fix-up launches cost more than they save


def auto_segments(B: int, T: int, batched: bool, min_length: int = SEGMENT_MIN_LENGTH,
                  min_samples: int = SEGMENT_MIN_SAMPLES, min_rows: int = SEGMENT_MIN_ROWS) -> int:
    """Segments per row for B rows of T samples (measured on B200, fwd+bwd replayed from a CUDA graph:
    32 rows x 2^20: 0.219 ms plain, 0.184 ms with 8 segments; 64 rows: 0.386 -> 0.342 ms with 4)."""
    if not batched or B * T < min_samples:
        return 1   # coefficients shared by the rows cannot be reshaped into more rows
    S = 1
    while B * S < min_rows and T % (2 * S) == 0 and T // (2 * S) >= min_length:
        S *= 2
    return S


# 2x2 matrices: tiles are a few thousand samples and a sample moves 80 bytes, so shorter segments and
# smaller problems already pay
SEGMENT2_MAX_BATCH = 96        # 128 rows already run at 0.96 of the copy bandwidth: segments gain nothing there
SEGMENT2_MIN_LENGTH = 1 << 16
SEGMENT2_MIN_SAMPLES = 1 << 23


def auto_segments2(B: int, T: int) -> int:
    """Segments per row for the time-varying 2x2 recurrence with per-row matrices (measured on B200,
    T = 2^20, fp32, eager fwd+bwd: 16 rows 0.403 ms plain, 0.313 ms with 8 segments; 32 rows
    0.659 -> 0.519 ms with 8; 64 rows 1.107 -> 0.942 ms with 4; 128 rows 1.778 ms either way)."""
    if B >= SEGMENT2_MAX_BATCH:
        return 1
    return auto_segments(B, T, True, SEGMENT2_MIN_LENGTH, SEGMENT2_MIN_SAMPLES)


def _rank_world(group):
    if group is LOCAL or (group is None and not dist.is_initialized()):
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


LOCAL = object()   # `group` value: this device alone, whatever process groups exist


class TimeShardedLPVRecurrence(Function):
    @staticmethod
    def forward(ctx: Any, a: Tensor, zi: Tensor, x: Tensor, group, kernels, segments) -> Tensor:
        k = kernels or _GpuKernels
        rank, world = _rank_world(group)
        B, T = x.shape
        S = segments if segments is not None else auto_segments(B, T, a.dim() == 2)
        if S > 1 and (a.dim() != 2 or T % S != 0):
            raise ValueError("segments need per-row coefficients (B, T) and a row length divisible by them")
        L = T // S
        av = a.contiguous().view(B * S, L) if S > 1 else a.contiguous()
        xv = x.contiguous().view(B * S, L)
        zi_c = zi.contiguous()
        if world * S > 1:
            y, maps = k.scan_zero(av, xv)                         # (B*S, L), (B*S, 2) = {prod a, y[:, -1]}
            rank_maps = None
            if world > 1:                                         # this rank's total map; ONE all-gather
                rank_maps = _all_gather(k.fold_maps(maps, B, S, False), group)
            s_v = k.fixup_forward(av, y, maps, zi_c, rank_maps, rank, world, B, S)
            ctx.P = maps[:, 0]
        else:
            s_v = zi_c
            y = k.forward(av, s_v, xv)
            ctx.P = None
        ctx.group, ctx.kernels, ctx.rank, ctx.world, ctx.S, ctx.shape = group, k, rank, world, S, (B, T)
        out = y.view(B, T)
        ctx.save_for_backward(a, zi, out, s_v)
        return out

    @staticmethod
    def backward(ctx: Any, gy: Tensor):
        a, zi, out, s_v = ctx.saved_tensors
        k, S, (B, T) = ctx.kernels, ctx.S, ctx.shape
        need_a, need_zi, need_x = ctx.needs_input_grad[:3]
        if torch.is_grad_enabled():
            # a higher-order graph is being recorded: the adjoint written with differentiable pieces
            # (philtorch/lpv/ssm.py:64-99 with M = 1), on one device only
            if ctx.world > 1:
                raise RuntimeError("double backward through the time-sharded recurrence is not supported")
            from .autograd import LPVRecurrence
            a_rev = torch.roll(a, shifts=-1, dims=-1).flip(-1)
            g = LPVRecurrence.apply(a_rev, torch.zeros_like(zi), gy.flip(1)).flip(1)
            prev = torch.cat([zi.unsqueeze(1), out[:, :-1]], dim=1)
            ga = prev * g
            return ((ga if a.dim() == 2 else ga.sum(0)) if need_a else None, g[:, 0] * a[..., 0] if need_zi else None,
                    g if need_x else None, None, None, None)
        av = a.contiguous().view(B * S, T // S) if S > 1 else a.contiguous()
        y = out.view(B * S, T // S)
        gyv = gy.contiguous().view(B * S, T // S)
        ga, gs, gx = k.backward(av, s_v, y, gyv, None, need_a)   # adjoint with nothing entering from the right
        if ctx.world * S > 1:
            maps = torch.stack([ctx.P, gs], dim=1)                # (B*S, 2) adjoint maps of the pieces
            rank_maps = None
            if ctx.world > 1:
                rank_maps = _all_gather(k.fold_maps(maps, B, S, True), ctx.group)
            gs = k.fixup_backward(av, y, s_v, maps, rank_maps, ctx.rank, ctx.world, gx, ga if need_a else None, B, S)
        # only rank 0's is the gradient of zi (sum over ranks = the gradient)
        gzi = gs if ctx.rank == 0 else torch.zeros_like(gs)
        return (ga.view(a.shape) if need_a else None, gzi if need_zi else None,
                gx.view(B, T) if need_x else None, None, None, None)


def time_sharded_linear_recurrence(a: Tensor, zi: Tensor, x: Tensor, group=None, *, segments=None,
                                   _kernels=None) -> Tensor:
    """``lpv.linear_recurrence`` on a sequence whose time axis is sharded over ``group``.

    Args:
        a: this rank's coefficients, (B, T_local) (or (T_local,) shared by the batch).
        zi: initial state of the WHOLE sequence, (B,), identical on every rank.
        x: this rank's samples, (B, T_local).
        group: process group (default: the world; without an initialised process group: one rank).
            Ranks own consecutive time ranges in rank order.
        segments: segments per row inside a rank (a power of two dividing T_local); default: as many
            as give the kernels 256 rows, 1 for batches that are large enough.

    Returns:
        this rank's outputs, (B, T_local).  The gradient w.r.t. ``zi`` is returned on rank 0 and is
        zero elsewhere (sum over ranks = the gradient).
    """
    return TimeShardedLPVRecurrence.apply(a, zi, x, group, _kernels, segments)


class SegmentedMatrixRecurrence(Function):
    """h[t] = A[t] h[t-1] + x[t] with 2x2 matrices per row and sample, every row cut into S segments
    that the kernels see as B*S independent rows (one device; A (B,T,2,2), zi (B,2), x (B,T,2) or
    (B,T) feeding state 0).  Forward: the zero-start scan of all segments (which also yields every
    segment's matrix product), then ONE fix-up launch that folds the states entering the segments
    and corrects y in place until the correction is exactly zero.  Backward: the adjoint kernel on
    the segments with nothing entering from the right, then the mirrored fix-up of grad_x / grad_A.
    Same values as ``MatrixRecurrence`` (philtorch/lpv/ssm.py:34-115 of the reference) up to rounding."""

    @staticmethod
    def forward(ctx: Any, A: Tensor, zi: Tensor, x: Tensor, S: int) -> Tensor:
        B, T = x.shape[0], x.shape[1]
        xs = x.dim() == 2
        if A.dim() != 4 or T % S != 0:
            raise ValueError("segments need per-row matrices (B, T, 2, 2) and a row length divisible by them")
        dev = _lib.require_cuda(A, zi, x)
        L, R = T // S, B * S
        code = _lib.dtype_code(x)
        Av, xv, zi_c = A.contiguous().view(R, L, 2, 2), x.contiguous().view((R, L) if xs else (R, L, 2)), zi.contiguous()
        y = x.new_empty(R, L, 2)
        nch = lib.ptb_lpv_recur2_carry_chunks(code, L)
        tile_prod, e = x.new_empty(R, nch, 4), x.new_empty(R, 2)
        _lib.call(lib.ptb_lpv_recur2_zero_carry, dev, R, L, code, R, L, ptr(Av), ptr(xv), int(xs), ptr(y),
                  ptr(tile_prod), ptr(e))
        P, states = x.new_empty(R, 4), x.new_empty(R, 2)
        _stream_call(lib.ptb_lpv_recur2_fold_products, dev, code, R, nch, ptr(tile_prod), ptr(P))
        _stream_call(lib.ptb_lpv_recur2_fixup_fwd, dev, code, B, S, L, ptr(Av), ptr(y), ptr(P), ptr(e), ptr(zi_c),
                     ptr(states))
        out = y.view(B, T, 2)
        ctx.S, ctx.xs = S, xs
        ctx.save_for_backward(A, zi, out, states, P)
        return out

    @staticmethod
    def backward(ctx: Any, gy: Tensor):
        A, zi, out, states, P = ctx.saved_tensors
        S, xs = ctx.S, ctx.xs
        need_A, need_zi, need_x = ctx.needs_input_grad[:3]
        B, T = out.shape[0], out.shape[1]
        if torch.is_grad_enabled():
            # a higher-order graph is being recorded: the adjoint written with differentiable pieces
            # (philtorch/lpv/ssm.py:64-99)
            from .autograd import MatrixRecurrence
            AmT = A.mT
            A_rev = torch.roll(AmT, shifts=-1, dims=-3).flip(-3)
            g = MatrixRecurrence.apply(A_rev, torch.zeros_like(zi), gy.flip(1)).flip(1)
            prev = torch.cat([zi.unsqueeze(1), out[:, :-1]], dim=1)
            return (g.unsqueeze(-1) * prev.unsqueeze(-2) if need_A else None,
                    (AmT[:, 0] @ g[:, 0, :, None]).squeeze(-1) if need_zi else None,
                    (g[..., 0] if xs else g) if need_x else None, None)
        dev = out.device
        L, R = T // S, B * S
        code = _lib.dtype_code(out)
        Av, yv, gyv = A.contiguous().view(R, L, 2, 2), out.view(R, L, 2), gy.contiguous().view(R, L, 2)
        gA, e_adj, gx = torch.ops.philtorch_b200.recur2_bwd(Av, states, yv, gyv, None, xs, need_A, True)
        gzi = out.new_empty(B, 2)
        _stream_call(lib.ptb_lpv_recur2_fixup_bwd, dev, code, B, S, L, ptr(Av), ptr(yv), ptr(states), ptr(P),
                     ptr(e_adj), int(xs), ptr(gx), ptr(gA) if need_A else None, ptr(gzi))
        return (gA.view(A.shape) if need_A else None, gzi if need_zi else None,
                gx.view((B, T) if xs else (B, T, 2)) if need_x else None, None)
