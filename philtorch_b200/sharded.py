"""First-order per-sample-coefficient recurrence with the TIME axis split across devices.

The reference has no multi-device code; this mode exists for rows too long for one GPU
(e.g. B = 8, T = 2^28).  Rank r of W owns the contiguous samples [r T/W, (r+1) T/W) of every row.

Forward, per rank
  (1) ONE pass over the shard: the scan started from a zero state, y0, together with the shard's
      total affine map (P_r, e_r) = (product of a, y0's last sample);
  (2) ONE all-gather of the (B, 2) maps; every rank folds the maps of the ranks before it into its
      true incoming state  s_r = P_{r-1} s_{r-1} + e_{r-1}  (s_0 = zi);
  (3) fix-up  y[t] = y0[t] + (prod_{u<=t} a[u]) s_r.  The running product normally underflows to
      exactly zero after a few thousand samples (|a| < 1), from where the correction is exactly
      zero: it is applied block by block from the shard's start and stops at the first block that
      ends with an all-zero correction (one tiny device->host read per block).  If the products
      never vanish the blocks double until the whole shard has been corrected: still exact.
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
The fold over the segments is the same recurrence over the (B, S) maps and runs as one more
launch of the kernel, queued behind the scan (folding on the host would stall the stream twice
per direction, and a Python loop over the segments is launch-bound for S >= 32).
"""
from __future__ import annotations

from typing import Any, Optional

import torch
import torch.distributed as dist
from torch import Tensor
from torch.autograd import Function

FIXUP_BLOCK = 1 << 16     # first fix-up block (samples per row) at most; later blocks double
FIXUP_SAMPLES = 1 << 20   # ... and about this many samples over all rows (more rows: shorter first block)


def _first_block(rows: int) -> int:
    return max(min(FIXUP_BLOCK, 1024), min(FIXUP_BLOCK, FIXUP_SAMPLES // max(rows, 1)))


class _GpuKernels:
    """The compiled kernels (default).  Tests substitute a CPU stand-in with the same methods to
    exercise the rank logic without a GPU."""

    @staticmethod
    def scan_zero(a: Tensor, x: Tensor):
        """(y from a zero state, carry (B,2) = {prod a, y[:, -1]})"""
        return torch.ops.philtorch_b200.lpv_recur_zero_carry(a, x)

    @staticmethod
    def forward(a: Tensor, zi: Tensor, x: Tensor) -> Tensor:
        return torch.ops.philtorch_b200.lpv_recur(a, zi, x)

    @staticmethod
    def backward(a, zi, y, gy, g_in, need_a: bool):
        return torch.ops.philtorch_b200.lpv_recur_bwd(a, zi, y, gy, g_in, need_a, True)


def _all_gather(t: Tensor, group) -> Tensor:
    world = dist.get_world_size(group)
    out = t.new_empty((world * t.shape[0],) + tuple(t.shape[1:]))   # concatenated along dim 0
    dist.all_gather_into_tensor(out, t.contiguous(), group=group)
    return out.view((world,) + tuple(t.shape))


def fold_carries_forward(carries: Tensor, zi: Tensor, rank: int) -> Tensor:
    """State entering shard ``rank``: s_0 = zi, s_{q+1} = P_q s_q + e_q.  carries: (W, B, 2)."""
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


def _rows(a: Tensor, lo: int, hi: int) -> Tensor:
    return a[..., lo:hi].contiguous()


def fixup_forward(k, a: Tensor, y: Tensor, s: Tensor) -> None:
    """In place: y[t] += (prod_{u<=t} a[u]) s, block by block until the correction has died out."""
    T = y.shape[1]
    lo, blk = 0, _first_block(y.shape[0])
    while lo < T:
        hi = min(T, lo + blk)
        z = k.forward(_rows(a, lo, hi), s.contiguous(), torch.zeros_like(y[:, lo:hi]))
        y[:, lo:hi] += z
        s = z[:, -1]
        if not bool((s != 0).any()):
            break
        lo, blk = hi, blk * 2


def fixup_backward(k, a: Tensor, s_in: Tensor, y: Tensor, c: Tensor, gx: Tensor, ga: Optional[Tensor]) -> None:
    """In place: adds to grad_x (and grad_a) the adjoint driven by the state ``c`` entering the shard
    from the right, suffix block by suffix block until it has died out."""
    T = y.shape[1]
    hi, blk = T, _first_block(y.shape[0])
    while hi > 0:
        lo = max(0, hi - blk)
        y_prev = s_in if lo == 0 else y[:, lo - 1]
        ga_b, c, gx_b = k.backward(_rows(a, lo, hi), y_prev.contiguous(), y[:, lo:hi].contiguous(),
                                   torch.zeros_like(y[:, lo:hi]), c.contiguous(), ga is not None)
        gx[:, lo:hi] += gx_b
        if ga is not None:
            ga[..., lo:hi] += ga_b   # (B,T) per row, or (T,) when the coefficients are shared
        if not bool((c != 0).any()):
            break
        hi, blk = lo, blk * 2


SEGMENT_MIN_ROWS = 256        # segments are added until the kernels see at least this many rows ...
SEGMENT_MIN_LENGTH = 1 << 20  # ... of at least this many samples


def auto_segments(B: int, T: int, batched: bool) -> int:
    if not batched:
        return 1   # coefficients shared by the rows cannot be reshaped into more rows
    S = 1
    while B * S < SEGMENT_MIN_ROWS and T % (2 * S) == 0 and T // (2 * S) >= SEGMENT_MIN_LENGTH:
        S *= 2
    return S


def _rank_world(group):
    if group is None and not dist.is_initialized():
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


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
        if world * S > 1:
            y, carry = k.scan_zero(av, xv)                       # (B*S, L), (B*S, 2) = {prod a, y[:, -1]}
            c = carry.view(B, S, 2)
            P_seg, e_seg = c[:, :, 0].contiguous(), c[:, :, 1].contiguous()
            if world > 1:                                         # this rank's total map, then the fold over ranks
                e_tot = k.forward(P_seg, torch.zeros_like(zi), e_seg)[:, -1] if S > 1 else e_seg[:, 0]
                mine = torch.stack([P_seg.prod(dim=1), e_tot], dim=1)
                s = fold_carries_forward(_all_gather(mine, group), zi, rank)
            else:
                s = zi
            states = s.reshape(B, 1)                              # states entering the segments: the same
            if S > 1:                                             # recurrence over the segments' maps, one launch
                after = k.forward(P_seg, s.contiguous(), e_seg)
                states = torch.cat([states, after[:, :-1]], dim=1)
            s_v = states.reshape(B * S).contiguous()
            fixup_forward(k, av, y, s_v)
            ctx.P = carry[:, 0].contiguous()
        else:
            s_v = zi.contiguous()
            y = k.forward(av, s_v, xv)
            ctx.P = None
        ctx.group, ctx.kernels, ctx.rank, ctx.world, ctx.S, ctx.shape = group, k, rank, world, S, (B, T)
        ctx.a_shape = a.shape
        ctx.save_for_backward(av, s_v, y)
        return y.view(B, T)

    @staticmethod
    def backward(ctx: Any, gy: Tensor):
        av, s_v, y = ctx.saved_tensors
        k, S, (B, T) = ctx.kernels, ctx.S, ctx.shape
        need_a, need_zi, need_x = ctx.needs_input_grad[:3]
        gyv = gy.contiguous().view(B * S, T // S)
        ga, gs, gx = k.backward(av, s_v, y, gyv, None, need_a)   # adjoint with nothing entering from the right
        if ctx.world * S > 1:
            Pr = ctx.P.view(B, S).flip(1).contiguous()            # segments from the right
            gr = gs.view(B, S).flip(1).contiguous()
            zero = torch.zeros_like(gr[:, 0])
            if ctx.world > 1:                                     # this rank's total adjoint map, then the fold
                e_tot = k.forward(Pr, zero, gr)[:, -1] if S > 1 else gr[:, 0]
                mine = torch.stack([Pr.prod(dim=1), e_tot], dim=1)
                c = fold_carries_backward(_all_gather(mine, ctx.group), ctx.rank)
            else:
                c = zero
            after = k.forward(Pr, c.contiguous(), gr)             # adjoint leaving each segment on its left
            cs = torch.cat([c.reshape(B, 1), after[:, :-1]], dim=1).flip(1)   # ... = entering the one before it
            c_v = cs.reshape(B * S).contiguous()
            fixup_backward(k, av, s_v, y, c_v, gx, ga if need_a else None)
            gs = after[:, -1]                                     # adjoint state leaving this rank on the left
        # only rank 0's is the gradient of zi (sum over ranks = the gradient)
        gzi = gs if ctx.rank == 0 else torch.zeros_like(gs)
        return (ga.view(ctx.a_shape) if need_a else None, gzi if need_zi else None,
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
