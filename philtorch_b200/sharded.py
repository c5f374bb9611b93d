"""First-order per-sample-coefficient recurrence with the TIME axis split across devices.

The reference has no multi-device code; this mode exists for rows too long for one GPU
(e.g. B = 8, T = 2^28).  Rank r of W owns the contiguous samples [r T/W, (r+1) T/W) of every row.

Forward, per rank:  (1) carry pass over the shard -> per row (P_r, e_r) = (product of a, end state
from a zero start);  (2) ONE all-gather of the (B, 2) carries;  (3) every rank folds the carries
of the ranks before it into its true incoming state s_r = P_{r-1} s_{r-1} + e_{r-1} (s_0 = zi);
(4) the ordinary forward scan started from s_r.
Backward mirrors it with the adjoint recurrence run from the right: carries flow from rank W-1
down, the incoming adjoint state enters the local adjoint kernel as ``g_in``.

The collective is tiny (W x B x 2 scalars) and latency-bound; everything else is local.
"""
from __future__ import annotations

from typing import Any, Optional

import torch
import torch.distributed as dist
from torch import Tensor
from torch.autograd import Function


class _GpuKernels:
    """The compiled kernels (default).  Tests substitute a CPU stand-in with the same methods to
    exercise the rank logic without a GPU."""

    @staticmethod
    def carry(a: Tensor, x: Tensor, reverse: bool) -> Tensor:
        return torch.ops.philtorch_b200.lpv_recur_carry(a, x, reverse)

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


class TimeShardedLPVRecurrence(Function):
    @staticmethod
    def forward(ctx: Any, a: Tensor, zi: Tensor, x: Tensor, group, kernels) -> Tensor:
        k = kernels or _GpuKernels
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        if world > 1:
            carries = _all_gather(k.carry(a, x, False), group)
            s = fold_carries_forward(carries, zi, rank)
        else:
            s = zi
        y = k.forward(a, s.contiguous(), x)
        ctx.group, ctx.kernels, ctx.rank, ctx.world = group, k, rank, world
        ctx.save_for_backward(a, s, y)
        return y

    @staticmethod
    def backward(ctx: Any, gy: Tensor):
        a, s, y = ctx.saved_tensors
        k = ctx.kernels
        need_a, need_zi, need_x = ctx.needs_input_grad[:3]
        gy = gy.contiguous()
        g_in: Optional[Tensor] = None
        if ctx.world > 1:
            carries = _all_gather(k.carry(a, gy, True), ctx.group)
            g_in = fold_carries_backward(carries, ctx.rank).contiguous()
        ga, gs, gx = k.backward(a, s, y, gy, g_in, need_a)
        # gs = adjoint state leaving this shard on the left; only rank 0's is the gradient of zi
        gzi = gs if ctx.rank == 0 else torch.zeros_like(gs)
        return (ga if need_a else None, gzi if need_zi else None, gx if need_x else None, None, None)


def time_sharded_linear_recurrence(a: Tensor, zi: Tensor, x: Tensor, group=None, *, _kernels=None) -> Tensor:
    """``lpv.linear_recurrence`` on a sequence whose time axis is sharded over ``group``.

    Args:
        a: this rank's coefficients, (B, T_local) (or (T_local,) shared by the batch).
        zi: initial state of the WHOLE sequence, (B,), identical on every rank.
        x: this rank's samples, (B, T_local).
        group: process group (default: the world).  Ranks own consecutive time ranges in rank order.

    Returns:
        this rank's outputs, (B, T_local).  The gradient w.r.t. ``zi`` is returned on rank 0 and is
        zero elsewhere (sum over ranks = the gradient).
    """
    return TimeShardedLPVRecurrence.apply(a, zi, x, group, _kernels)
