"""Helpers shared by the time-sharding tests (CPU stand-in kernels built on the oracle)."""
import torch

from oracle import cport


class OracleKernels:
    """CPU stand-in for the three kernels the time-sharded recurrence calls (test use only)."""

    @staticmethod
    def carry(a, x, reverse):
        B = x.shape[0]
        ab = a if a.dim() == 2 else a.expand(B, -1)
        P = ab.prod(dim=1)
        zero = torch.zeros(B, dtype=x.dtype)
        if not reverse:
            e = cport.recur1(a, zero, x)[:, -1]
        else:
            _, e, _ = cport.recur1_bwd(a, zero, torch.zeros_like(x), x)
        return torch.stack([P, e], dim=1)

    @staticmethod
    def scan_zero(a, x):
        y = cport.recur1(a, torch.zeros(x.shape[0], dtype=x.dtype), x)
        ab = a if a.dim() == 2 else a.expand(x.shape[0], -1)
        return y, torch.stack([ab.prod(dim=1), y[:, -1]], dim=1)

    @staticmethod
    def forward(a, zi, x):
        return cport.recur1(a, zi, x)

    @staticmethod
    def backward(a, zi, y, gy, g_in, need_a):
        ga, gzi, gx = cport.recur1_bwd(a, zi, y, gy, g_in)
        return ga, gzi, gx

    # ---- the fix-up kernels, restated with loops (small cases only)
    @staticmethod
    def fold_maps(maps, B, S, reverse):
        m = maps.view(B, S, 2)
        P, e = torch.ones(B, dtype=maps.dtype), torch.zeros(B, dtype=maps.dtype)
        for k in (range(S - 1, -1, -1) if reverse else range(S)):
            e = m[:, k, 0] * e + m[:, k, 1]
            P = P * m[:, k, 0]
        return torch.stack([P, e], dim=1)

    @staticmethod
    def fixup_forward(a, y, maps, zi, rank_maps, rank, world, B, S):
        m = maps.view(B, S, 2)
        s = zi.clone()
        for q in range(rank if rank_maps is not None else 0):
            s = rank_maps[q, :, 0] * s + rank_maps[q, :, 1]
        states = torch.empty(B, S, dtype=y.dtype)
        for j in range(S):
            states[:, j] = s
            s = m[:, j, 0] * s + m[:, j, 1]
        states = states.reshape(B * S)
        z = cport.recur1(a, states, torch.zeros_like(y))     # z[t] = a[t] z[t-1], z[-1] = state
        y += z
        return states

    @staticmethod
    def fixup_backward(a, y, states, maps, rank_maps, rank, world, gx, ga, B, S):
        m = maps.view(B, S, 2)
        c = torch.zeros(B, dtype=y.dtype)
        if rank_maps is not None:
            for q in range(world - 1, rank, -1):
                c = rank_maps[q, :, 0] * c + rank_maps[q, :, 1]
        cs = torch.empty(B, S, dtype=y.dtype)
        for j in range(S - 1, -1, -1):
            cs[:, j] = c
            c = m[:, j, 0] * c + m[:, j, 1]
        ga_b, _, gx_b = cport.recur1_bwd(a, states, y, torch.zeros_like(y), cs.reshape(B * S))
        gx += gx_b
        if ga is not None:
            ga += ga_b
        return c


def full_reference(a, zi, x, gy):
    y = cport.recur1(a, zi, x)
    ga, gzi, gx = cport.recur1_bwd(a, zi, y, gy)
    return y, ga, gzi, gx
