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


def full_reference(a, zi, x, gy):
    y = cport.recur1(a, zi, x)
    ga, gzi, gx = cport.recur1_bwd(a, zi, y, gy)
    return y, ga, gzi, gx
