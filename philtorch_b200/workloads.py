"""Seeded synthetic inputs for the five benchmark configurations of the recurrence path.

The reference project ships no dataset and no benchmark inputs; its tests draw unseeded
random tensors (e.g. tests/test_recur_ext.py:24-44 of the reference).  The generators
below produce tensors with the shapes and value distributions of the five named
configurations, from a fixed seed, in fp64 and then cast to the requested dtype, so the
CPU checker and the GPU kernels see identical bits when generated on the same device
and copied.

Each generator returns a dict of tensors plus ``gy`` (the upstream gradient, N(0,1),
same shape as the output) so forward+backward runs are reproducible.
"""
from __future__ import annotations

import math

import torch

SEED_BASE = 1234


def _gen(device, idx, shard=0):
    """Generator of configuration ``idx``; ``shard`` > 0 gives an independent stream for another
    shard (rows or time range) of the same configuration."""
    g = torch.Generator(device=device)
    g.manual_seed(SEED_BASE + idx + 1000 * shard)
    return g


def _rand(shape, g, device):
    return torch.rand(shape, generator=g, device=device, dtype=torch.float64)


def _randn(shape, g, device):
    return torch.randn(shape, generator=g, device=device, dtype=torch.float64)


def lti_first_order(B=64, T=65536, dtype=torch.float32, device="cpu", shard=0):
    """Config 1: y[n] = a*y[n-1] + x[n]; a per channel ~U(0.5,0.99) with random sign,
    x ~ N(0,1), zero initial state."""
    g = _gen(device, 1, shard)
    mag = 0.5 + 0.49 * _rand((B,), g, device)
    sgn = torch.where(_rand((B,), g, device) < 0.5, -1.0, 1.0)
    return dict(a=(mag * sgn).to(dtype), zi=torch.zeros(B, dtype=dtype, device=device),
                x=_randn((B, T), g, device).to(dtype), gy=_randn((B, T), g, device).to(dtype))


def lpv_first_order(B=256, T=1 << 20, dtype=torch.float32, device="cpu", shard=0):
    """Config 2: per-sample coefficients a[b,n] ~ U(-0.99,0.99) i.i.d., x ~ N(0,1),
    initial state ~ N(0,1) per channel."""
    g = _gen(device, 2, shard)
    return dict(a=(-0.99 + 1.98 * _rand((B, T), g, device)).to(dtype),
                zi=_randn((B,), g, device).to(dtype),
                x=_randn((B, T), g, device).to(dtype), gy=_randn((B, T), g, device).to(dtype))


def sos_cascade(B=512, T=1 << 18, sections=6, dtype=torch.float32, device="cpu", shard=0):
    """Config 3: cascade of second-order sections; poles at radius ~U(0.5,0.99), angle
    ~U(0,pi); zeros at radius ~U(0,1.2), angle ~U(0,pi); gain 1, a0 = 1.
    b: (sections, B, 3), a: (sections, B, 2)."""
    g = _gen(device, 3, shard)
    r = 0.5 + 0.49 * _rand((sections, B), g, device)
    th = math.pi * _rand((sections, B), g, device)
    rho = 1.2 * _rand((sections, B), g, device)
    phi = math.pi * _rand((sections, B), g, device)
    a = torch.stack([-2 * r * torch.cos(th), r * r], dim=-1)
    b = torch.stack([torch.ones_like(rho), -2 * rho * torch.cos(phi), rho * rho], dim=-1)
    return dict(b=b.to(dtype), a=a.to(dtype), x=_randn((B, T), g, device).to(dtype),
                gy=_randn((B, T), g, device).to(dtype))


def lpv_second_order(B=128, T=1 << 20, dtype=torch.float32, device="cpu", shard=0):
    """Config 4: time-varying 2x2 companion matrix; per-sample pole radius ~U(0.6,0.98),
    pole angle a random walk (step ~N(0,0.01)) reflected into (0,pi); x ~ N(0,1) into
    state 0; zero initial state.  A[b,n] = [[2 r cos(th), -r^2], [1, 0]]."""
    g = _gen(device, 4, shard)
    r = 0.6 + 0.38 * _rand((B, T), g, device)
    th0 = math.pi * _rand((B, 1), g, device)
    walk = th0 + torch.cumsum(0.01 * _randn((B, T), g, device), dim=1)
    th = torch.remainder(walk, 2 * math.pi)
    th = torch.where(th > math.pi, 2 * math.pi - th, th)  # reflection at 0 and pi
    A = torch.empty(B, T, 2, 2, dtype=torch.float64, device=device)
    A[..., 0, 0] = 2 * r * torch.cos(th)
    A[..., 0, 1] = -(r * r)
    A[..., 1, 0] = 1.0
    A[..., 1, 1] = 0.0
    return dict(A=A.to(dtype), zi=torch.zeros(B, 2, dtype=dtype, device=device),
                x=_randn((B, T), g, device).to(dtype),
                gy=_randn((B, T, 2), g, device).to(dtype))


def long_first_order(B=8, T=1 << 28, dtype=torch.float32, device="cpu", shard=0):
    """Config 5: long-sequence first-order LPV; a[b,n] ~ U(0.9,0.999), x ~ N(0,1),
    zero initial state."""
    g = _gen(device, 5, shard)
    return dict(a=(0.9 + 0.099 * _rand((B, T), g, device)).to(dtype),
                zi=torch.zeros(B, dtype=dtype, device=device),
                x=_randn((B, T), g, device).to(dtype), gy=_randn((B, T), g, device).to(dtype))
