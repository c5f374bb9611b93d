"""numpy restatements of the reference's callers that are pure first-order passes.
TEST INFRASTRUCTURE ONLY (the package never imports this file).

* ``comb_filter(a, delay, x, zi)``  -- philtorch/lti/filtering.py:15-71:
  y[t] = x[t] - a * y[t - delay], evaluated sequentially in blocks of ``delay`` samples;
  ``zi[..., k]`` is the output k + 1 samples before the signal starts.
* ``cspline(x, scipy_padding)``     -- philtorch/lti/interp.py:23-57: cubic B-spline coefficients
  by the causal / anticausal recursion with the pole sqrt(3) - 2, written as the textbook
  sequential loops over the mirrored signal (Unser, "B-Spline Signal Processing: Part II").
* ``cubic_spline(x, m, scipy_padding)`` -- philtorch/lti/interp.py:101-139: evaluation of the
  spline sum_k c[k] beta3(t - k) at t = j / m with the coefficients continued by mirroring.

Pinned against vectors produced by running the reference (tests/golden/cspline_*.npz,
comb_*.npz) and against scipy.signal.cspline1d in tests/test_oracle.py.
"""
from __future__ import annotations

import numpy as np


def comb_filter(a, delay: int, x, zi=None):
    a = np.asarray(a, dtype=np.float64)
    x = np.asarray(x, dtype=np.float64)
    rows, n = x.shape
    coef = a.reshape(-1, 1) if a.ndim == 1 else a
    past = np.zeros((rows, delay))                       # past[:, d] = y[t0 - delay + d]
    if zi is not None:
        zi = np.asarray(zi, dtype=np.float64)
        past = np.broadcast_to(zi[..., ::-1], (rows, delay)).copy()
    y = np.empty_like(x)
    for t0 in range(0, n, delay):
        k = min(delay, n - t0)
        y[:, t0:t0 + k] = x[:, t0:t0 + k] - coef * past[:, :k]
        past = np.concatenate([past[:, k:], y[:, t0:t0 + k]], axis=1)
    return y


def cspline(x, scipy_padding: bool):
    x = np.asarray(x, dtype=np.float64)
    rows, n = x.shape
    r = np.sqrt(3.0) - 2.0
    ext = np.concatenate([x, x[:, ::-1] if scipy_padding else x[:, -2::-1]], axis=1)   # one mirrored period
    # causal state before the first sample: sum over the mirrored past, r^k x_past[k]
    past = x if scipy_padding else x[:, 1:]
    h = past @ (r ** np.arange(past.shape[1]))
    out = np.empty_like(ext)
    for t in range(ext.shape[1]):
        h = r * h + ext[:, t]
        out[:, t] = h
    causal, anticausal = out[:, :n], out[:, -n:][:, ::-1]
    return -6.0 * r / (1.0 - r * r) * (causal + anticausal - x)


def _beta3(t):
    u = np.abs(t)
    return np.where(u <= 1, (4 - 6 * u ** 2 + 3 * u ** 3) / 6, np.where(u < 2, (2 - u) ** 3 / 6, 0.0))


def cubic_spline(x, m: int, scipy_padding: bool):
    c = cspline(x, scipy_padding)
    rows, n = c.shape
    if scipy_padding:      # c[-1] = c[0], c[n] = c[n-1], c[n+1] = c[n-2]
        ext = np.concatenate([c[:, :1], c, c[:, -1:], c[:, -2:-1]], axis=1)
    else:                  # c[-1] = c[1], c[n] = c[n-2], c[n+1] = c[n-3]
        ext = np.concatenate([c[:, 1:2], c, c[:, -2:-1], c[:, -3:-2]], axis=1)
    t = np.arange((n - 1) * m + 1) / m
    y = np.zeros((rows, t.size))
    base = np.floor(t).astype(int)
    for k in range(-1, 3):                               # the four coefficients around each output
        idx = base + k
        y += ext[:, idx + 1] * _beta3(t - idx)
    return y


def state_space(A, x, B, C, D=None, zi=None):
    """Sequential h[t+1] = A h[t] + B x[t], y[t] = C h[t] + D x[t] for x (rows, N), B (M,), C (M,),
    A (M, M) or (rows, M, M): what philtorch/lti/ssm.py:590-850 (``diag_state_space``) evaluates in
    the eigenbasis, restated in the original basis.  Returns (y, final state)."""
    A = np.asarray(A, dtype=np.float64)
    x = np.asarray(x, dtype=np.float64)
    B, C = np.asarray(B, dtype=np.float64), np.asarray(C, dtype=np.float64)
    rows, n = x.shape
    M = A.shape[-1]
    h = np.zeros((rows, M)) if zi is None else np.broadcast_to(np.asarray(zi, dtype=np.float64), (rows, M)).copy()
    y = np.empty((rows, n))
    for t in range(n):
        y[:, t] = h @ C
        h = (np.einsum("rij,rj->ri", A, h) if A.ndim == 3 else h @ A.T) + x[:, t:t + 1] * B
    if D is not None:
        y = y + np.asarray(D, dtype=np.float64) * x
    return y, h
