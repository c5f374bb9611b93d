"""Full-size parity of the five benchmark configurations against the CPU oracle.

The reduced-size golden vectors pin the arithmetic; these cases check what only the full sizes
show: rounding-error growth over 2^18 - 2^26 samples per row within the tolerance of the path
(max|out - ref| / max|ref| <= 1e-4 in float32, <= 1e-10 in float64, for the output and every
gradient).  The measurements come from the benchmark's own configuration runners, so the test
and the benchmark line cannot drift apart.
"""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import bench  # noqa: E402
import philtorch_b200 as ptb  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _check(entry):
    assert "error" not in entry, entry
    assert entry["parity_ok"], (entry["parity"], entry["parity_tolerance"])
    ptb.check_errors()


def test_config1_full_size():
    _check(bench.config1(DEV, 3, 0))


def test_config2_full_size():
    from philtorch_b200 import workloads

    ops = torch.ops.philtorch_b200
    w = workloads.lpv_first_order(device=DEV)
    a, zi, x, gy = w["a"], w["zi"], w["x"], w["gy"]
    y = ops.lpv_recur(a, zi, x)
    ga, gzi, gx = ops.lpv_recur_bwd(a, zi, y, gy, None, True, True)
    par = bench.config2_parity(DEV, a, zi, x, gy, y, ga, gzi, gx)
    assert max(par.values()) <= 1e-4, par
    ptb.check_errors()


def test_config3_full_size():
    chained, fused = bench.config3(DEV, 3, 0)
    _check(chained)
    _check(fused)


@pytest.mark.parametrize("f64", [False, True])
def test_config4_full_size(f64):
    _check(bench.config4(DEV, 3, 0, f64))


def test_config5_long_rows():
    """B = 8 rows of 2^26 samples (a quarter of the benchmark's length keeps the test short; the
    benchmark itself checks 2^28) through the segmented path, against the time-chunked oracle."""
    _check(bench.config5(DEV, 3, 0, log2_T=26))
