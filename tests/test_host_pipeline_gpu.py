"""The host-buffer entry point (philtorch_b200.host): inputs and results in pinned host memory, row
blocks streamed through three CUDA streams with recycled staging buffers.  Checked against the
CPU oracle: a batch that is not a multiple of the block size, more blocks than staging buffers,
and two runs in a row with different inputs through the same pipeline object."""
import pytest
import torch

import philtorch_b200 as ptb
from philtorch_b200.host import HostPipeline, linear_recurrence_fwd_bwd_host
from conftest import rel_err, tol
from sharded_common import full_reference

pytestmark = pytest.mark.gpu


def _inputs(B, T, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    a = (torch.rand(B, T, generator=g, dtype=torch.float64) * 1.98 - 0.99).to(dtype).pin_memory()
    zi = torch.randn(B, generator=g, dtype=torch.float64).to(dtype).pin_memory()
    x = torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype).pin_memory()
    gy = torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype).pin_memory()
    return a, zi, x, gy


def _check(out, a, zi, x, gy, dtype):
    y, ga, gzi, gx = full_reference(a, zi, x, gy)
    t = tol(dtype)
    assert rel_err(out["y"], y) <= t and rel_err(out["grad_x"], gx) <= t
    assert rel_err(out["grad_a"], ga) <= t and rel_err(out["grad_zi"], gzi) <= t


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("B,rows", [(70, 16), (5, 32), (33, 8)])
def test_pipeline_two_runs(dtype, B, rows):
    T = 20000
    pipe = HostPipeline(B, T, dtype, "cuda", rows_per_block=rows)
    assert pipe.nblk == -(-B // min(rows, B))
    out = {k: torch.full((B, T) if k != "grad_zi" else (B,), float("nan"), dtype=dtype).pin_memory()
           for k in ("y", "grad_a", "grad_x", "grad_zi")}
    for seed in (1, 2):   # the second run reuses every staging buffer and stream
        a, zi, x, gy = _inputs(B, T, dtype, seed)
        pipe.run(a, zi, x, gy, out)
        torch.cuda.synchronize()
        _check(out, a, zi, x, gy, dtype)
    assert pipe.h2d_bytes == (3 * B * T + B) * a.element_size()
    assert pipe.d2h_bytes == (3 * B * T + B) * a.element_size()
    ptb.check_errors()


def test_one_shot_wrapper():
    a, zi, x, gy = _inputs(19, 9217, torch.float32, 3)
    out = linear_recurrence_fwd_bwd_host(a, zi, x, gy, rows_per_block=4)
    _check(out, a, zi, x, gy, torch.float32)
    ptb.check_errors()
