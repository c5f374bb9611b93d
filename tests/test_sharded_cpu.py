"""Time-sharded recurrence: rank logic (carry folding, all-gather, gradient routing) on two gloo
ranks on CPU, with the oracle standing in for the GPU kernels."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import rel_err

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, B, T, q, slow_decay, segments=1):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from philtorch_b200 import sharded
        from philtorch_b200.sharded import time_sharded_linear_recurrence
        from sharded_common import OracleKernels

        g = torch.Generator().manual_seed(7)
        a = torch.rand(B, T, generator=g, dtype=torch.float64) * 1.9 - 0.95
        if slow_decay:
            a = 0.98 + 0.04 * a   # products never vanish: the fix-up must cover the whole shard
        zi = torch.randn(B, generator=g, dtype=torch.float64)
        x = torch.randn(B, T, generator=g, dtype=torch.float64)
        gy = torch.randn(B, T, generator=g, dtype=torch.float64)
        Tl = T // world
        sl = slice(rank * Tl, (rank + 1) * Tl)
        a_l = a[:, sl].clone().requires_grad_()
        x_l = x[:, sl].clone().requires_grad_()
        zi_l = zi.clone().requires_grad_()
        y = time_sharded_linear_recurrence(a_l, zi_l, x_l, segments=segments, _kernels=OracleKernels)
        ga, gzi, gx = torch.autograd.grad(y, (a_l, zi_l, x_l), gy[:, sl].contiguous())
        # numpy arrays are pickled by value; a tensor travels as a file descriptor its sender must outlive
        q.put((rank,) + tuple(t.detach().numpy() for t in (y, ga, gzi, gx)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,slow_decay,segments", [(2, False, 1), (3, False, 1), (2, True, 1), (2, False, 4),
                                                       (2, True, 2)])
def test_two_rank_gloo(world, slow_decay, segments):
    from sharded_common import full_reference

    B, T = 3, 96 * world
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000 + world + 10 * int(slow_decay) + 20 * segments
    procs = [ctx.Process(target=_worker, args=(r, world, port, B, T, q, slow_decay, segments)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=60) for _ in range(world)], key=lambda t: t[0])
    res = [(r[0],) + tuple(torch.from_numpy(v) for v in r[1:]) for r in res]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    g = torch.Generator().manual_seed(7)
    a = torch.rand(B, T, generator=g, dtype=torch.float64) * 1.9 - 0.95
    if slow_decay:
        a = 0.98 + 0.04 * a
    zi = torch.randn(B, generator=g, dtype=torch.float64)
    x = torch.randn(B, T, generator=g, dtype=torch.float64)
    gy = torch.randn(B, T, generator=g, dtype=torch.float64)
    y_ref, ga_ref, gzi_ref, gx_ref = full_reference(a, zi, x, gy)
    assert rel_err(torch.cat([r[1] for r in res], 1), y_ref) <= 1e-12
    assert rel_err(torch.cat([r[2] for r in res], 1), ga_ref) <= 1e-12
    assert rel_err(torch.cat([r[4] for r in res], 1), gx_ref) <= 1e-12
    assert rel_err(sum(r[3] for r in res), gzi_ref) <= 1e-12       # zi gradient: rank 0 only, zeros elsewhere
    assert all(float(r[3].abs().max()) == 0.0 for r in res[1:])


def test_fold_helpers():
    from philtorch_b200.sharded import fold_carries_backward, fold_carries_forward

    c = torch.tensor([[[0.5, 1.0]], [[2.0, -1.0]], [[0.25, 4.0]]])   # (W=3, B=1, 2)
    zi = torch.tensor([3.0])
    assert fold_carries_forward(c, zi, 0).item() == 3.0
    assert fold_carries_forward(c, zi, 1).item() == 0.5 * 3.0 + 1.0
    assert fold_carries_forward(c, zi, 2).item() == 2.0 * 2.5 - 1.0
    assert fold_carries_backward(c, 2).item() == 0.0
    assert fold_carries_backward(c, 1).item() == 4.0
    assert fold_carries_backward(c, 0).item() == 2.0 * 4.0 - 1.0


@pytest.mark.parametrize("segments,slow_decay", [(1, False), (4, False), (8, True)])
def test_single_process_segments(segments, slow_decay):
    """Without a process group the function is one rank; its local segments use the same carry algebra."""
    from philtorch_b200 import sharded
    from sharded_common import OracleKernels, full_reference

    if True:
        g = torch.Generator().manual_seed(11)
        B, T = 3, 256
        a = torch.rand(B, T, generator=g, dtype=torch.float64) * 1.9 - 0.95
        if slow_decay:
            a = 0.98 + 0.04 * a
        zi = torch.randn(B, generator=g, dtype=torch.float64)
        x = torch.randn(B, T, generator=g, dtype=torch.float64)
        gy = torch.randn(B, T, generator=g, dtype=torch.float64)
        ins = [t.clone().requires_grad_() for t in (a, zi, x)]
        y = sharded.time_sharded_linear_recurrence(ins[0], ins[1], ins[2], segments=segments, _kernels=OracleKernels)
        ga, gzi, gx = torch.autograd.grad(y, ins, gy)
        y_ref, ga_ref, gzi_ref, gx_ref = full_reference(a, zi, x, gy)
        assert rel_err(y, y_ref) <= 1e-12 and rel_err(ga, ga_ref) <= 1e-12
        assert rel_err(gx, gx_ref) <= 1e-12 and rel_err(gzi, gzi_ref) <= 1e-12


def test_auto_segments():
    from philtorch_b200.sharded import auto_segments

    assert auto_segments(8, 1 << 26, True) == 32
    assert auto_segments(256, 1 << 20, True) == 1
    assert auto_segments(8, 1 << 26, False) == 1
    assert auto_segments(32, 1 << 20, True) == 8     # 256 kernel rows of 2^17 samples
    assert auto_segments(64, 1 << 20, True) == 4
    assert auto_segments(8, 1 << 22, True) == 32     # segments stay at least 2^17 samples long
    assert auto_segments(8, 1 << 20, True) == 1      # small problems are launch-bound: no extra launches
