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


def _worker(rank, world, port, B, T, q, slow_decay):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from philtorch_b200 import sharded
        from philtorch_b200.sharded import time_sharded_linear_recurrence
        from sharded_common import OracleKernels

        sharded.FIXUP_BLOCK = 16   # several (doubling) fix-up blocks inside a 96-sample shard
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
        y = time_sharded_linear_recurrence(a_l, zi_l, x_l, _kernels=OracleKernels)
        ga, gzi, gx = torch.autograd.grad(y, (a_l, zi_l, x_l), gy[:, sl].contiguous())
        q.put((rank, y.detach(), ga, gzi, gx))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,slow_decay", [(2, False), (3, False), (2, True)])
def test_two_rank_gloo(world, slow_decay):
    from sharded_common import full_reference

    B, T = 3, 96 * world
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000 + world + 10 * int(slow_decay)
    procs = [ctx.Process(target=_worker, args=(r, world, port, B, T, q, slow_decay)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=60) for _ in range(world)], key=lambda t: t[0])
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
