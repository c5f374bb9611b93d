"""Time-sharded first-order scan on the GPU: the carry kernel against the oracle, the shard
composition emulated on one GPU (shards processed one after another with the same folding code
the ranks run), and -- when at least two GPUs are visible -- real ranks under torchrun/NCCL."""
import os
import subprocess
import sys

import pytest
import torch

import philtorch_b200 as ptb
from philtorch_b200 import workloads
from philtorch_b200.sharded import fold_carries_backward, fold_carries_forward
from conftest import rel_err, tol
from sharded_common import OracleKernels, full_reference

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ops = torch.ops.philtorch_b200


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("T", [1, 5, 3072, 3073, 20000, 100001])
@pytest.mark.parametrize("reverse", [False, True])
def test_carry_kernel(dtype, T, reverse):
    B = 5
    g = torch.Generator().manual_seed(T + reverse)
    a = (0.9 + 0.0999 * torch.rand(B, T, generator=g, dtype=torch.float64)).to(dtype)
    x = torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype)
    got = ops.lpv_recur_carry(a.to(DEV), x.to(DEV), reverse)
    ref = OracleKernels.carry(a, x, reverse)
    t = tol(dtype)
    assert rel_err(got[:, 1], ref[:, 1]) <= t
    assert ((got[:, 0].cpu().double() - ref[:, 0].double()).abs() <= t * ref[:, 0].double().abs() + 1e-300).all()
    ptb.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("T", [7, 4608, 9217, 50000])
def test_zero_start_scan_with_carry(dtype, T):
    B = 4
    g = torch.Generator().manual_seed(T)
    a = (0.7 + 0.2999 * torch.rand(B, T, generator=g, dtype=torch.float64)).to(dtype)
    x = torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype)
    y, carry = ops.lpv_recur_zero_carry(a.to(DEV), x.to(DEV))
    y_ref, carry_ref = OracleKernels.scan_zero(a, x)
    t = tol(dtype)
    assert rel_err(y, y_ref) <= t and rel_err(carry[:, 1], carry_ref[:, 1]) <= t
    assert ((carry[:, 0].cpu().double() - carry_ref[:, 0].double()).abs() <= t * carry_ref[:, 0].double().abs() + 1e-300).all()
    ptb.check_errors()


@pytest.mark.parametrize("world", [2, 8])
def test_shards_emulated_on_one_gpu(world):
    """Config-5 distribution (a ~ U(0.9, 0.999)), B = 8, shards of 2^17 samples."""
    B, Tl = 8, 1 << 17
    T = Tl * world
    w = workloads.long_first_order(B=B, T=T)
    a, zi, x, gy = w["a"], torch.randn(B, generator=torch.Generator().manual_seed(1)), w["x"], w["gy"]
    sh = [slice(r * Tl, (r + 1) * Tl) for r in range(world)]
    a_s = [a[:, s].contiguous().to(DEV) for s in sh]
    x_s = [x[:, s].contiguous().to(DEV) for s in sh]
    gy_s = [gy[:, s].contiguous().to(DEV) for s in sh]
    zi_d = zi.to(DEV)
    carries = torch.stack([ops.lpv_recur_carry(a_s[r], x_s[r], False) for r in range(world)])
    s_in = [fold_carries_forward(carries, zi_d, r).contiguous() for r in range(world)]
    y_s = [ops.lpv_recur(a_s[r], s_in[r], x_s[r]) for r in range(world)]
    bc = torch.stack([ops.lpv_recur_carry(a_s[r], gy_s[r], True) for r in range(world)])
    outs = [ops.lpv_recur_bwd(a_s[r], s_in[r], y_s[r], gy_s[r], fold_carries_backward(bc, r).contiguous(), True, True)
            for r in range(world)]
    ptb.check_errors()
    y_ref, ga_ref, gzi_ref, gx_ref = full_reference(a, zi, x, gy)
    assert rel_err(torch.cat(y_s, 1), y_ref) <= 1e-4
    assert rel_err(torch.cat([o[0] for o in outs], 1), ga_ref) <= 1e-4
    assert rel_err(torch.cat([o[2] for o in outs], 1), gx_ref) <= 1e-4
    assert rel_err(outs[0][1], gzi_ref) <= 1e-4


_RANK_SCRIPT = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["PTB_ROOT"]); sys.path.insert(0, os.path.join(os.environ["PTB_ROOT"], "tests"))
from philtorch_b200 import workloads
from philtorch_b200.sharded import time_sharded_linear_recurrence
import philtorch_b200 as ptb
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl")
B, Tl = 8, 1 << 18
w = workloads.long_first_order(B=B, T=Tl * world)
sl = slice(rank * Tl, (rank + 1) * Tl)
a = w["a"][:, sl].contiguous().cuda().requires_grad_()
x = w["x"][:, sl].contiguous().cuda().requires_grad_()
zi = torch.randn(B, generator=torch.Generator().manual_seed(1)).cuda().requires_grad_()
y = time_sharded_linear_recurrence(a, zi, x)
ga, gzi, gx = torch.autograd.grad(y, (a, zi, x), w["gy"][:, sl].contiguous().cuda())
ptb.check_errors()
parts = [torch.empty_like(t) for t in (y, ga, gx)]
gathered = []
for t in (y.detach(), ga, gx):
    buf = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(buf, t.contiguous())
    gathered.append(torch.cat(buf, 1).cpu())
dist.all_reduce(gzi)
if rank == 0:
    from sharded_common import full_reference
    y_ref, ga_ref, gzi_ref, gx_ref = full_reference(w["a"], zi.detach().cpu(), w["x"], w["gy"])
    def rel(o, r): return ((o.double() - r.double()).abs().max() / r.double().abs().max()).item()
    errs = [rel(gathered[0], y_ref), rel(gathered[1], ga_ref), rel(gathered[2], gx_ref), rel(gzi.cpu(), gzi_ref)]
    print("ERRS", errs)
    assert max(errs) <= 1e-4, errs
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_real_ranks_nccl(tmp_path):
    n = min(torch.cuda.device_count(), 4)
    script = tmp_path / "rank.py"
    script.write_text(_RANK_SCRIPT)
    env = dict(os.environ, PTB_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                          "--master-addr", "127.0.0.1", "--master-port", "29611", str(script)],
                         env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "ERRS" in out.stdout


@pytest.mark.parametrize("segments", [1, 4, 16])
@pytest.mark.parametrize("slow_decay", [False, True])
def test_single_gpu_segments(segments, slow_decay):
    """One rank, its rows cut into segments that the kernels see as more rows: same results as the
    plain kernels; with coefficients so close to one that the correction never dies out the fix-up
    walks whole segments."""
    from philtorch_b200 import sharded

    B, T = 4, 1 << 16
    g = torch.Generator().manual_seed(5)
    # the never-decaying case is ill-conditioned in float32 (a random walk of 65536 steps): float64 there
    dt = torch.float64 if slow_decay else torch.float32
    a = ((0.99995 + 0.0001 * torch.rand(B, T, generator=g, dtype=dt)) if slow_decay
         else (0.9 + 0.0999 * torch.rand(B, T, generator=g))).cuda()
    x = torch.randn(B, T, generator=g, dtype=dt).cuda()
    zi = torch.randn(B, generator=g, dtype=dt).cuda()
    gy = torch.randn(B, T, generator=g, dtype=dt).cuda()
    ins = [t.clone().requires_grad_() for t in (a, zi, x)]
    y = sharded.time_sharded_linear_recurrence(ins[0], ins[1], ins[2], sharded.LOCAL, segments=segments)
    ga, gzi, gx = torch.autograd.grad(y, ins, gy)
    y_r, ga_r, gzi_r, gx_r = full_reference(a.cpu(), zi.cpu(), x.cpu(), gy.cpu())
    t = 1e-9 if slow_decay else 1e-4
    assert rel_err(y, y_r) <= t and rel_err(gx, gx_r) <= t
    assert rel_err(ga, ga_r) <= t and rel_err(gzi, gzi_r) <= t
    ptb.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("world,S,L,shared,slow_decay", [
    (2, 1, 5000, False, False), (3, 4, 3001, False, False), (2, 8, 1024, False, True), (4, 2, 2500, False, True),
    (2, 1, 4099, True, False), (3, 1, 2048, True, True), (8, 32, 1500, False, False)])
def test_fixup_kernels_emulated_ranks(dtype, world, S, L, shared, slow_decay):
    """The device-side fold + fix-up with several time shards emulated on one GPU: every shard runs
    the calls a rank makes (zero-start scan, fold of its segment maps, fix-up with the gathered
    shard maps; then the same from the right for the adjoint), the stacked maps standing in for the
    all-gather.  Lengths that are not multiples of the fix-up block or of 16 bytes included."""
    from philtorch_b200.sharded import _GpuKernels as K

    B = 3
    T = world * S * L
    g = torch.Generator().manual_seed(world * 100 + S)
    lo, width = (0.999, 0.001) if slow_decay else (0.6, 0.39)   # slow: the correction outlives every piece
    a = (lo + width * torch.rand((T,) if shared else (B, T), generator=g, dtype=torch.float64)).to(dtype)
    x = torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype)
    zi = torch.randn(B, generator=g, dtype=torch.float64).to(dtype)
    gy = torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype)
    Tl = T // world
    a_s = [a[..., r * Tl:(r + 1) * Tl].contiguous().to(DEV) for r in range(world)]
    av = [t if shared else t.view(B * S, L) for t in a_s]
    xv = [x[:, r * Tl:(r + 1) * Tl].contiguous().to(DEV).view(B * S, L) for r in range(world)]
    gv = [gy[:, r * Tl:(r + 1) * Tl].contiguous().to(DEV).view(B * S, L) for r in range(world)]
    zi_d = zi.to(DEV)
    ys, maps = zip(*[K.scan_zero(av[r], xv[r]) for r in range(world)])
    rank_maps = torch.stack([K.fold_maps(maps[r], B, S, False) for r in range(world)])
    states = [K.fixup_forward(av[r], ys[r], maps[r], zi_d, rank_maps, r, world, B, S) for r in range(world)]
    outs = [K.backward(av[r], states[r], ys[r], gv[r], None, True) for r in range(world)]
    bmaps = [torch.stack([maps[r][:, 0], outs[r][1]], dim=1) for r in range(world)]
    brank = torch.stack([K.fold_maps(bmaps[r], B, S, True) for r in range(world)])
    gz = [K.fixup_backward(av[r], ys[r], states[r], bmaps[r], brank, r, world, outs[r][2], outs[r][0], B, S)
          for r in range(world)]
    ptb.check_errors()
    y_ref, ga_ref, gzi_ref, gx_ref = full_reference(a, zi, x, gy)
    t = tol(dtype) * (10 if slow_decay else 1)
    assert rel_err(torch.cat([v.view(B, Tl) for v in ys], 1), y_ref) <= t
    assert rel_err(torch.cat([o[2].view(B, Tl) for o in outs], 1), gx_ref) <= t
    ga = torch.cat([o[0].view(-1, Tl) if not shared else o[0].view(1, Tl) for o in outs], 1)
    assert rel_err(ga.view(ga_ref.shape), ga_ref) <= t
    assert rel_err(gz[0], gzi_ref) <= t


def test_few_long_rows_take_the_segmented_path():
    """lpv.linear_recurrence cuts a handful of long rows into segments by itself (same values and
    gradients as the oracle; double backward still works through the differentiable form)."""
    B, T = 4, 1 << 22
    w = workloads.long_first_order(B=B, T=T)
    a, x, gy = w["a"], w["x"], w["gy"]
    zi = torch.randn(B, generator=torch.Generator().manual_seed(3))
    from philtorch_b200.sharded import auto_segments
    assert auto_segments(B, T, True) == 32
    ins = [t.to(DEV).requires_grad_() for t in (a, zi, x)]
    y = ptb.lpv.linear_recurrence(*ins)
    assert type(y.grad_fn).__name__.startswith("TimeShardedLPVRecurrence")
    ga, gzi, gx = torch.autograd.grad(y, ins, gy.to(DEV))
    y_r, ga_r, gzi_r, gx_r = full_reference(a, zi, x, gy)
    assert rel_err(y, y_r) <= 1e-4 and rel_err(gx, gx_r) <= 1e-4
    assert rel_err(ga, ga_r) <= 1e-4 and rel_err(gzi, gzi_r) <= 1e-4
    ptb.check_errors()


def test_segmented_path_double_backward():
    from philtorch_b200 import sharded

    g = torch.Generator().manual_seed(9)
    B, T = 2, 64
    a = (torch.rand(B, T, generator=g, dtype=torch.float64) * 1.6 - 0.8).to(DEV).requires_grad_()
    zi = torch.randn(B, generator=g, dtype=torch.float64).to(DEV).requires_grad_()
    x = torch.randn(B, T, generator=g, dtype=torch.float64).to(DEV).requires_grad_()
    fn = lambda a_, zi_, x_: sharded.time_sharded_linear_recurrence(a_, zi_, x_, sharded.LOCAL, segments=4)  # noqa: E731
    assert torch.autograd.gradcheck(fn, (a, zi, x))
    assert torch.autograd.gradgradcheck(fn, (a, zi, x))
