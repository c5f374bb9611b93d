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
def test_single_gpu_segments(segments):
    """One rank, its rows cut into segments that the kernels see as more rows: same results as the
    plain kernels, for coefficients near one (the fix-up runs over several blocks) too."""
    import philtorch_b200 as ptb
    from philtorch_b200 import sharded

    B, T = 4, 1 << 16
    g = torch.Generator().manual_seed(5)
    a = (0.9 + 0.0999 * torch.rand(B, T, generator=g)).cuda()
    x = torch.randn(B, T, generator=g).cuda()
    zi = torch.randn(B, generator=g).cuda()
    gy = torch.randn(B, T, generator=g).cuda()
    old = sharded.FIXUP_BLOCK
    sharded.FIXUP_BLOCK = 1 << 10
    try:
        ins = [t.clone().requires_grad_() for t in (a, zi, x)]
        y = sharded.time_sharded_linear_recurrence(ins[0], ins[1], ins[2], segments=segments)
        ga, gzi, gx = torch.autograd.grad(y, ins, gy)
    finally:
        sharded.FIXUP_BLOCK = old
    ref = [t.clone().requires_grad_() for t in (a, zi, x)]
    y_r = ptb.lpv.linear_recurrence(ref[0], ref[1], ref[2])
    ga_r, gzi_r, gx_r = torch.autograd.grad(y_r, ref, gy)
    assert rel_err(y, y_r) <= 1e-4 and rel_err(gx, gx_r) <= 1e-4
    assert rel_err(ga, ga_r) <= 1e-4 and rel_err(gzi, gzi_r) <= 1e-4
    ptb.check_errors()
