#!/usr/bin/env python
"""Benchmark of the linear-recurrence hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step = one forward + one backward pass of the first-order recurrence with per-sample
coefficients (B = 256 channels, T = 2^20 samples, fp32; gradients w.r.t. x, a and the initial
state) over one batch of seeded synthetic input.  One JSON line is printed by rank 0.

* ``value``        samples/s of the whole job (all ranks), inputs resident in HBM, timed with CUDA
                   events between a barrier + synchronize on both sides, max over ranks.
* ``e2e``          the same metric through the host-buffer entry point: every step uploads the
                   inputs from pinned host memory and downloads all results.
* ``roofline``     algorithmic bytes of the backward launch / its mean duration (CUDA events on the
                   launching stream inside the timed region) against the measured copy bandwidth.
* ``cpu_baseline`` the reference project's own CPU extension (compiled into oracle/_ref), forward
                   + backward on a bounded sample of the same workload, on this machine's cores.

Multi-GPU (launched by torchrun): the batch axis is sharded, every rank runs the full per-GPU
workload on its own rows (weak scaling, no data-path collective).

``--impl reference`` times only the reference CPU extension (rank 0; other ranks exit).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fwd+bwd filter samples/s"
UNIT = "samples/s"
B, T = 256, 1 << 20
WORKLOAD = "LPV first-order linear_recurrence fwd+bwd (grads x, a, zi), fp32, B=256, T=2^20"
BYTES_FWD, BYTES_BWD = 12, 20          # algorithmic bytes per sample: r a,x w y | r gy,a,y w gx,ga
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one backward launch at the bench size, scaled
# from the ncu capture summarised in profiles/first_order_lpv_fwd_bwd_ncu.md.
NCU_TRAFFIC_BWD_BYTES = 4 * 1300032256   # 64-row capture x 4 (traffic is proportional to rows)


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.gpu = gpu_index
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            f = [s.strip() for s in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        # samples under load = the upper half of the clock readings
        sm_sorted = sorted(sm)
        load = sm_sorted[len(sm_sorted) // 2:] if sm_sorted else []
        return {"sm_mhz": statistics.median(load) if load else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------ CPU reference
def cpu_reference_run(steps: int, warmup: int, sample_T: int):
    """Forward + backward of the same op on the host cores with the reference's own CPU extension
    (oracle/_ref, compiled from its sources) or, if that binary is absent, the C oracle port."""
    import torch
    from philtorch_b200 import workloads
    from oracle import cport, refext

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    w = workloads.lpv_first_order(B=B, T=sample_T)
    a, zi, x, gy = w["a"], w["zi"], w["x"], w["gy"]
    if refext.available():
        kind = "reference"

        def step():
            y = refext.recur1(a, zi, x)
            return refext.recur1_bwd(a, zi, y, gy)
    else:
        kind = "port"

        def step():
            y = cport.recur1(a, zi, x)
            return cport.recur1_bwd(a, zi, y, gy)
    for _ in range(max(1, warmup)):
        step()
    ts = []
    for _ in range(max(1, steps)):
        t0 = time.perf_counter()
        step()
        ts.append(time.perf_counter() - t0)
    t = statistics.median(ts)
    return {"value": B * sample_T / t, "unit": UNIT, "cores": min(cores, B), "kind": kind,
            "sample": f"B={B}, T={sample_T} (1/{T // sample_T} of the workload's time axis), "
                      f"median of {len(ts)} fwd+bwd passes, {1e3 * t:.1f} ms each"}, t


def run_reference_arm(args, rank: int):
    if rank != 0:
        return
    steps = max(1, args.steps)
    base, t = cpu_reference_run(steps, args.warmup, sample_T=1 << 16)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": steps, "warmup": args.warmup, "ms_per_step": 1e3 * t, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded)",
            "config": {"workload": WORKLOAD, "note": "each step is a bounded sample: " + base["sample"]},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------ GPU arm
def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist

    import philtorch_b200 as ptb
    from philtorch_b200 import workloads
    from philtorch_b200.host import HostPipeline

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ops = torch.ops.philtorch_b200

    B = args.rows
    w = workloads.lpv_first_order(B=B, T=T, device=dev)   # this rank's rows (batch-sharded job)
    a, zi, x, gy = w["a"], w["zi"], w["x"], w["gy"]

    def step(ev=None):
        if ev:
            ev[0].record()
        y = ops.lpv_recur(a, zi, x)
        if ev:
            ev[1].record()
        out = ops.lpv_recur_bwd(a, zi, y, gy, None, True, True)
        if ev:
            ev[2].record()
        return y, out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_start.record()
    for k in range(args.steps):
        step(evs[k])
    t_end.record()
    barrier()
    ms_total = t_start.elapsed_time(t_end)
    clocks = sampler.stop() if sampler else None
    ptb.check_errors(dev)
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in evs)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in evs)

    if args.kernels_only:
        if rank == 0:
            print(json.dumps({"profile_case": True, "rows": B, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
                              "fwd_gbs": BYTES_FWD * B * T / fwd_ms / 1e6, "bwd_gbs": BYTES_BWD * B * T / bwd_ms / 1e6}))
        if world > 1:
            dist.destroy_process_group()
        return
    # ---- end to end through the host-buffer entry point (pinned host memory in and out)
    e2e_steps = max(1, min(args.steps, 3))
    host = {k: v.cpu().pin_memory() for k, v in (("a", a), ("zi", zi), ("x", x), ("gy", gy))}
    out = {"y": torch.empty_like(host["x"]).pin_memory(), "grad_a": torch.empty_like(host["x"]).pin_memory(),
           "grad_x": torch.empty_like(host["x"]).pin_memory(), "grad_zi": torch.empty_like(host["zi"]).pin_memory()}
    pipe = HostPipeline(B, T, torch.float32, dev)
    pipe.run(host["a"], host["zi"], host["x"], host["gy"], out)   # warm-up
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        pipe.run(host["a"], host["zi"], host["x"], host["gy"], out)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    ptb.check_errors(dev)

    times = torch.tensor([ms_total, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms = times.tolist()

    if rank == 0:
        peak, peak_kind = measured_peak()
        nsamp = B * T
        achieved = BYTES_BWD * nsamp / (bwd_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": world * nsamp * args.steps / (ms_total * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded, generated on device)",
            "config": {"workload": WORKLOAD if B == 256 else WORKLOAD.replace("B=256", f"B={B}"), "rows_per_gpu": B, "sharding": "batch axis, no collective",
                       "l2": "inputs (1 GiB per array) exceed the 126 MB L2, no flush needed"},
            "roofline": {"bound": "hbm", "kernel": "scan_kernel<FoBwd<float,LPV>> (adjoint scan)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": f"{peak_kind} copy bandwidth", "traffic": NCU_TRAFFIC_BWD_BYTES,
                         "algorithmic_bytes_per_launch": BYTES_BWD * nsamp, "launch_ms": bwd_ms,
                         "forward": {"achieved": BYTES_FWD * nsamp / (fwd_ms * 1e-3) / 1e9, "launch_ms": fwd_ms,
                                     "frac": BYTES_FWD * nsamp / (fwd_ms * 1e-3) / 1e9 / peak},
                         "fwd_plus_bwd_frac": (BYTES_FWD + BYTES_BWD) * nsamp / ((fwd_ms + bwd_ms) * 1e-3) / 1e9 / peak},
            "e2e": {"value": world * nsamp * e2e_steps / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": pipe.h2d_bytes, "d2h_bytes_per_step": pipe.d2h_bytes,
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                    "api": "philtorch_b200.host.HostPipeline.run (pinned host buffers in and out)"},
            "gpu_launches": 2 * args.steps,
            "clocks": clocks,
        }
        if world == 1:
            base, _ = cpu_reference_run(steps=3, warmup=1, sample_T=1 << 18)
            line["cpu_baseline"] = base
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_time_sharded(args, rank: int, world: int, local_rank: int):
    """Secondary line (not the headline metric): the long-sequence configuration, B = 8 rows of
    T = 2^28 samples split along TIME over the ranks (strong scaling): per rank and direction one pass
    over the shard (cut into segments the kernels see as rows), one all-gather of (B,2) maps when
    there is more than one rank, and a fix-up over the few thousand samples the incoming state reaches."""
    import torch
    import torch.distributed as dist

    import philtorch_b200 as ptb
    from philtorch_b200 import workloads
    from philtorch_b200.sharded import time_sharded_linear_recurrence

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    Bl, Ttot = 8, 1 << args.log2_T
    Tl = Ttot // world
    w = workloads.long_first_order(B=Bl, T=Tl, device=dev)   # this rank's time range (seeded per rank)
    a, x, gy = w["a"].requires_grad_(), w["x"].requires_grad_(), w["gy"]
    zi = torch.zeros(Bl, device=dev, requires_grad=True)

    def step():
        y = time_sharded_linear_recurrence(a, zi, x)
        return torch.autograd.grad(y, (a, zi, x), gy)

    for _ in range(max(3, args.warmup)):
        step()
    dist.barrier(); torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    dist.barrier(); torch.cuda.synchronize(dev)
    ptb.check_errors(dev)
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = t.item() / args.steps
        peak, kind = measured_peak()
        print(json.dumps({"metric": METRIC, "value": Bl * Ttot / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
                          "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
                          "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                          "data": "synthetic (seeded, generated on device)",
                          "config": {"workload": f"time-sharded LPV first-order fwd+bwd, fp32, B=8, T=2^{args.log2_T}",
                                     "sharding": "time axis, one (B,2) all-gather per direction"},
                          "roofline": {"bound": "hbm", "achieved": 32 * Bl * Ttot / world / (ms * 1e-3) / 1e9,
                                       "peak": peak, "unit": "GB/s", "peak_source": f"{kind} copy bandwidth",
                                       "frac": 32 * Bl * Ttot / world / (ms * 1e-3) / 1e9 / peak,
                                       "note": "algorithmic 32 B/sample per GPU; folds and fix-ups are overhead"}}),
              flush=True)
    dist.destroy_process_group()


def run_sos_cascade(args):
    """Secondary line (not the headline metric): six second-order sections, B = 512, T = 2^18, fp32,
    forward + backward with gradients for x, b and a, through ``lti.sosfilt`` (fused passes) and,
    for comparison, through six chained ``lti.lfilter`` calls (how the reference runs a cascade)."""
    import torch

    import philtorch_b200 as ptb
    from philtorch_b200 import workloads

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    Bc, Tc, K = args.rows if args.rows != B else 512, 1 << 18, 6
    w = workloads.sos_cascade(B=Bc, T=Tc, sections=K, device=dev)
    b, a, x, gy = w["b"].requires_grad_(), w["a"].requires_grad_(), w["x"].requires_grad_(), w["gy"]

    def fused():
        return torch.autograd.grad(ptb.lti.sosfilt(b, a, x), (b, a, x), gy)

    def chained():
        u = x
        for k in range(K):
            u = ptb.lti.lfilter(b[k], a[k], u)
        return torch.autograd.grad(u, (b, a, x), gy)

    def timed(fn):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / args.steps

    ms, ms_chain = timed(fused), timed(chained)
    ptb.check_errors(dev)
    peak, kind = measured_peak()
    n = Bc * Tc
    # bytes per input sample: forward one pass reading x and writing the K section outputs (kept for
    # the backward), backward one pass reading gy, x and the K outputs and writing grad_x
    alg = (4 * (K + 1) + 4 * (K + 3)) * n
    print(json.dumps({"metric": METRIC, "value": n / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
                      "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                      "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded, generated on device)",
                      "config": {"workload": f"cascade of {K} second-order sections fwd+bwd (x, b, a grads), fp32, "
                                             f"B={Bc}, T=2^18", "inputs": "larger than L2"},
                      "chained_single_sections_ms": ms_chain,
                      "roofline": {"bound": "hbm", "achieved": alg / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                                   "peak_source": f"{kind} copy bandwidth", "frac": alg / (ms * 1e-3) / 1e9 / peak,
                                   "note": f"algorithmic {alg // n} B per input sample (chained sections: {24 * K} B)"}}),
          flush=True)


def _secondary_line(args, workload: str, n: int, ms: float, alg_bytes_per_sample: int, extra: dict):
    peak, kind = measured_peak()
    alg = alg_bytes_per_sample * n
    line = {"metric": METRIC, "value": n / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": extra.pop("dtype", "f32"), "data": "synthetic (seeded, generated on device)",
            "config": {"workload": workload, "inputs": "larger than L2"},
            "roofline": {"bound": "hbm", "achieved": alg / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "peak_source": f"{kind} copy bandwidth", "frac": alg / (ms * 1e-3) / 1e9 / peak,
                         "note": f"algorithmic {alg_bytes_per_sample} B per sample"}}
    line.update(extra)
    print(json.dumps(line), flush=True)


def _timed(fn, args, dev):
    import torch
    for _ in range(max(3, args.warmup)):
        fn()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize(dev)
    return e0.elapsed_time(e1) / args.steps


def run_state_space(args):
    """Secondary line: time-varying 2x2 state-space recursion (scalar input into state 0), B = 128,
    T = 2^20, forward + backward with gradients for x and A, fp32 or fp64 (--f64)."""
    import torch

    import philtorch_b200 as ptb
    from philtorch_b200 import workloads

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dt = torch.float64 if args.f64 else torch.float32
    Bc, Tc = (args.rows if args.rows != B else 128), 1 << 20
    w = workloads.lpv_second_order(B=Bc, T=Tc, dtype=dt, device=dev)
    A, x, zi, gy = w["A"].requires_grad_(), w["x"].requires_grad_(), w["zi"], w["gy"]

    def step():
        return torch.autograd.grad(ptb.lpv.state_space_recursion(A, zi, x), (A, x), gy)

    ms = _timed(step, args, dev)
    ptb.check_errors(dev)
    s = 8 if args.f64 else 4
    _secondary_line(args, f"LPV 2x2 state_space_recursion fwd+bwd (grads x, A), {'fp64' if args.f64 else 'fp32'}, "
                          f"B={Bc}, T=2^20", Bc * Tc, ms, 20 * s, {"dtype": "f64" if args.f64 else "f32"})


def run_lpv_lfilter(args):
    """Secondary line: time-varying second-order filter ``lpv.lfilter(form='df2')``, B = 128, T = 2^20,
    fp32, forward + backward with gradients for b, a and x."""
    import math

    import torch

    import philtorch_b200 as ptb

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    Bc, Tc = (args.rows if args.rows != B else 128), 1 << 20
    g = torch.Generator(device=dev).manual_seed(SEED_LPV)
    r = 0.3 + 0.65 * torch.rand(Bc, Tc, device=dev, generator=g)
    th = math.pi * torch.rand(Bc, Tc, device=dev, generator=g)
    a = torch.stack([-2 * r * torch.cos(th), r * r], -1).requires_grad_()
    b = torch.randn(Bc, Tc, 3, device=dev, generator=g).requires_grad_()
    x = torch.randn(Bc, Tc, device=dev, generator=g).requires_grad_()
    gy = torch.randn(Bc, Tc, device=dev, generator=g)
    del r, th

    def step():
        return torch.autograd.grad(ptb.lpv.lfilter(b, a, x), (b, a, x), gy)

    ms = _timed(step, args, dev)
    ptb.check_errors(dev)
    _secondary_line(args, f"LPV lfilter df2 (order 2) fwd+bwd (grads b, a, x), fp32, B={Bc}, T=2^20", Bc * Tc, ms,
                    36 + 60, {})


def run_complex_poles(args):
    """Secondary line: complex first-order recurrence, the inner call of ``diag_state_space`` on
    complex poles: 256 rows (e.g. 64 signals x 4 poles) of 2^19 complex samples, forward + backward
    with gradients for the poles and x; complex64, or complex128 with --f64.  With --per-sample the
    poles vary per sample (the per-sample-coefficient kernels)."""
    import math

    import torch

    import philtorch_b200 as ptb

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    rdt = torch.float64 if args.f64 else torch.float32
    Bc, Tc = (args.rows if args.rows != B else 256), 1 << 19
    g = torch.Generator(device=dev).manual_seed(SEED_LPV + 1)
    shape = (Bc, Tc) if args.per_sample else (Bc,)
    a = torch.polar(0.9 + 0.099 * torch.rand(*shape, device=dev, generator=g, dtype=rdt),
                    2 * math.pi * torch.rand(*shape, device=dev, generator=g, dtype=rdt)).requires_grad_()
    x = torch.view_as_complex(torch.randn(Bc, Tc, 2, device=dev, generator=g, dtype=rdt)).requires_grad_()
    gy = torch.view_as_complex(torch.randn(Bc, Tc, 2, device=dev, generator=g, dtype=rdt))
    zi = torch.zeros(Bc, device=dev, dtype=x.dtype)
    fn = ptb.lpv.linear_recurrence if args.per_sample else ptb.lti.linear_recurrence

    def step():
        return torch.autograd.grad(fn(a, zi, x), (a, x), gy)

    ms = _timed(step, args, dev)
    ptb.check_errors(dev)
    s = 16 if args.f64 else 8
    units = (3 + 5) if args.per_sample else (2 + 3)   # arrays read or written, forward + backward
    name = "complex128" if args.f64 else "complex64"
    _secondary_line(args, f"complex first-order {'per-sample' if args.per_sample else 'time-invariant'} recurrence "
                          f"fwd+bwd (grads a, x), {name}, B={Bc}, T=2^19", Bc * Tc, ms, units * s,
                    {"dtype": "c128" if args.f64 else "c64"})


def run_callers(args):
    """Secondary lines for the callers that are pure first-order passes (one per invocation):
    --comb-filter   y[t] = x[t] - a y[t-1000], B = 64, T = 2^22, fp32, fwd+bwd (grads a, x);
    --cubic-spline  cspline coefficients (parallel form), B = 64, T = 2^22, fp32, fwd+bwd (grad x);
    --diag-ssm      4th-order real system with complex poles through diag_state_space (B (M,), C (M,)),
                    B = 64, T = 2^20, fp32, fwd+bwd (grads x, L)."""
    import math

    import torch

    import philtorch_b200 as ptb
    from philtorch_b200.lti.interp import cspline

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(SEED_LPV + 2)
    Bc = args.rows if args.rows != B else 64
    if args.comb_filter:
        Tc, delay = 1 << 22, 1000
        a = (torch.rand(Bc, device=dev, generator=g) * 1.8 - 0.9).requires_grad_()
        x = torch.randn(Bc, Tc, device=dev, generator=g).requires_grad_()
        gy = torch.randn(Bc, Tc, device=dev, generator=g)
        step = lambda: torch.autograd.grad(ptb.lti.comb_filter(a, delay, x), (a, x), gy)   # noqa: E731
        name, alg = f"comb_filter delay={delay} fwd+bwd (grads a, x), fp32, B={Bc}, T=2^22", 8 + 12
    elif args.cubic_spline:
        Tc = 1 << 22
        x = torch.randn(Bc, Tc, device=dev, generator=g).requires_grad_()
        gy = torch.randn(Bc, Tc, device=dev, generator=g)
        step = lambda: torch.autograd.grad(cspline(x), (x,), gy)   # noqa: E731
        # two kernel passes per direction: causal (read x, write h) and reverse-time with the fused
        # combination (read x and h, write c); a single pass (16 B in total) cannot form a two-sided filter
        name, alg = f"cspline (parallel form) fwd+bwd (grad x), fp32, B={Bc}, T=2^22", 2 * (8 + 12)
    else:
        Tc, M = 1 << 20, 4
        r = 0.9 + 0.09 * torch.rand(M // 2, device=dev, generator=g)
        th = math.pi * torch.rand(M // 2, device=dev, generator=g)
        half = torch.polar(r, th)
        L = torch.cat([half, half.conj()]).requires_grad_()                     # conjugate pole pairs
        V = torch.view_as_complex(torch.randn(M // 2, M, 2, device=dev, generator=g))
        V = torch.cat([V, V.conj()]).T.contiguous()                              # conjugate eigenvector pairs
        x = torch.randn(Bc, Tc, device=dev, generator=g).requires_grad_()
        gy = torch.randn(Bc, Tc, device=dev, generator=g)
        Bm, Cm = torch.randn(M, device=dev, generator=g), torch.randn(M, device=dev, generator=g)
        step = lambda: torch.autograd.grad(ptb.lti.diag_state_space(x, L=L, V=V, B=Bm, C=Cm), (x, L), gy)   # noqa: E731
        name, alg = f"diag_state_space M={M} (complex pole pairs, B (M,), C (M,)) fwd+bwd (grads x, L), fp32, " \
                    f"B={Bc}, T=2^20", 8 + 8
    ms = _timed(step, args, dev)
    ptb.check_errors(dev)
    _secondary_line(args, name, Bc * Tc, ms, alg, {})


SEED_LPV = 1240


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    # reduced cases for profiler captures (never a bench value): fewer rows, device-resident loop only
    ap.add_argument("--rows", type=int, default=B, help="rows per GPU (default: the benchmark's 256)")
    ap.add_argument("--kernels-only", action="store_true", help="skip the host-buffer and CPU legs")
    ap.add_argument("--time-sharded", action="store_true",
                    help="secondary workload: B=8 long rows split along time over the ranks")
    ap.add_argument("--log2-T", type=int, default=28, dest="log2_T", help="total row length of --time-sharded")
    ap.add_argument("--state-space", action="store_true",
                    help="secondary workload: LPV 2x2 state-space recursion, B=128, T=2^20 (one GPU)")
    ap.add_argument("--lpv-lfilter", action="store_true",
                    help="secondary workload: time-varying second-order lfilter, B=128, T=2^20 (one GPU)")
    ap.add_argument("--f64", action="store_true", help="float64 for --state-space, complex128 for --complex-poles")
    ap.add_argument("--complex-poles", action="store_true",
                    help="secondary workload: complex first-order recurrence, B=256, T=2^19 (one GPU)")
    ap.add_argument("--per-sample", action="store_true", help="--complex-poles with per-sample coefficients")
    ap.add_argument("--comb-filter", action="store_true", help="secondary workload: comb filter (one GPU)")
    ap.add_argument("--cubic-spline", action="store_true", help="secondary workload: cubic spline coefficients (one GPU)")
    ap.add_argument("--diag-ssm", action="store_true", help="secondary workload: diag_state_space, 4 complex modes (one GPU)")
    ap.add_argument("--sos-cascade", action="store_true",
                    help="secondary workload: six fused second-order sections, B=512, T=2^18 (one GPU)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    secondary = [fn for flag, fn in ((args.sos_cascade, run_sos_cascade), (args.state_space, run_state_space),
                                     (args.lpv_lfilter, run_lpv_lfilter), (args.complex_poles, run_complex_poles),
                                     (args.comb_filter or args.cubic_spline or args.diag_ssm, run_callers))
                 if flag]
    if secondary:
        if rank == 0:
            secondary[0](args)
        return
    if args.time_sharded:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29512")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        run_time_sharded(args, rank, world, local_rank)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
