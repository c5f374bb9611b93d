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
* ``configs``      (one GPU) the five benchmark configurations, each forward + backward through the
                   public API at full size: ms per step, samples/s, algorithmic bytes, fraction of
                   the measured copy bandwidth and of the nominal 8 TB/s, and ``parity`` =
                   max|out - ref| / max|ref| of the output and of every gradient against the CPU
                   oracle at full size.
* ``callers``      (one GPU) the filters that reduce to first-order passes (comb_filter at 64 and 16
                   rows, cspline, diag_state_space): ms per step and fraction of the copy bandwidth.

Multi-GPU (launched by torchrun): the headline ``value`` is the batch-sharded job, every rank
running the full per-GPU workload on its own rows (weak scaling, no data-path collective).  The
same line then carries two strong-scaling measurements: ``time_sharded`` (B = 8 rows of 2^28
samples split along time over the ranks: local scan, one all-gather of (B,2) maps per direction,
fix-up; parity of every rank's shard edges against the oracle) and ``strong`` (the rows of
configurations 1-4 split evenly over the ranks).

``--impl reference`` times only the reference CPU extension (rank 0; other ranks exit).
"""
from __future__ import annotations

import argparse
import importlib.util
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
NOMINAL_HBM_GBS = 8000.0               # the peak the target fraction (>= 0.70) is stated against
# dram__bytes_read.sum + dram__bytes_write.sum of one backward launch at the bench size, scaled
# from an ncu capture of a 64-row case (traffic is proportional to rows).
NCU_TRAFFIC_BWD_BYTES = 4 * 1300032256


def bench_config(rows: int) -> dict:
    """The ``config`` object; identical in both arms for the same rows per GPU."""
    return {"workload": WORKLOAD if rows == 256 else WORKLOAD.replace("B=256", f"B={rows}"),
            "rows_per_gpu": rows, "sharding": "batch axis, no collective",
            "l2": "inputs (1 GiB per array) exceed the 126 MB L2, no flush needed"}


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def load_workloads():
    """The input generators, loaded from their file: importing the package would load the CUDA
    library, which the reference arm must not touch."""
    spec = importlib.util.spec_from_file_location("_ptb_workloads", os.path.join(ROOT, "philtorch_b200", "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


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
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
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
    (oracle/_ref, compiled from its sources) or, if that binary is absent, the C oracle port.
    Loads nothing of the product: the inputs come from the generator file, the arithmetic from
    oracle/."""
    import torch
    from oracle import cport, refext

    workloads = load_workloads()
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
    frac = "the whole workload" if sample_T == T else f"1/{T // sample_T} of the workload's time axis"
    return {"value": B * sample_T / t, "unit": UNIT, "cores": min(cores, B), "kind": kind,
            "sample": f"B={B}, T={sample_T} ({frac}), median of {len(ts)} fwd+bwd passes, {1e3 * t:.1f} ms each; "
                      f"host has {cores} logical cores, the extension runs one row per OpenMP thread"}, t


def run_reference_arm(args, rank: int):
    if rank != 0:
        return
    steps = max(1, args.steps)
    base, t = cpu_reference_run(steps, args.warmup, sample_T=T)   # the workload itself, every step
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": steps, "warmup": args.warmup, "ms_per_step": 1e3 * t, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded)",
            "config": bench_config(B),
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------ GPU arm: helpers
def _events(n):
    import torch
    return [torch.cuda.Event(enable_timing=True) for _ in range(n)]


def _time_steps(fn, steps: int, warmup: int, dev, barrier=None) -> float:
    """ms per call of fn: warm-up, then `steps` calls between two events on the current stream."""
    import torch
    for _ in range(max(3, warmup)):
        fn()
    (barrier or (lambda: torch.cuda.synchronize(dev)))()
    e0, e1 = _events(2)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    (barrier or (lambda: torch.cuda.synchronize(dev)))()
    return e0.elapsed_time(e1) / steps


class Parity:
    """max|out - ref| / max|ref| per named quantity, accumulated over row or time blocks; the
    differences are taken on the device in float64."""

    def __init__(self, dev):
        self.dev, self.err, self.ref = dev, {}, {}

    def add(self, name: str, out, ref_cpu):
        import torch
        ref = ref_cpu.to(self.dev, non_blocking=False).to(torch.float64)
        e = (out.detach().to(torch.float64) - ref).abs().max().item() if ref.numel() else 0.0
        r = ref.abs().max().item() if ref.numel() else 0.0
        self.err[name] = max(self.err.get(name, 0.0), e)
        self.ref[name] = max(self.ref.get(name, 0.0), r)

    def result(self) -> dict:
        return {k: self.err[k] / (self.ref[k] if self.ref[k] > 0 else 1.0) for k in self.err}


def _entry(workload, api, n_samples, ms, alg_bytes, parity, dtype="f32", **extra):
    peak, kind = measured_peak()
    gbs = alg_bytes * n_samples / (ms * 1e-3) / 1e9
    tol = 1e-4 if dtype == "f32" else 1e-10
    e = {"workload": workload, "api": api, "dtype": dtype, "ms_per_step": ms, "samples_per_s": n_samples / (ms * 1e-3),
         "algorithmic_bytes_per_sample": alg_bytes, "achieved_gbs": gbs, "frac": gbs / peak,
         "frac_of": f"{kind} copy bandwidth {peak:.1f} GB/s", "frac_of_nominal_8tbs": gbs / NOMINAL_HBM_GBS}
    if parity is not None:
        e["parity"] = parity
        e["parity_max"] = max(parity.values()) if parity else None
        e["parity_tolerance"] = tol
        e["parity_ok"] = bool(parity) and max(parity.values()) <= tol
        e["parity_against"] = extra.pop("parity_against", "CPU oracle at full size")
    e.update(extra)
    return e


def _free():
    import gc
    import torch
    gc.collect()
    torch.cuda.empty_cache()


def _oracle_kind():
    from oracle import refext
    return "reference CPU extension (oracle/_ref)" if refext.available() else "C oracle (oracle/recur_oracle.c)"


def _graph_ms(fn, dev, reps: int = 50):
    """ms per replay of fn captured in a CUDA graph (launch overhead of the host removed), or None."""
    import torch
    try:
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize(dev)
        e0, e1 = _events(2)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / reps
    except Exception:
        return None


# ------------------------------------------------------------------------------------ the five configurations
def config1(dev, steps, warmup, rows=64, shard=0, parity=True):
    """LTI first order, B=64, T=65536, fp32; grads x, a (20 B/sample)."""
    import torch
    import philtorch_b200 as ptb
    from philtorch_b200 import workloads
    ops = torch.ops.philtorch_b200
    Tc = 65536
    w = workloads.lti_first_order(B=rows, T=Tc, device=dev, shard=shard)
    a, zi, x, gy = w["a"].requires_grad_(), w["zi"], w["x"].requires_grad_(), w["gy"]

    def step():
        return torch.autograd.grad(ptb.lti.linear_recurrence(a, zi, x), (a, x), gy)

    ms = _time_steps(step, steps, warmup, dev)
    ad, xd = a.detach(), x.detach()

    def raw():
        y = ops.lti_recur(ad, zi, xd)
        return ops.lti_recur_bwd(ad, zi, y, gy, None, True, False)

    ms_raw = _time_steps(raw, steps, warmup, dev)
    ms_graph = _graph_ms(raw, dev)

    class Floor(torch.autograd.Function):   # the same call pattern with no kernel behind it
        @staticmethod
        def forward(ctx, a_, zi_, x_):
            ctx.save_for_backward(a_, zi_, x_)
            return torch.empty_like(x_)

        @staticmethod
        def backward(ctx, g):
            a_, _, _ = ctx.saved_tensors
            return torch.empty_like(a_), None, torch.empty_like(g)

    ms_floor = _time_steps(lambda: torch.autograd.grad(Floor.apply(a, zi, x), (a, x), gy), steps, warmup, dev)
    par = None
    if parity:
        from oracle import cport, refext
        o = refext if refext.available() else cport
        y = ptb.lti.linear_recurrence(a, zi, x)
        ga, gx = torch.autograd.grad(y, (a, x), gy)
        ac, zc, xc, gc = ad.cpu(), zi.cpu(), xd.cpu(), gy.cpu()
        y_r = o.lti_recur(ac, zc, xc)
        ga_r, _, gx_r = o.lti_recur_bwd(ac, zc, y_r, gc)
        P = Parity(dev)
        P.add("y", y, y_r); P.add("grad_a", ga, ga_r); P.add("grad_x", gx, gx_r)
        par = P.result()
    return _entry(f"LTI first-order linear_recurrence fwd+bwd (grads x, a), fp32, B={rows}, T=65536",
                  "lti.linear_recurrence + autograd.grad (eager)", rows * Tc, ms, 20, par,
                  eager_ops_ms=ms_raw, cuda_graph_ms=ms_graph, torch_autograd_floor_ms=ms_floor,
                  note="84 MB in total: launch- and latency-bound; cuda_graph_ms = the two ops replayed from a CUDA "
                       "graph; torch_autograd_floor_ms = an autograd.Function that only allocates its outputs, "
                       "called and differentiated the same way (host time of torch itself)",
                  **({"parity_against": _oracle_kind() + " at full size"} if parity else {}))


def config2_parity(dev, a, zi, x, gy, y, ga, gzi, gx, block=64):
    """Full-size parity of the headline workload, row block by row block (rows are independent)."""
    from oracle import cport, refext
    o = refext if refext.available() else cport
    P = Parity(dev)
    for r0 in range(0, x.shape[0], block):
        sl = slice(r0, min(x.shape[0], r0 + block))
        ac, zc, xc, gc = a[sl].cpu(), zi[sl].cpu(), x[sl].cpu(), gy[sl].cpu()
        y_r = o.recur1(ac, zc, xc)
        ga_r, gzi_r, gx_r = o.recur1_bwd(ac, zc, y_r, gc)
        P.add("y", y[sl], y_r); P.add("grad_a", ga[sl], ga_r); P.add("grad_x", gx[sl], gx_r)
        P.add("grad_zi", gzi[sl], gzi_r)
    return P.result()


def config3(dev, steps, warmup, rows=512, shard=0, parity=True, graph=False):
    """Six TDF-II sections, B=512, T=2^18, fp32; grads b, a, x.  Two routes: six lti.lfilter calls (how
    the reference API runs a cascade, 24 B/sample per section) and lti.sosfilt (one fused pass per
    direction, 64 B/sample)."""
    import torch
    import philtorch_b200 as ptb
    from philtorch_b200 import workloads
    Tc, K = 1 << 18, 6
    w = workloads.sos_cascade(B=rows, T=Tc, sections=K, device=dev, shard=shard)
    b, a, x, gy = w["b"].requires_grad_(), w["a"].requires_grad_(), w["x"].requires_grad_(), w["gy"]

    def chained():
        u = x
        for bk, ak in zip(b, a):          # iterating a tensor unbinds it: one stack in the backward pass
            u = ptb.lti.lfilter(bk, ak, u)
        return u

    def fused():
        return ptb.lti.sosfilt(b, a, x)

    ms_c = _time_steps(lambda: torch.autograd.grad(chained(), (b, a, x), gy), steps, warmup, dev)
    ms_f = _time_steps(lambda: torch.autograd.grad(fused(), (b, a, x), gy), steps, warmup, dev)
    ms_fg = _graph_ms(lambda: torch.autograd.grad(fused(), (b, a, x), gy), dev, reps=steps) if graph else None
    par_c = par_f = None
    if parity:
        from oracle import cport
        outs = {}
        for name, fn in (("lfilter", chained), ("sosfilt", fused)):
            y = fn()
            outs[name] = (y.detach(),) + torch.autograd.grad(y, (b, a, x), gy)
        Pc, Pf = Parity(dev), Parity(dev)
        bd, ad, xd = b.detach(), a.detach(), x.detach()
        for r0 in range(0, rows, 128):
            sl = slice(r0, min(rows, r0 + 128))
            bc, ac = bd[:, sl].cpu(), ad[:, sl].cpu()
            ins, y_r = cport.sos_chain(bc, ac, xd[sl].cpu())
            gb_r, ga_r, gx_r = cport.sos_chain_bwd(bc, ac, ins, gy[sl].cpu())
            for P, (y, gb, ga, gx) in ((Pc, outs["lfilter"]), (Pf, outs["sosfilt"])):
                P.add("y", y[sl], y_r); P.add("grad_x", gx[sl], gx_r)
                for k in range(K):   # per section: their gradients differ by orders of magnitude
                    P.add(f"grad_b[{k}]", gb[k, sl], gb_r[k]); P.add(f"grad_a[{k}]", ga[k, sl], ga_r[k])
        par_c, par_f = Pc.result(), Pf.result()
    name = f"cascade of 6 second-order sections (TDF-II) fwd+bwd (grads b, a, x), fp32, B={rows}, T=2^18"
    against = {"parity_against": "C oracle (oracle/recur_oracle.c, pinned to the reference's golden vectors) at full size"} \
        if parity else {}
    return (_entry(name, "six chained lti.lfilter calls + autograd.grad", rows * Tc, ms_c, 144, par_c, **against),
            _entry(name, "lti.sosfilt + autograd.grad (fused cascade)", rows * Tc, ms_f, 64, par_f, cuda_graph_ms=ms_fg,
                   note="64 B per input sample: forward reads x and writes the 6 section outputs, backward reads "
                        "gy, x and those outputs and writes grad_x; against the 144 B of six separate sections "
                        "the achieved rate would read %.0f GB/s" % (144 * rows * Tc / (ms_f * 1e-3) / 1e9), **against))


def config4(dev, steps, warmup, f64: bool, rows=128, shard=0, parity=True, graph=False):
    """LPV 2x2 state_space_recursion, B=128, T=2^20, scalar input into state 0; grads x, A (80 / 160 B/sample)."""
    import torch
    import philtorch_b200 as ptb
    from philtorch_b200 import workloads
    Tc = 1 << 20
    dt = torch.float64 if f64 else torch.float32
    w = workloads.lpv_second_order(B=rows, T=Tc, dtype=dt, device=dev, shard=shard)
    A, x, zi, gy = w["A"].requires_grad_(), w["x"].requires_grad_(), w["zi"], w["gy"]

    def fwd():
        return ptb.lpv.state_space_recursion(A, zi, x)

    ms = _time_steps(lambda: torch.autograd.grad(fwd(), (A, x), gy), steps, warmup, dev)
    ms_g = _graph_ms(lambda: torch.autograd.grad(fwd(), (A, x), gy), dev, reps=steps) if graph else None
    par = None
    if parity:
        from oracle import cport, refext
        o = refext if refext.available() else cport
        y = fwd()
        gA, gx = torch.autograd.grad(y, (A, x), gy)
        P = Parity(dev)
        Ad, xd = A.detach(), x.detach()
        blk = 16 if f64 else 32
        for r0 in range(0, rows, blk):
            sl = slice(r0, min(rows, r0 + blk))
            Ac, zc, gc = Ad[sl].cpu(), zi[sl].cpu(), gy[sl].cpu()
            xc = torch.stack([xd[sl].cpu(), torch.zeros_like(xd[sl].cpu())], -1)   # as _ext_ss_recur pads it
            y_r = o.recur2(Ac, zc, xc)
            gA_r, _, gx_r = o.recur2_bwd(Ac, zc, y_r, gc)
            P.add("y", y[sl], y_r); P.add("grad_A", gA[sl], gA_r); P.add("grad_x", gx[sl], gx_r[..., 0])
        par = P.result()
    tag = "fp64" if f64 else "fp32"
    return _entry(f"LPV 2x2 state_space_recursion fwd+bwd (grads x, A), {tag}, B={rows}, T=2^20",
                  "lpv.state_space_recursion + autograd.grad", rows * Tc, ms, 160 if f64 else 80, par,
                  dtype="f64" if f64 else "f32", cuda_graph_ms=ms_g,
                  **({"parity_against": _oracle_kind() + " at full size"} if parity else {}))


def config5_parity(dev, a, zi, x, gy, y, ga, gx, chunk=1 << 24):
    """Full-length parity of the long rows through the time-chunked oracle: forward chunks chain
    zi <- y[:, -1] (sequential arithmetic, so identical to one pass over the whole row), the adjoint
    runs over the chunks from the right chaining the adjoint state entering each chunk."""
    import torch
    from oracle import cport
    Tt = x.shape[1]
    P = Parity(dev)
    y_or = torch.empty(x.shape, dtype=x.dtype)          # the oracle's outputs, kept on the host
    state = zi.cpu()
    for t0 in range(0, Tt, chunk):
        sl = slice(t0, min(Tt, t0 + chunk))
        yc = cport.recur1(a[:, sl].cpu(), state, x[:, sl].cpu())
        P.add("y", y[:, sl], yc)
        y_or[:, sl] = yc
        state = yc[:, -1].clone()
    g_in = None
    for t0 in reversed(range(0, Tt, chunk)):
        sl = slice(t0, min(Tt, t0 + chunk))
        prev = zi.cpu() if t0 == 0 else y_or[:, t0 - 1].clone()
        ga_r, g_in, gx_r = cport.recur1_bwd(a[:, sl].cpu(), prev, y_or[:, sl], gy[:, sl].cpu(), g_in)
        P.add("grad_a", ga[:, sl], ga_r); P.add("grad_x", gx[:, sl], gx_r)
    return P.result()


def config5(dev, steps, warmup, log2_T=28, parity=True):
    """Long rows on ONE GPU: B=8, T=2^28, fp32, through lpv.linear_recurrence (which cuts few long rows
    into segments the kernels see as independent rows); 32 B/sample."""
    import torch
    import philtorch_b200 as ptb
    from philtorch_b200 import workloads
    Bc, Tc = 8, 1 << log2_T
    w = workloads.long_first_order(B=Bc, T=Tc, device=dev)
    a, x, gy = w["a"].requires_grad_(), w["x"].requires_grad_(), w["gy"]
    zi = torch.zeros(Bc, device=dev, requires_grad=True)
    del w
    _free()

    def fwd():
        return ptb.lpv.linear_recurrence(a, zi, x)

    ms = _time_steps(lambda: torch.autograd.grad(fwd(), (a, zi, x), gy), min(steps, 5), warmup, dev)
    par = None
    if parity:
        y = fwd()
        ga, _, gx = torch.autograd.grad(y, (a, zi, x), gy)
        par = config5_parity(dev, a.detach(), zi.detach(), x.detach(), gy, y.detach(), ga, gx)
    return _entry(f"long-sequence LPV first-order fwd+bwd (grads x, a, zi), fp32, B={Bc}, T=2^{log2_T}, one GPU",
                  "lpv.linear_recurrence + autograd.grad", Bc * Tc, ms, 32, par,
                  **({"parity_against": "time-chunked C oracle over the full length (2^24-sample chunks chaining "
                                        "zi <- y[:, -1]; adjoint chunks chained from the right)"} if parity else {}))


def run_configs(dev, args, main_entry):
    """The five configurations on one GPU; a failing configuration is reported, not fatal."""
    out = {"2": main_entry}
    steps = max(3, min(args.steps, 10))
    jobs = [("1", lambda: config1(dev, max(steps, 20), args.warmup)),
            ("3", lambda: config3(dev, steps, args.warmup)),
            ("4_fp32", lambda: config4(dev, steps, args.warmup, False)),
            ("4_fp64", lambda: config4(dev, steps, args.warmup, True)),
            ("5", lambda: config5(dev, steps, args.warmup))]
    for key, job in jobs:
        t0 = time.perf_counter()
        try:
            res = job()
            if key == "3":
                out["3_lfilter"], out["3_sosfilt"] = res
                res[0]["wall_s"] = res[1]["wall_s"] = round(time.perf_counter() - t0, 1)
            else:
                res["wall_s"] = round(time.perf_counter() - t0, 1)
                out[key] = res
        except Exception as e:   # keep the headline line alive
            out[key] = {"error": f"{type(e).__name__}: {e}"[:300]}
        _free()
    return out


# ------------------------------------------------------------------------------------ multi-GPU strong scaling
def time_sharded_entry(dev, args, rank, world, barrier, log2_T=28):
    """Config 5 split along time over the ranks (strong scaling), with the parity of every rank's
    shard edges: the first and last 2^22 samples of the shard against the sequential oracle run over
    a window that starts 2^16 samples inside the neighbouring shard (whose data this rank
    regenerates from the neighbour's seed; with a <= 0.999 the state entering a window has no
    influence after ~1e5 samples, so a zero state there is exact to far below the tolerance)."""
    import torch
    import torch.distributed as dist
    import philtorch_b200 as ptb
    from philtorch_b200 import workloads
    from philtorch_b200.sharded import time_sharded_linear_recurrence
    from oracle import cport

    Bl, Ttot = 8, 1 << log2_T
    Tl = Ttot // world
    w = workloads.long_first_order(B=Bl, T=Tl, device=dev, shard=rank)
    a, x, gy = w["a"].requires_grad_(), w["x"].requires_grad_(), w["gy"]
    zi = torch.zeros(Bl, device=dev, requires_grad=True)
    del w
    _free()

    def step():
        y = time_sharded_linear_recurrence(a, zi, x)
        return y, torch.autograd.grad(y, (a, zi, x), gy)

    steps = max(3, min(args.steps, 10))
    ms = _time_steps(step, steps, args.warmup, dev, barrier)
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item()
    ptb.check_errors(dev)

    # ---- parity at the shard edges
    Wn, Wu = min(1 << 22, Tl // 2), min(1 << 16, Tl // 4)
    y, (ga, gzi, gx) = step()
    y, ad, xd = y.detach(), a.detach(), x.detach()
    P = Parity(dev)
    zeros = torch.zeros(Bl)
    # forward: the first Wn samples, entered through the neighbour's last Wu samples
    if rank > 0:
        nb = workloads.long_first_order(B=Bl, T=Tl, device=dev, shard=rank - 1)
        a_w = torch.cat([nb["a"][:, -Wu:], ad[:, :Wn]], 1).cpu()
        x_w = torch.cat([nb["x"][:, -Wu:], xd[:, :Wn]], 1).cpu()
        del nb
        P.add("y", y[:, :Wn], cport.recur1(a_w, zeros, x_w)[:, Wu:])
    else:
        P.add("y", y[:, :Wn], cport.recur1(ad[:, :Wn].cpu(), zeros, xd[:, :Wn].cpu()))
    # adjoint: the last Wn samples, entered through the neighbour's first Wu samples
    lo = Tl - Wn - Wu
    y_w = cport.recur1(ad[:, lo:].cpu(), zeros, xd[:, lo:].cpu())       # oracle outputs from a warmed-up state
    a_t, g_t = ad[:, Tl - Wn:], gy[:, Tl - Wn:]
    if rank < world - 1:
        nb = workloads.long_first_order(B=Bl, T=Tl, device=dev, shard=rank + 1)
        a_t, g_t = torch.cat([a_t, nb["a"][:, :Wu]], 1), torch.cat([g_t, nb["gy"][:, :Wu]], 1)
        del nb
    y_t = torch.cat([y_w[:, Wu:], torch.zeros(Bl, a_t.shape[1] - Wn)], 1)   # beyond the shard only grad_a reads y
    ga_r, _, gx_r = cport.recur1_bwd(a_t.cpu(), y_w[:, Wu - 1].clone(), y_t, g_t.cpu())
    P.add("grad_x", gx[:, Tl - Wn:], gx_r[:, :Wn]); P.add("grad_a", ga[:, Tl - Wn:], ga_r[:, :Wn])
    par = P.result()
    errs = torch.tensor([par["y"], par["grad_x"], par["grad_a"]], dtype=torch.float64, device=dev)
    dist.all_reduce(errs, op=dist.ReduceOp.MAX)
    par = dict(zip(("y", "grad_x", "grad_a"), errs.tolist()))
    _free()
    peak, kind = measured_peak()
    gbs = 32 * Bl * Tl / (ms * 1e-3) / 1e9
    return {"workload": f"time-sharded LPV first-order fwd+bwd, fp32, B=8, T=2^{log2_T} split over {world} GPUs "
                        f"(2^{Tl.bit_length() - 1} samples per row and GPU)",
            "api": "sharded.time_sharded_linear_recurrence + autograd.grad", "scaling": "strong",
            "collective": "one NCCL all-gather of (B,2) maps per direction", "ms_per_step": ms,
            "samples_per_s": Bl * Ttot / (ms * 1e-3), "algorithmic_bytes_per_sample": 32,
            "per_gpu_achieved_gbs": gbs, "per_gpu_frac": gbs / peak, "frac_of": f"{kind} copy bandwidth {peak:.1f} GB/s",
            "parity": par, "parity_max": max(par.values()), "parity_tolerance": 1e-4,
            "parity_ok": max(par.values()) <= 1e-4,
            "parity_against": f"sequential C oracle on the first and last {Wn} samples of every rank's shard "
                              f"(windows reach {Wu} samples into the neighbouring shards), max over ranks"}


def strong_entries(dev, args, rank, world, barrier):
    """Configurations 1-4 with their rows split evenly over the ranks (B/W rows per GPU, no collective)."""
    import torch
    import torch.distributed as dist
    from philtorch_b200 import workloads
    ops = torch.ops.philtorch_b200
    peak, kind = measured_peak()
    steps = max(3, min(args.steps, 20))
    out = {}

    def finish(key, name, rows_total, Tc, alg, eager_ms, graph_ms):
        """ms_per_step = the forward+backward step replayed from a CUDA graph (per-GPU work of a few hundred
        microseconds is otherwise bound by the host's launch rate), max over ranks; eager beside it."""
        best = graph_ms if graph_ms is not None else eager_ms
        t = torch.tensor([best, eager_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, eager = t.tolist()
        rows = rows_total // world
        gbs = alg * rows * Tc / (ms * 1e-3) / 1e9
        out[key] = {"workload": name, "rows_total": rows_total, "rows_per_gpu": rows, "ms_per_step": ms,
                    "timed": "CUDA-graph replay" if graph_ms is not None else "eager", "eager_ms_per_step": eager,
                    "samples_per_s": rows * world * Tc / (ms * 1e-3), "algorithmic_bytes_per_sample": alg,
                    "per_gpu_achieved_gbs": gbs, "per_gpu_frac": gbs / peak,
                    "frac_of": f"{kind} copy bandwidth {peak:.1f} GB/s"}

    import philtorch_b200 as ptb
    rows = B // world
    w = workloads.lpv_first_order(B=rows, T=T, device=dev, shard=rank)
    a, zi, x, gy = w["a"].requires_grad_(), w["zi"].requires_grad_(), w["x"].requires_grad_(), w["gy"]

    def step2():   # the public function: it cuts a handful of long rows into segments by itself
        return torch.autograd.grad(ptb.lpv.linear_recurrence(a, zi, x), (a, zi, x), gy)

    eager = _time_steps(step2, steps, args.warmup, dev, barrier)
    finish("2", WORKLOAD + f", rows split {rows} per GPU", B, T, 32, eager, _graph_ms(step2, dev, reps=steps))
    del w, a, zi, x, gy
    _free()
    for key, fn, rows_total, Tc, alg in (
            ("1", lambda r: config1(dev, steps, args.warmup, rows=r, shard=rank, parity=False), 64, 65536, 20),
            ("3_sosfilt", lambda r: config3(dev, steps, args.warmup, rows=r, shard=rank, parity=False, graph=True)[1],
             512, 1 << 18, 64),
            ("4_fp32", lambda r: config4(dev, steps, args.warmup, False, rows=r, shard=rank, parity=False, graph=True),
             128, 1 << 20, 80)):
        try:
            barrier()
            e = fn(rows_total // world)
            finish(key, e["workload"], rows_total, Tc, alg, e["ms_per_step"], e.get("cuda_graph_ms"))
        except Exception as ex:
            out[key] = {"error": f"{type(ex).__name__}: {ex}"[:300]}
        _free()
    return out


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
    w = workloads.lpv_first_order(B=B, T=T, device=dev, shard=rank)   # this rank's rows (batch-sharded job)
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
    evs = [_events(3) for _ in range(args.steps)]
    t_start, t_end = _events(2)
    barrier()
    t_start.record()
    for k in range(args.steps):
        step(evs[k])
    t_end.record()
    barrier()
    ms_total = t_start.elapsed_time(t_end)
    # keep the device under the same load for about a second more: tens of clock samples instead
    # of the two or three that fit into the timed region itself
    t_load = time.perf_counter()
    while time.perf_counter() - t_load < 1.0:
        for _ in range(20):
            step()
        torch.cuda.synchronize(dev)
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
    e2e_steps = max(1, min(args.steps, 7))
    host = {k: v.cpu().pin_memory() for k, v in (("a", a), ("zi", zi), ("x", x), ("gy", gy))}
    out = {"y": torch.empty_like(host["x"]).pin_memory(), "grad_a": torch.empty_like(host["x"]).pin_memory(),
           "grad_x": torch.empty_like(host["x"]).pin_memory(), "grad_zi": torch.empty_like(host["zi"]).pin_memory()}
    pipe = HostPipeline(B, T, torch.float32, dev)
    pipe.run(host["a"], host["zi"], host["x"], host["gy"], out)   # warm-up
    barrier()
    # every step between its own pair of events; the reported time is the median step times the number of
    # steps (host memory and PCIe are shared with the box's other tenants: one disturbed step does not count)
    marks = _events(e2e_steps + 1)
    marks[0].record()
    for i in range(e2e_steps):
        pipe.run(host["a"], host["zi"], host["x"], host["gy"], out)
        marks[i + 1].record()
    barrier()
    e2e_ms = statistics.median(marks[i].elapsed_time(marks[i + 1]) for i in range(e2e_steps)) * e2e_steps
    ptb.check_errors(dev)
    del host, out, pipe
    _free()

    times = torch.tensor([ms_total, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms = times.tolist()

    peak, peak_kind = measured_peak()
    nsamp = B * T
    achieved = BYTES_BWD * nsamp / (bwd_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": world * nsamp * args.steps / (ms_total * 1e-3), "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded, generated on device)",
        "config": bench_config(B),
        "roofline": {"bound": "hbm", "kernel": "scan_kernel<FoBwd<float,LPV>> (adjoint scan)",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": f"{peak_kind} copy bandwidth (a 1:1 read:write copy; this kernel reads 3 arrays "
                                    "per 2 written, so fractions slightly above 1 occur)",
                     "frac_of_nominal_8tbs": achieved / NOMINAL_HBM_GBS, "traffic": NCU_TRAFFIC_BWD_BYTES,
                     "algorithmic_bytes_per_launch": BYTES_BWD * nsamp, "launch_ms": bwd_ms,
                     "forward": {"achieved": BYTES_FWD * nsamp / (fwd_ms * 1e-3) / 1e9, "launch_ms": fwd_ms,
                                 "frac": BYTES_FWD * nsamp / (fwd_ms * 1e-3) / 1e9 / peak},
                     "fwd_plus_bwd_frac": (BYTES_FWD + BYTES_BWD) * nsamp / ((fwd_ms + bwd_ms) * 1e-3) / 1e9 / peak},
        "e2e": {"value": world * nsamp * e2e_steps / (e2e_ms * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": (3 * nsamp + B) * 4, "d2h_bytes_per_step": (3 * nsamp + B) * 4,
                "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                "api": "philtorch_b200.host.HostPipeline.run (pinned host buffers in and out)",
                "timing": "median of the per-step times (CUDA events around every step), max over ranks"},
        "gpu_launches": 2 * args.steps,
        "clocks": clocks,
    }
    if world == 1 and not args.no_configs:
        # the headline workload's own entry: same numbers, plus its full-size parity
        y, (ga, gzi, gx) = step()
        t0 = time.perf_counter()
        par = config2_parity(dev, a, zi, x, gy, y, ga, gzi, gx)
        main_entry = _entry(WORKLOAD, "ops lpv_recur + lpv_recur_bwd (the ops behind lpv.linear_recurrence)", nsamp,
                            ms_total / args.steps, 32, par, parity_against=_oracle_kind() + " at full size",
                            wall_s=round(time.perf_counter() - t0, 1))
        del y, ga, gzi, gx
    del w, a, zi, x, gy
    _free()
    if world == 1:
        if not args.no_configs:
            line["configs"] = run_configs(dev, args, main_entry)
            line["callers"] = callers_entries(dev, max(3, min(args.steps, 10)), args.warmup)
        if rank == 0:
            base, _ = cpu_reference_run(steps=3, warmup=1, sample_T=1 << 18)
            line["cpu_baseline"] = base
    elif not args.no_configs:
        try:
            line["time_sharded"] = time_sharded_entry(dev, args, rank, world, barrier)
        except Exception as e:
            line["time_sharded"] = {"error": f"{type(e).__name__}: {e}"[:300]}
        _free()
        line["strong"] = strong_entries(dev, args, rank, world, barrier)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
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
        for bk, ak in zip(b, a):
            u = ptb.lti.lfilter(bk, ak, u)
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


def caller_case(dev, kind: str, Bc: int):
    """(step, workload name, algorithmic bytes per sample, samples per row) of a caller workload."""
    import math

    import torch

    import philtorch_b200 as ptb
    from philtorch_b200.lti.interp import cspline

    g = torch.Generator(device=dev).manual_seed(SEED_LPV + 2)
    if kind == "comb":
        Tc, delay = 1 << 22, 1000
        a = (torch.rand(Bc, device=dev, generator=g) * 1.8 - 0.9).requires_grad_()
        x = torch.randn(Bc, Tc, device=dev, generator=g).requires_grad_()
        gy = torch.randn(Bc, Tc, device=dev, generator=g)
        step = lambda: torch.autograd.grad(ptb.lti.comb_filter(a, delay, x), (a, x), gy)   # noqa: E731
        name, alg = f"comb_filter delay={delay} fwd+bwd (grads a, x), fp32, B={Bc}, T=2^22", 8 + 12
    elif kind == "cspline":
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
    return step, name, alg, Tc


def callers_entries(dev, steps: int, warmup: int):
    """The callers that are first-order passes, for the main line: time and fraction of the copy
    bandwidth each (their parity is the GPU tests' business: oracle, golden vectors, scipy)."""
    out = {}
    for key, kind, rows in (("comb_filter", "comb", 64), ("comb_filter_16_rows", "comb", 16), ("cspline", "cspline", 64),
                            ("diag_state_space", "diag_ssm", 64)):
        try:
            step, name, alg, Tc = caller_case(dev, kind, rows)
            ms = _time_steps(step, steps, warmup, dev)
            out[key] = _entry(name, "public API + autograd.grad", rows * Tc, ms, alg, None)
            if kind == "diag_ssm":
                out[key]["note"] = ("bound by instruction issue, not by HBM: four complex modes per sample are "
                                    "scanned in registers while x is read and y written once per pass")
            del step
        except Exception as e:   # keep the headline line alive
            out[key] = {"error": f"{type(e).__name__}: {e}"[:300]}
        _free()
    return out


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
    Bc = args.rows if args.rows != B else 64
    kind = "comb" if args.comb_filter else ("cspline" if args.cubic_spline else "diag_ssm")
    step, name, alg, Tc = caller_case(dev, kind, Bc)
    ms = _timed(step, args, dev)
    ptb.check_errors(dev)
    _secondary_line(args, name, Bc * Tc, ms, alg, {})


SEED_LPV = 1240


def run_profile_case(args):
    """Reduced cases for profiler captures (never a bench value): a few launches of one kernel family
    on inputs larger than L2 but of a few hundred MB, so that a multi-pass capture ends in a minute.
      biquad   one TDF-II section forward + backward, fp32, B=128, T=2^19
      half     first-order per-sample recurrence on float16 arrays, forward + backward, B=64, T=2^20
      modal    fused bank of 4 complex modes, forward + backward, B=32, T=2^20
      dense    4x4 per-sample recurrence forward + adjoint scan, fp32, B=16, T=2^18
      dense-lti  8x8 constant-matrix recurrence forward + adjoint scan + grad_A sums, fp32, B=64, T=2^17
      segments2  2x2 per-sample recurrence cut into segments, fwd+bwd, fp32, B=16, T=2^20
      fixup    8 rows of 2^24 samples cut into 32 segments: zero-start scans, fold, fix-up, fp32"""
    import math

    import torch

    import philtorch_b200 as ptb
    from philtorch_b200 import workloads

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    ops = torch.ops.philtorch_b200
    g = torch.Generator(device=dev).manual_seed(SEED_LPV + 9)
    case = args.profile_case
    if case == "biquad":
        w = workloads.sos_cascade(B=128, T=1 << 19, sections=1, device=dev)
        b, a, x, gy = w["b"][0], w["a"][0], w["x"], w["gy"]

        def step():
            y, _ = ops.biquad_tdf2(b, a, None, x)
            return ops.biquad_tdf2_bwd(b, a, x, y, gy, None, True, False)
    elif case == "half":
        w = workloads.lpv_first_order(B=64, T=1 << 20, device=dev)
        a, zi, x, gy = (w[k].half() for k in ("a", "zi", "x", "gy"))

        def step():
            y = ops.lpv_recur(a, zi, x)
            return ops.lpv_recur_bwd(a, zi, y, gy, None, True, True)
    elif case == "modal":
        R, N, M = 32, 1 << 20, 4
        lam = torch.polar(0.9 + 0.09 * torch.rand(R, M, device=dev, generator=g),
                          2 * math.pi * torch.rand(R, M, device=dev, generator=g))
        gain, coef, w0 = (torch.view_as_complex(torch.randn(R, M, 2, device=dev, generator=g)) for _ in range(3))
        x, gy = torch.randn(R, N, device=dev, generator=g), torch.randn(R, N, device=dev, generator=g)

        def step():
            y, wf, chk = ops.modal_bank(x, lam, gain, coef, None, w0)
            return ops.modal_bank_bwd(x, lam, gain, coef, None, chk, gy, None, 7)
    elif case == "dense":
        Bn, Tn, n = 16, 1 << 18, 4
        A = torch.randn(Bn, Tn, n, n, device=dev, generator=g) * 0.25
        zi = torch.randn(Bn, n, device=dev, generator=g)
        x, gy = torch.randn(Bn, Tn, n, device=dev, generator=g), torch.randn(Bn, Tn, n, device=dev, generator=g)

        def step():
            y = ops.recur_n(A, zi, x)
            return ops.recur_n_adj(A, gy, None, True)
    elif case == "dense-lti":
        Bn, Tn, n = 64, 1 << 17, 8
        A = torch.randn(Bn, n, n, device=dev, generator=g) * (0.5 / n ** 0.5)
        zi = torch.randn(Bn, n, device=dev, generator=g)
        x, gy = torch.randn(Bn, Tn, n, device=dev, generator=g), torch.randn(Bn, Tn, n, device=dev, generator=g)

        def step():
            y = ops.lti_recur_n(A, zi, x)
            g_, _ = ops.recur_n_adj(A, gy, None, False)
            return ops.outer_prev_sum(g_, y, zi)
    elif case == "segments2":
        w = workloads.lpv_second_order(B=16, T=1 << 20, device=dev)
        A2, x2, zi2, gy2 = w["A"].requires_grad_(), w["x"].requires_grad_(), w["zi"], w["gy"]

        def step():
            return torch.autograd.grad(ptb.lpv.state_space_recursion(A2, zi2, x2), (A2, x2), gy2)
    elif case == "fixup":
        w = workloads.long_first_order(B=8, T=1 << 24, device=dev)
        a, x, gy = w["a"].requires_grad_(), w["x"].requires_grad_(), w["gy"]
        zi = torch.zeros(8, device=dev, requires_grad=True)

        def step():
            return torch.autograd.grad(ptb.lpv.linear_recurrence(a, zi, x), (a, zi, x), gy)
    else:
        raise SystemExit(f"unknown profile case {case!r}")
    ms = _time_steps(step, max(1, args.steps), args.warmup, dev)
    ptb.check_errors(dev)
    print(json.dumps({"profile_case": case, "ms_per_step": ms}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    # reduced cases for profiler captures (never a bench value): fewer rows, device-resident loop only
    ap.add_argument("--rows", type=int, default=B, help="rows per GPU (default: the benchmark's 256)")
    ap.add_argument("--kernels-only", action="store_true", help="skip the host-buffer and CPU legs")
    ap.add_argument("--no-configs", action="store_true", dest="no_configs",
                    help="headline workload only (skip the five-configuration / strong-scaling entries)")
    ap.add_argument("--profile-case", default=None, dest="profile_case",
                    help="reduced case for a profiler capture: biquad | half | modal | dense | dense-lti | segments2 | fixup (one GPU)")
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
    if args.profile_case:
        if rank == 0:
            run_profile_case(args)
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
