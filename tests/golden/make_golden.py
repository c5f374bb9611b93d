"""Generate the golden vectors in this folder by RUNNING THE REFERENCE.

Run where the reference checkout and its compiled CPU extension exist:

    python oracle/build_ref.py            # compiles oracle/_ref/philtorch_ref_C.so
    python tests/golden/make_golden.py    # writes tests/golden/*.npz

The reference Python package is imported from its checkout (nothing is copied): its
compiled module ``philtorch._C`` is replaced by the extension built from its own C++
sources, and its third-party dependency ``torchlpc`` (not installed here, not used by
any call below) by a stub that raises.

Every case stores inputs, outputs and gradients produced by the reference's public
API and autograd Functions; names of the callables are recorded in each file's
``case`` entry.
"""
from __future__ import annotations

import os
import sys
import types
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import build_ref  # noqa: E402


def import_reference():
    so = build_ref.build_reference_ext()
    ref_dir = build_ref.reference_dir()
    assert so and ref_dir, "reference checkout not found"
    torch.ops.load_library(so)
    sys.modules["philtorch._C"] = types.ModuleType("philtorch._C")
    stub = types.ModuleType("torchlpc")

    def _missing(*a, **k):
        raise RuntimeError("torchlpc is not installed")

    stub.sample_wise_lpc = _missing
    sys.modules["torchlpc"] = stub
    sys.path.insert(0, ref_dir)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        import philtorch  # noqa: F401
        import philtorch.lti
        import philtorch.lpv
    assert philtorch.EXTENSION_LOADED
    return philtorch


def _np(t):
    return None if t is None else t.detach().cpu().numpy()


def save(name, **arrays):
    arrays = {k: v for k, v in arrays.items() if v is not None}
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrays)
    if len(arrays) > 40:
        print(name, f"{len(arrays)} arrays")
    else:
        print(name, {k: getattr(v, "shape", None) for k, v in arrays.items()})


def grads(out, gy, *inputs):
    gs = torch.autograd.grad(out, inputs, gy, allow_unused=True)
    return [_np(g) for g in gs]


def lpv_lfilter_cases(pt):
    """Time-varying filters of order 1 and 2 through philtorch.lpv.lfilter (backend 'ssm', the
    extension route), forms df2 and tdf2, per-row and shared coefficients."""
    import math
    g = torch.Generator().manual_seed(20240611)
    B, N = 3, 300
    for dt, tag in ((torch.float64, "f64"), (torch.float32, "f32")):
        for order in (1, 2):
            for mode in ("batched", "shared"):
                lead = (B, N) if mode == "batched" else (N,)
                r = 0.3 + 0.6 * torch.rand(lead, generator=g, dtype=torch.float64)
                th = math.pi * torch.rand(lead, generator=g, dtype=torch.float64)
                if order == 2:
                    a = torch.stack([-2 * r * torch.cos(th), r * r], -1)
                else:
                    a = (-r * torch.cos(th)).unsqueeze(-1)
                b = torch.randn(lead + (order + 1,), generator=g, dtype=torch.float64)
                x = torch.randn(B, N, generator=g, dtype=torch.float64)
                zi = torch.randn(B, order, generator=g, dtype=torch.float64)
                gy = torch.randn(B, N, generator=g, dtype=torch.float64)
                b, a, x, zi, gy = (t.to(dt) for t in (b, a, x, zi, gy))
                out = {}
                # order 2 goes through the reference's compiled extension (unroll_factor=1); order 1
                # would go to torchlpc there, so it takes the reference's blocked pure-PyTorch scan
                uf = 1 if order == 2 else 8
                for form in ("df2", "tdf2"):
                    bb, aa, xx, zz = (t.clone().requires_grad_() for t in (b, a, x, zi))
                    y = pt.lpv.lfilter(bb, aa, xx, form=form, unroll_factor=uf)
                    gb, ga, gx = grads(y, gy, bb, aa, xx)
                    y_zi, zf = pt.lpv.lfilter(bb, aa, xx, zi=zz, form=form, unroll_factor=uf)
                    (gzi,) = grads(y_zi, gy, zz)
                    out.update({f"y_{form}": _np(y), f"grad_b_{form}": gb, f"grad_a_{form}": ga,
                                f"grad_x_{form}": gx, f"y_zi_{form}": _np(y_zi), f"zf_{form}": _np(zf),
                                f"grad_zi_{form}": gzi})
                save(f"lpv_lfilter_order{order}_{mode}_{tag}", b=_np(b), a=_np(a), x=_np(x), zi=_np(zi),
                     gy=_np(gy), case=np.array(f"philtorch.lpv.lfilter(backend='ssm', unroll_factor={uf})"), **out)


def complex_first_order_cases(pt):
    """Complex first-order recurrences: the reference's ``LTIRecurrence`` (op ``lti_recur``, which
    ``diag_state_space`` runs on complex poles) with its conjugating backward, and the per-sample
    form through ``MatrixRecurrence`` with 1x1 matrices."""
    from philtorch.lti.recur import LTIRecurrence
    from philtorch.lpv.ssm import MatrixRecurrence

    torch.manual_seed(20240611)

    def poles(shape, rdt):
        r = 0.2 + 0.79 * torch.rand(*shape, dtype=rdt)
        return torch.polar(r, 2 * np.pi * torch.rand(*shape, dtype=rdt))

    for dt, rdt, tag in ((torch.complex128, torch.float64, "c128"), (torch.complex64, torch.float32, "c64")):
        for mode in ("batched", "shared1", "scalar"):
            B, T = 3, 101
            a = poles((B if mode == "batched" else 1,), rdt)
            if mode == "scalar":
                a = a[0]
            a = a.clone().requires_grad_()
            zi = torch.randn(B, dtype=dt, requires_grad=True)
            x = torch.randn(B, T, dtype=dt, requires_grad=True)
            gy = torch.randn(B, T, dtype=dt)
            y = LTIRecurrence.apply(a, zi, x)
            ga, gzi, gx = grads(y, gy, a, zi, x)
            save(f"lti_recur_{mode}_{tag}", a=_np(a), zi=_np(zi), x=_np(x), gy=_np(gy), y=_np(y),
                 grad_a=ga, grad_zi=gzi, grad_x=gx)
        for mode in ("batched", "shared"):
            B, T = 3, 257
            a = poles((B, T) if mode == "batched" else (T,), rdt).requires_grad_()
            zi = torch.randn(B, dtype=dt, requires_grad=True)
            x = torch.randn(B, T, dtype=dt, requires_grad=True)
            gy = torch.randn(B, T, dtype=dt)
            y = MatrixRecurrence.apply(a[..., None, None], zi[:, None], x[..., None])[..., 0]
            ga, gzi, gx = grads(y, gy, a, zi, x)
            y_loop = pt.lpv.linear_recurrence(a.detach(), zi.detach(), x.detach())
            save(f"lpv_recur1_{mode}_{tag}", a=_np(a), zi=_np(zi), x=_np(x), gy=_np(gy), y=_np(y),
                 y_python_loop=_np(y_loop), grad_a=ga, grad_zi=gzi, grad_x=gx)


def first_order_caller_cases(pt):
    """Callers that are pure first-order passes: ``cspline`` / ``cubic_spline``
    (philtorch/lti/interp.py) and ``comb_filter`` (philtorch/lti/filtering.py)."""
    from philtorch.lti.interp import cspline, cubic_spline
    from philtorch.lti import comb_filter

    torch.manual_seed(20240612)
    for dt, tag in ((torch.float64, "f64"), (torch.float32, "f32")):
        out = {}
        x = torch.randn(3, 61, dtype=dt, requires_grad=True)
        gy = torch.randn(3, 61, dtype=dt)
        out["x"], out["gy"] = _np(x), _np(gy)
        for pfe in (True, False):
            for sp in (True, False):
                c = cspline(x, parallel_form=pfe, scipy_padding=sp)
                key = f"{'parallel' if pfe else 'cascade'}_{'scipy' if sp else 'reflect'}"
                out["c_" + key] = _np(c)
                out["grad_x_" + key] = grads(c, gy, x)[0]
        for m in (2, 3, 7):
            for sp in (True, False):
                y = cubic_spline(x, m, scipy_padding=sp)
                gu = torch.linspace(-1, 1, y.shape[1], dtype=dt).expand_as(y)
                key = f"m{m}_{'scipy' if sp else 'reflect'}"
                out["up_" + key] = _np(y)
                out["up_grad_x_" + key] = grads(y, gu, x)[0]
        save(f"cspline_{tag}", **out)

    B, T = 5, 97
    for dt, tag in ((torch.float64, "f64"), (torch.float32, "f32")):
        for delay, zi_shape in ((1, None), (5, None), (13, (13,)), (5, (5, 5)), (32, None)):
            for batched in (True, False):
                a = (torch.rand(B, dtype=dt) * 1.8 - 0.9) if batched else (torch.rand((), dtype=dt) * 1.8 - 0.9)
                a = a.clone().requires_grad_()
                x = torch.randn(B, T, dtype=dt, requires_grad=True)
                gy = torch.randn(B, T, dtype=dt)
                zi = torch.randn(*zi_shape, dtype=dt) if zi_shape else None
                res = comb_filter(a, delay, x, zi=zi)
                y, zf = res if isinstance(res, tuple) else (res, None)
                ga, gx = grads(y, gy, a, x)
                zs = "none" if zi is None else ("shared" if zi.dim() == 1 else "batched")
                save(f"comb_d{delay}_zi{zs}_{'batched' if batched else 'scalar'}_{tag}", a=_np(a), x=_np(x), gy=_np(gy),
                     zi=_np(zi), y=_np(y), zf=_np(zf), grad_a=ga, grad_x=gx)


def diag_state_space_cases(pt):
    """``philtorch.lti.diag_state_space`` (philtorch/lti/ssm.py:590-850): real matrices with complex
    eigenvalues, given eigen-decompositions, vector inputs, a selected state."""
    from philtorch.lti import diag_state_space

    torch.manual_seed(20240613)
    Bn, N, M = 5, 97, 3

    def stable(*lead):
        A = torch.randn(*lead, M, M, dtype=torch.float64)
        return A / (1.1 * torch.linalg.eigvals(A).abs().amax(-1)[..., None, None])

    for dt, tag in ((torch.float64, "f64"), (torch.float32, "f32")):
        cdt = torch.complex128 if dt == torch.float64 else torch.complex64
        # (1) real system from its matrix: B (M,), C (M,), scalar D, zi per row
        A = stable().to(dt).requires_grad_()
        x = torch.randn(Bn, N, dtype=dt, requires_grad=True)
        Bm = torch.randn(M, dtype=dt, requires_grad=True)
        Cm = torch.randn(M, dtype=dt, requires_grad=True)
        Dm = torch.randn(1, dtype=dt)
        zi = torch.randn(Bn, M, dtype=dt)
        gy = torch.randn(Bn, N, dtype=dt)
        y, zf = diag_state_space(x, A=A, B=Bm, C=Cm, D=Dm, zi=zi, unroll_factor=1)   # 1: its compiled op
        gA, gx, gB, gC = grads(y, gy, A, x, Bm, Cm)
        save(f"diag_ssm_matrix_{tag}", A=_np(A), x=_np(x), B=_np(Bm), C=_np(Cm), D=_np(Dm), zi=_np(zi), gy=_np(gy),
             y=_np(y), zf=_np(zf), grad_A=gA, grad_x=gx, grad_B=gB, grad_C=gC)
        # (2) batched eigen-decomposition given: complex L (batch, M), V (batch, M, M); vector input and output
        Ab = stable(Bn)
        Lb, Vb = torch.linalg.eig(Ab)
        Lb, Vb = Lb.to(cdt).requires_grad_(), Vb.to(cdt)
        x3 = torch.randn(Bn, N, 2, dtype=dt, requires_grad=True)
        B3 = torch.randn(M, 2, dtype=dt)
        C3 = torch.randn(2, M, dtype=dt)
        gy3 = torch.randn(Bn, N, 2, dtype=dt)
        y3 = diag_state_space(x3, L=Lb, V=Vb, B=B3, C=C3, unroll_factor=1)
        gL, gx3 = grads(y3, gy3, Lb, x3)
        save(f"diag_ssm_eig_batched_{tag}", L=_np(Lb), V=_np(Vb), x=_np(x3), B=_np(B3), C=_np(C3), gy=_np(gy3),
             y=_np(y3), grad_L=gL, grad_x=gx3)
        # (3) independent modes (L only), complex states returned; and one selected state of a matrix system
        Ls = torch.polar(0.5 + 0.45 * torch.rand(M, dtype=dt), 3.0 * torch.rand(M, dtype=dt)).requires_grad_()
        xs = torch.randn(Bn, N, M, dtype=cdt)
        ys = diag_state_space(xs, L=Ls, unroll_factor=1)
        gys = torch.randn(Bn, N, M, dtype=cdt)
        (gLs,) = grads(ys, gys, Ls)
        A2 = stable().to(dt)
        x2 = torch.randn(Bn, N, dtype=dt)
        y_idx = diag_state_space(x2, A=A2, out_idx=1)   # default unroll factor: its pure-PyTorch scan
        save(f"diag_ssm_modes_{tag}", L=_np(Ls), x=_np(xs), gy=_np(gys), y=_np(ys), grad_L=gLs,
             A2=_np(A2), x2=_np(x2), y_idx=_np(y_idx))


def newton_cases(pt):
    """``philtorch.prototype.nl.newton_solve`` on the feed-forward compressor smoother of the
    reference's tests/test_nl.py (first order) and on a two-state nonlinear recurrence."""
    from philtorch.prototype.nl import newton_solve

    torch.manual_seed(20240614)
    Bn, N = 3, 100
    g = torch.rand(Bn, N, 1, dtype=torch.float64)
    at, rt = torch.rand(Bn, 1, 1, dtype=torch.float64), torch.rand(Bn, 1, 1, dtype=torch.float64)
    init = torch.ones(Bn, 1, dtype=torch.float64)

    def smoother(prev, x):
        coeff = torch.where(x < prev, at, rt)
        return coeff * x + (1 - coeff) * prev

    def smoother_jac(prev, x):
        return (1 - torch.where(x < prev, at, rt)).unsqueeze(-2)

    y, iters = newton_solve(smoother, g, torch.ones(Bn, N, 1, dtype=torch.float64), init=init, max_iter=10,
                            atol=1e-8, rtol=1e-6, fprime=smoother_jac,
                            unroll_factor=4)   # its pure-PyTorch scan: order 1 with factor 1 needs torchlpc
    seq, h = [], init
    for t in range(N):
        h = smoother(h.unsqueeze(1), g[:, t:t + 1]).squeeze(1)
        seq.append(h)
    W = 0.4 * torch.randn(2, 2, dtype=torch.float64)
    x2 = torch.randn(Bn, N, 2, dtype=torch.float64)
    init2 = torch.zeros(Bn, 2, dtype=torch.float64)

    def cell(prev, x):
        return torch.tanh(prev @ W.T + x)

    def cell_jac(prev, x):
        return (1 - torch.tanh(prev @ W.T + x) ** 2).unsqueeze(-1) * W

    y2, iters2 = newton_solve(cell, x2, torch.zeros(Bn, N, 2, dtype=torch.float64), init=init2, max_iter=12,
                              atol=1e-10, rtol=1e-8, fprime=cell_jac)
    seq2, h = [], init2
    for t in range(N):
        h = cell(h.unsqueeze(1), x2[:, t:t + 1]).squeeze(1)
        seq2.append(h)
    save("newton_solve_f64", g=_np(g), at=_np(at), rt=_np(rt), init=_np(init), y=_np(y),
         iters=np.array(iters), y_sequential=_np(torch.stack(seq, 1)),
         W=_np(W), x2=_np(x2), init2=_np(init2), y2=_np(y2), iters2=np.array(iters2),
         y2_sequential=_np(torch.stack(seq2, 1)))


def low_precision_cases(pt):
    """float16 / bfloat16 through the reference's ``LTIRecurrence`` (its ops dispatch both,
    philtorch/csrc/host_lti_recur.cpp:61-78); the reference rounds after every step."""
    from philtorch.lti.recur import LTIRecurrence

    torch.manual_seed(20240615)
    for dt, tag in ((torch.float16, "f16"), (torch.bfloat16, "bf16")):
        B, T = 3, 101
        a = (torch.rand(B) * 1.8 - 0.9).to(dt).requires_grad_()
        zi = torch.randn(B).to(dt).requires_grad_()
        x = torch.randn(B, T).to(dt).requires_grad_()
        gy = torch.randn(B, T).to(dt)
        y = LTIRecurrence.apply(a, zi, x)
        ga, gzi, gx = torch.autograd.grad(y, (a, zi, x), gy)
        f = lambda t: t.detach().float().numpy()   # noqa: E731  (npz has no 16-bit float types for bf16)
        save(f"lti_recur_batched_{tag}", a=f(a), zi=f(zi), x=f(x), gy=f(gy), y=f(y), grad_a=f(ga), grad_zi=f(gzi),
             grad_x=f(gx))


def state_space_cases(pt):
    """philtorch.lpv.state_space with every accepted shape of B, C and D (extension route,
    unroll_factor=1), state dimensions 2 and 3, scalar and feature inputs; all tensors of one case go
    into one file, keyed "<case>/<name>"."""
    g = torch.Generator().manual_seed(777)
    batch, N, F, P = 3, 12, 2, 4
    dt = torch.float64

    def rnd(*shape):
        return torch.randn(tuple(shape), generator=g, dtype=dt)

    store = {}
    names = []
    for M in (2, 3):
        B2 = [None, (M,), (N, M), (batch, M), (batch, N, M)]                     # x (batch, N)
        B3 = [(M, F), (N, M, F), (batch, M, F), (batch, N, M, F)]                # x (batch, N, F)
        C_scalar = [(M,), (N, M), (batch, M), (batch, N, M)]                      # y (batch, N)
        C_vector = [(P, M), (N, P, M), (batch, P, M), (batch, N, P, M)]           # y (batch, N, P)
        D2_scalar = [None, (), (N,), (batch,), (batch, N)]
        D3_scalar = [None, (F,), (N, F), (batch, F), (batch, N, F)]
        D2_vector = [None, (P,), (N, P), (batch, P), (batch, N, P)]
        D3_vector = [None, (P, F), (N, P, F), (batch, P, F), (batch, N, P, F)]
        cases = []

        def cycle(kind, Bs, Cs, Ds):   # every shape of every list at least once, consistent output ranks
            for i in range(max(len(Bs), len(Cs), len(Ds))):
                cases.append((kind, Bs[i % len(Bs)], Cs[i % len(Cs)], Ds[i % len(Ds)]))

        cycle("2d", B2, C_scalar, D2_scalar)
        cycle("2d", B2, C_vector, D2_vector)
        cycle("3d", B3, C_scalar, D3_scalar)
        cycle("3d", B3, C_vector, D3_vector)
        cases.append(("2d", (M,), None, None))          # all states out
        cases.append(("2d-outidx", (M,), None, ()))
        for ci, (kind, bs, cs, ds) in enumerate(cases):
            for A_batched in (True, False):
                r = 0.5 * torch.rand((batch, N, M, M) if A_batched else (N, M, M), generator=g, dtype=dt) / M
                A = (r - r.mean()).requires_grad_()
                x = (rnd(batch, N) if kind.startswith("2d") else rnd(batch, N, F)).requires_grad_()
                Bm = None if bs is None else rnd(*bs).requires_grad_()
                Cm = None if cs is None else rnd(*cs).requires_grad_()
                Dm = None if ds is None else rnd(*ds).requires_grad_()
                zi = rnd(batch, M).requires_grad_()
                out_idx = 1 if kind == "2d-outidx" else None
                y, zf = pt.lpv.state_space(A, x, B=Bm, C=Cm, D=Dm, zi=zi, unroll_factor=1, out_idx=out_idx)
                y2 = pt.lpv.state_space(A, x, B=Bm, C=Cm, D=Dm, unroll_factor=1, out_idx=out_idx)
                gy, gzf = rnd(*y.shape), rnd(*zf.shape)
                ins = [t for t in (A, x, Bm, Cm, Dm, zi) if t is not None]
                gs = torch.autograd.grad([y, zf], ins, [gy, gzf], allow_unused=True)
                key = f"M{M}_{ci}_{'Ab' if A_batched else 'As'}"
                names.append(key)
                store[f"{key}/out_idx"] = np.array(-1 if out_idx is None else out_idx)
                for nm, t in (("A", A), ("x", x), ("B", Bm), ("C", Cm), ("D", Dm), ("zi", zi), ("gy", gy), ("gzf", gzf),
                              ("y", y), ("zf", zf), ("y_nozi", y2)):
                    if t is not None:
                        store[f"{key}/{nm}"] = _np(t)
                for t, gt in zip(ins, gs):
                    nm = next(n for n, u in (("A", A), ("x", x), ("B", Bm), ("C", Cm), ("D", Dm), ("zi", zi)) if u is t)
                    if gt is not None:
                        store[f"{key}/grad_{nm}"] = _np(gt)
    store["cases"] = np.array(names)
    save("lpv_state_space_f64", **store)


def dense_recurrence_cases(pt):
    """State dimensions above two through the reference's recurN / lti_recurN ops and its autograd
    Functions (CPU extension): N = 3, 4, 5, 8, per-row and shared matrices, float64 and float32;
    and time-invariant filters of order 3 and 5 through lti.lfilter(unroll_factor=1)."""
    from philtorch.lti.ssm import LTIMatrixRecurrence
    from philtorch.lpv.ssm import MatrixRecurrence
    g = torch.Generator().manual_seed(4242)
    Bn, T = 2, 150
    for dt, tag in ((torch.float64, "f64"), (torch.float32, "f32")):
        store = {}
        for n in (3, 5, 8):
            for lpv in (True, False):
                for batched in (True, False):
                    lead = ((Bn,) if batched else ()) + ((T,) if lpv else ())
                    A = (torch.randn(lead + (n, n), generator=g, dtype=torch.float64) * (0.55 / n ** 0.5)).to(dt)
                    zi = torch.randn(Bn, n, generator=g, dtype=torch.float64).to(dt)
                    x = torch.randn(Bn, T, n, generator=g, dtype=torch.float64).to(dt)
                    gy = torch.randn(Bn, T, n, generator=g, dtype=torch.float64).to(dt)
                    Ar, zr, xr = (t.clone().requires_grad_() for t in (A, zi, x))
                    y = (MatrixRecurrence if lpv else LTIMatrixRecurrence).apply(Ar, zr, xr)
                    gA, gzi, gx = grads(y, gy, Ar, zr, xr)
                    key = f"n{n}_{'lpv' if lpv else 'lti'}_{'batched' if batched else 'shared'}"
                    for nm, t in (("A", _np(A)), ("zi", _np(zi)), ("x", _np(x)), ("gy", _np(gy)), ("y", _np(y)),
                                  ("grad_A", gA), ("grad_zi", gzi), ("grad_x", gx)):
                        store[f"{key}/{nm}"] = t
        for order in (3, 5):
            rad = 0.4 + 0.5 * torch.rand(Bn, order, generator=g, dtype=torch.float64)
            poles = torch.polar(rad, 3.0 * torch.rand(Bn, order, generator=g, dtype=torch.float64))
            a = torch.stack([torch.from_numpy(np.poly(np.concatenate([p.numpy()[: order // 2], p.numpy()[: order // 2].conj(),
                                                                      p.numpy()[order - 1:].real])).real[1:])
                             for p in poles]).to(dt)
            b = torch.randn(Bn, order + 1, generator=g, dtype=torch.float64).to(dt)
            x = torch.randn(Bn, T, generator=g, dtype=torch.float64).to(dt)
            gy = torch.randn(Bn, T, generator=g, dtype=torch.float64).to(dt)
            for form in ("tdf2", "df2"):
                br, ar, xr = (t.clone().requires_grad_() for t in (b, a, x))
                y = pt.lti.lfilter(br, ar, xr, form=form, unroll_factor=1)
                gb, ga, gx = grads(y, gy, br, ar, xr)
                key = f"lfilter{order}_{form}"
                for nm, t in (("b", _np(b)), ("a", _np(a)), ("x", _np(x)), ("gy", _np(gy)), ("y", _np(y)),
                              ("grad_b", gb), ("grad_a", ga), ("grad_x", gx)):
                    store[f"{key}/{nm}"] = t
        save(f"dense_recurrence_{tag}", **store)


def main():
    pt = import_reference()
    if len(sys.argv) > 1 and sys.argv[1] == "state_space":     # only this group
        state_space_cases(import_reference())
        return
    if len(sys.argv) > 1 and sys.argv[1] == "dense":           # only this group
        dense_recurrence_cases(import_reference())
        return
    if len(sys.argv) > 1 and sys.argv[1] == "low_precision":   # only this group
        low_precision_cases(pt)
        return
    if len(sys.argv) > 1 and sys.argv[1] == "newton":        # only this group
        newton_cases(pt)
        return
    if len(sys.argv) > 1 and sys.argv[1] == "diag_ssm":      # only this group
        diag_state_space_cases(pt)
        return
    if len(sys.argv) > 1 and sys.argv[1] == "callers":       # only this group
        first_order_caller_cases(pt)
        return
    if len(sys.argv) > 1 and sys.argv[1] == "complex":       # only this group
        complex_first_order_cases(pt)
        return
    if len(sys.argv) > 1 and sys.argv[1] == "lpv_lfilter":   # only this group (the others are unchanged)
        lpv_lfilter_cases(pt)
        return
    from philtorch.lti.recur import LTIRecurrence
    from philtorch.lti.ssm import LTIMatrixRecurrence
    from philtorch.lpv.ssm import MatrixRecurrence
    from philtorch.mat import companion

    torch.manual_seed(20240607)

    # ---- first-order LTI: LTIRecurrence (op lti_recur) ------------------------------
    for dt, tag in ((torch.float64, "f64"), (torch.float32, "f32")):
        for mode in ("batched", "shared1", "scalar"):
            B, T = 3, 101
            a = (torch.rand(B if mode == "batched" else 1, dtype=dt) * 2 - 1)
            if mode == "scalar":
                a = a[0]
            a = a.clone().requires_grad_()
            zi = torch.randn(B, dtype=dt, requires_grad=True)
            x = torch.randn(B, T, dtype=dt, requires_grad=True)
            gy = torch.randn(B, T, dtype=dt)
            y = LTIRecurrence.apply(a, zi, x)
            ga, gzi, gx = grads(y, gy, a, zi, x)
            save(f"lti_recur_{mode}_{tag}", a=_np(a), zi=_np(zi), x=_np(x), gy=_np(gy), y=_np(y),
                 grad_a=ga, grad_zi=gzi, grad_x=gx)

    # ---- first-order LPV through recurN with N = 1 and the pure-Python loop ----------
    for dt, tag in ((torch.float64, "f64"), (torch.float32, "f32")):
        for mode in ("batched", "shared"):
            B, T = 3, 257
            a = (torch.rand(*((B, T) if mode == "batched" else (T,)), dtype=dt) * 1.98 - 0.99)
            a.requires_grad_()
            zi = torch.randn(B, dtype=dt, requires_grad=True)
            x = torch.randn(B, T, dtype=dt, requires_grad=True)
            gy = torch.randn(B, T, dtype=dt)
            y = MatrixRecurrence.apply(a[..., None, None], zi[:, None], x[..., None])[..., 0]
            ga, gzi, gx = grads(y, gy, a, zi, x)
            y_loop = pt.lpv.linear_recurrence(a.detach(), zi.detach(), x.detach())
            y_unrolled = pt.lpv.linear_recurrence(a.detach(), zi.detach(), x.detach(), unroll_factor=8)
            save(f"lpv_recur1_{mode}_{tag}", a=_np(a), zi=_np(zi), x=_np(x), gy=_np(gy), y=_np(y),
                 y_python_loop=_np(y_loop), y_python_unrolled=_np(y_unrolled),
                 grad_a=ga, grad_zi=gzi, grad_x=gx)

    # ---- 2x2 LTI: LTIMatrixRecurrence (op lti_recur2) -------------------------------
    def rand_stable_a(n):
        r = 0.5 + 0.49 * torch.rand(n, dtype=torch.float64)
        th = np.pi * torch.rand(n, dtype=torch.float64)
        return torch.stack([-2 * r * torch.cos(th), r * r], -1)

    for dt, tag in ((torch.float64, "f64"), (torch.float32, "f32")):
        for mode in ("batched", "shared"):
            B, T = 3, 101
            A = companion(rand_stable_a(B if mode == "batched" else 1)).to(dt)
            if mode == "shared":
                A = A[0]
            A = A.clone().requires_grad_()
            zi = torch.randn(B, 2, dtype=dt, requires_grad=True)
            x = torch.randn(B, T, 2, dtype=dt, requires_grad=True)
            gy = torch.randn(B, T, 2, dtype=dt)
            y = LTIMatrixRecurrence.apply(A, zi, x)
            gA, gzi, gx = grads(y, gy, A, zi, x)
            save(f"lti_recur2_{mode}_{tag}", A=_np(A), zi=_np(zi), x=_np(x), gy=_np(gy), y=_np(y),
                 grad_A=gA, grad_zi=gzi, grad_x=gx)

    # ---- 2x2 LPV: MatrixRecurrence (op recur2) --------------------------------------
    for dt, tag in ((torch.float64, "f64"), (torch.float32, "f32")):
        for mode in ("batched", "shared"):
            B, T = 3, 77
            n = (B, T) if mode == "batched" else (T,)
            r = 0.6 + 0.38 * torch.rand(*n, dtype=torch.float64)
            th = np.pi * torch.rand(*n, dtype=torch.float64)
            A = companion(torch.stack([-2 * r * torch.cos(th), r * r], -1)).to(dt)
            A = (A + 0.05 * torch.randn_like(A)).requires_grad_()   # general, not only companion
            zi = torch.randn(B, 2, dtype=dt, requires_grad=True)
            x = torch.randn(B, T, 2, dtype=dt, requires_grad=True)
            gy = torch.randn(B, T, 2, dtype=dt)
            y = MatrixRecurrence.apply(A, zi, x)
            gA, gzi, gx = grads(y, gy, A, zi, x)
            y_loop = pt.lpv.state_space_recursion(A.detach(), zi.detach(), x.detach())
            y_loop_idx = pt.lpv.state_space_recursion(A.detach(), zi.detach(), x.detach()[..., 0], out_idx=1)
            save(f"lpv_recur2_{mode}_{tag}", A=_np(A), zi=_np(zi), x=_np(x), gy=_np(gy), y=_np(y),
                 y_python_loop=_np(y_loop), y_python_loop_x2d_idx1=_np(y_loop_idx),
                 grad_A=gA, grad_zi=gzi, grad_x=gx)

    # ---- public scalar API: lti.linear_recurrence ------------------------------------
    B, T = 4, 130
    a = torch.rand(B, dtype=torch.float64) * 1.8 - 0.9
    zi = torch.randn(B, dtype=torch.float64)
    x = torch.randn(B, T, dtype=torch.float64)
    save("lti_linear_recurrence_f64", a=_np(a), zi=_np(zi), x=_np(x),
         y=_np(pt.lti.linear_recurrence(a, zi, x)),
         y_unrolled=_np(pt.lti.linear_recurrence(a, zi, x, unroll_factor=7)),
         y_scalar_a=_np(pt.lti.linear_recurrence(a[0], zi[0], x)))

    # ---- public matrix API: lti.state_space_recursion --------------------------------
    A = companion(rand_stable_a(B))
    zi2 = torch.randn(B, 2, dtype=torch.float64)
    x2 = torch.randn(B, T, 2, dtype=torch.float64)
    save("lti_state_space_recursion_f64", A=_np(A), zi=_np(zi2), x=_np(x2),
         y=_np(pt.lti.state_space_recursion(A, zi2, x2)),
         y_shared=_np(pt.lti.state_space_recursion(A[0], zi2, x2)),
         y_x2d_idx0=_np(pt.lti.state_space_recursion(A, zi2, x2[..., 0], out_idx=0)),
         y_unrolled=_np(pt.lti.state_space_recursion(A, zi2, x2, unroll_factor=5)))

    # ---- lfilter / filtfilt through the extension route (unroll_factor=1) -------------
    for dt, tag in ((torch.float64, "f64"), (torch.float32, "f32")):
        for order in (1, 2):
            for mode in ("batched", "shared"):
                B, T = 4, 300
                nb = B if mode == "batched" else 1
                if order == 2:
                    a = rand_stable_a(nb)
                else:
                    a = (torch.rand(nb, 1, dtype=torch.float64) * 1.8 - 0.9)
                b = torch.randn(nb, order + 1, dtype=torch.float64)
                if mode == "shared":
                    a, b = a[0], b[0]
                a = a.to(dt).requires_grad_()
                b = b.to(dt).requires_grad_()
                x = torch.randn(B, T, dtype=dt, requires_grad=True)
                zi = torch.randn(B, order, dtype=dt, requires_grad=True)
                gy = torch.randn(B, T, dtype=dt)
                gzf = torch.randn(B, order, dtype=dt)
                out = {}
                for form in ("tdf2", "df2"):
                    y = pt.lti.lfilter(b, a, x, form=form, unroll_factor=1)
                    gb, ga, gx = grads(y, gy, b, a, x)
                    y_zi, zf = pt.lti.lfilter(b, a, x, zi=zi, form=form, unroll_factor=1)
                    gs = torch.autograd.grad([y_zi, zf], [b, a, x, zi], [gy, gzf])
                    out.update({f"{form}_y": _np(y), f"{form}_grad_b": gb, f"{form}_grad_a": ga,
                                f"{form}_grad_x": gx, f"{form}_y_zi": _np(y_zi), f"{form}_zf": _np(zf),
                                f"{form}_zi_grad_b": _np(gs[0]), f"{form}_zi_grad_a": _np(gs[1]),
                                f"{form}_zi_grad_x": _np(gs[2]), f"{form}_zi_grad_zi": _np(gs[3])})
                ff = pt.lti.filtfilt(b.detach(), a.detach(), x.detach(), unroll_factor=1)
                ffg = pt.lti.filtfilt(b, a, x, unroll_factor=1)
                gb, ga, gx = grads(ffg, gy, b, a, x)
                save(f"lfilter_order{order}_{mode}_{tag}", b=_np(b), a=_np(a), x=_np(x), zi=_np(zi),
                     gy=_np(gy), gzf=_np(gzf), filtfilt_y=_np(ff), filtfilt_grad_b=gb,
                     filtfilt_grad_a=ga, filtfilt_grad_x=gx, **out)

    # ---- the five benchmark configurations at reduced size ----------------------------
    from philtorch_b200 import workloads as W

    w = W.lti_first_order(B=8, T=4096)
    a, zi, x = (w[k].clone().requires_grad_() for k in ("a", "zi", "x"))
    y = LTIRecurrence.apply(a, zi, x)
    ga, gzi, gx = grads(y, w["gy"], a, zi, x)
    save("config1_small", y=_np(y), grad_a=ga, grad_x=gx, B=8, T=4096)

    w = W.lpv_first_order(B=4, T=8192)
    a, zi, x = (w[k].clone().requires_grad_() for k in ("a", "zi", "x"))
    y = MatrixRecurrence.apply(a[..., None, None], zi[:, None], x[..., None])[..., 0]
    ga, gzi, gx = grads(y, w["gy"], a, zi, x)
    save("config2_small", y=_np(y), grad_a=ga, grad_zi=gzi, grad_x=gx, B=4, T=8192)

    w = W.sos_cascade(B=4, T=4096, sections=6)
    b, a, x = (w[k].clone().requires_grad_() for k in ("b", "a", "x"))
    u = x
    for k in range(6):
        u = pt.lti.lfilter(b[k], a[k], u, form="tdf2", unroll_factor=1)
    gb, ga, gx = grads(u, w["gy"], b, a, x)
    save("config3_small", y=_np(u), grad_b=gb, grad_a=ga, grad_x=gx, B=4, T=4096)

    for dt, tag in ((torch.float32, "f32"), (torch.float64, "f64")):
        w = W.lpv_second_order(B=2, T=4096, dtype=dt)
        A, x = (w[k].clone().requires_grad_() for k in ("A", "x"))
        xp = torch.stack([x, torch.zeros_like(x)], -1)
        y = MatrixRecurrence.apply(A, w["zi"], xp)
        gA, gx = grads(y, w["gy"], A, x)
        save(f"config4_small_{tag}", y=_np(y), grad_A=gA, grad_x=gx, B=2, T=4096)

    w = W.long_first_order(B=2, T=16384)
    a, zi, x = (w[k].clone().requires_grad_() for k in ("a", "zi", "x"))
    y = MatrixRecurrence.apply(a[..., None, None], zi[:, None], x[..., None])[..., 0]
    ga, gzi, gx = grads(y, w["gy"], a, zi, x)
    save("config5_small", y=_np(y), grad_a=ga, grad_x=gx, B=2, T=16384)

    lpv_lfilter_cases(pt)


if __name__ == "__main__":
    main()
