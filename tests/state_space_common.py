"""Shared driver of the lpv.state_space tests: runs every case of the reference-made golden file
through ``philtorch_b200.lpv.state_space`` on a given device and compares outputs and gradients."""
import os

import numpy as np
import torch

from conftest import GOLDEN, rel_err


def load_cases():
    z = np.load(os.path.join(GOLDEN, "lpv_state_space_f64.npz"))
    cases = {}
    for key in z.files:
        if "/" not in key:
            continue
        case, name = key.split("/", 1)
        cases.setdefault(case, {})[name] = z[key]
    return cases


def run_case(c, device, state_space, tol=1e-10):
    t = {k: torch.from_numpy(np.asarray(v)).to(device) for k, v in c.items() if k != "out_idx"}
    out_idx = int(c["out_idx"])
    out_idx = None if out_idx < 0 else out_idx
    names = [n for n in ("A", "x", "B", "C", "D", "zi") if n in t]
    ins = {n: t[n].clone().requires_grad_() for n in names}
    kw = {k: ins.get(k) for k in ("B", "C", "D")}
    y, zf = state_space(ins["A"], ins["x"], zi=ins["zi"], out_idx=out_idx, **kw)
    assert y.shape == t["y"].shape and rel_err(y, t["y"]) <= tol
    assert rel_err(zf, t["zf"]) <= tol
    y2 = state_space(ins["A"], ins["x"], out_idx=out_idx, **kw)
    assert rel_err(y2, t["y_nozi"]) <= tol
    gs = torch.autograd.grad([y, zf], [ins[n] for n in names], [t["gy"], t["gzf"]], allow_unused=True)
    for n, g in zip(names, gs):
        if f"grad_{n}" in t:
            assert g is not None and g.shape == t[f"grad_{n}"].shape, n
            assert rel_err(g, t[f"grad_{n}"]) <= tol * 10, n
