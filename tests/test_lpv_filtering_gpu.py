"""Parameter-varying ``lpv.lfilter`` (orders 1 and 2, forms df2 / tdf2) against golden vectors made
by running the reference's ``philtorch.lpv.lfilter`` (tests/golden/make_golden.py)."""
import pytest
import torch

import philtorch_b200 as ptb
from conftest import load_golden, rel_err, tol

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("tag", ["f32", "f64"])
@pytest.mark.parametrize("mode", ["batched", "shared"])
@pytest.mark.parametrize("order", [1, 2])
@pytest.mark.parametrize("form", ["df2", "tdf2"])
def test_lfilter_matches_reference(form, order, mode, tag):
    g = load_golden(f"lpv_lfilter_order{order}_{mode}_{tag}")
    dtype = torch.float32 if tag == "f32" else torch.float64
    t = tol(dtype)
    b, a, x, zi = (g[k].to(DEV).requires_grad_() for k in ("b", "a", "x", "zi"))
    gy = g["gy"].to(DEV)
    y = ptb.lpv.lfilter(b, a, x, form=form)
    gb, ga, gx = torch.autograd.grad(y, (b, a, x), gy)
    assert rel_err(y, g[f"y_{form}"]) <= t
    assert rel_err(gx, g[f"grad_x_{form}"]) <= t
    assert rel_err(gb, g[f"grad_b_{form}"]) <= t
    assert rel_err(ga, g[f"grad_a_{form}"]) <= t
    y2, zf = ptb.lpv.lfilter(b, a, x, zi=zi, form=form)
    (gzi,) = torch.autograd.grad(y2, (zi,), gy)
    assert rel_err(y2, g[f"y_zi_{form}"]) <= t
    assert rel_err(zf, g[f"zf_{form}"]) <= t
    assert rel_err(gzi, g[f"grad_zi_{form}"]) <= t
    ptb.check_errors()


def test_one_dimensional_call_and_errors():
    g = load_golden("lpv_lfilter_order2_shared_f64")
    b, a, x = g["b"].to(DEV), g["a"].to(DEV), g["x"][0].to(DEV)
    y = ptb.lpv.lfilter(b, a, x)
    assert y.shape == x.shape and rel_err(y, g["y_df2"][0]) <= 1e-10
    with pytest.raises(NotImplementedError):
        ptb.lpv.lfilter(b, a, x, form="df1")
    with pytest.raises(NotImplementedError):
        ptb.lpv.lfilter(b, a, x, backend="torchlpc")
    with pytest.raises(NotImplementedError):
        ptb.lpv.lfilter(torch.ones(300, 4, device=DEV), torch.zeros(300, 3, device=DEV), x.float())
    with pytest.raises(ValueError):
        ptb.lpv.lfilter(b, a, x, form="nope")
    with pytest.raises(RuntimeError):
        ptb.lpv.lfilter(b.cpu(), a.cpu(), x.cpu())
