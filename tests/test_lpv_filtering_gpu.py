"""Parameter-varying ``lpv.lfilter`` (orders 1 and 2, forms df2 / tdf2) against golden vectors made
by running the reference's ``philtorch.lpv.lfilter`` (tests/golden/make_golden.py)."""
import pytest
import torch

import philtorch_b200 as ptb
from conftest import load_golden, rel_err, tol

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True, params=[10**9, 1], ids=["scan+glue", "fused"])
def df2_path(request, monkeypatch):
    """The filter has two implementations, normally picked by the batch size: every case runs on both."""
    from philtorch_b200.lpv import filtering
    monkeypatch.setattr(filtering, "FUSED_MIN_ROWS", request.param)
    return request.param


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


@pytest.mark.parametrize("form", ["df2", "tdf2"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("B,T,shared", [(40, 5000, False), (33, 961, False), (64, 20003, False), (48, 7000, True),
                                        (130, 12000, False)])
def test_fused_matches_scan_path(form, dtype, B, T, shared, monkeypatch):
    """The fused kernels against the 2x2 scan kernels plus elementwise maps (pinned above to the
    reference) on batches, lengths (ragged, unaligned) and coefficient layouts the golden files lack."""
    from philtorch_b200.lpv import filtering
    g = torch.Generator().manual_seed(B * 7 + T)
    lead = (T,) if shared else (B, T)
    r = 0.3 + 0.65 * torch.rand(lead, generator=g, dtype=torch.float64)
    th = 3.14159 * torch.rand(lead, generator=g, dtype=torch.float64)
    a = torch.stack([-2 * r * torch.cos(th), r * r], -1).to(dtype)
    b = torch.randn(lead + (3,), generator=g, dtype=torch.float64).to(dtype)
    x = torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype)
    zi = torch.randn(B, 2, generator=g, dtype=torch.float64).to(dtype)
    gy = torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype)
    gzf = torch.randn(B, 2, generator=g, dtype=torch.float64).to(dtype)
    outs = []
    for min_rows in (1, 10**9):
        monkeypatch.setattr(filtering, "FUSED_MIN_ROWS", min_rows)
        ins = [t.to(DEV).requires_grad_() for t in (b, a, x, zi)]
        y, zf = ptb.lpv.lfilter(ins[0], ins[1], ins[2], zi=ins[3], form=form)
        outs.append((y, zf) + torch.autograd.grad([y, zf], ins, [gy.to(DEV), gzf.to(DEV)]))
    t = tol(dtype)
    for got, ref, name in zip(outs[0], outs[1], ("y", "zf", "grad_b", "grad_a", "grad_x", "grad_zi")):
        # shared coefficients: the gradient sums over the rows, in another order
        assert rel_err(got, ref) <= (10 * t if shared and name in ("grad_b", "grad_a") else t), name
    ptb.check_errors()


@pytest.mark.parametrize("form", ["df2", "tdf2"])
@pytest.mark.parametrize("order", [1, 2])
@pytest.mark.parametrize("shared", ["b", "a"])
def test_one_coefficient_shared_one_per_row(form, order, shared, df2_path):
    """b shared by the rows and a per row (or the reverse), as the reference's broadcasting allows:
    the same values and gradient shapes on the fused kernels (32 rows) as on the scan route."""
    from philtorch_b200.lpv import filtering

    B, N = 32, 700
    g = torch.Generator().manual_seed(order * 10 + (shared == "a"))
    bs = (N, order + 1) if shared == "b" else (B, N, order + 1)
    as_ = (N, order) if shared == "a" else (B, N, order)
    b = torch.randn(bs, generator=g, dtype=torch.float64).to(DEV).requires_grad_()
    a = (0.4 * (torch.rand(as_, generator=g, dtype=torch.float64) - 0.5)).to(DEV).requires_grad_()
    x = torch.randn(B, N, generator=g, dtype=torch.float64).to(DEV).requires_grad_()
    gy = torch.randn(B, N, generator=g, dtype=torch.float64).to(DEV)
    y = ptb.lpv.lfilter(b, a, x, form=form)
    grads = torch.autograd.grad(y, (b, a, x), gy)
    assert grads[0].shape == b.shape and grads[1].shape == a.shape
    old = filtering.FUSED_MIN_ROWS
    filtering.FUSED_MIN_ROWS = 10**9 if df2_path == 1 else 1      # the other implementation
    try:
        y2 = ptb.lpv.lfilter(b, a, x, form=form)
        grads2 = torch.autograd.grad(y2, (b, a, x), gy)
    finally:
        filtering.FUSED_MIN_ROWS = old
    assert rel_err(y, y2) <= 1e-10
    for g1, g2 in zip(grads, grads2):
        assert rel_err(g1, g2) <= 1e-9
    ptb.check_errors()
