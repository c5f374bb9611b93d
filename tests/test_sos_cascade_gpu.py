"""Fused cascade of second-order sections (one pass per direction for up to eight sections)
against the chain of single sections: the CPU oracle forward, the golden vectors of the reference
for the six-section configuration, and the chained single-section kernels for the gradients."""
import pytest
import torch

import philtorch_b200 as ptb
from philtorch_b200 import workloads
from conftest import load_golden, rel_err, tol
from oracle import cport

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True, params=[1, 2], ids=["decoupled", "chained"])
def kernel_family(request):
    """Every case runs on both kernel families (normally picked by the batch size)."""
    from philtorch_b200 import _lib
    assert _lib.lib.ptb_sos_cascade_set_mode(request.param) == 0
    yield request.param
    assert _lib.lib.ptb_sos_cascade_set_mode(0) == 0


def _workload(K, B, T, dtype, shared=False, seed=0):
    w = workloads.sos_cascade(B=B, T=T, sections=K, dtype=dtype)
    g = torch.Generator().manual_seed(seed)
    b, a = w["b"], w["a"]
    if shared:
        b, a = b[:, 0].contiguous(), a[:, 0].contiguous()
    zi = torch.randn(K, B, 2, generator=g, dtype=torch.float64).to(dtype)
    gzf = torch.randn(K, B, 2, generator=g, dtype=torch.float64).to(dtype)
    return b, a, w["x"], zi, w["gy"], gzf


def _oracle_chain(b, a, x, zi):
    u, zfs = x, []
    for k in range(b.shape[0]):
        u, zf = cport.biquad_tdf2(b[k], a[k], None if zi is None else zi[k], u)
        zfs.append(zf)
    return u, torch.stack(zfs)


def _chain(b, a, x, zi):
    """the single-section kernels chained (each verified against the oracle on its own)"""
    u, zfs = x, []
    for k in range(b.shape[0]):
        if zi is None:
            u = ptb.lti.lfilter(b[k], a[k], u)
        else:
            u, zf = ptb.lti.lfilter(b[k], a[k], u, zi=zi[k])
            zfs.append(zf)
    return u, (torch.stack(zfs) if zfs else None)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("K", [1, 2, 3, 4, 5, 6, 8, 9, 11])
def test_forward_section_counts(dtype, K):
    b, a, x, zi, _, _ = _workload(K, 5, 3000, dtype)
    y_ref, zf_ref = _oracle_chain(b, a, x, zi)
    y, zf = ptb.lti.sosfilt(b.to(DEV), a.to(DEV), x.to(DEV), zi=zi.to(DEV))
    assert rel_err(y, y_ref) <= tol(dtype)
    assert rel_err(zf, zf_ref) <= tol(dtype)
    y0 = ptb.lti.sosfilt(b.to(DEV), a.to(DEV), x.to(DEV))
    assert rel_err(y0, _oracle_chain(b, a, x, None)[0]) <= tol(dtype)
    ptb.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("T", [1, 2, 3, 35, 36, 37, 1000, 4608, 9215, 9216, 9217, 9220, 30001, 70000])
def test_forward_lengths(dtype, T):
    """short rows, tile boundaries, lengths off the 16-byte grid (plain-load path), many tiles"""
    b, a, x, zi, _, _ = _workload(6, 3, T, dtype, seed=T)
    y_ref, zf_ref = _oracle_chain(b, a, x, zi)
    y, zf = ptb.lti.sosfilt(b.to(DEV), a.to(DEV), x.to(DEV), zi=zi.to(DEV))
    assert rel_err(y, y_ref) <= tol(dtype)
    assert rel_err(zf, zf_ref) <= tol(dtype)
    ptb.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_forward_shared_coefficients_and_mixed(dtype):
    b, a, x, zi, _, _ = _workload(4, 7, 20000, dtype, shared=True)
    y_ref, zf_ref = _oracle_chain(b, a, x, zi)
    y, zf = ptb.lti.sosfilt(b.to(DEV), a.to(DEV), x.to(DEV), zi=zi.to(DEV))
    assert rel_err(y, y_ref) <= tol(dtype) and rel_err(zf, zf_ref) <= tol(dtype)
    # b shared, a per row
    a_rows = a.unsqueeze(1).expand(-1, 7, -1).contiguous()
    y2 = ptb.lti.sosfilt(b.to(DEV), a_rows.to(DEV), x.to(DEV))
    assert rel_err(y2, _oracle_chain(b, a, x, None)[0]) <= tol(dtype)
    ptb.check_errors()


def test_unaligned_views():
    """rows that do not start on 16-byte boundaries take the plain-load path"""
    b, a, x, zi, _, _ = _workload(6, 4, 12001, torch.float32)
    xd = torch.zeros(4, 12002, device=DEV)[:, 1:]
    xd.copy_(x)
    y = ptb.lti.sosfilt(b.to(DEV), a.to(DEV), xd)
    assert rel_err(y, _oracle_chain(b, a, x, None)[0]) <= 1e-4
    ptb.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("K,B,T,shared", [(6, 4, 4096, False), (6, 3, 30001, False), (2, 5, 9217, False),
                                          (4, 6, 20000, True), (8, 2, 12000, False), (3, 4, 5000, False),
                                          (6, 2, 70000, False), (6, 3, 37, False)])
def test_gradients_match_chained_sections(dtype, K, B, T, shared):
    b, a, x, zi, gy, gzf = _workload(K, B, T, dtype, shared=shared)
    ins = [t.to(DEV).requires_grad_() for t in (b, a, x, zi)]
    y, zf = ptb.lti.sosfilt(ins[0], ins[1], ins[2], zi=ins[3])
    grads = torch.autograd.grad([y, zf], ins, [gy.to(DEV), gzf.to(DEV)])
    ref_ins = [t.to(DEV).requires_grad_() for t in (b, a, x, zi)]
    y_r, zf_r = _chain(*[ref_ins[i] for i in (0, 1, 2, 3)])
    ref = torch.autograd.grad([y_r, zf_r], ref_ins, [gy.to(DEV), gzf.to(DEV)])
    assert rel_err(y, y_r) <= tol(dtype)
    ctol = tol(dtype) * (10 if dtype == torch.float64 else 1)   # sums of many O(1) terms, other order
    for g, r, name in zip(grads, ref, ("b", "a", "x", "zi")):
        assert rel_err(g, r) <= (ctol if name in ("b", "a") else tol(dtype)), name
    # input gradient only (no intermediate outputs are kept on this path)
    x2 = x.to(DEV).requires_grad_()
    y2 = ptb.lti.sosfilt(b.to(DEV), a.to(DEV), x2)
    (gx2,) = torch.autograd.grad(y2, x2, gy.to(DEV))
    x3 = x.to(DEV).requires_grad_()
    (gx3,) = torch.autograd.grad(_chain(b.to(DEV), a.to(DEV), x3, None)[0], x3, gy.to(DEV))
    assert rel_err(gx2, gx3) <= tol(dtype)
    ptb.check_errors()


def test_config3_against_reference_golden():
    g = load_golden("config3_small")
    w = workloads.sos_cascade(B=4, T=4096, sections=6)
    b, a, x = (w[k].to(DEV).requires_grad_() for k in ("b", "a", "x"))
    y = ptb.lti.sosfilt(b, a, x)
    gb, ga, gx = torch.autograd.grad(y, (b, a, x), w["gy"].to(DEV))
    assert rel_err(y, g["y"]) <= 1e-4 and rel_err(gb, g["grad_b"]) <= 1e-4
    assert rel_err(ga, g["grad_a"]) <= 1e-4 and rel_err(gx, g["grad_x"]) <= 1e-4
    ptb.check_errors()


def test_double_backward_and_opcheck():
    b, a, x, zi, gy, _ = _workload(2, 2, 40, torch.float64)
    ins = [t.to(DEV).requires_grad_() for t in (b, a, x, zi)]
    torch.autograd.gradcheck(lambda *t: ptb.lti.sosfilt(t[0], t[1], t[2], zi=t[3]), ins)
    torch.autograd.gradgradcheck(lambda *t: ptb.lti.sosfilt(t[0], t[1], t[2], zi=t[3])[0], ins)
    args = (b.to(DEV), a.to(DEV), zi.to(DEV), x.to(DEV), True)
    torch.library.opcheck(torch.ops.philtorch_b200.sos_cascade.default, args)
    y, mid, _ = torch.ops.philtorch_b200.sos_cascade(*args)
    torch.library.opcheck(torch.ops.philtorch_b200.sos_cascade_bwd.default,
                          (args[0], args[1], args[3], mid, y, gy.to(DEV), None, True, True))


def test_errors():
    b, a, x, zi, _, _ = _workload(2, 3, 100, torch.float32)
    with pytest.raises(RuntimeError):
        ptb.lti.sosfilt(b, a, x)                                    # CPU tensors
    with pytest.raises(ValueError):
        ptb.lti.sosfilt(b.to(DEV), a[:1].to(DEV), x.to(DEV))        # section counts differ
    with pytest.raises(RuntimeError):
        ptb.lti.sosfilt(b.to(DEV).double(), a.to(DEV).double(), x.to(DEV))   # dtype mismatch
