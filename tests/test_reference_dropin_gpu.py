"""The kernels behind the reference package's own ops (philtorch_b200.compat).

Two levels.  (1) Op level, needs only the reference's compiled CPU extension (oracle/_ref, built
from the reference's C++ sources): with ``compat.register()`` the very ops
``torch.ops.philtorch.*`` answer CUDA tensors with this package's kernels and CPU tensors with the
reference's kernels, so the same call on both devices must agree.  (2) Package level, needs an
installed copy of the UNMODIFIED reference package (``PHILTORCH_REFERENCE_PKG``, or the offline
install under baseline/_ref): its autograd Functions, ``lfilter(..., unroll_factor=1)`` and
``state_space_recursion`` run with ``device="cuda"`` -- the CUDA parametrisations of the reference's
own tests/test_recur_ext.py and tests/test_grad.py -- against their CPU results and gradcheck.
"""
import os
import sys
import types
import warnings

import pytest
import torch

import philtorch_b200 as ptb
from philtorch_b200 import compat
from conftest import rel_err, tol

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_package():
    """Imports the reference package if a copy is available; returns the module or None."""
    if "philtorch" in sys.modules:
        return sys.modules["philtorch"]
    cand = [os.environ.get("PHILTORCH_REFERENCE_PKG"), os.path.join(ROOT, "baseline", "_ref")]
    for d in cand:
        if d and os.path.isdir(os.path.join(d, "philtorch")):
            stub = types.ModuleType("torchlpc")     # third-party dependency of philtorch.lpv, unused here

            def _missing(*a, **k):
                raise RuntimeError("torchlpc is not installed")

            stub.sample_wise_lpc = _missing
            sys.modules.setdefault("torchlpc", stub)
            if hasattr(torch.ops.philtorch, "lti_recur"):
                # an earlier test loaded the reference's extension (oracle/_ref) already: the package
                # must not load its own copy of the same op library on top of it
                sys.modules["philtorch._C"] = types.ModuleType("philtorch._C")
            sys.path.insert(0, d)
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                import philtorch
                import philtorch.lti
                import philtorch.lpv
            return philtorch if philtorch.EXTENSION_LOADED else None
    return None


@pytest.fixture(scope="module")
def ref_ops():
    pt = _reference_package()
    if pt is None:
        from oracle import refext
        if not refext.available():
            pytest.skip("neither the reference package nor its compiled extension is available")
        refext.load()
    compat.register()
    return torch.ops.philtorch


@pytest.fixture(scope="module")
def ref_pkg(ref_ops):
    pt = _reference_package()
    if pt is None:
        pytest.skip("no installed copy of the reference package")
    return pt


def _both(op, *cpu_args):
    out_cpu = op(*cpu_args)
    out_gpu = op(*[a.cuda() for a in cpu_args])
    assert out_gpu.is_cuda and out_gpu.shape == out_cpu.shape
    return out_gpu, out_cpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_ops_cuda_against_reference_cpu(ref_ops, dtype):
    g = torch.Generator().manual_seed(0)
    B, T = 4, 3001
    t = tol(dtype)

    def rn(*s):
        return torch.randn(*s, generator=g, dtype=torch.float64).to(dtype)

    x1, zi1 = rn(B, T), rn(B)
    for a in (torch.tensor(0.7, dtype=dtype), torch.tensor([-0.6], dtype=dtype), (torch.rand(B, generator=g) * 1.8 - 0.9).to(dtype)):
        assert rel_err(*_both(ref_ops.lti_recur, a, zi1, x1)) <= t
    x2, zi2 = rn(B, T, 2), rn(B, 2)
    for A in (rn(2, 2) * 0.4, rn(B, 2, 2) * 0.4):
        assert rel_err(*_both(ref_ops.lti_recur2, A, zi2, x2)) <= t
        assert rel_err(*_both(ref_ops.lti_recurN, A, zi2, x2)) <= t
    for A in (rn(T, 2, 2) * 0.4, rn(B, T, 2, 2) * 0.4):
        assert rel_err(*_both(ref_ops.recur2, A, zi2, x2)) <= t
        assert rel_err(*_both(ref_ops.recurN, A, zi2, x2)) <= t
    for n in (1, 3, 5):
        xn, zin = rn(B, T, n), rn(B, n)
        s = 0.5 / n ** 0.5
        for A in (rn(T, n, n) * s, rn(B, T, n, n) * s):
            assert rel_err(*_both(ref_ops.recurN, A, zin, xn)) <= t
        for A in (rn(n, n) * s, rn(B, n, n) * s):
            assert rel_err(*_both(ref_ops.lti_recurN, A, zin, xn)) <= t
    ptb.check_errors()


def test_lti_recur2_equals_recur2_on_cuda(ref_ops):
    """tests/test_recur_ext.py::test_lti_recur2_equiv of the reference, device = cuda."""
    B, T = 3, 101
    for batch in (True, False):
        A = (torch.randn(B, 2, 2, dtype=torch.float64) * 0.4).cuda() if batch else (torch.randn(2, 2, dtype=torch.float64) * 0.4).cuda()
        x = torch.randn(B, T, 2, dtype=torch.float64).cuda()
        zi = torch.randn(B, 2, dtype=torch.float64).cuda()
        lti_y = ref_ops.lti_recur2(A, zi, x)
        ltv_y = ref_ops.recur2(A.unsqueeze(1).expand(-1, T, -1, -1) if batch else A.expand(T, -1, -1), zi, x)
        assert torch.allclose(lti_y, ltv_y)


def test_opcheck_on_cuda(ref_pkg):
    """tests/test_pt2_comp.py of the reference, device = cuda (needs the package's fake impls)."""
    B, T = 2, 33
    x, zi = torch.randn(B, T, 2, device="cuda"), torch.randn(B, 2, device="cuda")
    torch.library.opcheck(torch.ops.philtorch.lti_recur2.default, (torch.randn(2, 2, device="cuda") * 0.3, zi, x))
    torch.library.opcheck(torch.ops.philtorch.recur2.default, (torch.randn(B, T, 2, 2, device="cuda") * 0.3, zi, x))
    torch.library.opcheck(torch.ops.philtorch.lti_recur.default,
                          (torch.rand(B, device="cuda") - 0.5, zi[:, 0].contiguous(), x[..., 0].contiguous()))


def test_reference_autograd_functions_on_cuda(ref_pkg):
    """The reference's own Functions (its backward re-enters the ops) pass gradcheck / gradgradcheck
    on CUDA tensors: tests/test_grad.py:73-112,151-186,225-258 of the reference with device = cuda."""
    from philtorch.lti.recur import LTIRecurrence
    from philtorch.lti.ssm import LTIMatrixRecurrence
    from philtorch.lpv.ssm import MatrixRecurrence

    g = torch.Generator().manual_seed(3)
    B, T = 2, 17

    def rn(*s, scale=1.0):
        return (torch.randn(*s, generator=g, dtype=torch.float64) * scale).cuda().requires_grad_()

    for a in (rn(B, scale=0.5), rn(1, scale=0.5)):
        args = (a, rn(B), rn(B, T))
        assert torch.autograd.gradcheck(LTIRecurrence.apply, args)
        assert torch.autograd.gradgradcheck(LTIRecurrence.apply, args)
    for n in (2, 3):
        for A in (rn(n, n, scale=0.3), rn(B, n, n, scale=0.3)):
            args = (A, rn(B, n), rn(B, T, n))
            assert torch.autograd.gradcheck(LTIMatrixRecurrence.apply, args)
            assert torch.autograd.gradgradcheck(LTIMatrixRecurrence.apply, args)
        for A in (rn(T, n, n, scale=0.3), rn(B, T, n, n, scale=0.3)):
            args = (A, rn(B, n), rn(B, T, n))
            assert torch.autograd.gradcheck(MatrixRecurrence.apply, args)
            assert torch.autograd.gradgradcheck(MatrixRecurrence.apply, args)
    ptb.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_reference_public_api_on_cuda(ref_pkg, dtype):
    """lfilter / state_space_recursion of the reference with unroll_factor = 1 (its extension route):
    the same call on CUDA tensors (these kernels) and on CPU tensors (its own kernels), values and
    gradients."""
    pt = ref_pkg
    g = torch.Generator().manual_seed(4)
    B, T = 3, 5000
    t = tol(dtype) * 10
    r = 0.3 + 0.6 * torch.rand(B, generator=g, dtype=torch.float64)
    th = 3.0 * torch.rand(B, generator=g, dtype=torch.float64)
    a = torch.stack([-2 * r * torch.cos(th), r * r], -1).to(dtype)
    b = torch.randn(B, 3, generator=g, dtype=torch.float64).to(dtype)
    x = torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype)
    gy = torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype)
    res = {}
    for dev in ("cpu", "cuda"):
        ins = [v.to(dev).requires_grad_() for v in (b, a, x)]
        y = pt.lti.lfilter(*ins, form="tdf2", unroll_factor=1)
        res[dev] = (y,) + torch.autograd.grad(y, ins, gy.to(dev))
    for got, ref in zip(res["cuda"], res["cpu"]):
        assert got.is_cuda and rel_err(got, ref) <= t
    A = (torch.randn(B, T, 2, 2, generator=g, dtype=torch.float64) * 0.4).to(dtype)
    zi = torch.randn(B, 2, generator=g, dtype=torch.float64).to(dtype)
    x2 = torch.randn(B, T, 2, generator=g, dtype=torch.float64).to(dtype)
    gy2 = torch.randn(B, T, 2, generator=g, dtype=torch.float64).to(dtype)
    res = {}
    for dev in ("cpu", "cuda"):
        ins = [v.to(dev).requires_grad_() for v in (A, zi, x2)]
        y = pt.lpv.ssm.MatrixRecurrence.apply(*ins)
        res[dev] = (y,) + torch.autograd.grad(y, ins, gy2.to(dev))
    for got, ref in zip(res["cuda"], res["cpu"]):
        assert got.is_cuda and rel_err(got, ref) <= t
    ptb.check_errors()
