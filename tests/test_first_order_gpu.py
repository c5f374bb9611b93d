"""GPU parity of the first-order kernels (through the torch ops -> ctypes -> C ABI) against the
CPU oracle and the golden vectors made by the reference.  Tolerance: max|out-ref|/max|ref|
<= 1e-4 (fp32), <= 1e-10 (fp64)."""
import pytest
import torch

import philtorch_b200 as ptb
from philtorch_b200 import workloads
from philtorch_b200.autograd import LPVRecurrence, LTIRecurrence
from conftest import load_golden, rel_err, tol
from oracle import cport

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = {"f32": torch.float32, "f64": torch.float64}

# tile sizes are a few thousand samples (e.g. 9216 forward / 5120 backward in fp32, half that in
# fp64): cover below / at / above one and several tiles, and lengths that are not a multiple of
# 16 bytes (plain-load path)
LENGTHS = [1, 2, 3, 4, 5, 31, 32, 33, 101, 1535, 1536, 1537, 2560, 2561, 3072, 3073, 4608, 4609, 5119, 5120,
           5121, 9215, 9216, 9217, 12289, 18432, 40000]


def _cuda(*ts):
    return [t.to(DEV) for t in ts]


def _run_fo(kind, a, zi, x, gy):
    fn = LTIRecurrence if kind == "lti" else LPVRecurrence
    a_, zi_, x_ = (t.to(DEV).requires_grad_() for t in (a, zi, x))
    y = fn.apply(a_, zi_, x_)
    ga, gzi, gx = torch.autograd.grad(y, (a_, zi_, x_), gy.to(DEV))
    ptb.check_errors()
    return y, ga, gzi, gx


def _check_fo(kind, a, zi, x, gy, dtype):
    t = tol(dtype)
    y, ga, gzi, gx = _run_fo(kind, a, zi, x, gy)
    if kind == "lti":
        y_ref = cport.lti_recur(a, zi, x)
        ga_ref, gzi_ref, gx_ref = cport.lti_recur_bwd(a, zi, y_ref, gy)
    else:
        y_ref = cport.recur1(a, zi, x)
        ga_ref, gzi_ref, gx_ref = cport.recur1_bwd(a, zi, y_ref, gy)
    assert rel_err(y, y_ref) <= t
    assert rel_err(gx, gx_ref) <= t
    assert rel_err(gzi, gzi_ref) <= t
    assert rel_err(ga, ga_ref.reshape(ga.shape)) <= t


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("T", LENGTHS)
@pytest.mark.parametrize("B", [1, 3])
def test_lpv_lengths(dtype, T, B):
    g = torch.Generator().manual_seed(T * 7 + B)
    a = (torch.rand(B, T, generator=g, dtype=torch.float64) * 1.98 - 0.99).to(dtype)
    zi = torch.randn(B, generator=g, dtype=torch.float64).to(dtype)
    x = torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype)
    gy = torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype)
    _check_fo("lpv", a, zi, x, gy, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("T", LENGTHS)
@pytest.mark.parametrize("mode", ["batched", "shared1", "scalar"])
def test_lti_lengths(dtype, T, mode):
    B = 3
    g = torch.Generator().manual_seed(T * 11 + len(mode))
    a = (torch.rand(B if mode == "batched" else 1, generator=g, dtype=torch.float64) * 1.9 - 0.95).to(dtype)
    if mode == "scalar":
        a = a[0]
    zi = torch.randn(B, generator=g, dtype=torch.float64).to(dtype)
    x = torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype)
    gy = torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype)
    _check_fo("lti", a, zi, x, gy, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_lpv_shared_coefficients(dtype):
    B, T = 5, 7000
    g = torch.Generator().manual_seed(3)
    a = (torch.rand(T, generator=g, dtype=torch.float64) * 1.98 - 0.99).to(dtype)
    zi = torch.randn(B, generator=g, dtype=torch.float64).to(dtype)
    x = torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype)
    gy = torch.randn(B, T, generator=g, dtype=torch.float64).to(dtype)
    _check_fo("lpv", a, zi, x, gy, dtype)


@pytest.mark.parametrize("tag", ["f32", "f64"])
@pytest.mark.parametrize("mode", ["batched", "shared1", "scalar"])
def test_lti_golden(tag, mode):
    g = load_golden(f"lti_recur_{mode}_{tag}")
    t = tol(DT[tag])
    y, ga, gzi, gx = _run_fo("lti", g["a"], g["zi"], g["x"], g["gy"])
    assert rel_err(y, g["y"]) <= t
    assert rel_err(ga, g["grad_a"]) <= t
    assert rel_err(gzi, g["grad_zi"]) <= t
    assert rel_err(gx, g["grad_x"]) <= t


@pytest.mark.parametrize("tag", ["f32", "f64"])
@pytest.mark.parametrize("mode", ["batched", "shared"])
def test_lpv_golden(tag, mode):
    g = load_golden(f"lpv_recur1_{mode}_{tag}")
    t = tol(DT[tag])
    y, ga, gzi, gx = _run_fo("lpv", g["a"], g["zi"], g["x"], g["gy"])
    assert rel_err(y, g["y"]) <= t
    assert rel_err(y, g["y_python_loop"]) <= t
    assert rel_err(ga, g["grad_a"]) <= t
    assert rel_err(gzi, g["grad_zi"]) <= t
    assert rel_err(gx, g["grad_x"]) <= t


def test_config_goldens():
    g = load_golden("config1_small")
    w = workloads.lti_first_order(B=8, T=4096)
    y, ga, _, gx = _run_fo("lti", w["a"], w["zi"], w["x"], w["gy"])
    assert rel_err(y, g["y"]) <= 1e-4 and rel_err(ga, g["grad_a"]) <= 1e-4 and rel_err(gx, g["grad_x"]) <= 1e-4
    g = load_golden("config2_small")
    w = workloads.lpv_first_order(B=4, T=8192)
    y, ga, gzi, gx = _run_fo("lpv", w["a"], w["zi"], w["x"], w["gy"])
    assert rel_err(y, g["y"]) <= 1e-4 and rel_err(ga, g["grad_a"]) <= 1e-4
    assert rel_err(gzi, g["grad_zi"]) <= 1e-4 and rel_err(gx, g["grad_x"]) <= 1e-4
    g = load_golden("config5_small")
    w = workloads.long_first_order(B=2, T=16384)
    y, ga, _, gx = _run_fo("lpv", w["a"], w["zi"], w["x"], w["gy"])
    assert rel_err(y, g["y"]) <= 1e-4 and rel_err(ga, g["grad_a"]) <= 1e-4 and rel_err(gx, g["grad_x"]) <= 1e-4


@pytest.mark.parametrize("kind,B,T", [("lpv", 64, 1 << 16), ("lti", 64, 1 << 16), ("lpv", 2, 1 << 21),
                                      ("lti", 1, 1 << 21), ("lpv", 300, 9000)])
def test_many_tiles(kind, B, T):
    """Enough tiles to keep every SM busy and make the look-back span several predecessors."""
    dtype = torch.float32
    w = workloads.lpv_first_order(B=B, T=T) if kind == "lpv" else workloads.lti_first_order(B=B, T=T)
    zi = torch.randn(B, generator=torch.Generator().manual_seed(5))
    _check_fo(kind, w["a"], zi, w["x"], w["gy"], dtype)


def test_slowly_decaying_long_row():
    """a close to 1 (config-5 distribution): carries travel far, in fp32 and fp64."""
    for dtype in (torch.float32, torch.float64):
        w = workloads.long_first_order(B=2, T=1 << 20, dtype=dtype)
        _check_fo("lpv", w["a"], w["zi"], w["x"], w["gy"], dtype)


def test_public_api_and_errors():
    g = load_golden("lti_linear_recurrence_f64")
    a, zi, x = _cuda(g["a"], g["zi"], g["x"])
    assert rel_err(ptb.lti.linear_recurrence(a, zi, x), g["y"]) <= 1e-10
    assert rel_err(ptb.lti.linear_recurrence(a, zi, x, unroll_factor=7), g["y_unrolled"]) <= 1e-10
    assert rel_err(ptb.lti.linear_recurrence(a[0], zi[0], x), g["y_scalar_a"]) <= 1e-10
    with pytest.raises(ValueError):
        ptb.lti.linear_recurrence(a[:2], zi, x)
    with pytest.raises(ValueError):
        ptb.lti.linear_recurrence(a, zi, x, unroll_factor=0)
    with pytest.raises(RuntimeError):
        ptb.lti.linear_recurrence(a.float(), zi, x)          # dtype mismatch
    with pytest.raises(RuntimeError):
        ptb.lti.linear_recurrence(a.cpu(), zi.cpu(), x.cpu())  # no CPU path
    with pytest.raises(RuntimeError):
        ptb.lti.linear_recurrence(a.long(), zi.long(), x.long())     # integer tensors have no kernels
    # empty inputs
    assert ptb.lti.linear_recurrence(a, zi, x[:, :0]).shape == (4, 0)
    assert ptb.lpv.linear_recurrence(x[:0], zi[:0], x[:0]).shape == (0, 130)


def test_non_contiguous_inputs():
    g = torch.Generator().manual_seed(9)
    B, T = 4, 5000
    a = (torch.rand(T, B, generator=g) * 1.9 - 0.95).t()       # (B,T) view, column-major
    x = torch.randn(B, 2 * T, generator=g)[:, ::2]
    zi = torch.randn(2 * B, generator=g)[::2]
    y = ptb.lpv.linear_recurrence(a.to(DEV), zi.to(DEV), x.to(DEV))
    assert rel_err(y, cport.recur1(a, zi, x)) <= 1e-4


def test_repeatable():
    w = workloads.lpv_first_order(B=32, T=1 << 16)
    a, zi, x = _cuda(w["a"], w["zi"], w["x"])
    y1 = ptb.lpv.linear_recurrence(a, zi, x)
    y2 = ptb.lpv.linear_recurrence(a, zi, x)
    assert rel_err(y1, y2) <= 1e-6   # look-back association may differ in the last bits only
    ptb.check_errors()


@pytest.mark.parametrize("tag,dtype,eps", [("f16", torch.float16, 2.0 ** -11), ("bf16", torch.bfloat16, 2.0 ** -8)])
def test_low_precision_storage(tag, dtype, eps):
    """float16 / bfloat16 inputs: float32 arithmetic, one rounding per result.  Against the float64
    oracle on the same 16-bit inputs the error is one rounding; the reference, which rounds after
    every step, is matched within a few of its own roundings (vectors made by running it)."""
    g = load_golden(f"lti_recur_batched_{tag}")
    a, zi, x, gy = (g[k].to(dtype) for k in ("a", "zi", "x", "gy"))     # exactly representable: stored from 16-bit values
    y, ga, gzi, gx = _run_fo("lti", a, zi, x, gy)
    assert y.dtype == dtype and ga.dtype == dtype and gx.dtype == dtype
    y64 = cport.lti_recur(a.double(), zi.double(), x.double())
    ga64, gzi64, gx64 = cport.lti_recur_bwd(a.double(), zi.double(), y64, gy.double())
    assert rel_err(y, y64) <= 1.01 * eps and rel_err(gx, gx64) <= 1.01 * eps
    assert rel_err(ga, ga64) <= 4 * eps and rel_err(gzi, gzi64) <= 1.01 * eps
    assert rel_err(y, g["y"]) <= 16 * eps and rel_err(gx, g["grad_x"]) <= 16 * eps
    assert rel_err(ga, g["grad_a"]) <= 64 * eps and rel_err(gzi, g["grad_zi"]) <= 16 * eps
    # per-sample coefficients take the same route
    al = a.unsqueeze(1).expand(-1, x.shape[1]).contiguous()
    yl, _, _, _ = _run_fo("lpv", al, zi, x, gy)
    assert yl.dtype == dtype and rel_err(yl, y64) <= 1.01 * eps


@pytest.mark.parametrize("dtype,eps", [(torch.float16, 2.0 ** -11), (torch.bfloat16, 2.0 ** -8)])
@pytest.mark.parametrize("kind", ["lti", "lpv"])
@pytest.mark.parametrize("T", [8, 20000, 65536])
def test_two_byte_tile_storage(dtype, eps, kind, T):
    """Rows of a multiple of 8 samples go through the kernels that stage and store 2-byte samples
    (the others through a float32 copy): both routes agree with the float64 oracle on the same
    16-bit inputs to one rounding, several tiles per row included."""
    from philtorch_b200 import ops as ops_mod

    B = 6
    g = torch.Generator().manual_seed(T)
    a = ((torch.rand(B, T, generator=g) * 1.6 - 0.8) if kind == "lpv" else (torch.rand(B, generator=g) * 1.6 - 0.8)).to(dtype)
    zi = torch.randn(B, generator=g).to(dtype)
    x, gy = torch.randn(B, T, generator=g).to(dtype), torch.randn(B, T, generator=g).to(dtype)
    assert ops_mod._two_byte_kernels_apply((a.cuda(), zi.cuda(), x.cuda()))
    y, ga, gzi, gx = _run_fo(kind, a, zi, x, gy)
    assert y.dtype == dtype and ga.dtype == dtype and gzi.dtype == dtype and gx.dtype == dtype
    fwd = cport.lti_recur if kind == "lti" else cport.recur1
    bwd = cport.lti_recur_bwd if kind == "lti" else cport.recur1_bwd
    y64 = fwd(a.double(), zi.double(), x.double())
    # the adjoint reads the ROUNDED outputs, as any caller that keeps y in 16 bits does
    ga64, gzi64, gx64 = bwd(a.double(), zi.double(), y.double().cpu(), gy.double())
    assert rel_err(y, y64) <= 1.01 * eps and rel_err(gx, gx64) <= 1.01 * eps
    assert rel_err(gzi, gzi64) <= 1.01 * eps
    assert rel_err(ga, ga64) <= (1.01 * eps if kind == "lpv" else 4 * eps)
    # the same call with a row length that is not a multiple of 8 takes the float32-copy route
    if T > 8:
        y2, *_ = _run_fo(kind, a[..., :T - 3].contiguous() if kind == "lpv" else a, zi, x[:, :T - 3].contiguous(),
                         gy[:, :T - 3].contiguous())
        assert rel_err(y2, y64[:, :T - 3]) <= 1.01 * eps
    ptb.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.complex64])
@pytest.mark.parametrize("T", [20000, 20001, 64])
def test_shared_coefficients_gradient_sum(dtype, T):
    """Per-sample coefficients shared by the rows, a (T,): grad_a is the sum over the rows
    (philtorch/__init__.py:62-65 of the reference).  Rows that qualify for bulk copies accumulate
    into the one (T,) array inside the kernel (TMA reduce copies), others sum per-row gradients
    afterwards: both against the oracle."""
    B = 7
    g = torch.Generator().manual_seed(T)
    real = torch.float64 if dtype == torch.float64 else torch.float32

    def rnd(*s):
        v = torch.randn(*s, generator=g, dtype=torch.float64)
        if dtype.is_complex:
            v = torch.complex(v, torch.randn(*s, generator=g, dtype=torch.float64))
        return v.to(dtype)

    a = (rnd(T) * 0.4).contiguous()
    zi, x, gy = rnd(B), rnd(B, T), rnd(B, T)
    y, ga, gzi, gx = _run_fo("lpv", a, zi, x, gy)
    y_ref = cport.recur1(a, zi, x)
    ga_ref, gzi_ref, gx_ref = cport.recur1_bwd(a, zi, y_ref, gy)
    t = tol(real)
    assert ga.shape == (T,)
    assert rel_err(y, y_ref) <= t and rel_err(gx, gx_ref) <= t and rel_err(gzi, gzi_ref) <= t
    assert rel_err(ga, ga_ref) <= t * (10 if real == torch.float64 else 1)
    ptb.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.complex64])
@pytest.mark.parametrize("kind,a_shape", [("lti", "batched"), ("lti", "scalar"), ("lpv", "batched"), ("lpv", "shared")])
def test_coefficient_gradients_without_grad_x(dtype, kind, a_shape):
    """Only the coefficients (and the initial state) require gradients: the adjoint kernels are told
    not to write grad_x at all; grad_a and grad_zi against the oracle."""
    B, T = 5, 20000
    g = torch.Generator().manual_seed(31)
    real = torch.float64 if dtype == torch.float64 else torch.float32

    def rnd(*s):
        v = torch.randn(*s, generator=g, dtype=torch.float64)
        if dtype.is_complex:
            v = torch.complex(v, torch.randn(*s, generator=g, dtype=torch.float64))
        return v.to(dtype)

    if kind == "lti":
        a = (rnd(B) if a_shape == "batched" else rnd(1)[0]) * 0.4
    else:
        a = (rnd(B, T) if a_shape == "batched" else rnd(T)) * 0.4
    zi, x, gy = rnd(B), rnd(B, T), rnd(B, T)
    a_, zi_ = a.to(DEV).requires_grad_(), zi.to(DEV).requires_grad_()
    fn = ptb.lti.linear_recurrence if kind == "lti" else ptb.lpv.linear_recurrence
    y = fn(a_, zi_, x.to(DEV))
    ga, gzi = torch.autograd.grad(y, (a_, zi_), gy.to(DEV))
    if kind == "lti":
        y_r = cport.lti_recur(a, zi, x)
        ga_r, gzi_r, _ = cport.lti_recur_bwd(a, zi, y_r, gy)
    else:
        y_r = cport.recur1(a, zi, x)
        ga_r, gzi_r, _ = cport.recur1_bwd(a, zi, y_r, gy)
    t = tol(real)
    assert rel_err(y, y_r) <= t
    assert rel_err(ga, ga_r.reshape(ga.shape)) <= t * 10 and rel_err(gzi, gzi_r) <= t
    ptb.check_errors()
