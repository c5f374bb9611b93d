"""The entry point that allocates nothing (``ptb_lpv_recur_fwd_static``).

Some callers cannot hand the library a workspace and must not allocate device memory in their
processing call either (a real-time audio callback, a host that gave all GPU memory to its own
pool).  For them the library keeps a fixed scratch array inside its own image.  This test calls
that entry point straight through the C ABI, twice in a row with different inputs -- the second
call finds the first call's records in the shared scratch and must clear them -- and compares each
result with the regular entry point that takes a caller-provided workspace.  It also checks that
a problem beyond the built-in scratch is refused with its own error code.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bind():
    from philtorch_b200 import _lib

    lib = _lib.lib
    vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    lib.ptb_lpv_recur_fwd_static.argtypes = [i32, i64, i64, vp, i32, vp, i32, vp, vp, vp, vp, vp]
    lib.ptb_lpv_recur_fwd_static.restype = i32
    lib.ptb_lpv_recur_fwd_static_max_tiles.argtypes = [i32]
    lib.ptb_lpv_recur_fwd_static_max_tiles.restype = i64
    return lib


def _inputs(B, T, seed, dtype):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = (torch.rand(B, T, generator=g, device="cuda", dtype=torch.float64) * 1.98 - 0.99).to(dtype)
    zi = torch.randn(B, generator=g, device="cuda", dtype=torch.float64).to(dtype)
    x = torch.randn(B, T, generator=g, device="cuda", dtype=torch.float64).to(dtype)
    return a, zi, x


@pytest.mark.parametrize("dtype,code,tol", [(torch.float32, 0, 1e-4), (torch.float64, 1, 1e-10)])
def test_static_scratch_matches_workspace_entry_point(dtype, code, tol):
    lib = _bind()
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for call, (B, T) in enumerate([(24, 40000), (7, 100003)]):   # second: other shape, unaligned rows
        a, zi, x = _inputs(B, T, 100 + call, dtype)
        y_static, zf_static = torch.empty_like(x), torch.empty_like(zi)
        rc = lib.ptb_lpv_recur_fwd_static(code, B, T, a.data_ptr(), 1, zi.data_ptr(), 1, x.data_ptr(),
                                          y_static.data_ptr(), zf_static.data_ptr(), status.data_ptr(), stream)
        assert rc == 0, lib.ptb_error_string(rc)
        nbytes = lib.ptb_workspace_bytes(B, T)
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        y_ws, zf_ws = torch.empty_like(x), torch.empty_like(zi)
        rc = lib.ptb_lpv_recur_fwd(code, B, T, a.data_ptr(), 1, zi.data_ptr(), 1, x.data_ptr(), y_ws.data_ptr(),
                                   zf_ws.data_ptr(), ws.data_ptr(), nbytes, status.data_ptr(), stream)
        assert rc == 0, lib.ptb_error_string(rc)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        scale = y_ws.abs().max().item()
        assert (y_static - y_ws).abs().max().item() / scale <= tol
        assert (zf_static - zf_ws).abs().max().item() / scale <= tol
        assert (zf_ws - y_ws[:, -1]).abs().max().item() / scale <= tol   # zf is the last sample


def test_static_scratch_limit_is_refused():
    lib = _bind()
    max_tiles = lib.ptb_lpv_recur_fwd_static_max_tiles(0)
    assert 50_000 < max_tiles < 200_000
    B = 2 * max_tiles   # one tile per row: twice as many records as are guaranteed to fit
    a, zi, x = _inputs(B, 8, 5, torch.float32)
    y = torch.empty_like(x)
    rc = lib.ptb_lpv_recur_fwd_static(0, B, 8, a.data_ptr(), 1, zi.data_ptr(), 1, x.data_ptr(), y.data_ptr(),
                                      None, None, torch.cuda.current_stream().cuda_stream)
    assert rc == 5
    assert b"scratch" in lib.ptb_error_string(rc)


def test_static_shared_coefficients_without_status_word():
    """Coefficients shared by the rows (a_batched = 0) and no status word (NULL): same results as the
    entry point with a workspace."""
    lib = _bind()
    stream = torch.cuda.current_stream().cuda_stream
    B, T = 5, 30001
    a, zi, x = _inputs(B, T, 9, torch.float32)
    a = a[0].contiguous()
    y_static, y_ws = torch.empty_like(x), torch.empty_like(x)
    rc = lib.ptb_lpv_recur_fwd_static(0, B, T, a.data_ptr(), 0, zi.data_ptr(), 1, x.data_ptr(), y_static.data_ptr(),
                                      None, None, stream)
    assert rc == 0, lib.ptb_error_string(rc)
    nbytes = lib.ptb_workspace_bytes(B, T)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    rc = lib.ptb_lpv_recur_fwd(0, B, T, a.data_ptr(), 0, zi.data_ptr(), 1, x.data_ptr(), y_ws.data_ptr(), None,
                               ws.data_ptr(), nbytes, None, stream)
    assert rc == 0, lib.ptb_error_string(rc)
    torch.cuda.synchronize()
    assert (y_static - y_ws).abs().max().item() / y_ws.abs().max().item() <= 1e-4


def test_static_entry_point_is_real_only():
    """Complex dtype codes are not dispatched here: the size query answers 0 and the call is refused."""
    lib = _bind()
    for code in (2, 3, 7):
        assert lib.ptb_lpv_recur_fwd_static_max_tiles(code) == 0
    a, zi, x = _inputs(2, 64, 1, torch.float32)
    y = torch.empty_like(x)
    rc = lib.ptb_lpv_recur_fwd_static(2, 2, 32, a.data_ptr(), 1, zi.data_ptr(), 1, x.data_ptr(), y.data_ptr(), None,
                                      None, torch.cuda.current_stream().cuda_stream)
    assert rc == 1
