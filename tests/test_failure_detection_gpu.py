"""Failure detection without a GPU fault: a bounded device-side wait is made to run out (a
look-back record that nothing writes), the kernel must report it in the status word, finish on
its own, and leave the context usable."""
import ctypes
import time

import pytest
import torch

import philtorch_b200 as ptb
from philtorch_b200 import _lib
from conftest import rel_err
from oracle import cport

pytestmark = pytest.mark.gpu


def test_expired_lookback_wait_is_reported_and_context_survives():
    lib = _lib.lib
    n = lib.ptb_selftest_wait_expiry_elems()
    buf = torch.rand(n, device="cuda") * 0.5
    ws = torch.empty(lib.ptb_workspace_bytes(1, n), dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.ptb_set_wait_limit_ms(100) == 0
    try:
        t0 = time.time()
        rc = lib.ptb_selftest_wait_expiry(ws.data_ptr(), ws.numel(), buf.data_ptr(), n, status.data_ptr(), stream)
        assert rc == 0, lib.ptb_error_string(rc)
        host = ctypes.c_uint32(0)
        assert lib.ptb_read_status(status.data_ptr(), stream, ctypes.byref(host)) == 0   # synchronises
        elapsed = time.time() - t0
    finally:
        assert lib.ptb_set_wait_limit_ms(2000) == 0
    assert host.value & 1, f"look-back timeout bit not set: {host.value}"
    assert 0.05 < elapsed < 5.0, elapsed          # gave up after about the limit, did not hang

    # the same path through the package: the sticky word makes check_errors raise once
    st = _lib.status_word(torch.device("cuda", torch.cuda.current_device()))
    st.fill_(1)
    with pytest.raises(RuntimeError, match="look-back wait expired"):
        ptb.check_errors()
    ptb.check_errors()   # cleared

    # the context is intact: a normal call still gives the right answer
    g = torch.Generator().manual_seed(0)
    a = torch.rand(4, 30000, generator=g) * 1.9 - 0.95
    zi, x = torch.randn(4, generator=g), torch.randn(4, 30000, generator=g)
    y = ptb.lpv.linear_recurrence(a.cuda(), zi.cuda(), x.cuda())
    assert rel_err(y, cport.recur1(a, zi, x)) <= 1e-4
    ptb.check_errors()


def test_wait_limit_argument_check():
    assert _lib.lib.ptb_set_wait_limit_ms(0) == 1
    assert _lib.lib.ptb_set_wait_limit_ms(2000) == 0
