"""ctypes binding of ``libphiltorch_b200.so`` (the C ABI declared in include/philtorch_b200.h).

There is no CPU fallback: if the library is missing the import fails, and every wrapper
raises for non-CUDA tensors.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# PHILTORCH_B200_LIB: load another build of the same library (kernel tuning experiments)
LIB_PATH = os.environ.get("PHILTORCH_B200_LIB") or os.path.join(_HERE, "libphiltorch_b200.so")

PTB_F32, PTB_F64 = 0, 1
PTB_C64, PTB_C128 = 2, 3
_DTYPES = {torch.float32: PTB_F32, torch.float64: PTB_F64}
PTB_F16, PTB_BF16 = 4, 5
_COMPLEX_DTYPES = {torch.complex64: PTB_C64, torch.complex128: PTB_C128,
                   torch.float16: PTB_F16, torch.bfloat16: PTB_BF16}   # first-order kernels only

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python philtorch_b200/build.py` "
        "(needs nvcc; philtorch_b200 has no CPU or pure-PyTorch fallback)")

lib = ctypes.CDLL(LIB_PATH)

_vp, _i64, _i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
_tail = [_vp, _i64, _vp, _vp]  # workspace, workspace_bytes, status, stream

lib.ptb_version.restype = ctypes.c_char_p
lib.ptb_error_string.restype = ctypes.c_char_p
lib.ptb_error_string.argtypes = [_i32]
lib.ptb_last_cuda_error.restype = _i32
lib.ptb_workspace_bytes.restype = _i64
lib.ptb_workspace_bytes.argtypes = [_i64, _i64]
lib.ptb_read_status.argtypes = [_vp, _vp, ctypes.POINTER(ctypes.c_uint32)]

_fo_fwd = [_i32, _i64, _i64, _vp, _i32, _vp, _i32, _vp, _vp, _vp] + _tail
_fo_bwd = [_i32, _i64, _i64, _vp, _i32, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp] + _tail
for _n in ("ptb_lti_recur_fwd", "ptb_lpv_recur_fwd"):
    getattr(lib, _n).argtypes = _fo_fwd
    getattr(lib, _n).restype = _i32
for _n in ("ptb_lti_recur_bwd", "ptb_lpv_recur_bwd"):
    getattr(lib, _n).argtypes = _fo_bwd
    getattr(lib, _n).restype = _i32

lib.ptb_lpv_recur_bwd_shared.argtypes = [_i32, _i64, _i64, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp] + _tail
lib.ptb_lpv_recur_bwd_shared.restype = _i32

_so_fwd = [_i32, _i64, _i64, _vp, _i32, _vp, _vp, _i32, _vp, _vp] + _tail
_so_bwd = [_i32, _i64, _i64, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp] + _tail
for _n in ("ptb_lti_recur2_fwd", "ptb_lpv_recur2_fwd"):
    getattr(lib, _n).argtypes = _so_fwd
    getattr(lib, _n).restype = _i32
for _n in ("ptb_lti_recur2_bwd", "ptb_lpv_recur2_bwd"):
    getattr(lib, _n).argtypes = _so_bwd
    getattr(lib, _n).restype = _i32
lib.ptb_lpv_recur2_bwd_shared.argtypes = [_i32, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp] + _tail
lib.ptb_lpv_recur2_bwd_shared.restype = _i32
lib.ptb_lpv_recur2_carry_chunks.argtypes = [_i32, _i64]
lib.ptb_lpv_recur2_carry_chunks.restype = _i64
lib.ptb_lpv_recur2_zero_carry.argtypes = [_i32, _i64, _i64, _vp, _vp, _i32, _vp, _vp, _vp] + _tail
lib.ptb_lpv_recur2_zero_carry.restype = _i32
lib.ptb_lpv_recur2_fold_products.argtypes = [_i32, _i64, _i64, _vp, _vp, _vp]
lib.ptb_lpv_recur2_fold_products.restype = _i32
lib.ptb_lpv_recur2_fixup_fwd.argtypes = [_i32, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp]
lib.ptb_lpv_recur2_fixup_fwd.restype = _i32
lib.ptb_lpv_recur2_fixup_bwd.argtypes = [_i32, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp]
lib.ptb_lpv_recur2_fixup_bwd.restype = _i32
lib.ptb_biquad_tdf2_fwd.argtypes = [_i32, _i64, _i64, _vp, _vp, _i32, _vp, _vp, _vp, _vp] + _tail
lib.ptb_biquad_tdf2_fwd.restype = _i32
lib.ptb_biquad_tdf2_bwd.argtypes = [_i32, _i64, _i64, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp] + _tail
lib.ptb_biquad_tdf2_bwd.restype = _i32

lib.ptb_lpv_recur_carry.argtypes = [_i32, _i64, _i64, _vp, _i32, _vp, _i32, _vp] + _tail
lib.ptb_lpv_recur_carry.restype = _i32
lib.ptb_lpv_recur_fwd_carry.argtypes = [_i32, _i64, _i64, _vp, _i32, _vp, _vp, _vp] + _tail
lib.ptb_lpv_recur_fwd_carry.restype = _i32

lib.ptb_recur_n_workspace_bytes.argtypes = [_i32, _i32, _i64, _i64]
lib.ptb_recur_n_workspace_bytes.restype = _i64
lib.ptb_outer_prev_sum_chunks.argtypes = [_i64, _i64]
lib.ptb_outer_prev_sum_chunks.restype = _i64
lib.ptb_outer_prev_sum.argtypes = [_i32, _i32, _i64, _i64, _vp, _vp, _vp, _vp, _vp]
lib.ptb_outer_prev_sum.restype = _i32
lib.ptb_recur_n_set_policy.argtypes = [_i32]
lib.ptb_recur_n_set_policy.restype = _i32
lib.ptb_recur_n_fwd.argtypes = [_i32, _i32, _i64, _i64, _vp, _i32, _i32, _vp, _vp, _vp, _vp] + _tail
lib.ptb_recur_n_fwd.restype = _i32
lib.ptb_recur_n_adj.argtypes = [_i32, _i32, _i64, _i64, _vp, _i32, _i32, _vp, _vp, _vp, _vp] + _tail
lib.ptb_recur_n_adj.restype = _i32
lib.ptb_lpv_recur_fold_maps.argtypes = [_i32, _i64, _i64, _vp, _i32, _vp, _vp]
lib.ptb_lpv_recur_fold_maps.restype = _i32
lib.ptb_lpv_recur_fixup_fwd.argtypes = [_i32, _i64, _i64, _i64, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _vp, _vp]
lib.ptb_lpv_recur_fixup_fwd.restype = _i32
lib.ptb_lpv_recur_fixup_bwd.argtypes = [_i32, _i64, _i64, _i64, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _vp, _vp,
                                        _vp, _vp]
lib.ptb_lpv_recur_fixup_bwd.restype = _i32

lib.ptb_lpv_recur2_set_small_cta_min_rows.argtypes = [_i64]
lib.ptb_lpv_recur2_set_small_cta_min_rows.restype = _i32
lib.ptb_biquad_set_policy.argtypes = [_i32]
lib.ptb_biquad_set_policy.restype = _i32
lib.ptb_set_wait_limit_ms.argtypes = [_i64]
lib.ptb_set_wait_limit_ms.restype = _i32
lib.ptb_selftest_wait_expiry_elems.restype = _i64
lib.ptb_selftest_wait_expiry.argtypes = [_vp, _i64, _vp, _i64, _vp, _vp]
lib.ptb_selftest_wait_expiry.restype = _i32

lib.ptb_sos_cascade_set_mode.argtypes = [_i32]
lib.ptb_sos_cascade_set_mode.restype = _i32
lib.ptb_sos_cascade_workspace_bytes.argtypes = [_i32, _i32, _i64, _i64]
lib.ptb_sos_cascade_workspace_bytes.restype = _i64
lib.ptb_sos_cascade_fwd.argtypes = [_i32, _i32, _i64, _i64, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp] + _tail
lib.ptb_sos_cascade_fwd.restype = _i32
lib.ptb_sos_cascade_bwd.argtypes = [_i32, _i32, _i64, _i64, _vp, _vp, _i32] + [_vp] * 9 + _tail
lib.ptb_sos_cascade_bwd.restype = _i32

lib.ptb_lti_recur_reverse_fused.argtypes = [_i32, _i64, _i64, _vp, _i32, _vp, _vp, _vp, ctypes.c_double, _vp, _vp] + _tail
lib.ptb_lti_recur_reverse_fused.restype = _i32
lib.ptb_modal_mix_partial_blocks.argtypes = [_i64]
lib.ptb_modal_mix_partial_blocks.restype = _i64
lib.ptb_modal_mix_fwd.argtypes = [_i32, _i64, _i64, _i64, _vp, _vp, _vp, _i32, _i32, _vp] + _tail
lib.ptb_modal_mix_fwd.restype = _i32
lib.ptb_modal_drive_fwd.argtypes = [_i32, _i64, _i64, _i64, _vp, _vp, _i32, _vp] + _tail
lib.ptb_modal_drive_fwd.restype = _i32
lib.ptb_modal_mix_bwd.argtypes = [_i32, _i64, _i64, _i64, _vp, _vp, _vp, _i32, _i32, _vp, _vp, _vp, _vp] + _tail
lib.ptb_modal_mix_bwd.restype = _i32
lib.ptb_modal_bank_tiles.argtypes = [_i64, _i64]
lib.ptb_modal_bank_tiles.restype = _i64
lib.ptb_modal_bank_fwd.argtypes = [_i32, _i64, _i64, _i64] + [_vp] * 10
lib.ptb_modal_bank_fwd.restype = _i32
lib.ptb_modal_bank_bwd.argtypes = [_i32, _i64, _i64, _i64] + [_vp] * 8 + [_i32] + [_vp] * 5
lib.ptb_modal_bank_bwd.restype = _i32
lib.ptb_comb_set_policy.argtypes = [_i32]
lib.ptb_comb_set_policy.restype = _i32
lib.ptb_comb_partial_blocks.argtypes = [_i64]
lib.ptb_comb_partial_blocks.restype = _i64
lib.ptb_comb_fwd.argtypes = [_i32, _i64, _i64, _i64, _vp, _i32, _vp, _i32, _vp, _vp] + _tail
lib.ptb_comb_fwd.restype = _i32
lib.ptb_comb_bwd.argtypes = [_i32, _i64, _i64, _i64, _vp, _i32, _vp, _i32, _vp, _vp, _vp, _vp, _vp] + _tail
lib.ptb_comb_bwd.restype = _i32

lib.ptb_lpv_biquad_workspace_bytes.argtypes = [_i32, _i64, _i64]
lib.ptb_lpv_biquad_workspace_bytes.restype = _i64
lib.ptb_lpv_biquad_df2_fwd.argtypes = [_i32, _i64, _i64, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp] + _tail
lib.ptb_lpv_biquad_df2_fwd.restype = _i32
lib.ptb_lpv_biquad_df2_bwd.argtypes = [_i32, _i64, _i64, _vp, _vp, _i32] + [_vp] * 8 + _tail
lib.ptb_lpv_biquad_df2_bwd.restype = _i32
lib.ptb_lpv_biquad_tdf2_fwd.argtypes = lib.ptb_lpv_biquad_df2_fwd.argtypes
lib.ptb_lpv_biquad_tdf2_fwd.restype = _i32
lib.ptb_lpv_biquad_tdf2_bwd.argtypes = lib.ptb_lpv_biquad_df2_bwd.argtypes
lib.ptb_lpv_biquad_tdf2_bwd.restype = _i32

_status: dict[int, torch.Tensor] = {}

ERROR_BITS = {1: "look-back wait expired", 2: "tile load wait expired", 4: "tile drain wait expired",
              8: "pipeline wait expired"}


def dtype_code(t: torch.Tensor, complex_ok: bool = False) -> int:
    """dtype code of the C ABI; complex64/complex128 and the 2-byte floats only where the kernels
    have them (first order)."""
    if complex_ok and t.dtype in _COMPLEX_DTYPES:
        return _COMPLEX_DTYPES[t.dtype]
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        kinds = "float32, float64, complex64 and complex128" if complex_ok else "float32 and float64"
        raise RuntimeError(f"these philtorch_b200 kernels support {kinds}, got {t.dtype}") from None


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("philtorch_b200 runs on CUDA tensors only (there is no CPU path); "
                               f"got a tensor on {t.device}")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"all tensors must be on the same device, got {dev} and {t.device}")
    return dev


def status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    s = _status.get(idx)
    if s is None:
        s = torch.zeros(1, dtype=torch.int32, device=device)
        _status[idx] = s
    return s


_ws_bytes: dict = {}


def workspace(B: int, T: int, device: torch.device) -> torch.Tensor:
    n = _ws_bytes.get((B, T))
    if n is None:
        n = _ws_bytes[(B, T)] = lib.ptb_workspace_bytes(B, T)
    return torch.empty(n, dtype=torch.uint8, device=device)


def ptr(t):
    return None if t is None else t.data_ptr()


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib.ptb_error_string(rc).decode()
        if rc == 3:
            msg += f" (cudaError {lib.ptb_last_cuda_error()})"
        raise RuntimeError(f"{what}: {msg}")


_current_device = torch._C._cuda_getDevice                # both skip the Python layers of torch.cuda.*:
_current_raw_stream = torch._C._cuda_getCurrentRawStream  # this function runs once per kernel launch


def call(fn, device: torch.device, B: int, T: int, *args, ws_bytes: int = -1) -> None:
    """Runs ``fn(*args, workspace, bytes, status, stream)`` on ``device``'s current stream."""
    ws = workspace(B, T, device) if ws_bytes < 0 else torch.empty(ws_bytes, dtype=torch.uint8, device=device)
    idx = device.index
    if idx is None:
        idx = _current_device()
    st = _status.get(idx)
    if st is None:
        st = status_word(device)
    if idx != _current_device():
        with torch.cuda.device(idx):
            rc = fn(*args, ws.data_ptr(), ws.numel(), st.data_ptr(), _current_raw_stream(idx))
    else:
        rc = fn(*args, ws.data_ptr(), ws.numel(), st.data_ptr(), _current_raw_stream(idx))
    if rc != 0:
        check(rc, fn.__name__)
    if CHECK_EVERY_CALL:
        check_errors(device)


# PHILTORCH_B200_CHECK=1: every call synchronises and raises at once if a device-side wait expired
# (a debugging aid: it serialises host and device).  Without it a kernel that gave up on a wait only
# sets a bit in the device's status word, and the results of that launch flow on until
# ``check_errors()`` is called.
CHECK_EVERY_CALL = os.environ.get("PHILTORCH_B200_CHECK", "0") not in ("", "0")


def check_errors(device=None) -> None:
    """Synchronises and raises if a kernel reported an expired device-side wait since the
    last check (results of such a launch are invalid)."""
    for idx, st in list(_status.items()):
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        v = int(st.item())
        if v:
            st.zero_()
            names = [n for b, n in ERROR_BITS.items() if v & b]
            raise RuntimeError(f"philtorch_b200 kernel error on cuda:{idx}: {', '.join(names)}")
