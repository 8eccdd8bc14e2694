"""ctypes binding of libmamba_b200.so (see include/mamba_b200.h for the contract).

There is no fallback: if the library has not been built, or a call returns an error code,
a RuntimeError is raised.  Nothing here computes anything on the CPU.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmamba_b200.so")

F32, BF16 = 0, 1
DELTA_SOFTPLUS = 1
REVERSE = 2
GENERAL_DECAY = 4
EUNSUPPORTED = -8

_i64, _int, _ptr = C.c_int64, C.c_int, C.c_void_p

_SIGNATURES = {
    "mb200_strerror": (C.c_char_p, [_int]),
    "mb200_version": (_int, []),
    "mb200_device_status": (_int, []),
    "mb200_selftest_wait_timeout": (_int, [_int, _ptr]),
    "mb200_sscan_chunk": (_int, []),
    "mb200_pscan_segments": (_int, [_i64] * 3),
    "mb200_pscan_fwd": (_int, [_ptr] * 3 + [_i64] * 9 + [_ptr] * 3 + [_int, _int, _ptr]),
    "mb200_pscan_noalloc_max_ws_floats": (_i64, []),
    "mb200_pscan_fwd_noalloc": (_int, [_ptr] * 3 + [_i64] * 9 + [_ptr] * 2 + [_int, _int, _ptr]),
    "mb200_pscan_bwd": (_int, [_ptr] * 5 + [_i64] * 13 + [_ptr] * 2 + [_int, _int, _ptr]),
    "mb200_sscan_fwd": (_int, [_ptr] * 12 + [_i64] * 3 + [_int] + [_i64] * 12 + [_int, _int, _ptr]),
    "mb200_sscan_bwd": (_int, [_ptr] * 20 + [_i64] * 3 + [_int] + [_i64] * 18 + [_int, _int, _ptr]),
    "mb200_sscan_bwd_carry": (_int, [_ptr] * 7 + [_i64] * 3 + [_int] + [_i64] * 8 + [_int, _int, _ptr]),
    "mb200_ssm_step": (_int, [_ptr] * 11 + [_i64] * 2 + [_int] + [_i64] * 6 + [_int, _int, _ptr]),
    "mb200_conv_step": (_int, [_ptr] * 6 + [_i64] * 2 + [_int, _i64, _int, _ptr]),
    "mb200_conv1d_silu_fwd": (_int, [_ptr] * 4 + [_i64] * 3 + [_int] + [_i64] * 4 + [_int, _ptr]),
    "mb200_conv1d_silu_bwd": (_int, [_ptr] * 7 + [_i64] * 3 + [_int] + [_i64] * 6 + [_int, _ptr]),
    "mb200_rmsnorm_fwd": (_int, [_ptr] * 4 + [_i64] * 4 + [C.c_float, _int, _ptr]),
    "mb200_rmsnorm_bwd": (_int, [_ptr] * 6 + [_i64] * 5 + [_int, _ptr]),
    "mb200_add_rmsnorm_fwd": (_int, [_ptr] * 6 + [_i64] * 6 + [C.c_float, _int, _int, _int, _ptr]),
    "mb200_add_rmsnorm_bwd": (_int, [_ptr] * 7 + [_i64] * 6 + [_int, _int, _ptr]),
    "mb200_carry_fold": (_int, [_ptr] * 3 + [_i64] * 2 + [_int, _int, _ptr]),
    "mb200_carry_fold_range": (_int, [_ptr] * 4 + [_i64] * 3 + [_int, _int, _int, _ptr]),
    "mb200_sscan_fwd_carry": (_int, [_ptr] * 7 + [_i64] * 3 + [_int] + [_i64] * 6 + [_int, _int, _ptr]),
    "mb200_decay_prod": (_int, [_ptr] * 4 + [_i64] * 3 + [_int] + [_i64] * 2 + [_int, _int, _ptr]),
}

_lib = None


def exported_symbols():
    """Names this binding expects the library to export (used by the CPU-side tests)."""
    return sorted(_SIGNATURES)


def load():
    """Return the loaded library, loading it on first use.  Raises if it was never built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m mamba_b200.build` "
                "(needs nvcc). mamba_b200 has no CPU or PyTorch fallback.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)          # AttributeError here = library/header mismatch
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(code: int, what: str) -> None:
    if code != 0:
        msg = load().mb200_strerror(code).decode()
        raise RuntimeError(f"{what} failed: {msg} (code {code})")


def device_status(device=None) -> int:
    """Read and clear the kernels' device-side status word on `device` (SYNCHRONISES it).

    0 = every bounded wait inside the kernels launched so far completed; 1 = one gave up, and the
    outputs of that launch are invalid.  The launches themselves never wait for this word: callers
    poll it at their own synchronisation points (or set MB200_CHECK_STATUS=1, see check_status)."""
    import torch
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        return load().mb200_device_status()


CHECK_STATUS = os.environ.get("MB200_CHECK_STATUS", "0") not in ("", "0")


def check_status(device, what: str) -> None:
    """With MB200_CHECK_STATUS=1 in the environment every fused-scan launch is followed by a device
    synchronisation and a read of the status word, and a give-up raises.  Off by default (it
    serialises host and device); meant for debugging a suspected hang."""
    if CHECK_STATUS:
        st = device_status(device)
        if st != 0:
            raise RuntimeError(f"{what}: a bounded wait inside the kernel gave up (device status {st}); "
                               "its outputs are invalid")


def dtype_code(dtype) -> int:
    import torch
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"mamba_b200 kernels take float32 or bfloat16 activations, got {dtype}")


def ptr(t) -> int | None:
    """Device address of a tensor (None stays NULL)."""
    return None if t is None else t.data_ptr()


def current_stream(device) -> int:
    import torch
    return torch.cuda.current_stream(device).cuda_stream
