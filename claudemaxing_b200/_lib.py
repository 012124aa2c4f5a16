"""ctypes binding of libsoup_b200.so (the C ABI declared in include/soup_b200.h).

There is no other execution path: if the shared library is missing or a call fails, the ops raise.
`lib()` loads the library once (building it first when nvcc is available and the file is absent);
`call(name, *args)` invokes an entry point and turns a negative return code into RuntimeError with
the library's own message.
"""

import ctypes
import os
import threading

import torch

from . import build as _build

F32, F16, BF16 = 0, 1, 2
_DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_int64
_F = ctypes.c_float

# name -> argument ctypes, in the order of include/soup_b200.h
SIGNATURES = {
    "soup_nf4_dequant": [_P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _P],
    "soup_nf4_dequant_batch": [_P, _I, _P, _I, _I, _I, _I, _P],
    "soup_rmsnorm_fwd": [_P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _F, _I, _I, _I, _P],
    "soup_rmsnorm_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _I, _I, _I, _I, _I, _P],
    "soup_rmsnorm_bwd_noalloc": [_P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _I, _I, _I, _I, _I, _P],
    "soup_rope": [_P, _P, _P, _P, _P, _P] + [_L] * 13 + [_I] * 6 + [_P],
    "soup_row_status": [_P, _P],
    "soup_wait_selftest": [_L, _P, _P, _P],
    "soup_silu_mul_fwd": [_P, _P, _P, _L, _I, _I, _I, _I, _P],
    "soup_silu_mul_bwd": [_P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _P],
    "soup_dropout_pack": [_P, _P, _P, _P, _L, _F, _I, _P],
    "soup_dropout_unpack": [_P, _P, _P, _P, _P, _L, _F, _I, _P],
    "soup_lmhead_workspace_bytes": [_L, _L, _L, _L],
    "soup_lmhead_ce": [_P] * 13 + [_L] * 6 + [_I, _P],
    "soup_lmhead_set_timing": [_P],
    "soup_lmhead_plan": [_L, _L, _L, _P, _P, _P],
    "soup_lmhead_status": [_P, _L, _L, _L, _P, _P],
    "soup_lmhead_merge": [_P] * 15 + [_L, _I, _P],
    "soup_lmhead_finish": [_P] * 12 + [_L] * 4 + [_P],
    "soup_lmhead_grad_scale": [_P, _P, _P, _L, _I, _P],
    "soup_xent_rows": [_P] * 5 + [_L, _L, _L, _I, _P],
}
_RESTYPE = {"soup_lmhead_workspace_bytes": _L, "soup_rmsnorm_bwd_partials": _L}
SIGNATURES["soup_rmsnorm_bwd_partials"] = [_L, _L]

class Nf4Item(ctypes.Structure):
    """soup_nf4_item of include/soup_b200.h."""

    _fields_ = [("packed", _P), ("absmax", _P), ("code2", _P), ("absmax2", _P), ("offset", _P),
                ("out", _P), ("n_elems", _L)]


_lock = threading.Lock()
_handle = None


def lib_path():
    return _build.LIB


def lib():
    """The loaded library. Raises if it cannot be found or built: there is no fallback."""
    global _handle
    if _handle is not None:
        return _handle
    with _lock:
        if _handle is not None:
            return _handle
        path = lib_path()
        if not os.path.exists(path):
            try:
                _build.build()
            except Exception as exc:  # noqa: BLE001
                raise RuntimeError(
                    f"libsoup_b200.so is missing and could not be built ({exc}); the sm_100a "
                    "kernels are the only implementation of these ops") from exc
        handle = ctypes.CDLL(path)
        handle.soup_version.restype = ctypes.c_int
        handle.soup_last_error_string.restype = ctypes.c_char_p
        for name, argtypes in SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is None:
                continue
            fn.argtypes = argtypes
            fn.restype = _RESTYPE.get(name, ctypes.c_int)
        _handle = handle
    return _handle


def dtype_code(dtype):
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"libsoup_b200 has no kernel for dtype {dtype}") from None


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def stream_of(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("libsoup_b200 ops run on CUDA tensors only (no CPU fallback)")


def call(name, *args):
    fn = getattr(lib(), name)
    rc = fn(*args)
    if rc < 0:
        msg = lib().soup_last_error_string().decode("utf-8", "replace")
        raise RuntimeError(f"{name} failed ({rc}): {msg}")
    return rc
