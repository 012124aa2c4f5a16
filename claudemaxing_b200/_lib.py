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
    "soup_rmsnorm_bwd_residual": [_P] * 9 + [_L] * 3 + [_P],
    "soup_rope": [_P, _P, _P, _P, _P, _P] + [_L] * 13 + [_I] * 6 + [_P],
    "soup_rope_sum": [_P, _P, _P, _P, _P, _P, _P] + [_L] * 22 + [_I] * 7 + [_P],
    "soup_attn_fwd": [_P, _P, _P, _P, _P, _P] + [_L] * 8 + [_F, _P],
    "soup_attn_bwd": [_P] * 10 + [_L] * 8 + [_F, _P],
    "soup_row_status": [_P, _P],
    "soup_device_status": [_P, _I, _P],
    "soup_wait_selftest": [_L, _P, _P, _P],
    "soup_silu_mul_fwd": [_P, _P, _P, _L, _I, _I, _I, _I, _P],
    "soup_silu_mul_bwd": [_P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _P],
    "soup_dropout_pack": [_P, _P, _P, _P, _L, _F, _I, _P],
    "soup_dropout_unpack": [_P, _P, _P, _P, _P, _L, _F, _I, _P],
    "soup_dropout_pack2": [_P] * 7 + [_L, _F, _F, _I, _P],
    "soup_dropout_unpack2": [_P] * 8 + [_L, _F, _F, _P],
    "soup_lmhead_workspace_bytes": [_L, _L, _L, _L],
    "soup_lmhead_ce": [_P] * 13 + [_L] * 6 + [_I, _P],
    "soup_lmhead_set_timing": [_P],
    "soup_lmhead_plan": [_L, _L, _L, _P, _P, _P],
    "soup_lmhead_status": [_P, _L, _L, _L, _P, _P],
    "soup_lmhead_merge": [_P] * 15 + [_L, _I, _P],
    "soup_lmhead_finish": [_P] * 12 + [_L] * 4 + [_P],
    "soup_lmhead_finish_to": [_P] * 13 + [_I] + [_L] * 4 + [_P],
    "soup_lmhead_grad_scale": [_P, _P, _P, _L, _I, _P],
    "soup_xent_rows": [_P] * 5 + [_L, _L, _L, _I, _P],
    "soup_nf4_gemm_workspace_bytes": [_L, _L],
    "soup_nf4_linear_fwd": [_P, _P, _I, _P, _L, _L, _I, _I, _I, _P, _L, _P],
    "soup_nf4_linear_dx": [_P, _I, _P, _P, _I, _L, _L, _I, _I, _I, _P, _L, _P],
}
_RESTYPE = {"soup_lmhead_workspace_bytes": _L, "soup_rmsnorm_bwd_partials": _L,
            "soup_nf4_gemm_workspace_bytes": _L}
SIGNATURES["soup_rmsnorm_bwd_partials"] = [_L, _L]

class Nf4Item(ctypes.Structure):
    """soup_nf4_item of include/soup_b200.h."""

    _fields_ = [("packed", _P), ("absmax", _P), ("code2", _P), ("absmax2", _P), ("offset", _P),
                ("out", _P), ("n_elems", _L)]


class Nf4GemmItem(ctypes.Structure):
    """soup_nf4_gemm_item of include/soup_b200.h."""

    _fields_ = [("packed", _P), ("absmax", _P), ("code2", _P), ("absmax2", _P), ("offset", _P),
                ("bias", _P), ("out", _P), ("dy", _P), ("n_out", _L)]


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


class _StreamOf(int):
    """A cudaStream_t value that remembers which device it belongs to, so that `call` can make
    that device current for the launch."""

    device_index = None


def stream_of(t):
    """The current torch stream of `t`'s device, as the void* the C ABI takes."""
    handle = _StreamOf(torch.cuda.current_stream(t.device).cuda_stream)
    handle.device_index = t.device.index
    return handle


def require_cuda(*tensors):
    """Every given tensor lives on one CUDA device (there is no CPU path and a launch reaches one
    device only)."""
    device = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("libsoup_b200 ops run on CUDA tensors only (no CPU fallback)")
        if device is None:
            device = t.device
        elif t.device != device:
            raise RuntimeError(f"libsoup_b200: tensors on {device} and {t.device} in one call")


def call(name, *args):
    """Invokes an entry point. The launch, the library's per-device caches (SM count, status word,
    built-in scratch) and the stream all belong to one device: the one of the tensor `stream_of`
    was asked about, which is made current for the duration of the call when it is not already."""
    fn = getattr(lib(), name)
    index = next((a.device_index for a in args if isinstance(a, _StreamOf)), None)
    if index is not None and index != torch.cuda.current_device():
        with torch.cuda.device(index):
            rc = fn(*args)
    else:
        rc = fn(*args)
    if rc < 0:
        msg = lib().soup_last_error_string().decode("utf-8", "replace")
        raise RuntimeError(f"{name} failed ({rc}): {msg}")
    return rc


_STATUS_MEANING = {
    11: "RMSNorm forward or LM-head logits producer: a bounded wait ran out",
    12: "RMSNorm backward or LM-head logits accumulator: a bounded wait ran out",
    13: "RoPE or LM-head logits operand: a bounded wait ran out",
    14: "LM-head logits epilogue: a bounded wait ran out",
    21: "LM-head gradient producer: a bounded wait ran out",
    22: "LM-head gradient accumulator: a bounded wait ran out",
    23: "LM-head gradient operand: a bounded wait ran out",
    24: "LM-head gradient epilogue: a bounded wait ran out",
    90: "LM-head row merge: non-finite sum of exponentials",
    99: "bounded-wait self-test",
}


def device_status(device=None, clear=True):
    """The sticky status word of `device` (default: the current one): 0, or the code of the first
    kernel since the last clear that gave up a bounded wait or met a non-finite sum. Synchronises
    the device's current stream, so call it where the host waits for the step anyway."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    word = ctypes.c_int(0)
    with torch.cuda.device(index):
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib().soup_device_status(ctypes.byref(word), int(bool(clear)), stream)
    if rc < 0:
        msg = lib().soup_last_error_string().decode("utf-8", "replace")
        raise RuntimeError(f"soup_device_status failed ({rc}): {msg}")
    return int(word.value)


def check_device_status(device=None):
    """Raises RuntimeError when a kernel on `device` reported a failure since the last check (and
    clears the word): the outputs of the steps since then may be unwritten. Returns None."""
    code = device_status(device, clear=True)
    if code != 0:
        what = _STATUS_MEANING.get(code, "unknown code")
        raise RuntimeError(f"libsoup_b200 device status {code}: {what}; results since the last "
                           "check are not valid")
