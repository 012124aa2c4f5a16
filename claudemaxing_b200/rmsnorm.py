"""Fused RMSNorm for Qwen2: one kernel forward, one backward (plus a tiny reduce when dw is needed).

Drop-in for the reference's solution/rmsnorm.py: `RMSNorm.apply(x, weight, eps)`, `rmsnorm(...)`,
`fp16_copy_of(t)` and `patch_qwen2_rmsnorm()`. The output reproduces Qwen2RMSNorm in dtype and in
rounding: the normalised value is rounded to the input dtype first and only then multiplied by the
weight, so the result dtype is torch.promote_types(x.dtype, weight.dtype). With an fp32 input and
a frozen fp32 weight (the 4-bit model), forward also writes the fp16 copy of the output that the
next layers cast to anyway; backward rebuilds the normalised value from that copy divided by the
weight, except in columns with |w| < 2^-10, whose normalised values are kept in a small side
buffer (solution/rmsnorm.py:106-134,160-172).
"""

import weakref

import torch

from . import _lib

MAX_COLS = 16384  # wider rows go to the original forward
_SUPPORTED = (torch.float16, torch.bfloat16, torch.float32)
MIN_ABS_WEIGHT = 2.0 ** -10
MAX_SMALL = 64

# (weakref to the last output, its version, weakref to its fp16 copy)
_LAST_LOW = [None, -1, None]
_SMALL = {}


def _small_columns(weight):
    """(slot map int32 [n_cols]: index among the tiny-|w| columns or -1, their count) for a frozen
    weight, or None when there are more than MAX_SMALL of them or a weight is not finite. Cached
    per weight object, version and storage."""
    key = id(weight)
    hit = _SMALL.get(key)
    if (hit is not None and hit[0]() is weight and hit[1] == weight._version
            and hit[2] == weight.data_ptr()):
        return hit[3]
    tiny = weight.detach().abs() < MIN_ABS_WEIGHT
    count = int(tiny.sum())
    result = None
    if count <= MAX_SMALL and bool(torch.isfinite(weight).all()):
        slots = torch.full(weight.shape, -1, dtype=torch.int32, device=weight.device)
        slots[tiny] = torch.arange(count, dtype=torch.int32, device=weight.device)
        result = (slots, count)
    _SMALL[key] = (weakref.ref(weight), weight._version, weight.data_ptr(), result)
    return result


def fp16_copy_of(t):
    """The fp16 copy of `t` if `t` is the last output of the fused RMSNorm (bit-identical to
    t.to(torch.float16)), else None."""
    ref, version, low_ref = _LAST_LOW
    if ref is None or ref() is not t or t._version != version:
        return None
    low = low_ref()
    return None if low is None else low.view(t.shape)


class RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        _lib.require_cuda(x, weight)
        shape = x.shape
        n_cols = shape[-1]
        x2 = x.contiguous().view(-1, n_cols)
        weight = weight.contiguous()
        n_rows = x2.shape[0]
        out_dtype = torch.promote_types(x.dtype, weight.dtype)
        out = torch.empty((n_rows, n_cols), dtype=out_dtype, device=x.device)
        rstd = torch.empty(n_rows, dtype=torch.float32, device=x.device)
        compress = (x.dtype == torch.float32 and weight.dtype == torch.float32
                    and not weight.requires_grad and ctx.needs_input_grad[0])
        small_cols = _small_columns(weight) if compress else None
        low = slots = small = None
        n_small = 1
        if small_cols is not None:
            slots, count = small_cols
            n_small = max(count, 1)
            low = torch.empty((n_rows, n_cols), dtype=torch.float16, device=x.device)
            small = torch.empty((n_rows, n_small), dtype=torch.float16, device=x.device)
        if n_rows:
            _lib.call("soup_rmsnorm_fwd", _lib.ptr(x2), _lib.ptr(weight), _lib.ptr(out),
                      _lib.ptr(rstd), _lib.ptr(low), _lib.ptr(slots), _lib.ptr(small), n_small,
                      n_rows, n_cols, float(eps), _lib.dtype_code(x2.dtype),
                      _lib.dtype_code(weight.dtype), _lib.dtype_code(out_dtype),
                      _lib.stream_of(x2))
        if low is not None:
            ctx.save_for_backward(low, weight, rstd, slots, small)
        else:
            ctx.save_for_backward(x2, weight, rstd, rstd, rstd)
        ctx.x_dtype = x.dtype
        ctx.shape = shape
        result = out.view(shape)
        if low is not None:
            _LAST_LOW[0], _LAST_LOW[1], _LAST_LOW[2] = (weakref.ref(result), result._version,
                                                         weakref.ref(low))
        return result

    @staticmethod
    def backward(ctx, grad):
        x2, weight, rstd, slots, small = ctx.saved_tensors
        n_rows, n_cols = x2.shape
        grad2 = grad.contiguous().view(n_rows, n_cols)
        dx = torch.empty(x2.shape, dtype=ctx.x_dtype, device=x2.device)
        need_dw = ctx.needs_input_grad[1]
        saved_output = x2.dtype != ctx.x_dtype
        dw = partial = None
        if need_dw:
            dw = torch.empty(n_cols, dtype=weight.dtype, device=x2.device)
            parts = _lib.lib().soup_rmsnorm_bwd_partials(n_rows, n_cols)
            partial = torch.empty((max(parts, 1), n_cols), dtype=torch.float32, device=x2.device)
        _lib.call("soup_rmsnorm_bwd", _lib.ptr(grad2), _lib.ptr(x2), _lib.ptr(weight),
                  _lib.ptr(rstd), _lib.ptr(dx), _lib.ptr(partial), _lib.ptr(dw),
                  _lib.ptr(slots) if saved_output else None,
                  _lib.ptr(small) if saved_output else None,
                  small.shape[-1] if saved_output else 1, n_rows, n_cols,
                  _lib.dtype_code(grad2.dtype), _lib.dtype_code(x2.dtype),
                  _lib.dtype_code(weight.dtype), _lib.dtype_code(ctx.x_dtype),
                  int(saved_output), _lib.stream_of(x2))
        return dx.view(ctx.shape), dw, None


def rmsnorm(x, weight, eps):
    return RMSNorm.apply(x, weight, eps)


def patch_qwen2_rmsnorm():
    """Send Qwen2RMSNorm.forward through the fused kernel. Class-level, so it works before or after
    the model is built. CPU tensors, unusual dtypes, very wide rows or a weight that does not match
    keep the installed forward."""
    from transformers.models.qwen2 import modeling_qwen2

    cls = getattr(modeling_qwen2, "Qwen2RMSNorm", None)
    if cls is None or getattr(cls.forward, "_fused_rmsnorm", False):
        return
    original = cls.forward

    def forward(self, hidden_states):
        w = self.weight
        covered = (isinstance(hidden_states, torch.Tensor) and hidden_states.is_cuda
                   and hidden_states.dtype in _SUPPORTED and w.dtype in _SUPPORTED
                   and w.dim() == 1 and w.device == hidden_states.device
                   and hidden_states.shape[-1] == w.shape[0]
                   and hidden_states.shape[-1] <= MAX_COLS)
        if not covered:
            return original(self, hidden_states)
        return rmsnorm(hidden_states, w, self.variance_epsilon)

    forward._fused_rmsnorm = True
    cls.forward = forward
