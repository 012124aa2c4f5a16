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


class _LastCopy:
    """The fp16 copy written by the most recent fused forward, findable from its fp32 output
    (weak references: neither tensor is kept alive by the cache)."""

    output = copy = None
    version = -1

    @classmethod
    def record(cls, output, copy):
        cls.output, cls.copy, cls.version = weakref.ref(output), weakref.ref(copy), output._version

    @classmethod
    def find(cls, tensor):
        if cls.output is None or cls.output() is not tensor or tensor._version != cls.version:
            return None
        return cls.copy()


def fp16_copy_of(t):
    """The fp16 copy of `t` if `t` is the last output of the fused RMSNorm and has not been
    written since (bit-identical to t.to(torch.float16)), else None."""
    low = _LastCopy.find(t)
    return None if low is None else low.view(t.shape)


def _forward_launch(rows, weight, eps, out_dtype, keep_copy):
    """Runs the forward kernel on `rows` [n, cols]; returns (out, rstd, low, slots, small) where
    the last three are None unless `keep_copy` found a usable slot map for the weight."""
    n, cols = rows.shape
    dev = rows.device
    out = torch.empty((n, cols), dtype=out_dtype, device=dev)
    rstd = torch.empty(n, dtype=torch.float32, device=dev)
    low = slots = small = None
    side = 1
    mapping = _small_columns(weight) if keep_copy else None
    if mapping is not None:
        slots, tiny_count = mapping
        side = max(tiny_count, 1)
        low = torch.empty((n, cols), dtype=torch.float16, device=dev)
        small = torch.empty((n, side), dtype=torch.float16, device=dev)
    if n:
        _lib.call("soup_rmsnorm_fwd", _lib.ptr(rows), _lib.ptr(weight), _lib.ptr(out), _lib.ptr(rstd),
                  _lib.ptr(low), _lib.ptr(slots), _lib.ptr(small), side, n, cols, float(eps),
                  _lib.dtype_code(rows.dtype), _lib.dtype_code(weight.dtype),
                  _lib.dtype_code(out_dtype), _lib.stream_of(rows))
    return out, rstd, low, slots, small


class RMSNorm(torch.autograd.Function):
    """`RMSNorm.apply(x, weight, eps)`. Saves x (any dtype) for backward, or, for an fp32 x with a
    frozen fp32 weight, only the fp16 copy of the output plus the normalised values of the
    tiny-|w| columns."""

    @staticmethod
    def forward(ctx, x, weight, eps):
        _lib.require_cuda(x, weight)
        rows = x.contiguous().view(-1, x.shape[-1])
        weight = weight.contiguous()
        fp32_frozen = (x.dtype == torch.float32 and weight.dtype == torch.float32
                       and not weight.requires_grad and ctx.needs_input_grad[0])
        out, rstd, low, slots, small = _forward_launch(
            rows, weight, eps, torch.promote_types(x.dtype, weight.dtype), fp32_frozen)
        ctx.from_copy = low is not None
        if ctx.from_copy:
            ctx.save_for_backward(low, weight, rstd, slots, small)
        else:
            ctx.save_for_backward(rows, weight, rstd)
        ctx.x_dtype, ctx.x_shape = x.dtype, x.shape
        result = out.view(x.shape)
        if ctx.from_copy:
            _LastCopy.record(result, low)
        return result

    @staticmethod
    def backward(ctx, grad):
        if ctx.from_copy:
            saved, weight, rstd, slots, small = ctx.saved_tensors
            side = small.shape[-1]
        else:
            saved, weight, rstd = ctx.saved_tensors
            slots = small = None
            side = 1
        n, cols = saved.shape
        dy = grad.contiguous().view(n, cols)
        dx = torch.empty((n, cols), dtype=ctx.x_dtype, device=saved.device)
        dw = partial = None
        if ctx.needs_input_grad[1]:   # trainable weight: per-CTA partial rows, reduced in fixed order
            dw = torch.empty(cols, dtype=weight.dtype, device=saved.device)
            n_partial = max(_lib.lib().soup_rmsnorm_bwd_partials(n, cols), 1)
            partial = torch.empty((n_partial, cols), dtype=torch.float32, device=saved.device)
        _lib.call("soup_rmsnorm_bwd", _lib.ptr(dy), _lib.ptr(saved), _lib.ptr(weight), _lib.ptr(rstd),
                  _lib.ptr(dx), _lib.ptr(partial), _lib.ptr(dw), _lib.ptr(slots), _lib.ptr(small),
                  side, n, cols, _lib.dtype_code(dy.dtype), _lib.dtype_code(saved.dtype),
                  _lib.dtype_code(weight.dtype), _lib.dtype_code(ctx.x_dtype), int(ctx.from_copy),
                  _lib.stream_of(saved))
        return dx.view(ctx.x_shape), dw, None


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
