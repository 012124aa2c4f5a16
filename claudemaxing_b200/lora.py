"""LoRA branch of a 4-bit linear (q_proj / v_proj) with a bit-packed dropout mask.

Drop-in for the reference's solution/lora.py: `LoRABranch.apply(x, x16, weight_a, weight_b, p,
scaling)`, `_pack(x, mask, scale) -> (xd, bits)`, `_unpack(x16, bits, g16, scale, dx_dtype) ->
(xd, dx)` and `patch_peft_lora_4bit()`. The mask comes from the same `torch.native_dropout` call
peft's nn.Dropout makes (same random stream), is packed to one bit per element by csrc/dropout.cu,
and lora_A's input is rebuilt in backward from the shared fp16 copy of x and the bits. The four
r=16 GEMMs of the adapter stay torch library calls.
"""

import weakref

import torch

from . import _lib


def _pack(x, mask, scale):
    """xd = fp16(keep ? x*scale : 0) and the mask as bits (bit l of byte r = element 8r + l)."""
    _lib.require_cuda(x, mask)
    n = x.numel()
    if n % 8:
        raise ValueError("the packed dropout mask needs a multiple of 8 elements")
    x, mask = x.contiguous(), mask.contiguous()
    xd = torch.empty(x.shape, dtype=torch.float16, device=x.device)
    bits = torch.empty(n // 8, dtype=torch.uint8, device=x.device)
    if n:
        _lib.call("soup_dropout_pack", _lib.ptr(x), _lib.ptr(mask), _lib.ptr(xd), _lib.ptr(bits),
                  n, float(scale), _lib.dtype_code(x.dtype), _lib.stream_of(x))
    return xd, bits


def _unpack(x16, bits, g16, scale, dx_dtype):
    """From the fp16 x and the bits: xd = fp16(keep ? x16*scale : 0), dx = keep ? g16*scale : 0."""
    _lib.require_cuda(x16, bits, g16)
    if x16.dtype != torch.float16 or g16.dtype != torch.float16:
        raise TypeError("_unpack takes fp16 x and fp16 gradient")
    n = x16.numel()
    x16, g16 = x16.contiguous(), g16.contiguous()
    xd = torch.empty_like(x16)
    dx = torch.empty(x16.shape, dtype=dx_dtype, device=x16.device)
    if n:
        _lib.call("soup_dropout_unpack", _lib.ptr(x16), _lib.ptr(bits), _lib.ptr(g16),
                  _lib.ptr(xd), _lib.ptr(dx), n, float(scale), _lib.dtype_code(dx_dtype),
                  _lib.stream_of(x16))
    return xd, dx


def _weight_gradient(grad_rows, input_rows, dtype):
    """grad_rows^T @ input_rows (both fp16, [rows, out] and [rows, in]) in `dtype`. For an fp32
    weight the GEMM writes its fp32 accumulator directly: no fp16 rounding (or overflow at a large
    loss scale) of a sum over thousands of rows, and no cast kernel behind the GEMM."""
    if dtype == torch.float32 and grad_rows.is_cuda and grad_rows.dtype == input_rows.dtype == torch.float16:
        return torch.mm(grad_rows.t(), input_rows, out_dtype=torch.float32)
    return grad_rows.t().mm(input_rows).to(dtype)


def _add_weight_gradient(weight, grad_rows, input_rows, alpha):
    """weight.grad += alpha * grad_rows^T @ input_rows inside the GEMM (fp32 accumulator added to
    the fp32 gradient in its epilogue): True when done, False when the caller has to return the
    gradient to autograd instead (no gradient tensor yet, or operands this form does not take)."""
    grad = weight.grad
    if (grad is None or grad.dtype != torch.float32 or not grad.is_cuda or not grad.is_contiguous()
            or grad_rows.dtype != torch.float16 or input_rows.dtype != torch.float16):
        return False
    torch.addmm(grad, grad_rows.t(), input_rows, out_dtype=torch.float32, alpha=alpha, out=grad)
    return True


class LoRABranch(torch.autograd.Function):
    """fp16 `lora_B(lora_A(dropout(x))) * scaling` for fp32 x under fp16 autocast.

    `LoRABranch.accumulate_in_place` (off by default; `CapturedStep` turns it on for the step it
    captures): backward adds the two weight gradients to `weight.grad` itself, in the epilogue of
    the GEMM that forms them, and returns None for them, so autograd launches no separate
    accumulation (and runs no hooks of those parameters: not for a model wrapped in
    DistributedDataParallel)."""

    accumulate_in_place = False

    @staticmethod
    def forward(ctx, x, x16, weight_a, weight_b, p, scaling, a16=None, b16=None, b16_scaled=False):
        """`a16`, `b16`: fp16 copies of the two weights when the caller has made them already (a
        model that casts all its adapters in one launch per forward); cast here otherwise. With
        `b16_scaled`, b16 is fp16(scaling * B): the branch output and the gradient that goes back
        through B then need no scaling pass over [tokens, out] (two of the branch's larger
        kernels); only B's own gradient, [out, r], is multiplied. For a power-of-two scaling the
        numbers are the same; otherwise B is rounded after the scaling instead of before."""
        dropped, mask = torch.native_dropout(x, p, True)
        del dropped  # only the mask is used
        scale = 1.0 / (1.0 - p)
        xd, bits = _pack(x, mask, scale)  # from the fp32 x: lora_A's input exactly as peft's
        del mask
        if a16 is None or b16 is None:
            a16, b16 = weight_a.to(torch.float16), weight_b.to(torch.float16)
        a = torch.nn.functional.linear(xd, a16)
        out = torch.nn.functional.linear(a, b16)
        if not b16_scaled:
            out = out * scaling
        ctx.save_for_backward(x16, bits, a, a16, b16)   # the fp16 adapter copies are 50 KB each
        ctx.scale, ctx.scaling, ctx.x_dtype, ctx.b16_scaled = scale, scaling, x.dtype, b16_scaled
        ctx.weight_dtypes = (weight_a.dtype, weight_b.dtype)
        ctx.weights = (weight_a, weight_b) if LoRABranch.accumulate_in_place else None
        return out

    @staticmethod
    def backward(ctx, grad):
        x16, bits, a, a16, b16 = ctx.saved_tensors
        g = grad.to(torch.float16)
        if not ctx.b16_scaled:
            g = g * ctx.scaling
        g2 = g.reshape(-1, g.shape[-1])
        a2 = a.reshape(-1, a.shape[-1])
        in_place = ctx.weights is not None and ctx.needs_input_grad[2] and ctx.needs_input_grad[3]
        grad_b = None
        if not (in_place and _add_weight_gradient(ctx.weights[1], g2, a2,
                                                  ctx.scaling if ctx.b16_scaled else 1.0)):
            grad_b = _weight_gradient(g2, a2, ctx.weight_dtypes[1])
            if ctx.b16_scaled:
                grad_b = grad_b * ctx.scaling
        grad_a_in = g.matmul(b16)
        ga2 = grad_a_in.reshape(-1, grad_a_in.shape[-1])
        grad_xd = grad_a_in.matmul(a16)
        xd, dx = _unpack(x16, bits, grad_xd.contiguous(), ctx.scale, ctx.x_dtype)
        xd2 = xd.reshape(-1, xd.shape[-1])
        grad_a = None
        if not (in_place and _add_weight_gradient(ctx.weights[0], ga2, xd2, 1.0)):
            grad_a = _weight_gradient(ga2, xd2, ctx.weight_dtypes[0])
        return dx, None, grad_a, grad_b, None, None, None, None, None


class LoRABranchPair(torch.autograd.Function):
    """Two LoRA branches on the same x (q_proj's and v_proj's adapters of a block), each with its
    own dropout draw, as one autograd node: one launch packs both dropped inputs (x read once),
    the two rank-r products with A are one batched GEMM, and backward unpacks both in one launch
    that also sums the two input gradients. Per adapter the numbers are LoRABranch's with
    `b16_scaled`; the dropout draws come in the same order (first adapter, then second).

    `a16_pair` is fp16 [2, r, in] (both A weights), `b16s_first` / `b16s_second` fp16
    scaling * B. Returns the two branch outputs."""

    @staticmethod
    def forward(ctx, x, x16, a_first, b_first, a_second, b_second, p_first, p_second,
                scaling_first, scaling_second, a16_pair, b16s_first, b16s_second):
        _lib.require_cuda(x, x16, a16_pair)
        n, hidden = x.numel(), x.shape[-1]
        rows = n // hidden
        mask_first = torch.native_dropout(x, p_first, True)[1]
        mask_second = torch.native_dropout(x, p_second, True)[1]
        scales = (1.0 / (1.0 - p_first), 1.0 / (1.0 - p_second))
        x = x.contiguous()
        xd = torch.empty((2, rows, hidden), dtype=torch.float16, device=x.device)
        bits = torch.empty((2, n // 8), dtype=torch.uint8, device=x.device)
        _lib.call("soup_dropout_pack2", _lib.ptr(x), _lib.ptr(mask_first), _lib.ptr(mask_second),
                  _lib.ptr(xd[0]), _lib.ptr(xd[1]), _lib.ptr(bits[0]), _lib.ptr(bits[1]), n,
                  scales[0], scales[1], _lib.dtype_code(x.dtype), _lib.stream_of(x))
        del mask_first, mask_second
        a = torch.bmm(xd, a16_pair.transpose(1, 2))          # [2, rows, r]
        out_first = torch.mm(a[0], b16s_first.t())
        out_second = torch.mm(a[1], b16s_second.t())
        ctx.save_for_backward(x16, bits, a, a16_pair, b16s_first, b16s_second)
        ctx.scales, ctx.scalings = scales, (scaling_first, scaling_second)
        ctx.x_shape, ctx.weight_dtypes = x.shape, (a_first.dtype, b_first.dtype, a_second.dtype, b_second.dtype)
        ctx.weights = ((a_first, b_first, a_second, b_second) if LoRABranch.accumulate_in_place else None)
        lead = x.shape[:-1]
        return out_first.view(*lead, -1), out_second.view(*lead, -1)

    @staticmethod
    def backward(ctx, grad_first, grad_second):
        x16, bits, a, a16_pair, b16s_first, b16s_second = ctx.saved_tensors
        rows, hidden = a.shape[1], x16.shape[-1]
        grads = [g.to(torch.float16).reshape(rows, -1) for g in (grad_first, grad_second)]
        b16s = (b16s_first, b16s_second)
        in_place = ctx.weights is not None and all(ctx.needs_input_grad[2:6])
        out = [None] * 4                                     # dA1, dB1, dA2, dB2
        gain = torch.empty((2, rows, a.shape[-1]), dtype=torch.float16, device=a.device)
        for i in (0, 1):
            if not (in_place and _add_weight_gradient(ctx.weights[2 * i + 1], grads[i], a[i], ctx.scalings[i])):
                out[2 * i + 1] = _weight_gradient(grads[i], a[i], ctx.weight_dtypes[2 * i + 1]) * ctx.scalings[i]
            torch.mm(grads[i], b16s[i], out=gain[i])
        grad_xd = torch.bmm(gain, a16_pair)                  # [2, rows, hidden]
        xd = torch.empty((2, rows, hidden), dtype=torch.float16, device=a.device)
        dx = torch.empty(ctx.x_shape, dtype=torch.float32, device=a.device)
        _lib.call("soup_dropout_unpack2", _lib.ptr(x16), _lib.ptr(bits[0]), _lib.ptr(bits[1]),
                  _lib.ptr(grad_xd[0]), _lib.ptr(grad_xd[1]), _lib.ptr(xd[0]), _lib.ptr(xd[1]),
                  _lib.ptr(dx), rows * hidden, ctx.scales[0], ctx.scales[1], _lib.stream_of(x16))
        for i in (0, 1):
            if not (in_place and _add_weight_gradient(ctx.weights[2 * i], gain[i], xd[i], 1.0)):
                out[2 * i] = _weight_gradient(gain[i], xd[i], ctx.weight_dtypes[2 * i])
        return (dx, None, out[0], out[1], out[2], out[3]) + (None,) * 7


def pair_covers(x, x16, first, second):
    """Whether LoRABranchPair takes these two adapter modules (LoRALinear-like: lora_A, lora_B, p,
    scaling) on this x: what LoRABranch needs, the same rank and input width, whole 16-element
    groups and an fp16 copy of x that is contiguous."""
    return (x.dtype == torch.float32 and x.numel() % 16 == 0 and x16 is not None
            and x16.dtype == torch.float16 and x16.is_contiguous()
            and first.lora_A.weight.shape == second.lora_A.weight.shape
            and 0.0 < first.p < 1.0 and 0.0 < second.p < 1.0)


class _SharedCopy:
    """The fp16 copy of the tensor the adapter layers of a block all see (q_proj and v_proj get the
    same hidden states): made once, found again by identity, version and storage of the source."""

    def __init__(self):
        self.source = self.copy = None
        self.stamp = None

    @staticmethod
    def _stamp(x):
        return x._version, x.data_ptr(), tuple(x.shape)

    def lookup(self, x):
        if self.source is None or self.copy is None:
            return None
        src, low = self.source(), self.copy()
        if src is x and low is not None and self.stamp == self._stamp(x):
            return low
        return None

    def remember(self, x, low):
        self.source, self.copy, self.stamp = weakref.ref(x), weakref.ref(low), self._stamp(x)


_COPY = _SharedCopy()


def _shared_fp16(x):
    """The fp16 copy of `x`: the one a previous adapter layer used, else the one the preceding
    RMSNorm wrote, else a fresh cast."""
    from .rmsnorm import fp16_copy_of

    low = _COPY.lookup(x)
    if low is None:
        low = fp16_copy_of(x)
        if low is None:
            low = x.detach().to(torch.float16).contiguous()
        _COPY.remember(x, low)
    return low


def _autocast_fp16():
    try:
        on, dtype = torch.is_autocast_enabled("cuda"), torch.get_autocast_dtype("cuda")
    except (TypeError, AttributeError):
        on, dtype = torch.is_autocast_enabled(), torch.get_autocast_gpu_dtype()
    return bool(on) and dtype == torch.float16


def branch_covers(x, p, training):
    """Whether LoRABranch reproduces the adapter for this input: training with gradients on under
    fp16 autocast, a contiguous fp32 CUDA tensor whose last dimension is a multiple of 8, and a
    dropout probability strictly between 0 and 1."""
    if not (training and torch.is_grad_enabled() and _autocast_fp16()):
        return False
    if not (isinstance(x, torch.Tensor) and x.is_cuda and x.dtype == torch.float32):
        return False
    return x.is_contiguous() and x.shape[-1] % 8 == 0 and 0.0 < p < 1.0


def _single_vanilla_adapter(layer):
    """Name of the layer's only active adapter when it is plain LoRA (bias-free fp32 nn.Linear A
    and B behind an nn.Dropout, no DoRA or other variant, not merged, not disabled), else None."""
    names = layer.active_adapters
    if len(names) != 1 or layer.disable_adapters or layer.merged:
        return None
    name = names[0]
    if name not in layer.lora_A or name not in getattr(layer, "lora_dropout", {}):
        return None
    if name in getattr(layer, "lora_variant", {}) or getattr(layer, "use_dora", {}).get(name, False):
        return None
    if getattr(layer, "fan_in_fan_out", False) or type(layer.lora_dropout[name]) is not torch.nn.Dropout:
        return None
    for part in (layer.lora_A[name], layer.lora_B[name]):
        if type(part) is not torch.nn.Linear or part.bias is not None or part.weight.dtype != torch.float32:
            return None
    return name


def _wrap_peft_forward(installed):
    def forward(self, x, *args, **kwargs):
        name = None if (args or kwargs) else _single_vanilla_adapter(self)
        if name is None or not branch_covers(x, self.lora_dropout[name].p, self.training):
            return installed(self, x, *args, **kwargs)
        self._check_forward_args(x)
        frozen_part = self.base_layer(x)
        adapter = LoRABranch.apply(x, _shared_fp16(x), self.lora_A[name].weight, self.lora_B[name].weight,
                                   float(self.lora_dropout[name].p), float(self.scaling[name]))
        return frozen_part + adapter

    forward._lora_branch = True
    forward._original = installed
    return forward


def patch_peft_lora_4bit():
    """peft's LoRA Linear layers (the bitsandbytes 4-bit one and the plain one): vanilla LoRA with
    dropout on an fp32 input under fp16 autocast in training goes through LoRABranch; everything
    else keeps peft's forward. Without peft there is nothing to patch."""
    import importlib

    for module_name, class_name in (("peft.tuners.lora.bnb", "Linear4bit"),
                                    ("peft.tuners.lora.layer", "Linear")):
        try:
            cls = getattr(importlib.import_module(module_name), class_name, None)
        except Exception:  # noqa: BLE001 - peft (or its bitsandbytes half) is not installed
            continue
        if cls is not None and not getattr(cls.forward, "_lora_branch", False):
            cls.forward = _wrap_peft_forward(cls.forward)
