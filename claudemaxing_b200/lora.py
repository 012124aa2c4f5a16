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


class LoRABranch(torch.autograd.Function):
    """fp16 `lora_B(lora_A(dropout(x))) * scaling` for fp32 x under fp16 autocast."""

    @staticmethod
    def forward(ctx, x, x16, weight_a, weight_b, p, scaling):
        dropped, mask = torch.native_dropout(x, p, True)
        del dropped  # only the mask is used
        scale = 1.0 / (1.0 - p)
        xd, bits = _pack(x, mask, scale)  # from the fp32 x: lora_A's input exactly as peft's
        del mask
        a16, b16 = weight_a.to(torch.float16), weight_b.to(torch.float16)
        a = torch.nn.functional.linear(xd, a16)
        out = torch.nn.functional.linear(a, b16) * scaling
        ctx.save_for_backward(x16, bits, a, weight_a, weight_b)
        ctx.scale, ctx.scaling, ctx.x_dtype = scale, scaling, x.dtype
        return out

    @staticmethod
    def backward(ctx, grad):
        x16, bits, a, weight_a, weight_b = ctx.saved_tensors
        a16, b16 = weight_a.to(torch.float16), weight_b.to(torch.float16)
        g = grad.to(torch.float16) * ctx.scaling
        g2 = g.reshape(-1, g.shape[-1])
        grad_b = g2.t().mm(a.reshape(-1, a.shape[-1]))
        grad_a_in = g.matmul(b16)
        ga2 = grad_a_in.reshape(-1, grad_a_in.shape[-1])
        grad_xd = grad_a_in.matmul(a16)
        xd, dx = _unpack(x16, bits, grad_xd.contiguous(), ctx.scale, ctx.x_dtype)
        grad_a = ga2.t().mm(xd.reshape(-1, xd.shape[-1]))
        return dx, None, grad_a.to(weight_a.dtype), grad_b.to(weight_b.dtype), None, None


# (weakref to x, (version, data_ptr, shape), weakref to its fp16 copy)
_X16 = [None, None, None]


def _shared_fp16(x):
    """One fp16 copy of `x` for all the adapter layers that see the same tensor (q and v of a
    block): the copy the preceding RMSNorm wrote if there is one, else a fresh cast."""
    ref, key, x16_ref = _X16
    now = (x._version, x.data_ptr(), tuple(x.shape))
    x16 = x16_ref() if x16_ref is not None else None
    if x16 is not None and ref is not None and ref() is x and key == now:
        return x16
    from .rmsnorm import fp16_copy_of

    x16 = fp16_copy_of(x)
    if x16 is None:
        x16 = x.detach().to(torch.float16).contiguous()
    _X16[0], _X16[1], _X16[2] = weakref.ref(x), now, weakref.ref(x16)
    return x16


def _autocast_fp16():
    try:
        return (torch.is_autocast_enabled("cuda")
                and torch.get_autocast_dtype("cuda") == torch.float16)
    except (TypeError, AttributeError):
        return torch.is_autocast_enabled() and torch.get_autocast_gpu_dtype() == torch.float16


def branch_covers(x, p, training):
    """Whether LoRABranch reproduces the adapter for this input: fp32 contiguous CUDA x under fp16
    autocast, training with gradients on, 0 < p < 1, last dim a multiple of 8."""
    return (training and torch.is_grad_enabled() and _autocast_fp16()
            and isinstance(x, torch.Tensor) and x.is_cuda and x.dtype == torch.float32
            and x.shape[-1] % 8 == 0 and x.is_contiguous() and 0.0 < p < 1.0)


def _make_forward(original):
    def forward(self, x, *args, **kwargs):
        active = self.active_adapters
        name = active[0] if len(active) == 1 else None
        drop = self.lora_dropout[name] if name in getattr(self, "lora_dropout", {}) else None
        plain = (not args and not kwargs and not self.disable_adapters and not self.merged
                 and name is not None and name in self.lora_A
                 and name not in getattr(self, "lora_variant", {})
                 and type(drop) is torch.nn.Dropout
                 and type(self.lora_A[name]) is torch.nn.Linear
                 and type(self.lora_B[name]) is torch.nn.Linear
                 and self.lora_A[name].bias is None and self.lora_B[name].bias is None
                 and self.lora_A[name].weight.dtype == torch.float32
                 and self.lora_B[name].weight.dtype == torch.float32
                 and not getattr(self, "use_dora", {}).get(name, False)
                 and not getattr(self, "fan_in_fan_out", False))
        if not plain or not branch_covers(x, drop.p, self.training):
            return original(self, x, *args, **kwargs)
        self._check_forward_args(x)
        result = self.base_layer(x)
        lora = LoRABranch.apply(x, _shared_fp16(x), self.lora_A[name].weight,
                                self.lora_B[name].weight, float(drop.p),
                                float(self.scaling[name]))
        return result + lora

    forward._lora_branch = True
    forward._original = original
    return forward


def patch_peft_lora_4bit():
    """peft's LoRA Linear layers (the bitsandbytes 4-bit one and the plain one): vanilla LoRA with
    dropout on an fp32 input under fp16 autocast in training goes through LoRABranch; everything
    else keeps peft's forward. Without peft there is nothing to patch."""
    classes = []
    try:
        from peft.tuners.lora import bnb as lora_bnb

        classes.append(getattr(lora_bnb, "Linear4bit", None))
    except Exception:  # noqa: BLE001
        pass
    try:
        from peft.tuners.lora import layer as lora_layer

        classes.append(getattr(lora_layer, "Linear", None))
    except Exception:  # noqa: BLE001
        pass
    for cls in classes:
        if cls is not None and not getattr(cls.forward, "_lora_branch", False):
            cls.forward = _make_forward(cls.forward)
