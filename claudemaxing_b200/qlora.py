"""Self-contained 4-bit linear and LoRA layers for running the hot path without bitsandbytes/peft.

The reference reaches its kernels through bitsandbytes' `Linear4bit` and peft's LoRA `Linear4bit`
(call sites solution/nf4.py:102-130 and solution/lora.py:137-160). Those packages are optional
here: `NF4Linear` and `LoRALinear` follow the same formulas

    base:  x.to(compute) -> dequantise W -> F.linear -> cast back to x.dtype   (dequantised again
           in backward for the input gradient, as bitsandbytes' MatMul4Bit does)
    lora:  base(x) + lora_B(lora_A(dropout(x))) * scaling

and route through this package's kernels (`dequantize_nf4`, `LoRABranch`). `quantize_nf4` builds
the packed weight and its double-quantised statistics in the bitsandbytes layout with plain torch
ops on whatever device the weight is on; it is set-up code, not part of the step.
"""

import math

import torch
import torch.nn.functional as F

from .lora import LoRABranch, _shared_fp16, branch_covers
from .nf4 import dequantize_nf4


class QuantState:
    """The fields of bitsandbytes' QuantState that `dequantize_nf4` reads."""

    def __init__(self, absmax, shape, code, blocksize, dtype, offset=None, state2=None):
        self.absmax, self.shape, self.code = absmax, torch.Size(shape), code
        self.blocksize, self.dtype, self.offset, self.state2 = blocksize, dtype, offset, state2
        self.quant_type = "nf4"
        self.nested = state2 is not None

    def to(self, device):
        s2 = self.state2.to(device) if self.state2 is not None else None
        off = self.offset.to(device) if self.offset is not None else None
        return QuantState(self.absmax.to(device), self.shape, self.code.to(device), self.blocksize,
                          self.dtype, off, s2)


def normal_float4_levels():
    """16 quantisation levels in [-1, 1] with an exact zero: 8 + 1 quantiles of N(0,1) on the
    positive side and 7 + 1 on the negative side (the NormalFloat construction of the QLoRA
    paper), computed with torch's inverse error function."""
    edge = 0.5 * ((1 - 1 / 32) + (1 - 1 / 30))
    icdf = lambda p: math.sqrt(2.0) * torch.erfinv(2 * p - 1)  # noqa: E731
    pos = icdf(torch.linspace(edge, 0.5, 9, dtype=torch.float64)[:-1])
    neg = -icdf(torch.linspace(edge, 0.5, 8, dtype=torch.float64)[:-1])
    levels = torch.cat([neg, torch.zeros(1, dtype=torch.float64), pos]).sort().values
    return (levels / levels.abs().max()).float()


def absmax_levels():
    """256 sorted levels in [-1, 1] for the 8-bit quantisation of the absmax: signed
    fraction * 10^-e over seven decades, denser towards zero."""
    vals = {0.0, 1.0, -1.0}
    for e in range(7):
        for j in range(18):
            f = (0.1 + 0.9 * (j + 0.5) / 18) * 10.0 ** -e
            vals.add(f)
            vals.add(-f)
    vals.add(5e-8)
    out = torch.tensor(sorted(vals), dtype=torch.float64)
    return out[:256].float() if out.numel() >= 256 else F.pad(out, (0, 256 - out.numel()), value=1.0).float()


def _nearest(levels, x):
    return torch.bucketize(x, (levels[1:] + levels[:-1]) / 2)


def quantize_nf4(w, blocksize=64, nested=True, blocksize2=256, code=None, code2=None):
    """(packed uint8 [n/2, 1], QuantState) of a 2-D weight: blocks of `blocksize` along the
    row-major flattening, fp32 absmax, nearest level of w/absmax, element 2i in the high nibble of
    byte i; nested: (absmax - mean) quantised to 8 bits per block of `blocksize2`."""
    dev = w.device
    code = (normal_float4_levels() if code is None else code).to(dev)
    flat = w.detach().float().reshape(-1)
    n = flat.numel()
    if n % 2:
        raise ValueError("NF4 packing needs an even number of elements")
    blocks = F.pad(flat, (0, (-n) % blocksize)).view(-1, blocksize)
    absmax = blocks.abs().amax(1)
    idx = _nearest(code, blocks / absmax.clamp(min=1e-30)[:, None]).reshape(-1)[:n].to(torch.uint8)
    packed = ((idx[0::2] << 4) | idx[1::2]).reshape(-1, 1).contiguous()
    if not nested:
        return packed, QuantState(absmax, w.shape, code, blocksize, w.dtype)
    code2 = (absmax_levels() if code2 is None else code2).to(dev)
    offset = absmax.mean()
    centred = absmax - offset
    b2 = F.pad(centred, (0, (-centred.numel()) % blocksize2)).view(-1, blocksize2)
    absmax2 = b2.abs().amax(1)
    q8 = _nearest(code2, b2 / absmax2.clamp(min=1e-30)[:, None]).reshape(-1)[:centred.numel()]
    inner = QuantState(absmax2, (absmax.numel(),), code2, blocksize2, torch.float32)
    return packed, QuantState(q8.to(torch.uint8), w.shape, code, blocksize, w.dtype,
                              offset=offset.reshape(1).clone(), state2=inner)


class _MatMul4Bit(torch.autograd.Function):
    """x @ dequant(W)^T; the weight is dequantised again in backward instead of being kept."""

    @staticmethod
    def forward(ctx, x, layer):
        ctx.layer = layer
        return F.linear(x, dequantize_nf4(layer.packed, layer.quant_state, x.dtype))

    @staticmethod
    def backward(ctx, grad):
        w = dequantize_nf4(ctx.layer.packed, ctx.layer.quant_state, grad.dtype)
        return torch.matmul(grad, w), None


class NF4Linear(torch.nn.Module):
    """Frozen, bias-free linear with an NF4 double-quantised weight."""

    _soup_nf4_linear = True

    def __init__(self, in_features, out_features, packed, quant_state, compute_dtype=torch.float16):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("packed", packed, persistent=False)
        self.quant_state = quant_state
        self.compute_dtype = compute_dtype
        self.bias = None

    @classmethod
    def from_weight(cls, weight, compute_dtype=torch.float16, blocksize=64):
        packed, state = quantize_nf4(weight.to(torch.float16), blocksize=blocksize, nested=True)
        return cls(weight.shape[1], weight.shape[0], packed, state, compute_dtype)

    def _apply(self, fn, *args, **kwargs):
        super()._apply(fn, *args, **kwargs)
        self.quant_state = self.quant_state.to(self.packed.device)
        return self

    def matmul_4bit(self, x_low):
        return _MatMul4Bit.apply(x_low, self)

    def forward(self, x):
        return self.matmul_4bit(x.to(self.compute_dtype)).to(x.dtype)


class LoRALinear(torch.nn.Module):
    """base(x) + lora_B(lora_A(dropout(x))) * scaling with fp32 adapter weights (peft's layout:
    A Kaiming-uniform, B zero)."""

    def __init__(self, base_layer, r=16, alpha=32, dropout=0.05):
        super().__init__()
        self.base_layer = base_layer
        self.lora_A = torch.nn.Linear(base_layer.in_features, r, bias=False, dtype=torch.float32)
        self.lora_B = torch.nn.Linear(r, base_layer.out_features, bias=False, dtype=torch.float32)
        torch.nn.init.kaiming_uniform_(self.lora_A.weight, a=math.sqrt(5))
        torch.nn.init.zeros_(self.lora_B.weight)
        self.p = float(dropout)
        self.scaling = alpha / r

    def forward(self, x):
        result = self.base_layer(x)
        if branch_covers(x, self.p, self.training):
            lora = LoRABranch.apply(x, _shared_fp16(x), self.lora_A.weight, self.lora_B.weight,
                                    self.p, float(self.scaling))
            return result + lora
        xa = F.dropout(x.to(self.lora_A.weight.dtype), self.p, self.training)
        return result + self.lora_B(self.lora_A(xa)) * self.scaling
