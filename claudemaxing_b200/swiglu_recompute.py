"""SwiGLU of the Qwen2 MLP, `silu(gate) * up`, with recomputation in backward.

Drop-in for the reference's solution/swiglu_recompute.py: `SwiGLURecompute.apply(gate, up,
inplace)`, `swiglu_recompute(gate, up, inplace=False)`, `MLPInputRecompute.apply(x, gate_proj,
up_proj, down_compute=None)` and `patch_qwen2_mlp_recompute()`. Backward keeps nothing but the two
inputs (silu is recomputed) and, with `inplace`, writes dgate over gate and dup over up.
`MLPInputRecompute` keeps only the MLP input and re-runs the two frozen projections in backward;
for 4-bit projections (bitsandbytes' Linear4bit or this package's NF4Linear) gate and up stay fp16
and the fp16 copy of the input written by the preceding RMSNorm is reused.
"""

import torch

from . import _lib
from .rmsnorm import fp16_copy_of

_SUPPORTED = (torch.float16, torch.bfloat16, torch.float32)


def _silu_mul_fwd(gate, up, out, round_silu):
    n = gate.numel()
    if n:
        _lib.require_cuda(gate, up, out)
        _lib.call("soup_silu_mul_fwd", _lib.ptr(gate), _lib.ptr(up), _lib.ptr(out), n,
                  _lib.dtype_code(gate.dtype), _lib.dtype_code(up.dtype),
                  _lib.dtype_code(out.dtype), int(round_silu), _lib.stream_of(gate))
    return out


def _silu_mul_bwd(dy, gate, up, d_gate, d_up, round_silu):
    """d_gate / d_up are output buffers (gate.dtype / up.dtype) or None when not wanted; they may
    be `gate` and `up` themselves."""
    n = gate.numel()
    if n:
        _lib.require_cuda(dy, gate, up)
        _lib.call("soup_silu_mul_bwd", _lib.ptr(dy), _lib.ptr(gate), _lib.ptr(up),
                  _lib.ptr(d_gate), _lib.ptr(d_up), n, _lib.dtype_code(dy.dtype),
                  _lib.dtype_code(gate.dtype), _lib.dtype_code(up.dtype), int(round_silu),
                  _lib.stream_of(gate))


class SwiGLURecompute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up, inplace):
        gate, up = gate.contiguous(), up.contiguous()
        out = torch.empty(gate.shape, dtype=torch.promote_types(gate.dtype, up.dtype),
                          device=gate.device)
        _silu_mul_fwd(gate, up, out, True)
        ctx.save_for_backward(gate, up)
        ctx.inplace = inplace
        return out

    @staticmethod
    def backward(ctx, grad):
        gate, up = ctx.saved_tensors
        want_gate, want_up = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if not (want_gate or want_up):
            return None, None, None
        if ctx.inplace:
            d_gate, d_up = (gate if want_gate else None), (up if want_up else None)
        else:
            d_gate = torch.empty_like(gate) if want_gate else None
            d_up = torch.empty_like(up) if want_up else None
        _silu_mul_bwd(grad.contiguous(), gate, up, d_gate, d_up, True)
        return d_gate, d_up, None


def swiglu_recompute(gate, up, inplace=False):
    """silu(gate) * up. With `inplace=True` backward overwrites the saved `gate` and `up`, so use it
    only when they are temporaries and backward runs once (no retain_graph)."""
    return SwiGLURecompute.apply(gate, up, inplace)


def _autocast_state():
    try:
        return torch.is_autocast_enabled("cuda"), torch.get_autocast_dtype("cuda")
    except (TypeError, AttributeError):
        return torch.is_autocast_enabled(), torch.get_autocast_gpu_dtype()


def _matmul_4bit(x_low, handle):
    """x_low @ dequant(W)^T for a 4-bit layer handle returned by `_nf4_layer`."""
    kind, weight, state = handle
    if kind == "bnb":
        import bitsandbytes as bnb

        return bnb.matmul_4bit(x_low, weight, quant_state=state)
    return weight.matmul_4bit(x_low)  # this package's NF4Linear


class MLPInputRecompute(torch.autograd.Function):
    """silu(gate_proj(x)) * up_proj(x) for frozen projections, keeping only `x` for backward
    (solution/swiglu_recompute.py:138-215 of the reference)."""

    @staticmethod
    def forward(ctx, x, gate_proj, up_proj, down_compute=None):
        nf4 = _nf4_pair(gate_proj, up_proj, x)
        if nf4 is not None:
            hg, hu, compute = nf4
            x_low = fp16_copy_of(x) if compute == torch.float16 else None
            if x_low is None:  # the norm before the MLP usually wrote this exact copy already
                x_low = x.to(compute)
            gate, up = _matmul_4bit(x_low, hg), _matmul_4bit(x_low, hu)
            out_dtype, round_silu = x.dtype, x.dtype == compute
            if down_compute == compute:
                out_dtype = compute  # the 4-bit down_proj casts its input to `compute` anyway
        else:
            gate, up = gate_proj(x), up_proj(x)
            out_dtype, round_silu = torch.promote_types(gate.dtype, up.dtype), True
        out = torch.empty(gate.shape, dtype=out_dtype, device=gate.device)
        _silu_mul_fwd(gate.contiguous(), up.contiguous(), out, round_silu)
        ctx.save_for_backward(x_low if nf4 is not None else x)
        ctx.x_dtype = x.dtype
        ctx.projs, ctx.nf4, ctx.round_silu = (gate_proj, up_proj), nf4, round_silu
        ctx.autocast = _autocast_state()
        return out

    @staticmethod
    def backward(ctx, grad):
        (x,) = ctx.saved_tensors
        enabled, dtype = ctx.autocast
        with torch.enable_grad(), torch.autocast("cuda", dtype=dtype, enabled=enabled):
            x_again = x.detach().requires_grad_(True)
            if ctx.nf4 is not None:
                hg, hu, _ = ctx.nf4
                gate, up = _matmul_4bit(x_again, hg), _matmul_4bit(x_again, hu)
            else:
                gate_proj, up_proj = ctx.projs
                gate, up = gate_proj(x_again), up_proj(x_again)
        g, u = gate.detach(), up.detach()
        if not (g.is_contiguous() and u.is_contiguous()):
            g, u = g.contiguous(), u.contiguous()
        # gradients written over the recomputed buffers, nothing else allocated
        _silu_mul_bwd(grad.contiguous(), g, u, g, u, ctx.round_silu)
        if ctx.nf4 is not None:
            (dx_gate,) = torch.autograd.grad(gate, x_again, g)
            (dx_up,) = torch.autograd.grad(up, x_again, u)
            return dx_gate.to(ctx.x_dtype) + dx_up.to(ctx.x_dtype), None, None, None
        torch.autograd.backward((gate, up), (g, u), inputs=[x_again])
        return x_again.grad, None, None, None


def _nf4_layer(linear):
    """(handle, compute dtype) of a bias-free 4-bit linear whose compute dtype is fixed, else None
    (then the module itself is called). Handles bitsandbytes' Linear4bit and this package's
    NF4Linear."""
    if getattr(linear, "bias", None) is not None:
        return None
    if linear._forward_hooks or linear._forward_pre_hooks or hasattr(linear, "_hf_hook"):
        return None  # calling the matmul directly would skip the hooks
    if getattr(linear, "_soup_nf4_linear", False):
        return ("soup", linear, None), linear.compute_dtype
    if type(linear).__name__ != "Linear4bit":
        return None
    try:
        import bitsandbytes as bnb
        from bitsandbytes.nn.modules import fix_4bit_weight_quant_state_from_module
    except Exception:  # noqa: BLE001
        return None
    if (not isinstance(linear, bnb.nn.Linear4bit) or not linear.compute_type_is_set
            or linear.compute_dtype is None):
        return None
    fix_4bit_weight_quant_state_from_module(linear)
    return ("bnb", linear.weight, linear.weight.quant_state), linear.compute_dtype


def _nf4_pair(gate_proj, up_proj, x):
    gate, up = _nf4_layer(gate_proj), _nf4_layer(up_proj)
    if gate is None or up is None or gate[1] != up[1] or x.dtype not in (torch.float32, gate[1]):
        return None
    return gate[0], up[0], gate[1]


def _frozen(module):
    return not any(p.requires_grad for p in module.parameters())


def patch_qwen2_mlp_recompute():
    """Send the activation of Qwen2MLP.forward through the recomputing kernels. Class-level. CPU
    tensors, another activation or unusual dtypes keep the installed behaviour."""
    from transformers.models.qwen2 import modeling_qwen2

    cls = getattr(modeling_qwen2, "Qwen2MLP", None)
    if cls is None or getattr(cls.forward, "_swiglu_recompute", False):
        return
    original = cls.forward

    def forward(self, x):
        act = getattr(getattr(self, "config", None), "hidden_act", "silu")
        if act != "silu" or not isinstance(x, torch.Tensor) or not x.is_cuda:
            return original(self, x)
        if (x.dtype in _SUPPORTED and _frozen(self.gate_proj) and _frozen(self.up_proj)
                and torch.is_grad_enabled() and x.requires_grad):
            down = _nf4_layer(self.down_proj)
            return self.down_proj(MLPInputRecompute.apply(x, self.gate_proj, self.up_proj,
                                                          down[1] if down else None))
        gate, up = self.gate_proj(x), self.up_proj(x)
        if (gate.shape != up.shape or gate.dtype not in _SUPPORTED
                or up.dtype not in _SUPPORTED):
            return self.down_proj(self.act_fn(gate) * up)
        return self.down_proj(swiglu_recompute(gate, up, True))

    forward._swiglu_recompute = True
    cls.forward = forward
