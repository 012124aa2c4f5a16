"""SwiGLU of the Qwen2 MLP, `silu(gate) * up`, with recomputation in backward.

Drop-in for the reference's solution/swiglu_recompute.py: `SwiGLURecompute.apply(gate, up,
inplace)`, `swiglu_recompute(gate, up, inplace=False)`, `MLPInputRecompute.apply(x, gate_proj,
up_proj, down_compute=None)` and `patch_qwen2_mlp_recompute()`. Backward keeps nothing but the two
inputs (silu is recomputed) and, with `inplace`, writes dgate over gate and dup over up.
`MLPInputRecompute` keeps only the MLP input and re-runs the two frozen projections in backward;
for 4-bit projections (bitsandbytes' Linear4bit or this package's NF4Linear, wrapped by
`_FourBitWeight`) gate and up stay fp16 and the fp16 copy of the input written by the preceding
RMSNorm is reused.
"""

import torch

from . import _lib
from .nf4 import nf4_linear, nf4_linear_dx
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


class _FourBitWeight:
    """A bias-free 4-bit projection reduced to what the MLP needs: `matmul(x_low)` = x_low @
    dequant(W)^T with the weight dequantised again in its own backward, and the fixed compute
    dtype. Wraps bitsandbytes' Linear4bit or this package's NF4Linear."""

    def __init__(self, compute_dtype, matmul):
        self.compute_dtype, self.matmul = compute_dtype, matmul

    @classmethod
    def of(cls, linear):
        """The wrapper for `linear`, or None when the module has to be called as a whole (bias,
        hooks that a direct matmul would skip, no fixed compute dtype, not a 4-bit layer)."""
        if getattr(linear, "bias", None) is not None or hasattr(linear, "_hf_hook"):
            return None
        if linear._forward_hooks or linear._forward_pre_hooks:
            return None
        if getattr(linear, "_soup_nf4_linear", False):
            return cls(linear.compute_dtype, linear.matmul_4bit)
        if type(linear).__name__ != "Linear4bit":
            return None
        try:
            import bitsandbytes as bnb
            from bitsandbytes.nn.modules import fix_4bit_weight_quant_state_from_module as restore_state
        except Exception:  # noqa: BLE001 - a look-alike class without bitsandbytes behind it
            return None
        if not isinstance(linear, bnb.nn.Linear4bit):
            return None
        if not linear.compute_type_is_set or linear.compute_dtype is None:
            return None
        restore_state(linear)
        weight = linear.weight
        return cls(linear.compute_dtype,
                   lambda x_low: bnb.matmul_4bit(x_low, weight, quant_state=weight.quant_state))


def _four_bit_pair(gate_proj, up_proj, x):
    """Both projections as _FourBitWeight when they share a compute dtype that x can be cast to."""
    gate, up = _FourBitWeight.of(gate_proj), _FourBitWeight.of(up_proj)
    if gate is None or up is None or gate.compute_dtype != up.compute_dtype:
        return None
    if x.dtype != torch.float32 and x.dtype != gate.compute_dtype:
        return None
    return gate, up


def _fused_pair(gate_proj, up_proj, x_low):
    """[(packed, state), (packed, state)] when gate_proj and up_proj are this package's NF4 layers
    and their products with `x_low` can share one launch of the NF4 GEMM (x is then read once and
    the two input gradients are summed in the accumulator), else None."""
    if not (getattr(gate_proj, "_soup_nf4_linear", False) and getattr(up_proj, "_soup_nf4_linear", False)):
        return None
    if not (gate_proj.takes_fused_gemm(x_low) and up_proj.takes_fused_gemm(x_low)):
        return None
    if gate_proj.out_features % 64 or up_proj.out_features % 64:
        return None
    return [(gate_proj.packed, gate_proj.quant_state), (up_proj.packed, up_proj.quant_state)]


class MLPInputRecompute(torch.autograd.Function):
    """silu(gate_proj(x)) * up_proj(x) for frozen projections, keeping only the MLP input for
    backward (the reference's solution/swiglu_recompute.py:138-215): backward runs the two
    projections again, lets the kernel write dgate / dup over the recomputed gate / up, and sends
    those back through the projections."""

    @staticmethod
    def forward(ctx, x, gate_proj, up_proj, down_compute=None):
        pair = _four_bit_pair(gate_proj, up_proj, x)
        if pair is None:
            kept = x
            gate, up = gate_proj(x), up_proj(x)
            out_dtype, round_silu = torch.promote_types(gate.dtype, up.dtype), True
        else:
            compute = pair[0].compute_dtype
            kept = fp16_copy_of(x) if compute == torch.float16 else None
            if kept is None:   # usually the norm before the MLP has written exactly this copy
                kept = x.to(compute)
            fused = _fused_pair(gate_proj, up_proj, kept)
            if fused is not None:
                gate, up = nf4_linear(kept, fused)
            else:
                gate, up = pair[0].matmul(kept), pair[1].matmul(kept)
            round_silu = x.dtype == compute
            # a 4-bit down_proj casts its input to `compute` anyway: hand it that dtype directly
            out_dtype = compute if down_compute == compute else x.dtype
        out = torch.empty(gate.shape, dtype=out_dtype, device=gate.device)
        _silu_mul_fwd(gate.contiguous(), up.contiguous(), out, round_silu)
        ctx.save_for_backward(kept)
        ctx.modules, ctx.pair = (gate_proj, up_proj), pair
        ctx.round_silu, ctx.x_dtype, ctx.autocast = round_silu, x.dtype, _autocast_state()
        return out

    @staticmethod
    def backward(ctx, grad):
        (kept,) = ctx.saved_tensors
        on, dtype = ctx.autocast
        fused = _fused_pair(*ctx.modules, kept) if ctx.pair is not None else None
        if fused is not None:
            # one launch recomputes gate and up, one forms dgate * Wg + dup * Wu in the accumulator
            d_gate, d_up = nf4_linear(kept, fused)
            _silu_mul_bwd(grad.contiguous(), d_gate, d_up, d_gate, d_up, ctx.round_silu)
            direct = ctx.x_dtype if ctx.x_dtype in (torch.float16, torch.float32) else torch.float16
            dx = nf4_linear_dx([d_gate, d_up], fused, direct)
            return dx.to(ctx.x_dtype), None, None, None
        leaf = kept.detach().requires_grad_(True)
        with torch.enable_grad(), torch.autocast("cuda", dtype=dtype, enabled=on):
            if ctx.pair is None:
                gate, up = ctx.modules[0](leaf), ctx.modules[1](leaf)
            else:
                gate, up = ctx.pair[0].matmul(leaf), ctx.pair[1].matmul(leaf)
        d_gate, d_up = gate.detach().contiguous(), up.detach().contiguous()
        # the two gradients overwrite the recomputed activations: nothing else is allocated
        _silu_mul_bwd(grad.contiguous(), d_gate, d_up, d_gate, d_up, ctx.round_silu)
        if ctx.pair is None:
            torch.autograd.backward((gate, up), (d_gate, d_up), inputs=[leaf])
            return leaf.grad, None, None, None
        from_gate = torch.autograd.grad(gate, leaf, d_gate)[0]
        from_up = torch.autograd.grad(up, leaf, d_up)[0]
        return from_gate.to(ctx.x_dtype) + from_up.to(ctx.x_dtype), None, None, None


def _all_frozen(*modules):
    return not any(p.requires_grad for m in modules for p in m.parameters())


def _mlp_forward(mlp, x, installed):
    """Qwen2MLP.forward with the activation (and, for frozen projections in training, the two
    projections' outputs) not kept for backward."""
    silu = getattr(getattr(mlp, "config", None), "hidden_act", "silu") == "silu"
    if not (silu and isinstance(x, torch.Tensor) and x.is_cuda):
        return installed(mlp, x)
    training_input = torch.is_grad_enabled() and x.requires_grad
    if training_input and x.dtype in _SUPPORTED and _all_frozen(mlp.gate_proj, mlp.up_proj):
        down = _FourBitWeight.of(mlp.down_proj)
        hidden = MLPInputRecompute.apply(x, mlp.gate_proj, mlp.up_proj,
                                         down.compute_dtype if down is not None else None)
        return mlp.down_proj(hidden)
    gate, up = mlp.gate_proj(x), mlp.up_proj(x)
    if gate.shape == up.shape and gate.dtype in _SUPPORTED and up.dtype in _SUPPORTED:
        return mlp.down_proj(swiglu_recompute(gate, up, True))
    return mlp.down_proj(mlp.act_fn(gate) * up)


def patch_qwen2_mlp_recompute():
    """Qwen2MLP.forward goes through `_mlp_forward` (class-level patch; CPU tensors, another
    activation or unusual dtypes keep the installed behaviour)."""
    from transformers.models.qwen2 import modeling_qwen2

    cls = getattr(modeling_qwen2, "Qwen2MLP", None)
    if cls is None or getattr(cls.forward, "_swiglu_recompute", False):
        return
    installed = cls.forward

    def forward(self, x):
        return _mlp_forward(self, x, installed)

    forward._swiglu_recompute = True
    cls.forward = forward
