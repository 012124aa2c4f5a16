"""Rotary position embedding for Qwen2 attention: q*cos + rotate_half(q)*sin, q and k in one launch.

Drop-in for the reference's solution/rope.py: `RoPE.apply(q, k, cos, sin) -> (q', k')`, `rope(...)`
and `patch_qwen2_rope()`. q and k are read through their strides (they arrive as transposed views
of the projection outputs), the outputs are contiguous [batch, heads, seq, head_dim] in
torch.promote_types(x.dtype, cos.dtype); backward is the same kernel with the transposed rotation
(csrc/rope.cu).
"""

import torch

from . import _lib

_SUPPORTED = (torch.float16, torch.bfloat16, torch.float32)


def _unit_last_stride(x):
    return x if x is None or x.stride(-1) == 1 else x.contiguous()


def _rotate_pair(q, k, cos, sin, q_dtype, k_dtype, backward):
    """Rotates q and/or k (either may be None) with one kernel launch."""
    q, k = _unit_last_stride(q), _unit_last_stride(k)
    ref = q if q is not None else k
    _lib.require_cuda(ref, cos, sin)
    b, _, t, d = ref.shape
    dev = ref.device
    q_out = torch.empty((b, q.shape[1], t, d), dtype=q_dtype, device=dev) if q is not None else None
    k_out = torch.empty((b, k.shape[1], t, d), dtype=k_dtype, device=dev) if k is not None else None
    if ref.numel() == 0 and (q is None or q.numel() == 0) and (k is None or k.numel() == 0):
        return q_out, k_out
    cs_b = cos.stride(0) if cos.shape[0] > 1 else 0  # batch 1: shared positions, broadcast
    f32 = _lib.F32
    _lib.call(
        "soup_rope", _lib.ptr(q), _lib.ptr(k), _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(q_out),
        _lib.ptr(k_out), b, q.shape[1] if q is not None else 0, k.shape[1] if k is not None else 0,
        t, d,
        *(q.stride()[:3] if q is not None else (0, 0, 0)),
        *(k.stride()[:3] if k is not None else (0, 0, 0)),
        cs_b, cos.stride(1),
        _lib.dtype_code(q.dtype) if q is not None else f32,
        _lib.dtype_code(k.dtype) if k is not None else f32,
        _lib.dtype_code(cos.dtype),
        _lib.dtype_code(q_dtype) if q is not None else f32,
        _lib.dtype_code(k_dtype) if k is not None else f32,
        int(backward), _lib.stream_of(ref))
    return q_out, k_out


class RoPE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, cos, sin):
        cos, sin = cos.contiguous(), sin.contiguous()
        q_dtype = torch.promote_types(q.dtype, cos.dtype)
        k_dtype = torch.promote_types(k.dtype, cos.dtype)
        ctx.save_for_backward(cos, sin)
        ctx.dtypes = (q.dtype, k.dtype)
        return _rotate_pair(q, k, cos, sin, q_dtype, k_dtype, False)

    @staticmethod
    def backward(ctx, grad_q, grad_k):
        cos, sin = ctx.saved_tensors
        q_dtype, k_dtype = ctx.dtypes
        gq = grad_q if ctx.needs_input_grad[0] and grad_q is not None else None
        gk = grad_k if ctx.needs_input_grad[1] and grad_k is not None else None
        if gq is None and gk is None:
            return None, None, None, None
        dq, dk = _rotate_pair(gq, gk, cos, sin, q_dtype, k_dtype, True)
        return dq, dk, None, None


def rope(q, k, cos, sin):
    """apply_rotary_pos_emb(q, k, cos, sin) for q/k of shape [batch, heads, seq, head_dim] and
    cos/sin of shape [batch, seq, head_dim]."""
    return RoPE.apply(q, k, cos, sin)


ORIGINAL = None


def _covered(q, k, cos, sin, unsqueeze_dim):
    if unsqueeze_dim != 1:
        return False
    if not all(isinstance(x, torch.Tensor) and x.is_cuda for x in (q, k, cos, sin)):
        return False
    d = q.shape[-1]
    half = d // 2
    return (q.dim() == 4 and k.dim() == 4 and cos.dim() == 3 and sin.shape == cos.shape
            and k.shape[-1] == d and cos.shape[-1] == d and d % 2 == 0 and d <= 256
            and half & (half - 1) == 0
            and cos.shape[0] in (1, q.shape[0]) and q.shape[2] == cos.shape[1]
            and k.shape[0] == q.shape[0] and k.shape[2] == q.shape[2]
            and not cos.requires_grad and not sin.requires_grad and sin.dtype == cos.dtype
            and len({x.device for x in (q, k, cos, sin)}) == 1
            and all(x.dtype in _SUPPORTED for x in (q, k, cos, sin)))


def patch_qwen2_rope():
    """Replace transformers.models.qwen2.modeling_qwen2.apply_rotary_pos_emb, which
    Qwen2Attention.forward looks up by name on every call. Layouts the kernel does not cover
    (CPU, another unsqueeze_dim, odd head_dim, gradients for cos/sin) keep the installed one."""
    global ORIGINAL
    from transformers.models.qwen2 import modeling_qwen2

    current = getattr(modeling_qwen2, "apply_rotary_pos_emb", None)
    if current is None or getattr(current, "_fused_rope", False):
        return
    ORIGINAL = original = current

    def apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim=1):
        if not _covered(q, k, cos, sin, unsqueeze_dim):
            return original(q, k, cos, sin, unsqueeze_dim)
        return rope(q, k, cos, sin)

    apply_rotary_pos_emb._fused_rope = True
    modeling_qwen2.apply_rotary_pos_emb = apply_rotary_pos_emb
