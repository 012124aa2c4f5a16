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


def rotate_into(q, q_add, k, cos, sin, q_out, k_out, backward=False):
    """Rotates `q` (+ `q_add`, summed in fp32 first, when given) and `k` into `q_out` and `k_out`.
    Every tensor is a [batch, heads, seq, head_dim] view with a unit last stride; the outputs are
    written through their strides, so they may be [batch, seq, heads, head_dim] buffers seen
    transposed, or column blocks of a wider matrix. One launch (csrc/rope.cu, soup_rope_sum)."""
    _lib.require_cuda(q, k, cos, sin, q_out, k_out)
    b, hq, t, d = q.shape
    if q_add is not None and q_add.shape != q.shape:
        raise ValueError("q's second term must have q's shape")
    for x in (q, k, q_out, k_out) + (() if q_add is None else (q_add,)):
        if x.stride(-1) != 1:
            raise ValueError("rotate_into needs a unit last stride")
    cs_b = cos.stride(0) if cos.shape[0] > 1 else 0
    _lib.call(
        "soup_rope_sum", _lib.ptr(q), _lib.ptr(q_add), _lib.ptr(k), _lib.ptr(cos), _lib.ptr(sin),
        _lib.ptr(q_out), _lib.ptr(k_out), b, hq, k.shape[1], t, d,
        *q.stride()[:3], *k.stride()[:3], cs_b, cos.stride(1),
        *((0, 0, 0) if q_add is None else q_add.stride()[:3]),
        *q_out.stride()[:3], *k_out.stride()[:3],
        _lib.dtype_code(q.dtype), _lib.dtype_code((q_add if q_add is not None else q).dtype),
        _lib.dtype_code(k.dtype), _lib.dtype_code(cos.dtype), _lib.dtype_code(q_out.dtype),
        _lib.dtype_code(k_out.dtype), int(backward), _lib.stream_of(q))


class RoPE(torch.autograd.Function):
    """`RoPE.apply(q, k, cos, sin) -> (q', k')`; the gradient of a rotation is the rotation by the
    opposite angle, so backward is the same kernel with its `backward` flag set."""

    @staticmethod
    def forward(ctx, q, k, cos, sin):
        tables = (cos.contiguous(), sin.contiguous())
        ctx.save_for_backward(*tables)
        ctx.in_dtypes = (q.dtype, k.dtype)           # what the gradients have to come back in
        out_dtypes = tuple(torch.promote_types(t.dtype, cos.dtype) for t in (q, k))
        return _rotate_pair(q, k, *tables, *out_dtypes, False)

    @staticmethod
    def backward(ctx, grad_q, grad_k):
        wanted = [g if (g is not None and ctx.needs_input_grad[i]) else None
                  for i, g in enumerate((grad_q, grad_k))]
        if wanted[0] is None and wanted[1] is None:
            return None, None, None, None
        dq, dk = _rotate_pair(*wanted, *ctx.saved_tensors, *ctx.in_dtypes, True)
        return dq, dk, None, None


def rope(q, k, cos, sin):
    """apply_rotary_pos_emb(q, k, cos, sin) for q/k of shape [batch, heads, seq, head_dim] and
    cos/sin of shape [batch, seq, head_dim]."""
    return RoPE.apply(q, k, cos, sin)


ORIGINAL = None   # the installed apply_rotary_pos_emb, once patched


def _why_not(q, k, cos, sin, unsqueeze_dim):
    """Why a call keeps the installed implementation ("" when the kernel covers it)."""
    tensors = (q, k, cos, sin)
    if unsqueeze_dim != 1:
        return "heads are not on dim 1"
    if not all(isinstance(t, torch.Tensor) and t.is_cuda for t in tensors):
        return "not CUDA tensors"
    if len({t.device for t in tensors}) != 1 or not all(t.dtype in _SUPPORTED for t in tensors):
        return "mixed devices or an unsupported dtype"
    if q.dim() != 4 or k.dim() != 4 or cos.dim() != 3 or sin.shape != cos.shape or sin.dtype != cos.dtype:
        return "unexpected ranks"
    d = q.shape[-1]
    if d != k.shape[-1] or d != cos.shape[-1] or d % 2 or d > 256 or (d // 2) & (d // 2 - 1):
        return "head_dim must be an even power of two up to 256, the same for q, k and the tables"
    if k.shape[0] != q.shape[0] or k.shape[2] != q.shape[2] or cos.shape[1] != q.shape[2]:
        return "batch or sequence sizes differ"
    if cos.shape[0] not in (1, q.shape[0]):
        return "tables neither shared nor per batch row"
    if cos.requires_grad or sin.requires_grad:
        return "the tables want a gradient"
    return ""


def patch_qwen2_rope():
    """Replace transformers.models.qwen2.modeling_qwen2.apply_rotary_pos_emb, which
    Qwen2Attention.forward looks up by name on every call. Calls the kernel does not cover (see
    `_why_not`) keep the installed function."""
    global ORIGINAL
    from transformers.models.qwen2 import modeling_qwen2 as qwen2

    installed = getattr(qwen2, "apply_rotary_pos_emb", None)
    if installed is None or getattr(installed, "_fused_rope", False):
        return

    def apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim=1):
        if _why_not(q, k, cos, sin, unsqueeze_dim):
            return installed(q, k, cos, sin, unsqueeze_dim)
        return rope(q, k, cos, sin)

    apply_rotary_pos_emb._fused_rope = True
    ORIGINAL = installed
    qwen2.apply_rotary_pos_emb = apply_rotary_pos_emb
