"""Attention of the packed training row, and grouped-query attention without repeating k/v.

Attention stays a library call, as in the reference (solution/attention.py:332-343 calls torch
SDPA). Two routes replace transformers' "sdpa" attention function:

* a packed row whose batch rows are given as segment offsets (`cu_seq_lens_q` / `cu_seq_lens_k`,
  the keyword names transformers uses for packed sequences) runs torch's variable-length causal
  attention: work and memory are linear in the packed length times the longest segment, and no
  [N, N] mask exists. The reference's packed route builds that mask (solution/lm_head_loss.py:
  300-337); this is the same attention pattern stated as segments.
* a boolean 4-D mask on a grouped-query model runs one SDPA call with `enable_gqa`, which gives
  the same products as transformers' repeat_kv path without materialising the repeated k and v.
"""

import os

import torch
import torch.nn.functional as F

from . import _lib

_LOW = (torch.float16, torch.bfloat16)
# SOUP_ATTN_KERNEL=0 keeps torch's variable-length kernel for forward and backward;
# SOUP_ATTN_BACKWARD=0 keeps it for the backward only
OWN_FORWARD = os.environ.get("SOUP_ATTN_KERNEL", "1") != "0"
OWN_BACKWARD = os.environ.get("SOUP_ATTN_BACKWARD", "1") != "0"


def attention_gradients(q, k, v, out, lse, grad, cu_rows, scale):
    """(dq fp16 [n, hq, 128], dk fp32 [n, hk, 128], dv fp32 [n, hk, 128]) of the segment attention
    from this library's backward kernel (csrc/attention.cu)."""
    n, hq, d = q.shape
    grad = grad if grad.is_contiguous() else grad.contiguous()
    dq = torch.empty((n, hq, d), dtype=q.dtype, device=q.device)
    dk, dv = torch.empty((2, n, k.shape[1], d), dtype=torch.float32, device=q.device)   # one clear
    _lib.call("soup_attn_bwd", _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(grad),
              _lib.ptr(lse), _lib.ptr(cu_rows), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), n,
              cu_rows.numel() - 1, hq, k.shape[1], d, q.stride(0), k.stride(0), v.stride(0),
              float(scale), _lib.stream_of(q))
    return dq, dk, dv


def mask_of_segments(cu_rows, n):
    """[1, 1, n, n] bool: key in the same segment as the query and not after it. `cu_rows` holds
    the segments' starts followed by the total."""
    idx = torch.arange(n, device=cu_rows.device)
    segment = torch.searchsorted(cu_rows[1:].to(torch.int64), idx, right=True)
    same = segment.unsqueeze(1).eq(segment.unsqueeze(0))
    return (same & idx.unsqueeze(0).le(idx.unsqueeze(1))).unsqueeze(0).unsqueeze(0)


def _varlen():
    try:
        from torch.nn.attention.varlen import varlen_attn
    except ImportError:
        return None
    return varlen_attn


def _autocast_dtype():
    try:
        on, dtype = torch.is_autocast_enabled("cuda"), torch.get_autocast_dtype("cuda")
    except (TypeError, AttributeError):
        on, dtype = torch.is_autocast_enabled(), torch.get_autocast_gpu_dtype()
    return dtype if on else None


def _grouped_sdpa(query, key, value, attention_mask, scaling):
    """One SDPA call for all heads; the kernel maps query head i to kv head i // group itself
    (`enable_gqa`), which is transformers' repeat_kv order. One call per layer matters: at a few
    thousand packed tokens every attention kernel is launch- and latency-bound."""
    out = F.scaled_dot_product_attention(query, key, value, attn_mask=attention_mask, dropout_p=0.0,
                                         scale=scaling, enable_gqa=query.shape[1] != key.shape[1])
    return out.transpose(1, 2).contiguous()


def _token_major(t):
    """[tokens, heads, 128] view of a [1, heads, tokens, 128] tensor if its heads are adjacent in
    memory (a transposed view of a [tokens, heads * 128] matrix), else None."""
    x = t.transpose(1, 2)[0]
    if x.stride(2) == 1 and x.stride(1) == x.shape[2] and x.stride(0) >= x.shape[1] * x.shape[2] \
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0:
        return x
    return None


class SegmentAttention(torch.autograd.Function):
    """Causal attention inside the segments of a packed row on fp16 [tokens, heads, 128] tensors:
    forward and backward by this library's tcgen05 kernels (csrc/attention.cu). The forward also
    returns the row log-sum-exps in the layout torch's variable-length flash-attention backward
    takes ([heads, tokens]), which `SOUP_ATTN_BACKWARD=0` uses instead of this library's."""

    @staticmethod
    def forward(ctx, q, k, v, cu_rows, longest, scale):
        n, hq, d = q.shape
        out = torch.empty((n, hq, d), dtype=q.dtype, device=q.device)
        lse = torch.empty((hq, n), dtype=torch.float32, device=q.device)
        _lib.call("soup_attn_fwd", _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(cu_rows),
                  _lib.ptr(out), _lib.ptr(lse), n, cu_rows.numel() - 1, hq, k.shape[1], d,
                  q.stride(0), k.stride(0), v.stride(0), float(scale), _lib.stream_of(q))
        ctx.save_for_backward(q, k, v, cu_rows, out, lse)
        ctx.longest, ctx.scale = int(longest), float(scale)
        return out

    @staticmethod
    def backward(ctx, grad):
        q, k, v, cu_rows, out, lse = ctx.saved_tensors
        if OWN_BACKWARD:
            dq, dk, dv = attention_gradients(q, k, v, out, lse, grad, cu_rows, ctx.scale)
            return dq, dk.to(k.dtype), dv.to(v.dtype), None, None, None
        rng_state = torch.empty(2, dtype=torch.uint64, device=q.device)   # no dropout: never read
        dq, dk, dv = torch.ops.torch_attn._varlen_attn_backward(
            grad.contiguous(), q, k, v, out, lse, cu_rows, cu_rows, ctx.longest, ctx.longest, True,
            rng_state, ctx.scale, [-1, 0])
        return dq, dk, dv, None, None, None


def _own_forward_covers(q, k, v, cu_rows):
    return (OWN_FORWARD and q is not None and k is not None and v is not None
            and q.dtype == torch.float16 and k.dtype == v.dtype == torch.float16
            and q.shape[2] == 128 and cu_rows.dtype == torch.int32 and cu_rows.is_cuda
            and hasattr(torch.ops, "torch_attn") and hasattr(torch.ops.torch_attn, "_varlen_attn_backward"))


def segment_attention(query, key, value, cu_rows, longest, scaling):
    """Causal attention inside each segment of one packed row. query [1, Hq, N, D], key and value
    [1, Hkv, N, D] (any strides with a contiguous last dimension), `cu_rows` int32 [S + 1] on the
    same device, `longest` >= the longest segment. Returns [1, N, Hq, D], contiguous. Under
    autocast the operands are cast as SDPA would cast them; operands the variable-length kernel
    does not take (fp32, CPU, head dimension over 256) go through SDPA with the mask instead."""
    varlen_attn = _varlen()
    dtype = _autocast_dtype() or query.dtype
    if (varlen_attn is None or not query.is_cuda or dtype not in _LOW or query.shape[-1] > 256
            or query.shape[-1] % 8 or query.shape[1] % key.shape[1]):
        return _grouped_sdpa(query, key, value, mask_of_segments(cu_rows, query.shape[2]), scaling)
    if dtype == torch.float16 and all(t.dtype == dtype for t in (query, key, value)):
        rows = [_token_major(t) for t in (query, key, value)]
        if _own_forward_covers(*rows, cu_rows):
            scale = query.shape[-1] ** -0.5 if scaling is None else scaling
            return SegmentAttention.apply(*rows, cu_rows, longest, scale).unsqueeze(0)
    q, k, v = (t.transpose(1, 2)[0] if t.dtype == dtype else t.transpose(1, 2)[0].to(dtype)
               for t in (query, key, value))
    out = varlen_attn(q, k, v, cu_rows, cu_rows, int(longest), int(longest),
                      scale=scaling, window_size=(-1, 0))
    return out.unsqueeze(0)


def segments_route_installed():
    """Whether transformers' "sdpa" attention function is the one that understands segments."""
    try:
        from transformers.modeling_utils import AttentionInterface
    except ImportError:
        return False
    return getattr(AttentionInterface._global_mapping.get("sdpa"), "_grouped_sdpa", False)


def segment_arguments(cu_rows, longest, n=None):
    """Keyword arguments that make a transformers decoder attend inside the segments of a packed
    row: the offsets under transformers' packed-sequence names and no mask at all when the "sdpa"
    function is this module's, else the [1, 1, N, N] mask."""
    if segments_route_installed():
        return {"attention_mask": {"full_attention": None}, "cu_seq_lens_q": cu_rows,
                "cu_seq_lens_k": cu_rows, "max_length_q": longest, "max_length_k": longest}
    total = int(cu_rows[-1]) if n is None else n
    return {"attention_mask": mask_of_segments(cu_rows, total)}


def patch_qwen2_grouped_sdpa():
    """transformers' "sdpa" attention: a packed row given as segment offsets goes through
    `segment_attention`, a grouped-query model with a boolean 4-D mask through `_grouped_sdpa`;
    everything else keeps the installed implementation."""
    from transformers.modeling_utils import AttentionInterface

    current = AttentionInterface._global_mapping.get("sdpa")
    if current is None or getattr(current, "_grouped_sdpa", False):
        return
    original = current

    def sdpa_attention_forward(module, query, key, value, attention_mask, dropout=0.0,
                               scaling=None, is_causal=None, **kwargs):
        groups = getattr(module, "num_key_value_groups", 1)
        tensors_ok = all(isinstance(x, torch.Tensor) and x.dim() == 4 for x in (query, key, value))
        plain = (dropout == 0.0 and kwargs.get("sliding_window") is None
                 and kwargs.get("position_bias") is None
                 and not kwargs.get("output_attentions", False))
        cu = kwargs.get("cu_seq_lens_q")
        if (attention_mask is None and isinstance(cu, torch.Tensor) and kwargs.get("cu_seq_lens_k") is cu
                and tensors_ok and plain and query.shape[0] == 1 and key.shape == value.shape
                and query.shape[2] == key.shape[2]):
            return segment_attention(query, key, value, cu, kwargs.get("max_length_q", query.shape[2]),
                                     scaling), None
        if attention_mask is None and isinstance(cu, torch.Tensor) and tensors_ok:
            # segments this route does not cover (attention dropout, a cache): state them as a mask
            attention_mask = mask_of_segments(cu, key.shape[2])[..., -query.shape[2]:, :]
        mask_ok = (isinstance(attention_mask, torch.Tensor)
                   and attention_mask.dtype == torch.bool and attention_mask.dim() == 4)
        if (groups > 1 and tensors_ok and mask_ok and plain and query.is_cuda
                and query.shape[1] == key.shape[1] * groups and key.shape == value.shape):
            return _grouped_sdpa(query, key, value, attention_mask, scaling), None
        return original(module, query, key, value, attention_mask, dropout=dropout,
                        scaling=scaling, is_causal=is_causal, **kwargs)

    sdpa_attention_forward._grouped_sdpa = True
    AttentionInterface._global_mapping["sdpa"] = sdpa_attention_forward
