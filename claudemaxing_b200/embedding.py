"""fp16 storage for the frozen, tied embedding / head weight of the 4-bit model.

`prepare_model_for_kbit_training` leaves the tied weight in fp32 although every value is an fp16
number (the checkpoint is fp16). The fused head reads the weight as fp16 anyway, so storing it in
fp16 halves 890 MiB without changing any value; the embedding lookup casts back to fp32 so the
residual stream keeps its dtype. Same behaviour as the reference's solution/embedding.py:56-79;
on a 180 GB part the point is no longer the memory but that the head kernel gets an fp16 operand
without a per-step cast of 467 MB.
"""

import types

import torch
import torch.nn.functional as F

_DONE = "_fp16_tied_embedding"
_CHECK_ROWS = 8192


def _lookup_as_fp32(self, input):
    out = F.embedding(input, self.weight, self.padding_idx, self.max_norm, self.norm_type,
                      self.scale_grad_by_freq, self.sparse)
    return out.to(torch.float32)


def _lossless_fp16(weight):
    """fp16 tensor equal in value to fp32 `weight`, or None if some value is not an fp16 number.
    Converted slab by slab so the check never holds a second full-size fp32 temporary."""
    low = torch.empty(weight.shape, dtype=torch.float16, device=weight.device)
    for r0 in range(0, weight.shape[0], _CHECK_ROWS):
        slab = weight.data[r0:r0 + _CHECK_ROWS]
        low[r0:r0 + _CHECK_ROWS] = slab
        if not torch.equal(low[r0:r0 + _CHECK_ROWS].float(), slab):
            return None
    return low


def _autocast_fp16():
    try:
        return (torch.is_autocast_enabled("cuda")
                and torch.get_autocast_dtype("cuda") == torch.float16)
    except (TypeError, AttributeError):
        return torch.is_autocast_enabled() and torch.get_autocast_gpu_dtype() == torch.float16


def shrink_tied_embedding(lm):
    """Store the tied fp32 embedding/head weight of `lm` in fp16 if that is lossless. Decided once
    per model, on the first call under fp16 autocast; returns whether the weight is fp16 by us."""
    done = getattr(lm, _DONE, None)
    if done is not None:
        return done
    if not _autocast_fp16():
        return False
    emb, head = lm.get_input_embeddings(), lm.get_output_embeddings()
    w = getattr(emb, "weight", None)
    eligible = (type(emb) is torch.nn.Embedding and type(head) is torch.nn.Linear
                and w is not None and head.weight is w and w.dtype == torch.float32
                and w.is_cuda and not w.requires_grad and emb.max_norm is None
                and not emb.sparse and not emb._forward_pre_hooks
                and "forward" not in emb.__dict__ and not hasattr(emb, "_hf_hook"))
    ok = False
    if eligible:
        with torch.no_grad():
            low = _lossless_fp16(w)
            if low is not None:
                w.data = low  # one Parameter, shared with the head
                emb.forward = types.MethodType(_lookup_as_fp32, emb)
                ok = True
    setattr(lm, _DONE, ok)
    return ok
