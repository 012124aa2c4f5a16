"""Grouped-query attention through torch SDPA without repeating k/v.

The hot path keeps torch's SDPA (a library call in the reference too, solution/attention.py:
332-343): one call per layer with `enable_gqa`, which gives the same products as transformers'
repeat_kv path without materialising the repeated k and v.
"""

import torch
import torch.nn.functional as F


def _grouped_sdpa(query, key, value, attention_mask, scaling):
    """One SDPA call for all heads; the kernel maps query head i to kv head i // group itself
    (`enable_gqa`), which is transformers' repeat_kv order. One call per layer matters: at a few
    thousand packed tokens every attention kernel is launch- and latency-bound."""
    out = F.scaled_dot_product_attention(query, key, value, attn_mask=attention_mask, dropout_p=0.0,
                                         scale=scaling, enable_gqa=True)
    return out.transpose(1, 2).contiguous()


def patch_qwen2_grouped_sdpa():
    """transformers' "sdpa" attention for grouped-query models with a boolean 4-D mask goes
    through `_grouped_sdpa`; everything else keeps the installed implementation."""
    from transformers.modeling_utils import AttentionInterface

    current = AttentionInterface._global_mapping.get("sdpa")
    if current is None or getattr(current, "_grouped_sdpa", False):
        return
    original = current

    def sdpa_attention_forward(module, query, key, value, attention_mask, dropout=0.0,
                               scaling=None, is_causal=None, **kwargs):
        groups = getattr(module, "num_key_value_groups", 1)
        tensors_ok = all(isinstance(x, torch.Tensor) and x.dim() == 4 and x.is_cuda
                         for x in (query, key, value))
        mask_ok = (isinstance(attention_mask, torch.Tensor)
                   and attention_mask.dtype == torch.bool and attention_mask.dim() == 4)
        plain = (dropout == 0.0 and kwargs.get("sliding_window") is None
                 and kwargs.get("position_bias") is None
                 and not kwargs.get("output_attentions", False))
        if (groups > 1 and tensors_ok and mask_ok and plain
                and query.shape[1] == key.shape[1] * groups and key.shape == value.shape):
            return _grouped_sdpa(query, key, value, attention_mask, scaling), None
        return original(module, query, key, value, attention_mask, dropout=dropout,
                        scaling=scaling, is_causal=is_causal, **kwargs)

    sdpa_attention_forward._grouped_sdpa = True
    AttentionInterface._global_mapping["sdpa"] = sdpa_attention_forward
