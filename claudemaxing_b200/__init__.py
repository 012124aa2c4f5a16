"""claudemaxing_b200: the QLoRA training hot path of arturbaimuratov1-sys/claudemaxing on B200.

`apply()` installs the same seven patches as the reference's `solution.apply()`
(solution/__init__.py:25-32), in the same order; each op module keeps the reference's
autograd.Function and functional signatures. Underneath, every op calls a hand-written sm_100a
kernel through the C ABI of libsoup_b200 (include/soup_b200.h); there is no Triton, no CPU
fallback and no backend dispatch. `import claudemaxing_b200 as solution` is the drop-in.
"""

from ._lib import check_device_status, device_status
from .attention import patch_qwen2_grouped_sdpa
from .lm_head_loss import fused_head_loss, patch_fused_head_loss
from .lora import patch_peft_lora_4bit
from .nf4 import dequantize_nf4, patch_bnb_nf4_dequant
from .rmsnorm import patch_qwen2_rmsnorm, rmsnorm
from .rope import patch_qwen2_rope, rope
from .swiglu_recompute import patch_qwen2_mlp_recompute, swiglu_recompute

__all__ = ["apply", "fused_head_loss", "dequantize_nf4", "rmsnorm", "rope", "swiglu_recompute",
           "check_device_status", "device_status"]


def apply():
    patch_qwen2_mlp_recompute()   # SwiGLU with recomputation
    patch_qwen2_rmsnorm()         # fused RMSNorm
    patch_fused_head_loss()       # head + loss + metrics without full logits
    patch_qwen2_rope()            # rotary embedding, q and k in one launch
    patch_bnb_nf4_dequant()       # NF4 weight dequantisation in one kernel
    patch_peft_lora_4bit()        # LoRA branch with a packed dropout mask
    patch_qwen2_grouped_sdpa()    # torch SDPA per kv head, no k/v copies
