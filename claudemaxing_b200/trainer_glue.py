"""Where the fused head meets transformers and TRL: batch packing, the Qwen2ForCausalLM.forward
route that builds the loss from hidden states, and the SFTTrainer.compute_loss route that asks
for it and logs TRL's metrics from the per-token terms.

Behaviour follows the reference's solution/lm_head_loss.py:300-517 (same conditions under which a
step keeps TRL's own path, same metric definitions, same trainer attributes); the code is organised
differently: every "can this step be fused" question is a small named rule, so a refused step can
say why (`explain_trainer_route`, `explain_batch_route`), and the per-token terms travel in a
dataclass.
"""

import dataclasses
import functools

import torch

from . import lm_head_loss as head
from .attention import segment_arguments
from .embedding import shrink_tied_embedding


StepTerms = head.StepTerms


@dataclasses.dataclass
class PackedRow:
    """A padded batch `[B, T]` reduced to its real tokens as one row `[1, N]`. The tokens of a
    batch row stay together and in order, so attention over the packed row is causal attention
    inside each of the `B` segments that `cu_rows` delimits."""

    B: int
    T: int
    index: torch.Tensor     # [N] flat positions of the real tokens in the [B*T] batch
    ids: torch.Tensor       # [1, N]
    pos: torch.Tensor       # [1, N] position ids (restart in every batch row)
    target: torch.Tensor    # [1, N] labels shifted left inside their batch row
    cu_rows: torch.Tensor   # [B + 1] int32: where each batch row's tokens start in the packed row
    longest: int            # an upper bound of the tokens of one batch row

    @property
    def mask(self):
        """[1, 1, N, N] bool, same batch row and key not after the query: the O(N^2) form of
        `cu_rows`, built only for an attention that cannot take the segments."""
        from .attention import mask_of_segments

        return mask_of_segments(self.cu_rows, self.ids.shape[1])


# --------------------------------------------------------------------------------- packing
def pack_tokens(ids, mask, labels, position_ids=None):
    """PackedRow of a padded batch, or None when there is nothing to drop (no padding, or no real
    token) or the position ids are of a kind this packing does not understand."""
    n_rows, width = ids.shape
    real = torch.nonzero(mask.reshape(-1), as_tuple=False).reshape(-1)
    n_real = real.numel()
    if n_real == 0 or n_real == n_rows * width:
        return None
    batch_row = torch.div(real, width, rounding_mode="floor")
    if position_ids is None:
        positions = real - batch_row * width
    elif isinstance(position_ids, torch.Tensor) and position_ids.shape == ids.shape:
        positions = position_ids.reshape(-1).index_select(0, real)
    else:
        return None
    cu_rows = torch.zeros(n_rows + 1, dtype=torch.int32, device=ids.device)
    cu_rows[1:] = torch.bincount(batch_row, minlength=n_rows).cumsum(0)
    shifted = head.shift_labels_left(labels.to(ids.device)).reshape(-1).index_select(0, real)
    return PackedRow(B=n_rows, T=width, index=real,
                     ids=ids.reshape(-1).index_select(0, real).unsqueeze(0),
                     pos=positions.unsqueeze(0), target=shifted.unsqueeze(0),
                     cu_rows=cu_rows, longest=width)


def _plain_frozen_linear(module):
    return type(module) is torch.nn.Linear and module.bias is None and not module.weight.requires_grad


# (name, predicate over (lm, kwargs, labels)) - the first that holds keeps the padded batch
_BATCH_RULES = (
    ("input_ids is not a 2-D CUDA tensor",
     lambda lm, kw, lab: not (isinstance(kw.get("input_ids"), torch.Tensor)
                              and kw["input_ids"].dim() == 2 and kw["input_ids"].is_cuda)),
    ("attention_mask missing or of another shape",
     lambda lm, kw, lab: not (isinstance(kw.get("attention_mask"), torch.Tensor)
                              and kw["attention_mask"].shape == kw["input_ids"].shape)),
    ("inputs_embeds or a kv cache is in use",
     lambda lm, kw, lab: kw.get("inputs_embeds") is not None or kw.get("past_key_values") is not None),
    ("labels of another shape", lambda lm, kw, lab: lab.shape != kw["input_ids"].shape),
    ("the output head is not a plain frozen linear", lambda lm, kw, lab: not _plain_frozen_linear(lm.lm_head)),
    ("attention is not sdpa", lambda lm, kw, lab: getattr(lm.config, "_attn_implementation", None) != "sdpa"),
    ("sliding-window attention", lambda lm, kw, lab: bool(getattr(lm.config, "use_sliding_window", False))),
)


def explain_batch_route(lm, kwargs, labels):
    """Why this batch is not packed ("" when it is eligible)."""
    for reason, holds in _BATCH_RULES:
        if holds(lm, kwargs, labels):
            return reason
    return ""


def _pack_batch(lm, kwargs, labels):
    if explain_batch_route(lm, kwargs, labels):
        return None
    return pack_tokens(kwargs["input_ids"], kwargs["attention_mask"], labels, kwargs.get("position_ids"))


def _unpacked(values, packed):
    """Per-token values of the packed row back at their [B, T] places, zeros at the padding."""
    full = values.new_zeros(packed.B * packed.T)
    full.index_copy_(0, packed.index, values.reshape(-1))
    return full.view(packed.B, packed.T)


def _packed_logits_loss(lm, hidden, target, num_items_in_batch=None):
    """The packed row's loss and per-token terms through the logits, for a step whose head does
    not compute in float16 (bf16 autocast, an fp32 model without autocast): the tensor-core head
    kernel takes fp16 operands only, and the reference's packed route accepts every compute dtype
    (solution/lm_head_loss.py:339-362), so such a step keeps the packing and builds the logits of
    the real tokens only. Sum of the per-token cross-entropies over `num_items_in_batch` (default:
    the labelled tokens), as ForCausalLMLoss divides."""
    logits = lm.lm_head(hidden)
    flat = target.reshape(-1).to(logits.device)
    total = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), flat,
                                              ignore_index=head.IGNORE_INDEX, reduction="sum")
    divisor = flat.ne(head.IGNORE_INDEX).sum() if num_items_in_batch is None else num_items_in_batch
    if torch.is_tensor(divisor):
        divisor = divisor.to(total.device)
    terms = head.head_metrics_from_logits(logits.detach(), None, target=target)
    return total / divisor, terms


def _packed_forward(lm, kwargs, packed):
    """Decoder on the packed row, fused head on its hidden states; the per-token terms return to
    the padded layout (every consumer masks the padding out). `packed` needs the attributes of
    PackedRow."""
    from transformers.modeling_outputs import CausalLMOutputWithPast

    passthrough = dict(kwargs)
    for replaced in ("input_ids", "attention_mask", "position_ids"):
        passthrough.pop(replaced, None)
    for name, value in segment_arguments(packed.cu_rows, packed.longest, packed.ids.shape[1]).items():
        passthrough.setdefault(name, value)
    decoded = lm.model(input_ids=packed.ids, position_ids=packed.pos, **passthrough)
    hidden, weight = decoded.last_hidden_state, lm.lm_head.weight
    if head.head_compute_dtype(hidden, weight) == torch.float16:
        loss, terms = head.fused_head_loss(hidden, weight, None,
                                           num_items_in_batch=kwargs.get("num_items_in_batch"),
                                           target=packed.target)
    else:
        loss, terms = _packed_logits_loss(lm, hidden, packed.target,
                                          kwargs.get("num_items_in_batch"))
    lm.__dict__[head._STEP_ATTR] = StepTerms(_unpacked(terms.token_loss, packed),
                                             _unpacked(terms.token_entropy, packed),
                                             terms.correct, terms.labelled)
    return CausalLMOutputWithPast(loss=loss, logits=None)


# --------------------------------------------------------------------- Qwen2ForCausalLM.forward
def _forward_wants_fused(lm, args, kwargs):
    """The trainer asked for it (one-shot flag) and the call is the plain training call."""
    asked = lm.__dict__.pop(head._REQUEST_ATTR, False)
    if not asked or args or kwargs.get("labels") is None:
        return False
    keep = kwargs.get("logits_to_keep", 0)
    if not isinstance(keep, int) or keep != 0:
        return False
    return "shift_labels" not in kwargs and kwargs.get("return_dict") is not False


def _fused_lm_forward(lm, kwargs):
    from transformers.modeling_outputs import CausalLMOutputWithPast

    labels = kwargs.pop("labels")
    kwargs.pop("logits_to_keep", None)
    shrink_tied_embedding(lm)
    packed = _pack_batch(lm, kwargs, labels)
    if packed is not None:
        return _packed_forward(lm, kwargs, packed)
    decoded = lm.model(**kwargs)
    hidden, out_head = decoded.last_hidden_state, lm.lm_head
    fusable = (_plain_frozen_linear(out_head) and hidden.is_cuda
               and head.head_compute_dtype(hidden, out_head.weight) == torch.float16)
    if fusable:
        loss, terms = head.fused_head_loss(hidden, out_head.weight, labels,
                                           num_items_in_batch=kwargs.get("num_items_in_batch"))
        lm.__dict__[head._STEP_ATTR] = terms
        logits = None
    else:  # finish the way the installed forward does; the trainer takes its metrics from the logits
        logits = out_head(hidden)
        loss = lm.loss_function(logits=logits, labels=labels, vocab_size=lm.config.vocab_size, **kwargs)
    return CausalLMOutputWithPast(loss=loss, logits=logits, past_key_values=decoded.past_key_values,
                                  hidden_states=decoded.hidden_states, attentions=decoded.attentions)


def patch_qwen2_causal_lm_head():
    """Qwen2ForCausalLM.forward builds the loss from the hidden states with the fused head and
    returns no logits, but only for a call the trainer flagged; every other call is the installed
    forward."""
    from transformers.models.qwen2 import modeling_qwen2

    cls = getattr(modeling_qwen2, "Qwen2ForCausalLM", None)
    if cls is None or getattr(cls.forward, "_fused_head", False):
        return
    installed = cls.forward

    @functools.wraps(installed)  # the trainer inspects the forward's signature
    def forward(self, *args, **kwargs):
        if _forward_wants_fused(self, args, kwargs):
            return _fused_lm_forward(self, kwargs)
        return installed(self, *args, **kwargs)

    forward._fused_head = True
    cls.forward = forward


# ------------------------------------------------------------------- SFTTrainer.compute_loss
def _innermost_lm(model):
    """Through DDP-style `.module` wrappers and a peft wrapper to the causal LM."""
    while isinstance(getattr(model, "module", None), torch.nn.Module):
        model = model.module
    unwrap = getattr(model, "get_base_model", None)
    return unwrap() if callable(unwrap) else model


# (name, predicate over (trainer, model, inputs)) - the first that holds keeps TRL's own path
_TRAINER_RULES = (
    ("not a training step of an nn.Module",
     lambda tr, m, inp: not isinstance(m, torch.nn.Module) or not getattr(tr.model, "training", False)),
    ("DataParallel or several GPUs in one process",
     lambda tr, m, inp: isinstance(m, torch.nn.DataParallel) or getattr(tr.args, "n_gpu", 1) > 1),
    ("inputs without labels, or with pre-shifted labels",
     lambda tr, m, inp: not isinstance(inp, dict) or "labels" not in inp or "shift_labels" in inp),
    ("liger kernel", lambda tr, m, inp: bool(getattr(tr.args, "use_liger_kernel", False))),
    ("prompt tuning", lambda tr, m, inp: bool(getattr(tr, "num_virtual_tokens", 0))),
    ("auxiliary loss", lambda tr, m, inp: bool(getattr(tr, "aux_loss_enabled", False))),
    ("custom loss function", lambda tr, m, inp: getattr(tr, "compute_loss_func", None) is not None),
    ("label smoothing", lambda tr, m, inp: getattr(tr, "label_smoother", None) is not None),
    ("trainer without TRL's metric store", lambda tr, m, inp: not hasattr(tr, "_metrics")),
)


def explain_trainer_route(trainer, model, inputs):
    """(causal LM, "") when the step can use the fused head, else (None, reason)."""
    for reason, holds in _TRAINER_RULES:
        if holds(trainer, model, inputs):
            return None, reason
    lm = _innermost_lm(model)
    if not getattr(type(lm).forward, "_fused_head", False):
        return None, "the model's forward is not the patched one"
    out_head = lm.get_output_embeddings()
    if not _plain_frozen_linear(out_head) or not out_head.weight.is_cuda:
        return None, "the output head is not a plain frozen CUDA linear"
    if getattr(lm.config, "final_logit_softcapping", None) is not None:
        return None, "logit soft-capping"
    return lm, ""


def _log_trl_metrics(trainer, mode, inputs, terms):
    """`entropy`, `num_tokens` and `mean_token_accuracy` with the masks, gathers and order of
    reductions SFTTrainer.compute_loss uses when it has logits."""
    across_ranks = trainer.accelerator.gather_for_metrics
    store = trainer._metrics[mode]
    masked = "attention_mask" in inputs
    if not masked and "position_ids" not in inputs:
        raise ValueError("Expected 'attention_mask' or 'position_ids' in inputs.")

    if masked:
        weights = inputs["attention_mask"]
        mean_entropy = (terms.token_entropy * weights).sum() / weights.sum()
    else:
        mean_entropy = terms.token_entropy.mean()
    store["entropy"].append(across_ranks(mean_entropy).mean().item())

    if mode == "train":
        if masked:
            seen_here = inputs["attention_mask"].sum()
        else:
            ids = inputs["position_ids"]
            seen_here = torch.tensor(ids.size(1), device=ids.device)
        trainer._total_train_tokens += across_ranks(seen_here).sum().item()
    store["num_tokens"] = [trainer._total_train_tokens]

    hits, scored = across_ranks(terms.correct).sum(), across_ranks(terms.labelled).sum()
    store["mean_token_accuracy"].append((hits / scored).item() if scored > 0 else 0.0)
    # the host has just waited for this step's numbers: the one place a kernel that gave up a
    # bounded wait (its outputs are then unwritten) is turned into an exception, per step
    if terms.token_entropy.is_cuda:
        from . import _lib

        _lib.check_device_status(terms.token_entropy.device)


@dataclasses.dataclass
class _LossOnly:
    """What Soup's rewind recorder reads from the trainer after a step without logits."""

    token_loss: torch.Tensor


def patch_sft_compute_loss():
    """TRL's SFTTrainer.compute_loss: a training step of a patched causal LM flags the model for
    the fused head, logs TRL's metrics from the per-token terms and leaves the per-token losses
    where Soup's rewind recorder reads them. Without TRL this does nothing."""
    try:
        from trl.trainer import sft_trainer
    except Exception:  # noqa: BLE001
        return
    trainer_cls = sft_trainer.SFTTrainer
    if getattr(trainer_cls.compute_loss, "_fused_head", False):
        return
    installed = trainer_cls.compute_loss

    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        setattr(self, head.SOUP_STEP_ATTR, None)
        lm, _reason = explain_trainer_route(self, model, inputs)
        if lm is None:
            return installed(self, model, inputs, return_outputs=return_outputs,
                             num_items_in_batch=num_items_in_batch)
        inputs.pop("_prediction_loss_only", None)
        inputs["use_cache"] = False
        labels = inputs["labels"]
        lm.__dict__[head._REQUEST_ATTR] = True
        try:  # the grandparent's compute_loss: TRL's own would want logits for its metrics
            loss, outputs = super(trainer_cls, self).compute_loss(
                model, inputs, return_outputs=True, num_items_in_batch=num_items_in_batch)
        finally:
            lm.__dict__.pop(head._REQUEST_ATTR, None)
        terms = lm.__dict__.pop(head._STEP_ATTR, None)
        if terms is None:  # the forward ended up building logits
            terms = head.head_metrics_from_logits(outputs.logits, labels)
        _log_trl_metrics(self, "train", inputs, terms)
        setattr(self, head.SOUP_STEP_ATTR, _LossOnly(terms.token_loss))
        return (loss, outputs) if return_outputs else loss

    compute_loss._fused_head = True
    trainer_cls.compute_loss = compute_loss


def patch_fused_head_loss():
    patch_qwen2_causal_lm_head()
    patch_sft_compute_loss()
