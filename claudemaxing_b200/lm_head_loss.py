"""The output head and everything the trainer reads from its logits, without the full logits.

Drop-in for the reference's solution/lm_head_loss.py: the same `_FusedHeadLoss.apply(hidden,
weight, target, denominator, compute_dtype, chunk_cols, want_grad)` returning `(loss, token_loss,
entropy, correct)`, the same `fused_head_loss(...) -> (loss, step)`, `head_metrics_from_logits`,
the batch packing and the two patches (Qwen2ForCausalLM.forward, TRL's SFTTrainer.compute_loss).
What runs underneath is different: instead of a cuBLAS GEMM plus a Triton row kernel per 8192
column chunk (solution/lm_head_loss.py:213-224), three sm_100a kernels per chunk from
libsoup_b200 (a tcgen05 GEMM with the softmax statistics in its epilogue, a row merge, a second
tcgen05 GEMM for the hidden-state gradient), see csrc/lmhead.cu. The arithmetic contract is the
reference's: fp16 operands, fp32 statistics, the gradient accumulated at GRAD_SCALE = 1024 against
the running log-sum-exp, the label's -1 restored at the end.
"""

import functools
from types import SimpleNamespace

import torch

from . import _lib
from .embedding import shrink_tied_embedding

IGNORE_INDEX = -100
GRAD_SCALE = 1024.0
TILE_COLS = 256  # vocabulary columns per GEMM tile; chunks are whole tiles
_REQUEST_ATTR = "_fused_head_request"
_STEP_ATTR = "_fused_head_step"
try:  # the trainer attribute Soup's rewind recorder reads when a step has no logits
    from soup_cli.utils.stream_loss_chunk import STEP_ATTR as SOUP_STEP_ATTR
except Exception:  # noqa: BLE001 - Soup missing: same name as in 0.77.0
    SOUP_STEP_ATTR = "_soup_chunked_step"


def head_compute_dtype(hidden, weight):
    """The dtype `F.linear(hidden, weight)` computes in: the autocast dtype when autocast is on,
    else the common dtype; None when the two differ and nothing would cast them
    (solution/lm_head_loss.py:175-184)."""
    try:
        enabled, dtype = torch.is_autocast_enabled("cuda"), torch.get_autocast_dtype("cuda")
    except (TypeError, AttributeError):
        enabled, dtype = torch.is_autocast_enabled(), torch.get_autocast_gpu_dtype()
    if enabled:
        return dtype
    return weight.dtype if hidden.dtype == weight.dtype else None


def shift_labels_left(labels):
    """Position t is scored against token t + 1, the last position against nothing."""
    return torch.nn.functional.pad(labels, (0, 1), value=IGNORE_INDEX)[..., 1:]


def _chunk_tiles(chunk_cols):
    if chunk_cols is None:
        return 0  # the library picks the chunk that fills whole waves of SMs
    return max(1, -(-int(chunk_cols) // TILE_COLS))


class HeadState:
    """Per-row state of one pass over a vocabulary range (fp32 / int32, all [n]). (run_max,
    run_sum, run_dot) mean mass = run_sum * e^run_max and dot mass = run_dot * e^run_max; best /
    best_val are the index and value of the largest logit; grad_ref is the log-sum-exp the
    range's raw gradient is relative to."""

    __slots__ = ("run_max", "run_sum", "run_dot", "best", "best_val", "label_logit", "grad_ref")

    def __init__(self, n, device):
        f32 = torch.float32
        self.run_max = torch.empty(n, dtype=f32, device=device)
        self.run_sum = torch.empty(n, dtype=f32, device=device)
        self.run_dot = torch.empty(n, dtype=f32, device=device)
        self.best = torch.empty(n, dtype=torch.int32, device=device)
        self.best_val = torch.empty(n, dtype=f32, device=device)
        self.label_logit = torch.empty(n, dtype=f32, device=device)
        self.grad_ref = torch.empty(n, dtype=f32, device=device)

    def tensors(self):
        return (self.run_max, self.run_sum, self.run_dot, self.best, self.best_val,
                self.label_logit, self.grad_ref)

    def lse(self):
        return self.run_max + torch.log(self.run_sum)


_BF16_COPIES = {}  # id(weight) -> (weakref, data_ptr, version, bf16 copy)


def bf16_copy_of_weight(w16):
    """The head weight rounded to bf16, made once per (frozen) weight and kept until the weight
    changes or dies. The gradient GEMM multiplies bf16 probabilities with it: the tensor core
    takes one element format for both operands."""
    import weakref

    key = id(w16)
    hit = _BF16_COPIES.get(key)
    if (hit is not None and hit[0]() is w16 and hit[1] == w16.data_ptr()
            and hit[2] == w16._version):
        return hit[3]
    copy = w16.detach().to(torch.bfloat16).contiguous()
    try:
        ref = weakref.ref(w16, lambda _r, k=key: _BF16_COPIES.pop(k, None))
    except TypeError:
        return copy
    _BF16_COPIES[key] = (ref, w16.data_ptr(), w16._version, copy)
    return copy


def head_partial(h16, w16, target, col_offset=0, chunk_cols=None, want_grad=True, w_bf16=None):
    """One pass of the fused head over the columns of `w16` (a shard of the head weight whose
    first row is vocabulary index `col_offset`). Returns (state, grad_raw): the per-row state of
    this range and, with `want_grad`, the raw fp32 [n, hidden] gradient sum_v exp(z_v -
    state.grad_ref) W[v] over the range's columns except the label's; `head_finish` completes
    it."""
    _lib.require_cuda(h16, w16, target)
    if h16.dtype != torch.float16 or w16.dtype != torch.float16:
        raise TypeError("the fused head computes in float16")
    n, hidden = h16.shape
    vocab = w16.shape[0]
    if w16.shape[1] != hidden:
        raise ValueError(f"hidden {hidden} does not match head weight {tuple(w16.shape)}")
    h16, w16 = h16.contiguous(), w16.contiguous()
    target = target.contiguous()
    if target.dtype != torch.int64:
        target = target.to(torch.int64)
    dev = h16.device
    state = HeadState(n, dev)
    grad_raw = torch.empty((n, hidden), dtype=torch.float32, device=dev) if want_grad else None
    if n == 0 or vocab == 0:  # an empty shard contributes nothing: max -inf, sums 0, gradient 0
        for t in state.tensors():
            t.zero_()
        state.run_max.fill_(float("-inf"))
        state.best_val.fill_(float("-inf"))
        if grad_raw is not None:
            grad_raw.zero_()
        return state, grad_raw
    tiles = _chunk_tiles(chunk_cols)
    nbytes = _lib.lib().soup_lmhead_workspace_bytes(n, hidden, vocab, tiles)
    workspace = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    if want_grad and w_bf16 is None:
        w_bf16 = bf16_copy_of_weight(w16)
    _lib.call("soup_lmhead_ce", _lib.ptr(h16), _lib.ptr(w16),
              _lib.ptr(w_bf16) if want_grad else None, _lib.ptr(target),
              *(_lib.ptr(t) for t in state.tensors()), _lib.ptr(grad_raw), _lib.ptr(workspace),
              nbytes, n, hidden, vocab, int(col_offset), tiles, int(bool(want_grad)),
              _lib.stream_of(h16))
    return state, grad_raw


def head_finish(state, target, w16, grad_raw=None, col_offset=0, grad_ref=None,
                want_metrics=True):
    """Turns a (merged) state into token_loss / entropy / correct and completes `grad_raw` in
    place: GRAD_SCALE * (exp(grad_ref - lse) * grad_raw + (p_label - 1) * W[label]), the label
    term where the label falls in `w16`'s range. `grad_ref` is the array of the state that
    `head_partial` returned together with `grad_raw` (default: `state.grad_ref`)."""
    n = target.numel()
    dev = target.device
    token_loss = entropy = correct = None
    if want_metrics:
        token_loss = torch.empty(n, dtype=torch.float32, device=dev)
        entropy = torch.empty(n, dtype=torch.float32, device=dev)
        correct = torch.empty(n, dtype=torch.int32, device=dev)
    if grad_ref is None:
        grad_ref = state.grad_ref
    if n:
        _lib.call("soup_lmhead_finish", _lib.ptr(state.run_max), _lib.ptr(state.run_sum),
                  _lib.ptr(state.run_dot), _lib.ptr(state.best), _lib.ptr(state.label_logit),
                  _lib.ptr(grad_ref), _lib.ptr(target), _lib.ptr(w16), _lib.ptr(token_loss),
                  _lib.ptr(entropy), _lib.ptr(correct), _lib.ptr(grad_raw), n, w16.shape[1],
                  w16.shape[0], int(col_offset), _lib.stream_of(target))
    return token_loss, entropy, correct


class _FusedHeadLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, target, denominator, compute_dtype, chunk_cols, want_grad):
        if compute_dtype != torch.float16:
            raise TypeError(f"the fused head computes in float16, not {compute_dtype}")
        shape = hidden.shape
        h2 = hidden.reshape(-1, shape[-1])
        tgt = target.reshape(-1).contiguous().to(torch.int64)
        h_low = h2.to(compute_dtype)
        w_low = weight.detach().to(compute_dtype)
        # cached on the weight object itself (detach() makes a new tensor object every call)
        w_bf16 = bf16_copy_of_weight(weight) if want_grad else None
        state, grad_raw = head_partial(h_low, w_low, tgt, 0, chunk_cols, want_grad, w_bf16)
        token_loss, entropy, correct = head_finish(state, tgt, w_low, grad_raw)
        loss = token_loss.sum() / denominator
        ctx.shape, ctx.hidden_dtype, ctx.denominator = shape, hidden.dtype, denominator
        if want_grad:
            ctx.save_for_backward(grad_raw)
        ctx.want_grad = want_grad
        token_loss, entropy, correct = (token_loss.view(shape[:-1]), entropy.view(shape[:-1]),
                                        correct.view(shape[:-1]))
        ctx.mark_non_differentiable(token_loss, entropy, correct)
        return loss, token_loss, entropy, correct

    @staticmethod
    def backward(ctx, grad_loss, _token_loss, _entropy, _correct):
        if not ctx.want_grad:
            return (None,) * 7
        (grad_raw,) = ctx.saved_tensors
        scale = (grad_loss.float() / (ctx.denominator * GRAD_SCALE)).reshape(1).contiguous()
        grad = torch.empty(grad_raw.shape, dtype=ctx.hidden_dtype, device=grad_raw.device)
        _lib.call("soup_lmhead_grad_scale", _lib.ptr(grad_raw), _lib.ptr(grad), _lib.ptr(scale),
                  grad_raw.numel(), _lib.dtype_code(ctx.hidden_dtype), _lib.stream_of(grad_raw))
        return grad.view(ctx.shape), None, None, None, None, None, None


def fused_head_loss(hidden, weight, labels, num_items_in_batch=None, chunk_cols=None,
                    target=None):
    """ForCausalLMLoss(linear(hidden, weight), labels) and the per-token terms the trainer's
    metrics need, without materialising the logits. `weight` must be frozen: the gradient goes to
    `hidden` only. Returns (loss, step) with step.token_loss and step.token_entropy of shape
    [batch, seq] (fp32), step.correct and step.labelled (counts). `target` (the labels already
    shifted, same leading shape as `hidden`) replaces `labels` when given."""
    if target is None:
        target = shift_labels_left(labels)
    target = target.to(hidden.device)
    labelled = (target != IGNORE_INDEX).sum()
    if num_items_in_batch is None:
        denominator = labelled
    elif torch.is_tensor(num_items_in_batch):
        denominator = num_items_in_batch.to(hidden.device)
    else:
        denominator = num_items_in_batch
    compute_dtype = head_compute_dtype(hidden, weight)
    if compute_dtype is None:
        raise TypeError(f"hidden {hidden.dtype} and head {weight.dtype} differ outside autocast")
    want_grad = torch.is_grad_enabled() and hidden.requires_grad
    loss, token_loss, entropy, correct = _FusedHeadLoss.apply(
        hidden, weight, target, denominator, compute_dtype, chunk_cols, want_grad)
    step = SimpleNamespace(token_loss=token_loss, token_entropy=entropy,
                           correct=correct.sum(), labelled=labelled)
    return loss, step


@torch.no_grad()
def head_metrics_from_logits(logits, labels):
    """The same per-token terms from logits that were built anyway (fallback path of the
    reference, solution/lm_head_loss.py:285-297): one warp per row over the full logits."""
    target = shift_labels_left(labels).to(logits.device).reshape(-1).contiguous().to(torch.int64)
    flat = logits.reshape(-1, logits.shape[-1]).contiguous()
    _lib.require_cuda(flat)
    n = flat.shape[0]
    token_loss = torch.empty(n, dtype=torch.float32, device=logits.device)
    entropy = torch.empty_like(token_loss)
    correct = torch.empty(n, dtype=torch.int32, device=logits.device)
    if n:
        _lib.call("soup_xent_rows", _lib.ptr(flat), _lib.ptr(target), _lib.ptr(token_loss),
                  _lib.ptr(entropy), _lib.ptr(correct), n, flat.shape[1], flat.stride(0),
                  _lib.dtype_code(flat.dtype), _lib.stream_of(flat))
    shape = logits.shape[:-1]
    return SimpleNamespace(token_loss=token_loss.view(shape), token_entropy=entropy.view(shape),
                           correct=correct.sum(), labelled=(target != IGNORE_INDEX).sum())


def _pack_batch(lm, kwargs, labels):
    """The real (non-pad) tokens of a padded batch as one row [1, N] with per-token position ids,
    a [1, 1, N, N] mask (same batch row, key column not after the query's) and the shifted
    targets; None to run the batch as it is (solution/lm_head_loss.py:300-336)."""
    ids, mask = kwargs.get("input_ids"), kwargs.get("attention_mask")
    head = lm.lm_head
    if (not isinstance(ids, torch.Tensor) or ids.dim() != 2 or not ids.is_cuda
            or not isinstance(mask, torch.Tensor) or mask.shape != ids.shape
            or kwargs.get("inputs_embeds") is not None or kwargs.get("past_key_values") is not None
            or labels.shape != ids.shape
            or type(head) is not torch.nn.Linear or head.bias is not None
            or head.weight.requires_grad
            or getattr(lm.config, "_attn_implementation", None) != "sdpa"
            or getattr(lm.config, "use_sliding_window", False)):
        return None
    return pack_tokens(ids, mask, labels, kwargs.get("position_ids"))


def pack_tokens(ids, mask, labels, position_ids=None):
    """The device-independent part of `_pack_batch` (also used to build synthetic packed rows)."""
    B, T = ids.shape
    keep = mask.reshape(-1) != 0
    index = keep.nonzero().squeeze(1)
    n = index.numel()
    if n == 0 or n == B * T:
        return None
    pos = position_ids
    if isinstance(pos, torch.Tensor) and pos.shape == ids.shape:
        pos = pos.reshape(-1)[index]
    elif pos is None:
        pos = index % T
    else:
        return None
    row, col = index // T, index % T
    allowed = (row[:, None] == row[None, :]) & (col[None, :] <= col[:, None])
    target = shift_labels_left(labels.to(ids.device)).reshape(-1)[index]
    return SimpleNamespace(B=B, T=T, index=index, ids=ids.reshape(-1)[index][None],
                           pos=pos[None], mask=allowed[None, None], target=target[None])


def _packed_forward(lm, kwargs, packed):
    """The fused training forward on the packed real tokens; the per-token terms go back to their
    [batch, seq] places (zeros at pads, which every consumer masks out)."""
    from transformers.modeling_outputs import CausalLMOutputWithPast

    rest = {k: v for k, v in kwargs.items()
            if k not in ("input_ids", "attention_mask", "position_ids")}
    outputs = lm.model(input_ids=packed.ids, attention_mask=packed.mask,
                       position_ids=packed.pos, **rest)
    hidden = outputs.last_hidden_state
    loss, step = fused_head_loss(hidden, lm.lm_head.weight, None,
                                 num_items_in_batch=kwargs.get("num_items_in_batch"),
                                 target=packed.target)
    full = packed.B * packed.T

    def spread(values):
        out = torch.zeros(full, dtype=values.dtype, device=values.device)
        out[packed.index] = values.reshape(-1)
        return out.view(packed.B, packed.T)

    step = SimpleNamespace(token_loss=spread(step.token_loss),
                           token_entropy=spread(step.token_entropy),
                           correct=step.correct, labelled=step.labelled)
    lm.__dict__[_STEP_ATTR] = step
    return CausalLMOutputWithPast(loss=loss, logits=None)


def _head_is_fusable(head):
    return (type(head) is torch.nn.Linear and head.bias is None
            and not head.weight.requires_grad)


def patch_qwen2_causal_lm_head():
    """Qwen2ForCausalLM.forward: when the trainer has asked for it (and only then), build the loss
    from the hidden states with the fused head and return no logits."""
    from transformers.modeling_outputs import CausalLMOutputWithPast
    from transformers.models.qwen2 import modeling_qwen2

    cls = getattr(modeling_qwen2, "Qwen2ForCausalLM", None)
    if cls is None or getattr(cls.forward, "_fused_head", False):
        return
    original = cls.forward

    @functools.wraps(original)  # the trainer reads the forward's signature
    def forward(self, *args, **kwargs):
        asked = self.__dict__.pop(_REQUEST_ATTR, False)
        labels = kwargs.get("labels")
        keep = kwargs.get("logits_to_keep", 0)
        if (not asked or args or labels is None or not isinstance(keep, int) or keep != 0
                or "shift_labels" in kwargs or kwargs.get("return_dict") is False):
            return original(self, *args, **kwargs)
        kwargs.pop("labels")
        kwargs.pop("logits_to_keep", None)
        shrink_tied_embedding(self)
        packed = _pack_batch(self, kwargs, labels)
        if packed is not None:
            return _packed_forward(self, kwargs, packed)
        outputs = self.model(**kwargs)
        hidden = outputs.last_hidden_state
        head = self.lm_head
        if (not _head_is_fusable(head) or not hidden.is_cuda
                or head_compute_dtype(hidden, head.weight) != torch.float16):
            logits = head(hidden)  # what the original forward does from here on
            loss = self.loss_function(logits=logits, labels=labels,
                                      vocab_size=self.config.vocab_size, **kwargs)
            return CausalLMOutputWithPast(loss=loss, logits=logits,
                                          past_key_values=outputs.past_key_values,
                                          hidden_states=outputs.hidden_states,
                                          attentions=outputs.attentions)
        loss, step = fused_head_loss(hidden, head.weight, labels,
                                     num_items_in_batch=kwargs.get("num_items_in_batch"))
        self.__dict__[_STEP_ATTR] = step
        return CausalLMOutputWithPast(loss=loss, logits=None,
                                      past_key_values=outputs.past_key_values,
                                      hidden_states=outputs.hidden_states,
                                      attentions=outputs.attentions)

    forward._fused_head = True
    cls.forward = forward


def _causal_lm(model):
    while isinstance(getattr(model, "module", None), torch.nn.Module):
        model = model.module
    get_base = getattr(model, "get_base_model", None)
    return get_base() if callable(get_base) else model


def _fused_target(trainer, model, inputs):
    """The causal LM to run with the fused head, or None to keep TRL's own path."""
    if (not isinstance(model, torch.nn.Module) or not getattr(trainer.model, "training", False)
            or isinstance(model, torch.nn.DataParallel)
            or getattr(trainer.args, "n_gpu", 1) > 1
            or not isinstance(inputs, dict) or "labels" not in inputs
            or "shift_labels" in inputs
            or getattr(trainer.args, "use_liger_kernel", False)
            or getattr(trainer, "num_virtual_tokens", 0)
            or getattr(trainer, "aux_loss_enabled", False)
            or getattr(trainer, "compute_loss_func", None) is not None
            or getattr(trainer, "label_smoother", None) is not None
            or not hasattr(trainer, "_metrics")):
        return None
    lm = _causal_lm(model)
    if not getattr(type(lm).forward, "_fused_head", False):
        return None
    head = lm.get_output_embeddings()
    if (not _head_is_fusable(head) or not head.weight.is_cuda
            or getattr(lm.config, "final_logit_softcapping", None) is not None):
        return None
    return lm


def _log_trl_metrics(trainer, mode, inputs, step):
    """entropy, num_tokens and mean_token_accuracy as SFTTrainer.compute_loss logs them from the
    logits: same masks, same gathers, same order of reductions
    (solution/lm_head_loss.py:449-472)."""
    gather = trainer.accelerator.gather_for_metrics
    if "attention_mask" in inputs:
        mask = inputs["attention_mask"]
        entropy = torch.sum(step.token_entropy * mask) / mask.sum()
    elif "position_ids" in inputs:
        entropy = torch.mean(step.token_entropy)
    else:
        raise ValueError("Expected 'attention_mask' or 'position_ids' in inputs.")
    trainer._metrics[mode]["entropy"].append(gather(entropy).mean().item())
    if mode == "train":
        if "attention_mask" in inputs:
            num_tokens = gather(inputs["attention_mask"].sum()).sum().item()
        else:
            local = torch.tensor(inputs["position_ids"].size(1),
                                 device=inputs["position_ids"].device)
            num_tokens = gather(local).sum().item()
        trainer._total_train_tokens += num_tokens
    trainer._metrics[mode]["num_tokens"] = [trainer._total_train_tokens]
    correct, total = gather(step.correct), gather(step.labelled)
    total_sum = total.sum()
    accuracy = (correct.sum() / total_sum).item() if total_sum > 0 else 0.0
    trainer._metrics[mode]["mean_token_accuracy"].append(accuracy)


def patch_sft_compute_loss():
    """TRL's SFTTrainer.compute_loss, for a training step of a patched causal LM: ask the model for
    the fused head, log TRL's metrics from the per-token terms and leave the per-token losses where
    Soup's rewind recorder looks for them. Without TRL there is nothing to patch."""
    try:
        from trl.trainer import sft_trainer as trl_sft
    except Exception:  # noqa: BLE001
        return
    cls = trl_sft.SFTTrainer
    if getattr(cls.compute_loss, "_fused_head", False):
        return
    original = cls.compute_loss

    def compute_loss(self, model, inputs, return_outputs=False, num_items_in_batch=None):
        lm = _fused_target(self, model, inputs)
        if lm is None:
            setattr(self, SOUP_STEP_ATTR, None)
            return original(self, model, inputs, return_outputs=return_outputs,
                            num_items_in_batch=num_items_in_batch)
        inputs.pop("_prediction_loss_only", None)
        labels = inputs["labels"]
        inputs["use_cache"] = False
        setattr(self, SOUP_STEP_ATTR, None)
        lm.__dict__[_REQUEST_ATTR] = True
        try:
            loss, outputs = super(cls, self).compute_loss(
                model, inputs, return_outputs=True, num_items_in_batch=num_items_in_batch)
        finally:
            lm.__dict__.pop(_REQUEST_ATTR, None)
        step = lm.__dict__.pop(_STEP_ATTR, None)
        if step is None:  # the forward built the logits after all
            step = head_metrics_from_logits(outputs.logits, labels)
        _log_trl_metrics(self, "train", inputs, step)
        setattr(self, SOUP_STEP_ATTR, SimpleNamespace(token_loss=step.token_loss))
        return (loss, outputs) if return_outputs else loss

    compute_loss._fused_head = True
    cls.compute_loss = compute_loss


def patch_fused_head_loss():
    patch_qwen2_causal_lm_head()
    patch_sft_compute_loss()
