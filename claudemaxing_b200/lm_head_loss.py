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

import dataclasses

import torch

from . import _lib

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


def head_partial(h16, w16, target, col_offset=0, chunk_cols=None, want_grad=True, w_bf16=None,
                 grad_out=None):
    """One pass of the fused head over the columns of `w16` (a shard of the head weight whose
    first row is vocabulary index `col_offset`). Returns (state, grad_raw): the per-row state of
    this range and, with `want_grad`, the raw fp32 [n, hidden] gradient sum_v exp(z_v -
    state.grad_ref) W[v] over the range's columns except the label's; `head_finish` completes
    it. `grad_out` (contiguous fp32 [n, hidden]) is used for the gradient instead of a new tensor."""
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
    grad_raw = None
    if want_grad:
        grad_raw = grad_out
        if grad_raw is None:
            grad_raw = torch.empty((n, hidden), dtype=torch.float32, device=dev)
        elif (grad_raw.shape != (n, hidden) or grad_raw.dtype != torch.float32
              or not grad_raw.is_contiguous()):
            raise ValueError("grad_out must be a contiguous fp32 [n, hidden] tensor")
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
                want_metrics=True, grad_out=None):
    """Turns a (merged) state into token_loss / entropy / correct and completes `grad_raw` in
    place: GRAD_SCALE * (exp(grad_ref - lse) * grad_raw + (p_label - 1) * W[label]), the label
    term where the label falls in `w16`'s range. `grad_ref` is the array of the state that
    `head_partial` returned together with `grad_raw` (default: `state.grad_ref`). With `grad_out`
    (same shape, any floating dtype) the completed gradient is written there, rounded once, and
    `grad_raw` is left as it was."""
    n = target.numel()
    dev = target.device
    token_loss = entropy = correct = None
    if want_metrics:
        token_loss = torch.empty(n, dtype=torch.float32, device=dev)
        entropy = torch.empty(n, dtype=torch.float32, device=dev)
        correct = torch.empty(n, dtype=torch.int32, device=dev)
    if grad_ref is None:
        grad_ref = state.grad_ref
    if n and grad_out is not None:
        _lib.call("soup_lmhead_finish_to", _lib.ptr(state.run_max), _lib.ptr(state.run_sum),
                  _lib.ptr(state.run_dot), _lib.ptr(state.best), _lib.ptr(state.label_logit),
                  _lib.ptr(grad_ref), _lib.ptr(target), _lib.ptr(w16), _lib.ptr(token_loss),
                  _lib.ptr(entropy), _lib.ptr(correct), _lib.ptr(grad_raw), _lib.ptr(grad_out),
                  _lib.dtype_code(grad_out.dtype), n, w16.shape[1], w16.shape[0], int(col_offset),
                  _lib.stream_of(target))
    elif n:
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


@dataclasses.dataclass
class StepTerms:
    """What the trainer's metrics need from a step: per-token loss and entropy `[batch, seq]`
    (fp32, zero at ignored positions), the number of correct argmax predictions and of labelled
    positions (0-d tensors)."""

    token_loss: torch.Tensor
    token_entropy: torch.Tensor
    correct: torch.Tensor
    labelled: torch.Tensor


def fused_head_loss(hidden, weight, labels, num_items_in_batch=None, chunk_cols=None,
                    target=None):
    """ForCausalLMLoss(linear(hidden, weight), labels) plus the per-token terms the trainer's
    metrics need, without the logits. `weight` must be frozen: only `hidden` gets a gradient.
    Returns (loss, StepTerms). `target` (labels already shifted, same leading shape as `hidden`)
    replaces `labels` when given; `num_items_in_batch` (number or tensor) replaces the count of
    labelled positions as the divisor of the loss."""
    dtype = head_compute_dtype(hidden, weight)
    if dtype is None:
        raise TypeError(f"hidden {hidden.dtype} and head {weight.dtype} differ outside autocast")
    scored = (shift_labels_left(labels) if target is None else target).to(hidden.device)
    n_scored = scored.ne(IGNORE_INDEX).sum()
    divisor = n_scored
    if num_items_in_batch is not None:
        divisor = (num_items_in_batch.to(hidden.device) if torch.is_tensor(num_items_in_batch)
                   else num_items_in_batch)
    needs_grad = hidden.requires_grad and torch.is_grad_enabled()
    loss, per_token, entropy, hits = _FusedHeadLoss.apply(hidden, weight, scored, divisor, dtype,
                                                          chunk_cols, needs_grad)
    return loss, StepTerms(per_token, entropy, hits.sum(), n_scored)


@torch.no_grad()
def head_metrics_from_logits(logits, labels, target=None):
    """StepTerms from logits that exist anyway (the route the reference keeps for steps that end
    up building them, solution/lm_head_loss.py:285-297): one warp per row over the full logits.
    `target` (labels already shifted) replaces `labels` when given."""
    rows = logits.reshape(-1, logits.shape[-1]).contiguous()
    _lib.require_cuda(rows)
    scored = shift_labels_left(labels) if target is None else target
    scored = scored.to(rows.device).reshape(-1).to(torch.int64).contiguous()
    n = rows.shape[0]
    per_token = torch.empty(n, dtype=torch.float32, device=rows.device)
    entropy = torch.empty(n, dtype=torch.float32, device=rows.device)
    hits = torch.empty(n, dtype=torch.int32, device=rows.device)
    if n:
        _lib.call("soup_xent_rows", _lib.ptr(rows), _lib.ptr(scored), _lib.ptr(per_token),
                  _lib.ptr(entropy), _lib.ptr(hits), n, rows.shape[1], rows.stride(0),
                  _lib.dtype_code(rows.dtype), _lib.stream_of(rows))
    lead = logits.shape[:-1]
    return StepTerms(per_token.view(lead), entropy.view(lead), hits.sum(),
                     scored.ne(IGNORE_INDEX).sum())


# The transformers / TRL side lives in trainer_glue.py; its names stay importable from here, where
# the reference keeps them.
from .trainer_glue import (  # noqa: E402,F401
    PackedRow,
    _pack_batch,
    _packed_forward,
    explain_batch_route,
    explain_trainer_route,
    pack_tokens,
    patch_fused_head_loss,
    patch_qwen2_causal_lm_head,
    patch_sft_compute_loss,
)
