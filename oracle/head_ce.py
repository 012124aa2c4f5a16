"""LM head + cross-entropy oracle: fp32 matmul + log_softmax, as benchmark config 1 prescribes and
as the reference's own test computes its expectation (tests_local/test_lm_head_loss.py:66-86, with
the autocast removed so that everything is fp32)."""

import torch
import torch.nn.functional as F

IGNORE = -100


def head_ce(hidden, weight, target, denominator=None, want_grad=True, grad_scale=1.0):
    """hidden [n, H], weight [V, H] (any float dtype, used as fp32), target [n] int64 (already
    shifted; -100 = ignore). Returns dict(loss, token_loss [n], entropy [n], correct [n] int32,
    lse [n], dhidden [n, H] fp32 = d(loss * grad_scale)/d hidden or None)."""
    h = hidden.detach().float().clone().requires_grad_(want_grad)
    w = weight.detach().float()
    logits = h @ w.t()
    logp = F.log_softmax(logits, dim=-1)
    labelled = target != IGNORE
    safe = target.clamp(min=0)
    nll = -logp.gather(1, safe[:, None]).squeeze(1)
    token_loss = torch.where(labelled, nll, torch.zeros_like(nll))
    denom = labelled.sum() if denominator is None else denominator
    loss = token_loss.sum() / denom
    dh = None
    if want_grad:
        (dh,) = torch.autograd.grad(loss * grad_scale, h)
    with torch.no_grad():
        entropy = -(logp.exp() * logp).sum(-1)  # tests_local/test_lm_head_loss.py:31-37
        correct = (labelled & (logits.argmax(-1) == target)).to(torch.int32)
        lse = torch.logsumexp(logits, -1)
    return dict(loss=loss.detach(), token_loss=token_loss.detach(), entropy=entropy,
                correct=correct, lse=lse, dhidden=dh)


def head_ce_chunked(hidden, weight, target, chunk_cols, grad_scale=1024.0):
    """The reference's own chunked algorithm (solution/lm_head_loss.py:194-245 with the kernel of
    :108-160) restated in fp32 torch: running (max, sum, dot, argmax, label logit) across column
    chunks, per-chunk softmax against the running lse with the label's -1 in its chunk, rescale by
    exp(lse_before - lse_after), label fix-up at the end. Returns the same dict as head_ce with
    dhidden = grad_raw / grad_scale / denominator."""
    h = hidden.detach().float()
    w = weight.detach().float()
    n, vocab = h.shape[0], w.shape[0]
    run_max = torch.full((n,), float("-inf"))
    run_sum = torch.zeros(n)
    run_dot = torch.zeros(n)
    best = torch.zeros(n, dtype=torch.int64)
    label_logit = torch.zeros(n)
    label_lse = torch.zeros(n)
    grad_raw = torch.zeros(n, h.shape[1])
    labelled = target != IGNORE
    rows = torch.arange(n)
    for c0 in range(0, vocab, chunk_cols):
        c1 = min(vocab, c0 + chunk_cols)
        z = h @ w[c0:c1].t()
        prev_lse = run_max + torch.log(run_sum)
        tile_max, tile_arg = z.max(1)
        best = torch.where(tile_max > run_max, tile_arg + c0, best)
        new_max = torch.maximum(run_max, tile_max)
        rescale = torch.exp(run_max - new_max)
        e = torch.exp(z - new_max[:, None])
        run_sum = run_sum * rescale + e.sum(1)
        run_dot = run_dot * rescale + (e * z).sum(1)
        run_max = new_max
        local = target - c0
        hit = labelled & (local >= 0) & (local < c1 - c0)
        label_logit = torch.where(hit, z[rows, local.clamp(0, c1 - c0 - 1)], label_logit)
        lse = run_max + torch.log(run_sum)
        factor = torch.exp(prev_lse - lse)
        label_lse = torch.where(hit, lse, label_lse)
        prob = torch.exp(z - lse[:, None])
        prob[rows[hit], local[hit]] -= 1.0
        prob = torch.where(labelled[:, None], prob * grad_scale, torch.zeros_like(prob))
        grad_raw = grad_raw * factor[:, None] + prob @ w[c0:c1]
    lse = run_max + torch.log(run_sum)
    token_loss = torch.where(labelled, lse - label_logit, torch.zeros_like(lse))
    entropy = lse - run_dot / run_sum
    correct = (labelled & (best == target)).to(torch.int32)
    missing = torch.where(labelled, 1.0 - torch.exp(label_lse - lse), torch.zeros_like(lse)) * grad_scale
    grad_raw = grad_raw - w[target.clamp(min=0)] * missing[:, None]
    denom = labelled.sum()
    return dict(loss=token_loss.sum() / denom, token_loss=token_loss, entropy=entropy,
                correct=correct, lse=lse, dhidden=grad_raw / (grad_scale * denom))
