"""CPU restatement of the vocabulary-parallel bookkeeping (test infrastructure): per-shard state
and gradient in fp32 torch, the merge rule, and the per-shard finish. The merge is the
chunk-to-chunk carry of solution/lm_head_loss.py:119-145 applied across shards instead of chunks;
the finish is :225-237 with the extra exp(lse_shard - lse) factor."""

import torch

IGNORE = -100
GRAD_SCALE = 1024.0


def shard_partial(hidden, w_shard, target, col_offset):
    """State of one shard and its gradient at GRAD_SCALE against the shard's own lse, with the
    label's -1 in place where the label falls in the shard."""
    h, w = hidden.float(), w_shard.float()
    n = h.shape[0]
    if w.shape[0] == 0:
        z = torch.zeros(n)
        return dict(run_max=torch.full((n,), float("-inf")), run_sum=z.clone(), run_dot=z.clone(),
                    best=torch.zeros(n, dtype=torch.int64), label_logit=z.clone(),
                    label_lse=z.clone(), grad_raw=torch.zeros(n, h.shape[1]))
    z = h @ w.t()
    run_max, arg = z.max(1)
    e = torch.exp(z - run_max[:, None])
    run_sum, run_dot = e.sum(1), (e * z).sum(1)
    lse = run_max + torch.log(run_sum)
    labelled = target != IGNORE
    local = target - col_offset
    hit = labelled & (local >= 0) & (local < w.shape[0])
    rows = torch.arange(n)
    label_logit = torch.where(hit, z[rows, local.clamp(0, w.shape[0] - 1)], torch.zeros(n))
    label_lse = torch.where(hit, lse, torch.zeros(n))
    p = torch.exp(z - lse[:, None])
    p[rows[hit], local[hit]] -= 1.0
    p = torch.where(labelled[:, None], p * GRAD_SCALE, torch.zeros_like(p))
    return dict(run_max=run_max, run_sum=run_sum, run_dot=run_dot, best=arg + col_offset,
                label_logit=label_logit, label_lse=label_lse, grad_raw=p @ w)


def merge(parts, target, bounds):
    """parts: list of shard states in ascending vocabulary order -> merged state + lse."""
    n = target.numel()
    m = torch.full((n,), float("-inf"))
    best = torch.zeros(n, dtype=torch.int64)
    for p in parts:
        better = p["run_max"] > m
        best = torch.where(better, p["best"], best)
        m = torch.maximum(m, p["run_max"])
    s, d = torch.zeros(n), torch.zeros(n)
    ll, lls = torch.zeros(n), torch.zeros(n)
    for r, p in enumerate(parts):
        wgt = torch.exp(p["run_max"] - m)
        s, d = s + p["run_sum"] * wgt, d + p["run_dot"] * wgt
        own = (target != IGNORE) & (target >= bounds[r]) & (target < bounds[r + 1])
        ll = torch.where(own, p["label_logit"], ll)
        lls = torch.where(own, p["label_lse"], lls)
    return dict(run_max=m, run_sum=s, run_dot=d, best=best, label_logit=ll, label_lse=lls,
                lse=m + torch.log(s))


def finish(merged, part, w_shard, target, col_offset):
    """(token_loss, entropy, correct, this shard's completed grad_raw)."""
    lse = merged["lse"]
    labelled = target != IGNORE
    token_loss = torch.where(labelled, lse - merged["label_logit"], torch.zeros_like(lse))
    entropy = lse - merged["run_dot"] / merged["run_sum"]
    correct = (labelled & (merged["best"] == target)).to(torch.int32)
    local_lse = part["run_max"] + torch.log(part["run_sum"])
    g = part["grad_raw"] * torch.exp(local_lse - lse)[:, None]
    local = target - col_offset
    mine = labelled & (local >= 0) & (local < w_shard.shape[0])
    missing = torch.where(mine, 1.0 - torch.exp(merged["label_lse"] - lse), torch.zeros_like(lse))
    if w_shard.shape[0]:
        g = g - w_shard.float()[local.clamp(0, w_shard.shape[0] - 1)] * (missing * GRAD_SCALE)[:, None]
    return token_loss, entropy, correct, g
