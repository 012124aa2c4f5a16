"""Oracle of the packed row's attention: causal attention inside every segment, written out with
explicit loops over segments and heads in float64, forward and backward, with the row
log-sum-exps. Test infrastructure only (tests, smoke, the bench's CPU leg): nothing shipped imports
it.

What it restates: transformers' sdpa path as the reference's own attention test states it
(tests_local/test_attention.py:23-32: repeat_kv, boolean mask "same batch row and key not after the
query", output [B, T, H, D]) on the packed layout of solution/lm_head_loss.py:300-337, i.e. one
row of N tokens whose batch rows are the segments. The formulas of the backward are those of the
reference's unused Triton kernels (solution/attention.py:75-168): P = exp(scale S - lse),
D = rowsum(dO o O), dS = P o (dP - D), dQ = scale dS K, dK = scale dS^T Q, dV = P^T dO.

Pinned by tests/test_oracle_golden.py against torch's scaled_dot_product_attention on the CPU in
float64 with the [N, N] mask (a library implementation of the same definition), values and all
three gradients.
"""

import torch


def segment_attention(q, k, v, cu_rows, scale=None):
    """q [N, Hq, D], k and v [N, Hk, D], cu_rows [S + 1] -> (out [N, Hq, D] float64, lse [Hq, N]
    float64: log(sum_j exp(scale * q_i . k_j)) over the visible j). Tokens outside every segment
    get zeros."""
    n, hq, d = q.shape
    hk = k.shape[1]
    group = hq // hk
    scale = d ** -0.5 if scale is None else scale
    q, k, v = q.double(), k.double(), v.double()
    out = torch.zeros(n, hq, d, dtype=torch.float64)
    lse = torch.zeros(hq, n, dtype=torch.float64)
    bounds = [int(x) for x in cu_rows]
    for b, e in zip(bounds, bounds[1:]):
        if e <= b:
            continue
        visible = torch.ones(e - b, e - b, dtype=torch.bool).tril()
        for h in range(hq):
            s = (q[b:e, h] @ k[b:e, h // group].t()) * scale
            s = s.masked_fill(~visible, float("-inf"))
            row_lse = torch.logsumexp(s, dim=-1)
            out[b:e, h] = torch.exp(s - row_lse[:, None]) @ v[b:e, h // group]
            lse[h, b:e] = row_lse
    return out, lse


def segment_attention_backward(q, k, v, cu_rows, d_out, scale=None):
    """(dq [N, Hq, D], dk [N, Hk, D], dv [N, Hk, D]) in float64 from the explicit formulas (the
    key/value gradients summed over the query heads of a group)."""
    n, hq, d = q.shape
    hk = k.shape[1]
    group = hq // hk
    scale = d ** -0.5 if scale is None else scale
    q, k, v, d_out = q.double(), k.double(), v.double(), d_out.double()
    out, lse = segment_attention(q, k, v, cu_rows, scale)
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    bounds = [int(x) for x in cu_rows]
    for b, e in zip(bounds, bounds[1:]):
        if e <= b:
            continue
        visible = torch.ones(e - b, e - b, dtype=torch.bool).tril()
        for h in range(hq):
            g = h // group
            s = (q[b:e, h] @ k[b:e, g].t()) * scale
            p = torch.exp(s - lse[h, b:e, None]).masked_fill(~visible, 0.0)
            delta = (d_out[b:e, h] * out[b:e, h]).sum(-1, keepdim=True)
            d_p = d_out[b:e, h] @ v[b:e, g].t()
            d_s = p * (d_p - delta)
            dq[b:e, h] = scale * (d_s @ k[b:e, g])
            dk[b:e, g] += scale * (d_s.t() @ q[b:e, h])
            dv[b:e, g] += p.t() @ d_out[b:e, h]
    return dq, dk, dv
