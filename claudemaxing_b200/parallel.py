"""Multi-GPU use of the hot path: a vocabulary-parallel LM head and the data-parallel LoRA step.

The reference is single-GPU (its fused head refuses n_gpu > 1, solution/lm_head_loss.py:426-428),
so nothing here replaces reference code; it extends the same arithmetic across ranks.

Vocabulary-parallel head: the weight is split into contiguous ranges of whole 256-column tiles,
rank r owning columns [bounds[r], bounds[r+1]); hidden states and targets are replicated. Each rank
runs `head_partial` on its shard and gets the per-row state (log-sum-exp bookkeeping, sum exp*z,
argmax index and value, label logit) and a raw gradient against its *own* reference lse. One
all-gather of the [6, n] states (24 bytes per row and rank) feeds the merge kernel; the finish
kernel rescales the rank's gradient by exp(lse_rank - lse_global) and restores the label term on
the rank that owns the label; one all-reduce sums the gradients. There is no other exchange.

Data-parallel step: every rank runs the whole step on its own batch; the LoRA gradients
(2.18 M fp32 values for Qwen2.5-1.5B, r = 16 on q/v) travel in one flat all-reduce.
"""

import torch
import torch.distributed as dist

from . import _lib
from .lm_head_loss import TILE_COLS, HeadState, head_finish, head_partial


def shard_bounds(vocab, world, tile=TILE_COLS):
    """world + 1 column indices: contiguous ranges of whole tiles, the first `rem` ranks one tile
    longer, the last range clipped to the vocabulary."""
    tiles = -(-vocab // tile)
    per, rem = divmod(tiles, world)
    bounds, t = [0], 0
    for r in range(world):
        t += per + (1 if r < rem else 0)
        bounds.append(min(t * tile, vocab))
    return bounds


N_FIELDS = 6  # run_max, run_sum, run_dot, best (bits), best_val, label_logit


def pack_state(state):
    """[6, n] fp32 view of a HeadState for one collective (the int32 argmax travels as bits;
    grad_ref stays local: only the rank itself needs it)."""
    return torch.stack([state.run_max, state.run_sum, state.run_dot,
                        state.best.view(torch.float32), state.best_val, state.label_logit])


_BOUNDS_ON_DEVICE = {}


def _bounds_tensor(bounds, device):
    """The shard bounds as an int64 device tensor, made once per (bounds, device): building it from
    the Python list on every call is a pageable host-to-device copy, which makes the host wait for
    everything enqueued before it and so ends the host's run-ahead twice per step."""
    key = (tuple(int(b) for b in bounds), str(device))
    hit = _BOUNDS_ON_DEVICE.get(key)
    if hit is None:
        hit = torch.tensor(key[0], dtype=torch.int64, device=device)
        _BOUNDS_ON_DEVICE[key] = hit
    return hit


def merge_states(gathered, target, bounds):
    """gathered [world, 6, n] (rank order) -> (merged HeadState, merged lse [n])."""
    world, _, n = gathered.shape
    dev = gathered.device
    fields = gathered.permute(1, 0, 2).contiguous()  # [6, world, n]
    merged = HeadState(n, dev)
    lse = torch.empty(n, dtype=torch.float32, device=dev)
    begin = _bounds_tensor(bounds, dev)
    if n:
        _lib.call("soup_lmhead_merge", *(_lib.ptr(fields[i]) for i in range(N_FIELDS)),
                  _lib.ptr(target), _lib.ptr(begin), _lib.ptr(merged.run_max),
                  _lib.ptr(merged.run_sum), _lib.ptr(merged.run_dot), _lib.ptr(merged.best),
                  _lib.ptr(merged.best_val), _lib.ptr(merged.label_logit), _lib.ptr(lse), n,
                  world, _lib.stream_of(target))
    return merged, lse


def _row_block(n, hidden, v_shard, chunk_cols):
    """The row block the kernels use for a shard `v_shard` columns wide (2048 for a wide shard, up
    to 8192 for a narrow one). Host arithmetic only."""
    import ctypes

    from .lm_head_loss import _chunk_tiles

    rows = ctypes.c_int64(2048)
    _lib.lib().soup_lmhead_plan(int(n), int(v_shard), _chunk_tiles(chunk_cols), ctypes.byref(rows),
                                None, None)
    return max(int(rows.value), 1)


def exchange_rows(n, hidden, bounds, chunk_cols=None):
    """Rows per exchange step, the same number on every rank. It is derived from the shard bounds
    (which all ranks hold), never from the local shard: shards differ by one column tile when the
    tiles do not divide evenly, the kernels' row block depends on the tile count (151936 columns
    over 4 ranks: 149 tiles -> 6144 rows, 148 tiles -> 8192), and ranks that walked the rows in
    different block sizes would issue different numbers of collectives and wait for each other
    forever. The widest shard has the smallest row block, so one exchange step is at most one
    pass of the kernels on every rank."""
    widest = max(int(bounds[r + 1]) - int(bounds[r]) for r in range(len(bounds) - 1))
    return _row_block(n, hidden, max(widest, 1), chunk_cols)


def _one_block(h16, w_shard, target, bounds, rank, world, group, want_grad, chunk_cols, w_bf16,
               grad_out):
    """Partial pass, state exchange, merge and finish for one block of rows; the gradient (not yet
    summed over ranks) lands in `grad_out`."""
    state, grad_raw = head_partial(h16, w_shard, target, bounds[rank], chunk_cols, want_grad,
                                   w_bf16, grad_out)
    mine = pack_state(state)
    # concatenated along dim 0: the output layout every backend accepts
    gathered = torch.empty((world * mine.shape[0], mine.shape[1]), dtype=mine.dtype,
                           device=mine.device)
    dist.all_gather_into_tensor(gathered, mine, group=group)
    merged, _ = merge_states(gathered.view(world, *mine.shape), target, bounds)
    terms = head_finish(merged, target, w_shard, grad_raw, bounds[rank], grad_ref=state.grad_ref)
    return terms, grad_raw


def vocab_parallel_head(h16, w_shard, target, bounds, group=None, want_grad=True,
                        reduce_grad=True, chunk_cols=None, w_bf16=None):
    """The fused head with the vocabulary split across the ranks of `group`. `w_shard` is this
    rank's rows [bounds[rank], bounds[rank+1]) of the head weight. Returns dict(token_loss,
    entropy, correct, grad_raw): per-row terms identical on every rank, grad_raw the fp32
    [n, hidden] gradient at GRAD_SCALE, summed over ranks when `reduce_grad`.

    Inputs of more rows than the kernels' row block are walked block by block: a block's gradient
    all-reduce is issued asynchronously and runs beside the GEMMs of the next block (the kernels
    process a row block at a time anyway), so only the last block's reduction is exposed."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    if len(bounds) != world + 1 or w_shard.shape[0] != bounds[rank + 1] - bounds[rank]:
        raise ValueError(f"rank {rank}: w_shard has {w_shard.shape[0]} rows, the bounds {list(bounds)} "
                         f"give this rank {bounds[rank + 1] - bounds[rank] if len(bounds) == world + 1 else '?'}")
    target = target.contiguous().to(torch.int64)
    n = h16.shape[0]
    block = exchange_rows(n, h16.shape[1], bounds, chunk_cols)
    if n <= block or not (want_grad and reduce_grad):
        (token_loss, entropy, correct), grad_raw = _one_block(
            h16, w_shard, target, bounds, rank, world, group, want_grad, chunk_cols, w_bf16, None)
        if want_grad and reduce_grad:
            dist.all_reduce(grad_raw, group=group)
        return dict(token_loss=token_loss, entropy=entropy, correct=correct, grad_raw=grad_raw)
    h16 = h16.contiguous()
    grad_raw = torch.empty((n, h16.shape[1]), dtype=torch.float32, device=h16.device)
    pieces, pending = [], []
    for r0 in range(0, n, block):
        rows = slice(r0, min(n, r0 + block))
        terms, block_grad = _one_block(h16[rows], w_shard, target[rows], bounds, rank, world, group,
                                       True, chunk_cols, w_bf16, grad_raw[rows])
        pieces.append(terms)
        pending.append(dist.all_reduce(block_grad, group=group, async_op=True))
    for work in pending:
        work.wait()
    token_loss, entropy, correct = (torch.cat([p[i] for p in pieces]) for i in range(3))
    return dict(token_loss=token_loss, entropy=entropy, correct=correct, grad_raw=grad_raw)


STEP_ROWS = 16384   # rows gathered per exchange step of the row-sharded head (all ranks together)


def step_rows(n_total, hidden, bounds, chunk_cols=None):
    """Rows (over all ranks) one exchange step of `vocab_parallel_head_rows` gathers: whole
    kernel row blocks, up to STEP_ROWS. A step has fixed costs (its first chunk's one-wave
    launches, a dozen small kernels, four collectives' launch latencies: 0.15-0.2 ms measured), so
    a job of 2048 rows per GPU runs as one step; a long job (65536 rows) as steps whose gather and
    reduce-scatter travel beside the neighbouring steps' GEMMs. SOUP_VP_STEP_ROWS overrides."""
    import os

    block = exchange_rows(n_total, hidden, bounds, chunk_cols)
    want = int(os.environ.get("SOUP_VP_STEP_ROWS", STEP_ROWS))
    return max(block, want // block * block)


def plan_exchange_steps(n_local, world, block_rows):
    """[(begin, end)] ranges of a rank's local rows, one per exchange step. A step gathers the
    same range from every rank (world * (end - begin) rows, at most `block_rows`, the kernels'
    row block) and the steps are of equal size up to rounding to 8 rows, so that no step is a
    sliver whose launches run the GPU half empty."""
    if n_local <= 0:
        return []
    per_rank = max(8, block_rows // world)
    steps = -(-n_local // per_rank)
    size = -(-n_local // steps)
    size = -(-size // 8) * 8
    return [(a, min(n_local, a + size)) for a in range(0, n_local, size)]


_ONE = {}


def _one(device):
    if device not in _ONE:
        _ONE[device] = torch.ones(1, dtype=torch.float32, device=device)
    return _ONE[device]


def _rounded(grad_raw, dtype):
    """`grad_raw` (fp32, at GRAD_SCALE) rounded to `dtype` in a new tensor, one pass."""
    low = torch.empty(grad_raw.shape, dtype=dtype, device=grad_raw.device)
    _lib.call("soup_lmhead_grad_scale", _lib.ptr(grad_raw), _lib.ptr(low),
              _lib.ptr(_one(grad_raw.device)), grad_raw.numel(), _lib.dtype_code(dtype),
              _lib.stream_of(grad_raw))
    return low


def vocab_parallel_head_rows(h_local, target_local, w_shard, bounds, group=None, want_grad=True,
                             chunk_cols=None, w_bf16=None, grad_dtype=torch.float16):
    """The vocabulary-parallel head for a data-parallel upstream: every rank brings its own rows
    (the same number on every rank), and gets back the terms and the hidden-state gradient of
    exactly those rows. Nothing of full size is replicated or all-reduced.

    Per exchange step (`plan_exchange_steps`): the ranks' row ranges are all-gathered over NVLink
    (hidden fp16 and targets), each rank runs `head_partial` over the gathered rows on its
    vocabulary shard, the per-row states are all-gathered and merged, `head_finish` rescales the
    rank's gradient to the global log-sum-exp, and the gradient, rounded to `grad_dtype` at
    GRAD_SCALE (values of order 1: fp16 keeps 11 bits of each partial), is reduce-scattered so
    that every rank receives the sum for its own rows. The gather of step s+1 and the
    reduce-scatter of step s run beside the GEMMs of the neighbouring steps; what stays exposed is
    the first gather and the last reduce-scatter (rows x hidden x 2 bytes each).

    Returns dict(token_loss, entropy, correct: [n_local] for this rank's rows; grad: `grad_dtype`
    [n_local, hidden] at GRAD_SCALE, summed over the ranks, or None; loss_sum, labelled, hits:
    0-d tensors over the rows of ALL ranks, identical on every rank, no further collective)."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    if len(bounds) != world + 1 or w_shard.shape[0] != bounds[rank + 1] - bounds[rank]:
        raise ValueError(f"rank {rank}: w_shard has {w_shard.shape[0]} rows, the bounds {list(bounds)} "
                         "give this rank another range")
    n_local, hidden = h_local.shape
    dev = h_local.device
    h_local = h_local.contiguous()
    target_local = target_local.contiguous().to(torch.int64)
    steps = plan_exchange_steps(n_local, world, step_rows(n_local * world, hidden, bounds, chunk_cols))
    f32 = torch.float32
    token_loss = torch.empty(n_local, dtype=f32, device=dev)
    entropy = torch.empty(n_local, dtype=f32, device=dev)
    correct = torch.empty(n_local, dtype=torch.int32, device=dev)
    grad = torch.empty((n_local, hidden), dtype=grad_dtype, device=dev) if want_grad else None
    loss_sum = torch.zeros((), dtype=f32, device=dev)
    labelled = torch.zeros((), dtype=torch.int64, device=dev)
    hits = torch.zeros((), dtype=torch.int64, device=dev)

    def gather(step):
        a, z = steps[step]
        hg = torch.empty((world * (z - a), hidden), dtype=h_local.dtype, device=dev)
        tg = torch.empty(world * (z - a), dtype=torch.int64, device=dev)
        works = (dist.all_gather_into_tensor(hg, h_local[a:z], group=group, async_op=True),
                 dist.all_gather_into_tensor(tg, target_local[a:z], group=group, async_op=True))
        return hg, tg, works

    pending, keep = [], []
    raw = None
    nxt = gather(0) if steps else None
    for step, (a, z) in enumerate(steps):
        hg, tg, works = nxt
        for work in works:
            work.wait()
        nxt = gather(step + 1) if step + 1 < len(steps) else None   # travels beside this step's GEMMs
        rows = z - a
        if want_grad and (raw is None or raw.shape[0] != world * rows):
            raw = torch.empty((world * rows, hidden), dtype=f32, device=dev)
        state, grad_raw = head_partial(hg, w_shard, tg, bounds[rank], chunk_cols, want_grad, w_bf16,
                                       raw if want_grad else None)
        mine = pack_state(state)
        gathered = torch.empty((world * mine.shape[0], mine.shape[1]), dtype=mine.dtype, device=dev)
        dist.all_gather_into_tensor(gathered, mine, group=group)
        merged, _ = merge_states(gathered.view(world, *mine.shape), tg, bounds)
        low = (torch.empty(grad_raw.shape, dtype=grad_dtype, device=dev)
               if want_grad and grad_dtype != torch.float32 else None)
        tl, en, co = head_finish(merged, tg, w_shard, grad_raw, bounds[rank], grad_ref=state.grad_ref,
                                 grad_out=low)   # the gradient leaves rounded to `grad_dtype`, in one pass
        own = slice(rank * rows, (rank + 1) * rows)
        token_loss[a:z], entropy[a:z], correct[a:z] = tl[own], en[own], co[own]
        loss_sum += tl.sum()
        labelled += tg.ne(-100).sum()
        hits += co.sum()
        if want_grad:
            if low is None:
                low = grad_raw if grad_raw.dtype == grad_dtype else _rounded(grad_raw, grad_dtype)
            pending.append(dist.reduce_scatter_tensor(grad[a:z], low, group=group, async_op=True))
            keep.append(low)
    for work in pending:
        work.wait()
    return dict(token_loss=token_loss, entropy=entropy, correct=correct, grad=grad,
                loss_sum=loss_sum, labelled=labelled, hits=hits)


def emulate_vocab_parallel(h16, w, target, n_shards, chunk_cols=None):
    """The same data flow as `vocab_parallel_head` with every rank's shard processed on this GPU
    in turn (no collective): for tests on a single device."""
    bounds = shard_bounds(w.shape[0], n_shards)
    target = target.contiguous().to(torch.int64)
    states, grads = [], []
    for r in range(n_shards):
        st, g = head_partial(h16, w[bounds[r]:bounds[r + 1]], target, bounds[r], chunk_cols, True)
        states.append(st)
        grads.append(g)
    gathered = torch.stack([pack_state(s) for s in states])
    merged, _ = merge_states(gathered, target, bounds)
    out = None
    for r in range(n_shards):
        res = head_finish(merged, target, w[bounds[r]:bounds[r + 1]], grads[r], bounds[r],
                          grad_ref=states[r].grad_ref, want_metrics=(r == 0))
        if r == 0:
            out = res
    return dict(token_loss=out[0], entropy=out[1], correct=out[2], grad_raw=torch.stack(grads).sum(0))


def allreduce_lora_grads(params, group=None, average=True):
    """One flat fp32 all-reduce of the gradients of `params` (the LoRA A/B matrices). Parameters
    without a gradient contribute zeros, so every rank sends the same layout."""
    params = [p for p in params if p.requires_grad]
    if not params:
        return 0
    flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1).float()
                      for p in params])
    dist.all_reduce(flat, group=group)
    if average:
        flat /= dist.get_world_size(group)
    offset = 0
    for p in params:
        n = p.numel()
        chunk = flat[offset:offset + n].view_as(p).to(p.dtype)
        if p.grad is None:
            p.grad = chunk.clone()
        else:
            p.grad.copy_(chunk)
        offset += n
    return flat.numel()
