"""World-size-2 run of the multi-rank data flow on CPU ranks (gloo): the vocabulary-parallel
state exchange and merge, and the flat LoRA-gradient all-reduce. The arithmetic on each rank is the
oracle's; what is tested is the exchange protocol of claudemaxing_b200/parallel.py."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from claudemaxing_b200 import parallel
        from oracle import head_ce, parallel as opar

        gen = torch.Generator().manual_seed(0)
        h = torch.randn(48, 32, generator=gen)
        w = torch.randn(1000, 32, generator=gen) * 0.3
        t = torch.randint(0, 1000, (48,), generator=gen)
        t[::5] = -100
        bounds = parallel.shard_bounds(1000, world)
        w_shard = w[bounds[rank]:bounds[rank + 1]]
        part = opar.shard_partial(h, w_shard, t, bounds[rank])
        keys = ("run_max", "run_sum", "run_dot", "best", "label_logit", "label_lse")
        mine = torch.stack([part[k].float() for k in keys])
        gathered = torch.empty((world * mine.shape[0], mine.shape[1]))
        dist.all_gather_into_tensor(gathered, mine)
        gathered = gathered.view(world, *mine.shape)
        parts = [dict(zip(keys, gathered[r])) for r in range(world)]
        for p in parts:
            p["best"] = p["best"].long()
        merged = opar.merge(parts, t, bounds)
        tl, en, co, g = opar.finish(merged, part, w_shard, t, bounds[rank])
        dist.all_reduce(g)
        ref = head_ce.head_ce(h, w, t)
        n_lab = (t != -100).sum()
        ok = (torch.allclose(tl, ref["token_loss"], atol=1e-5)
              and torch.allclose(en, ref["entropy"], atol=1e-5)
              and torch.equal(co, ref["correct"])
              and torch.allclose(g / (1024.0 * n_lab), ref["dhidden"], atol=1e-6))
        # flat LoRA-gradient all-reduce
        a = torch.nn.Parameter(torch.zeros(4, 8))
        b = torch.nn.Parameter(torch.zeros(8, 4))
        frozen = torch.nn.Parameter(torch.zeros(3), requires_grad=False)
        a.grad = torch.full((4, 8), float(rank + 1))
        n = parallel.allreduce_lora_grads([a, b, frozen])
        ok = ok and n == 64 and torch.allclose(a.grad, torch.full((4, 8), (1 + world) / 2))
        ok = ok and b.grad is not None and b.grad.abs().max() == 0 and frozen.grad is None
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_cpu_ranks_vocab_parallel_and_grad_allreduce():
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        assert dict(results) == {0: True, 1: True}


# --- the block-wise exchange of vocab_parallel_head itself, kernels replaced by torch on CPU -------

def _cpu_partial(h16, w, target, col_offset=0, chunk_cols=None, want_grad=True, w_bf16=None,
                 grad_out=None):
    from claudemaxing_b200.lm_head_loss import HeadState

    n = h16.shape[0]
    z = h16.float() @ w.float().t()
    st = HeadState(n, h16.device)
    st.best_val, idx = z.max(dim=1)
    st.best = (idx + col_offset).to(torch.int32)
    st.run_max = st.best_val.clone()
    e = torch.exp(z - st.run_max[:, None])
    st.run_sum, st.run_dot = e.sum(1), (e * z).sum(1)
    local = target - col_offset
    inside = (target >= 0) & (local >= 0) & (local < w.shape[0])
    rows = torch.arange(n)
    st.label_logit = torch.where(inside, z[rows, local.clamp(0, w.shape[0] - 1)], torch.zeros(n))
    st.grad_ref = st.run_max + torch.log(st.run_sum)
    p = torch.exp(z - st.grad_ref[:, None])
    p[rows[inside], local[inside]] = 0.0
    p[target < 0] = 0.0
    grad = p @ w.float()
    if grad_out is not None:
        grad_out.copy_(grad)
        grad = grad_out
    return st, grad


def _cpu_merge(gathered, target, bounds):
    from claudemaxing_b200.lm_head_loss import HeadState

    world, _, n = gathered.shape
    run_max, run_sum, run_dot, best, best_val, label_logit = (gathered[:, i] for i in range(6))
    top = run_max.max(dim=0).values
    scale = torch.exp(run_max - top)
    out = HeadState(n, gathered.device)
    out.run_max, out.run_sum, out.run_dot = top, (run_sum * scale).sum(0), (run_dot * scale).sum(0)
    first = best_val.argmax(dim=0)          # ties: the lowest rank, i.e. the lowest column
    cols = torch.arange(n)
    out.best = best.contiguous().view(torch.int32)[first, cols]
    out.best_val = best_val[first, cols]
    owner = torch.bucketize(target.clamp(min=0), torch.tensor(bounds[1:-1]), right=True)
    out.label_logit = label_logit[owner, cols]
    out.grad_ref = out.run_max + torch.log(out.run_sum)
    return out, out.grad_ref.clone()


def _cpu_finish(state, target, w, grad_raw=None, col_offset=0, grad_ref=None, want_metrics=True,
                grad_out=None):
    lse = state.run_max + torch.log(state.run_sum)
    labelled = target >= 0
    loss = torch.where(labelled, lse - state.label_logit, torch.zeros_like(lse))
    entropy = lse - state.run_dot / state.run_sum
    correct = (labelled & (state.best.long() == target)).to(torch.int32)
    if grad_raw is not None:
        grad_raw.mul_(torch.exp(grad_ref - lse)[:, None])
        local = target - col_offset
        inside = labelled & (local >= 0) & (local < w.shape[0])
        p_label = torch.exp(state.label_logit - lse)
        grad_raw[inside] += (p_label[inside] - 1.0)[:, None] * w.float()[local[inside]]
        grad_raw.mul_(1024.0)
        if grad_out is not None:
            grad_out.copy_(grad_raw)
    return loss, entropy, correct


def _block_worker(rank, world, port, results):
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=60))
    try:
        from claudemaxing_b200 import parallel
        from oracle import head_ce

        parallel.head_partial, parallel.merge_states = _cpu_partial, _cpu_merge
        parallel.head_finish = _cpu_finish
        # as in the kernels' plan, the row block shrinks with the shard's tile count: the ranks'
        # own shards (3, 3, 2, 2 tiles of 8 columns) would give 16, 16, 32, 32 rows
        parallel._row_block = lambda n, hidden, v_shard, chunk_cols: 16 if v_shard > 16 else 32
        gen = torch.Generator().manual_seed(1)
        h = (torch.randn(40, 32, generator=gen)).half()
        w = (torch.randn(77, 32, generator=gen) * 0.3).half()
        t = torch.randint(0, 77, (40,), generator=gen)
        t[::7] = -100
        bounds = parallel.shard_bounds(77, world, tile=8)
        widths = [bounds[r + 1] - bounds[r] for r in range(world)]
        assert len({16 if v > 16 else 32 for v in widths}) == 2, widths
        assert parallel.exchange_rows(40, 32, bounds) == 16
        out = parallel.vocab_parallel_head(h, w[bounds[rank]:bounds[rank + 1]], t, bounds)
        ref = head_ce.head_ce(h.float(), w.float(), t)
        n_lab = (t != -100).sum()
        results[rank] = bool(
            torch.allclose(out["token_loss"], ref["token_loss"], atol=1e-4)
            and torch.allclose(out["entropy"], ref["entropy"], atol=1e-4)
            and torch.equal(out["correct"], ref["correct"])
            and torch.allclose(out["grad_raw"] / (1024.0 * n_lab), ref["dhidden"], atol=1e-5))
    finally:
        dist.destroy_process_group()


def test_four_cpu_ranks_with_uneven_shards_walk_the_same_row_blocks():
    """Shards that differ by a column tile have different kernel row blocks; the exchange has to
    use one block size on all ranks or the ranks issue different numbers of collectives."""
    world = 4
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_block_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        assert dict(results) == {r: True for r in range(world)}


def test_exchange_rows_is_common_to_all_ranks_for_the_real_plan():
    """With the library's own plan: for every world size the exchange block computed from the
    bounds is one number, although the ranks' own shards can plan different row blocks."""
    from claudemaxing_b200 import parallel

    differing = 0
    for world in (2, 3, 4, 5, 6, 7, 8):
        bounds = parallel.shard_bounds(151936, world)
        for n in (2048 * world, 65536):
            own = {parallel._row_block(n, 1536, bounds[r + 1] - bounds[r], None) for r in range(world)}
            differing += len(own) > 1
            assert parallel.exchange_rows(n, 1536, bounds) == min(own)
    assert differing, "expected at least one world size (4) whose shards plan different row blocks"


# --- the row-sharded variant: every rank brings its own rows, gathers, reduce-scatters ------------

def _rows_worker(rank, world, port, results):
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=60))
    try:
        from claudemaxing_b200 import parallel
        from oracle import head_ce

        parallel.head_partial, parallel.merge_states = _cpu_partial, _cpu_merge
        parallel.head_finish = _cpu_finish
        parallel._rounded = lambda g, dtype: g.to(dtype)
        parallel._row_block = lambda n, hidden, v_shard, chunk_cols: 32
        os.environ["SOUP_VP_STEP_ROWS"] = "32"              # several exchange steps for a tiny job
        n_local, hidden, vocab = 27, 32, 77                 # 27 rows per rank: ragged last step
        gen = torch.Generator().manual_seed(5)
        h = torch.randn(world * n_local, hidden, generator=gen).half()
        w = (torch.randn(vocab, hidden, generator=gen) * 0.3).half()
        t = torch.randint(0, vocab, (world * n_local,), generator=gen)
        t[::6] = -100
        bounds = parallel.shard_bounds(vocab, world, tile=8)
        steps = parallel.plan_exchange_steps(n_local, world, 32)
        assert len(steps) > 2 and steps[0][0] == 0 and steps[-1][1] == n_local
        mine = slice(rank * n_local, (rank + 1) * n_local)   # any split of the rows over ranks works
        out = parallel.vocab_parallel_head_rows(h[mine], t[mine], w[bounds[rank]:bounds[rank + 1]],
                                                bounds, grad_dtype=torch.float32)
        ref = head_ce.head_ce(h.float(), w.float(), t)
        n_lab = int((t != -100).sum())
        results[rank] = bool(
            torch.allclose(out["token_loss"], ref["token_loss"][mine], atol=1e-4)
            and torch.allclose(out["entropy"], ref["entropy"][mine], atol=1e-4)
            and torch.equal(out["correct"], ref["correct"][mine])
            and torch.allclose(out["grad"] / (1024.0 * n_lab), ref["dhidden"][mine], atol=1e-5)
            and abs(float(out["loss_sum"]) / n_lab - float(ref["loss"])) < 1e-4
            and int(out["labelled"]) == n_lab
            and int(out["hits"]) == int(ref["correct"].sum()))
    finally:
        dist.destroy_process_group()


def test_four_cpu_ranks_row_sharded_head_gathers_and_reduce_scatters():
    """vocab_parallel_head_rows on 4 gloo ranks (kernels replaced by torch): each rank feeds its
    own rows, several exchange steps with a ragged last one, and gets its own rows' terms and
    gradient back; the job-wide sums are identical on every rank without another collective."""
    world = 4
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_rows_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        assert dict(results) == {r: True for r in range(world)}


def test_exchange_steps_cover_the_rows_in_near_equal_pieces():
    from claudemaxing_b200 import parallel

    for n_local, world, block in ((2048, 8, 8192), (8192, 8, 8192), (2048, 4, 6144), (2048, 2, 4096),
                                  (8192, 4, 6144), (27, 4, 32), (1, 8, 8192)):
        steps = parallel.plan_exchange_steps(n_local, world, block)
        assert steps[0][0] == 0 and steps[-1][1] == n_local
        assert all(a[1] == b[0] for a, b in zip(steps, steps[1:]))
        sizes = [z - a for a, z in steps]
        assert max(sizes) * world <= max(block, 8 * world) and max(sizes) - min(sizes[:-1] or sizes) <= 8
    assert parallel.plan_exchange_steps(0, 4, 4096) == []


def test_step_rows_are_whole_row_blocks_and_common_to_all_ranks():
    from claudemaxing_b200 import parallel

    for world in (2, 4, 8):
        bounds = parallel.shard_bounds(151936, world)
        block = parallel.exchange_rows(2048 * world, 1536, bounds)
        rows = parallel.step_rows(2048 * world, 1536, bounds)
        assert rows % block == 0 and block <= rows <= max(block, parallel.STEP_ROWS)
        # the weak-scaling job of 2048 rows per GPU is one exchange step
        assert len(parallel.plan_exchange_steps(2048, world, rows)) == 1
        assert len(parallel.plan_exchange_steps(65536 // world, world, rows)) >= 4
