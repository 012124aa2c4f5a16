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
