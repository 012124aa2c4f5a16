"""One rank of the multi-GPU parity run (launched by tests/test_gpu_multi.py through
torch.distributed.run, one process per GPU, NCCL):

  * vocabulary-parallel fused head against the single-GPU fused head on the full weight and
    against the oracle on a sample of rows, once within one exchange block and once over several;
  * the row-sharded variant (every rank feeds its own rows; fp16 reduce-scatter) against the oracle;
  * data-parallel captured QLoRA step: the all-reduced LoRA gradients equal the mean of the
    per-rank gradients, and the adapters stay identical across ranks after the optimizer step.

Prints "MULTI_GPU_OK" from rank 0 when every check passed on every rank.
"""

import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def rel(a, b):
    b = b.double()
    return ((a.double() - b).norm() / b.norm().clamp(min=1e-30)).item()


def check_head(rank, world, dev, n=1024, chunk_cols=None):
    from claudemaxing_b200 import parallel
    from claudemaxing_b200.lm_head_loss import GRAD_SCALE, fused_head_loss
    from oracle import head_ce

    hdim, vocab = 512, 50021   # vocabulary not a multiple of anything
    gen = torch.Generator().manual_seed(7)
    h = torch.randn(n, hdim, generator=gen).half()
    w = (torch.randn(vocab, hdim, generator=gen) * 0.05).half()
    t = torch.randint(0, vocab, (n,), generator=gen)
    t[torch.rand(n, generator=gen) < 0.1] = -100
    bounds = parallel.shard_bounds(vocab, world)
    hd, td = h.to(dev), t.to(dev)
    if chunk_cols is not None:   # the case is meant to walk several exchange blocks
        assert n > parallel.exchange_rows(n, hdim, bounds, chunk_cols)
    res = parallel.vocab_parallel_head(hd, w[bounds[rank]:bounds[rank + 1]].to(dev), td, bounds,
                                       chunk_cols=chunk_cols)
    n_lab = int((t != -100).sum())
    grad = res["grad_raw"] / (GRAD_SCALE * n_lab)
    # single-GPU fused head on the whole weight
    hs = hd.detach().requires_grad_(True)
    loss, step = fused_head_loss(hs[None], w.to(dev), None, target=td[None])
    loss.backward()
    errs = {
        "loss_vs_single": (res["token_loss"] - step.token_loss[0]).abs().max().item(),
        "entropy_vs_single": (res["entropy"] - step.token_entropy[0]).abs().max().item(),
        "grad_vs_single": rel(grad, hs.grad.float()),
        "correct_vs_single": abs(int(res["correct"].sum()) - int(step.correct)),
    }
    rows = slice(0, 64)
    ref = head_ce.head_ce(h[rows].float(), w.float(), t[rows])
    errs["loss_vs_oracle"] = (res["token_loss"][rows].cpu() - ref["token_loss"]).abs().max().item()
    errs["entropy_vs_oracle"] = (res["entropy"][rows].cpu() - ref["entropy"]).abs().max().item()
    ok = (errs["loss_vs_single"] < 1e-3 and errs["entropy_vs_single"] < 1e-3
          and errs["grad_vs_single"] < 1e-2 and errs["correct_vs_single"] == 0
          and errs["loss_vs_oracle"] < 1e-3 and errs["entropy_vs_oracle"] < 1e-3)
    return ok, errs


def check_rows(rank, world, dev, n_local=1100, chunk_cols=4096):
    """The row-sharded head: every rank feeds its own rows and gets their terms and their fp16
    gradient back (hidden all-gather, state all-gather, fp16 reduce-scatter per exchange step,
    several steps with a ragged last one), against the oracle on the whole job."""
    from claudemaxing_b200 import parallel
    from claudemaxing_b200.lm_head_loss import GRAD_SCALE
    from oracle import head_ce

    hdim, vocab = 256, 30011
    n = n_local * world
    gen = torch.Generator().manual_seed(9)
    h = torch.randn(n, hdim, generator=gen).half()
    w = (torch.randn(vocab, hdim, generator=gen) * 0.06).half()
    t = torch.randint(0, vocab, (n,), generator=gen)
    t[torch.rand(n, generator=gen) < 0.1] = -100
    bounds = parallel.shard_bounds(vocab, world)
    os.environ["SOUP_VP_STEP_ROWS"] = "2048"     # several exchange steps also for this small job
    steps = parallel.plan_exchange_steps(n_local, world, parallel.step_rows(n, hdim, bounds, chunk_cols))
    assert len(steps) >= 2, steps
    mine = slice(rank * n_local, (rank + 1) * n_local)
    res = parallel.vocab_parallel_head_rows(h[mine].to(dev), t[mine].to(dev),
                                            w[bounds[rank]:bounds[rank + 1]].to(dev), bounds,
                                            chunk_cols=chunk_cols)
    os.environ.pop("SOUP_VP_STEP_ROWS", None)
    ref = head_ce.head_ce(h.float(), w.float(), t)
    n_lab = int((t != -100).sum())
    grad = res["grad"].float().cpu() / (GRAD_SCALE * n_lab)
    scale = ref["dhidden"].abs().max().item()
    errs = {
        "loss": (res["token_loss"].cpu() - ref["token_loss"][mine]).abs().max().item(),
        "entropy": (res["entropy"].cpu() - ref["entropy"][mine]).abs().max().item(),
        "grad_rel_max": (grad - ref["dhidden"][mine]).abs().max().item() / scale,
        "job_loss": abs(float(res["loss_sum"]) / n_lab - float(ref["loss"])),
        "labelled": int(res["labelled"]) - n_lab,
        "hits": abs(int(res["hits"]) - int(ref["correct"].sum())),
        "steps": len(steps),
    }
    ok = (errs["loss"] < 1e-3 and errs["entropy"] < 1e-3 and errs["grad_rel_max"] < 1e-2
          and errs["job_loss"] < 1e-3 and errs["labelled"] == 0 and errs["hits"] <= 2)
    return ok, errs


TINY = dict(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, vocab_size=3000, max_position_embeddings=512)


def check_step(rank, world, dev):
    import claudemaxing_b200 as solution
    from claudemaxing_b200 import qlora

    solution.apply()
    model, lora = qlora.build_qlora_model(dev, TINY, dropout=0.05, seed=1)   # same on every rank
    torch.manual_seed(2)
    for m in model.modules():
        if isinstance(m, qlora.LoRALinear):
            m.lora_B.weight.data.normal_(0, 0.02)
    batch = qlora.synthetic_batch(batch=4, min_len=16, max_len=96, vocab=TINY["vocab_size"],
                                  seed=11 + rank)
    opt = torch.optim.AdamW(lora, lr=1e-3, fused=True, capturable=True)
    before = torch.cat([p.detach().reshape(-1).clone() for p in lora])
    step = qlora.CapturedStep(model, lora, opt, batch, bucket_tokens=384, loss_scale=1024.0)
    restored = torch.cat([p.detach().reshape(-1) for p in lora])
    assert torch.equal(before, restored), "construction must leave the adapters untouched"
    torch.manual_seed(100 + rank)          # the dropout masks of the step below
    step.graph_fb.replay()
    mine = step.flat_grad.clone()
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    want = torch.stack(gathered).mean(0)
    dist.all_reduce(step.flat_grad)
    step.flat_grad.div_(world)
    errs = {"allreduce_vs_mean": rel(step.flat_grad, want),
            "grad_norm": mine.norm().item()}
    step.graph_opt.replay()
    after = torch.cat([p.detach().reshape(-1) for p in lora])
    ref_after = after.clone()
    dist.broadcast(ref_after, 0)
    errs["adapters_differ"] = (after - ref_after).abs().max().item()
    errs["moved"] = (after - before).abs().max().item()
    # the public path does the same in one call
    loss = step.run()
    errs["loss"] = float(loss)
    ok = (errs["allreduce_vs_mean"] < 1e-6 and errs["adapters_differ"] == 0.0
          and errs["moved"] > 0 and errs["grad_norm"] > 0 and errs["loss"] == errs["loss"])
    return ok, errs


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    try:
        ok1, e1 = check_head(rank, world, dev)
        # more rows than one block: blocks' exchanges overlap the next block's GEMMs, ragged tail
        ok3, e3 = check_head(rank, world, dev, n=4500, chunk_cols=4096)
        ok4, e4 = check_rows(rank, world, dev)
        ok2, e2 = check_step(rank, world, dev)
        from claudemaxing_b200 import _lib

        _lib.check_device_status()
        flag = torch.tensor([int(ok1 and ok2 and ok3 and ok4)], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        print(f"rank {rank}: head {ok1} {e1} head-4500 {ok3} {e3} rows {ok4} {e4} step {ok2} {e2}",
              flush=True)
        if rank == 0 and int(flag) == 1:
            print("MULTI_GPU_OK", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
