"""The whole QLoRA training step through the patched model (packed tokens, NF4 linears, LoRA
branch, RoPE, RMSNorm, SwiGLU recompute, fused head) against the installed transformers code run
on the CPU in fp32 on the same weights. Criterion of the reference's end-to-end test
(tests_local/test_lm_head_trainer.py:186-188): loss within 1 %; here also the LoRA gradients."""

import pytest
import torch

from conftest import rel_norm

pytestmark = pytest.mark.gpu

TINY = dict(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, vocab_size=3000, max_position_embeddings=512)


class _RefLoRA(torch.nn.Module):
    def __init__(self, weight, bias, a, b, scaling):
        super().__init__()
        self.weight, self.bias, self.scaling = weight, bias, scaling
        self.a = torch.nn.Parameter(a.clone())
        self.b = torch.nn.Parameter(b.clone())

    def forward(self, x):
        base = torch.nn.functional.linear(x, self.weight, self.bias)
        return base + torch.nn.functional.linear(torch.nn.functional.linear(x, self.a), self.b) * self.scaling


def _cpu_reference(model_gpu, cfg):
    """fp32 CPU copy with plain nn.Linear layers holding the dequantised weights."""
    from transformers import Qwen2Config, Qwen2ForCausalLM

    from claudemaxing_b200.nf4 import dequantize_nf4
    from claudemaxing_b200.qlora import LoRALinear

    hf_cfg = Qwen2Config(**model_gpu.config.to_dict())  # the builder's defaults (rope_theta, eps) included
    hf_cfg._attn_implementation = "sdpa"
    ref = Qwen2ForCausalLM(hf_cfg).float()
    ref.model.embed_tokens.weight.data = model_gpu.model.embed_tokens.weight.detach().float().cpu()
    ref.lm_head.weight = ref.model.embed_tokens.weight
    ref.model.norm.weight.data = model_gpu.model.norm.weight.detach().float().cpu()
    refs = {}
    for lg, lr in zip(model_gpu.model.layers, ref.model.layers):
        lr.input_layernorm.weight.data = lg.input_layernorm.weight.detach().float().cpu()
        lr.post_attention_layernorm.weight.data = lg.post_attention_layernorm.weight.detach().float().cpu()
        for pg, pr, names in ((lg.self_attn, lr.self_attn, ("q_proj", "k_proj", "v_proj", "o_proj")),
                              (lg.mlp, lr.mlp, ("gate_proj", "up_proj", "down_proj"))):
            for name in names:
                mod = getattr(pg, name)
                base = mod.base_layer if isinstance(mod, LoRALinear) else mod
                w = dequantize_nf4(base.packed, base.quant_state, torch.float16).float().cpu()
                bias = None if base.bias is None else base.bias.detach().float().cpu()
                if isinstance(mod, LoRALinear):
                    r = _RefLoRA(w, bias, mod.lora_A.weight.detach().cpu(), mod.lora_B.weight.detach().cpu(),
                                 mod.scaling)
                    setattr(pr, name, r)
                    refs[id(mod)] = r
                else:
                    lin = getattr(pr, name)
                    lin.weight.data = w
                    if bias is not None:
                        lin.bias.data = bias
                    else:
                        lin.bias = None
    for p in ref.parameters():
        p.requires_grad_(False)
    for r in refs.values():
        r.a.requires_grad_(True)
        r.b.requires_grad_(True)
    return ref, refs


@pytest.mark.parametrize("fused_gemm", [False, True])
def test_step_matches_installed_transformers_on_cpu(fused_gemm, monkeypatch):
    """`fused_gemm`: the 4-bit projections as dequantise + cuBLAS (default) or on the tcgen05 GEMM
    that dequantises in its operand prologue (forward, MLP recompute and every input gradient)."""
    import claudemaxing_b200 as solution
    from claudemaxing_b200 import nf4 as nf4_mod, qlora
    from claudemaxing_b200.qlora import LoRALinear

    monkeypatch.setattr(qlora.NF4Linear, "fused_gemm", fused_gemm)
    launches = []
    real_fwd, real_dx = nf4_mod._lib.call, None

    def counting_call(name, *args):
        if name.startswith("soup_nf4_linear"):
            launches.append(name)
        return real_fwd(name, *args)

    monkeypatch.setattr(nf4_mod._lib, "call", counting_call)
    solution.apply()
    model, lora = qlora.build_qlora_model("cuda", TINY, dropout=1e-6, seed=1)
    # B = 0 would make the adapter output and dA vanish: give B small values
    torch.manual_seed(2)
    for m in model.modules():
        if isinstance(m, LoRALinear):
            m.lora_B.weight.data.normal_(0, 0.02)
    ref, refs = _cpu_reference(model, TINY)
    batch = qlora.synthetic_batch(batch=4, min_len=16, max_len=96, vocab=TINY["vocab_size"], seed=5)
    ref_out = ref(input_ids=batch["input_ids"], attention_mask=batch["attention_mask"],
                  labels=batch["labels"])
    ref_out.loss.backward()
    dev_batch = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in batch.items()}
    calls = []
    from claudemaxing_b200 import lm_head_loss

    original = lm_head_loss.fused_head_loss

    def spy(*args, **kwargs):  # the fused head must be what produced the loss
        calls.append(1)
        return original(*args, **kwargs)

    lm_head_loss.fused_head_loss = spy
    try:
        loss = qlora.qlora_step(model, dev_batch)
    finally:
        lm_head_loss.fused_head_loss = original
    assert calls, "the fused head did not run"
    if fused_gemm:   # q, k, v, o, gate+up, down forward; gate+up recompute; five input gradients
        assert launches.count("soup_nf4_linear_fwd") == 7 * TINY["num_hidden_layers"]
        assert launches.count("soup_nf4_linear_dx") >= 5 * TINY["num_hidden_layers"] - 3
    else:
        assert not launches
    assert abs(loss.item() - ref_out.loss.item()) <= 1e-2 * abs(ref_out.loss.item())
    checked = 0
    for m in model.modules():
        if isinstance(m, LoRALinear):
            r = refs[id(m)]
            assert rel_norm(m.lora_B.weight.grad.cpu(), r.b.grad) < 5e-2
            assert rel_norm(m.lora_A.weight.grad.cpu(), r.a.grad) < 5e-2
            checked += 1
    assert checked == 2 * TINY["num_hidden_layers"]


def test_fused_blocks_give_the_per_op_chain_s_step():
    """The same model with its decoder blocks run as the fused chain (decoder_block.py) and as
    transformers' block through the per-op patches: same dropout draws (same seed, same order),
    loss and LoRA gradients equal to fp16 rounding of the few intermediate results the fused
    GEMMs keep in fp32."""
    import claudemaxing_b200 as solution
    from claudemaxing_b200 import qlora
    from claudemaxing_b200.qlora import LoRALinear

    solution.apply()
    results = []
    for fused, keep in ((True, True), (False, None), (True, False)):
        model, lora = qlora.build_qlora_model("cuda", TINY, dropout=0.1, seed=1, fused_blocks=fused)
        taken = [l._soup_block for l in model.model.layers if getattr(l, "_soup_block", None) is not None]
        assert len(taken) == (TINY["num_hidden_layers"] if fused else 0)
        for plan in taken:     # keep gate and up for backward, or run the two projections again
            plan.keep_products = keep
        torch.manual_seed(2)
        for m in model.modules():
            if isinstance(m, LoRALinear):
                m.lora_B.weight.data.normal_(0, 0.02)
        batch = qlora.synthetic_batch(batch=4, min_len=16, max_len=96, vocab=TINY["vocab_size"],
                                      seed=5, device="cuda")
        torch.manual_seed(11)
        loss = qlora.qlora_step(model, batch)
        results.append((loss.item(), [p.grad.detach().float().cpu() for p in lora]))
    (loss_f, grads_f), (loss_p, grads_p), (loss_r, grads_r) = results
    assert abs(loss_f - loss_p) < 1e-3 * abs(loss_p)
    for a, b in zip(grads_f, grads_p):
        assert rel_norm(a, b) < 2e-2
    # recomputing the two products gives the numbers that were kept: same loss to the bit, and
    # gradients equal up to the order of the attention backward's atomic sums
    assert loss_r == loss_f
    for a, b in zip(grads_r, grads_f):
        assert rel_norm(a, b) < 1e-3


def test_step_trains():
    import claudemaxing_b200 as solution
    from claudemaxing_b200 import qlora

    solution.apply()
    model, lora = qlora.build_qlora_model("cuda", TINY, seed=3)
    batch = qlora.synthetic_batch(batch=4, min_len=16, max_len=96, vocab=TINY["vocab_size"],
                                  seed=6, device="cuda")
    opt = torch.optim.AdamW(lora, lr=2e-3)
    scaler = torch.amp.GradScaler("cuda")
    losses = [qlora.qlora_step(model, batch, opt, scaler).item() for _ in range(8)]
    assert all(torch.isfinite(torch.tensor(losses)))
    assert losses[-1] < losses[0]


def test_single_call_grouped_attention_matches_repeat_kv():
    from claudemaxing_b200.attention import _grouped_sdpa

    torch.manual_seed(0)
    n, hq, hk, d = 300, 12, 2, 128
    q = torch.randn(1, n, hq, d, device="cuda", dtype=torch.float16).transpose(1, 2)
    k = torch.randn(1, n, hk, d, device="cuda", dtype=torch.float16).transpose(1, 2)
    v = torch.randn(1, n, hk, d, device="cuda", dtype=torch.float16).transpose(1, 2)
    row = torch.arange(n, device="cuda") // 77
    col = torch.arange(n, device="cuda") % 77
    mask = ((row[:, None] == row[None, :]) & (col[None, :] <= col[:, None]))[None, None]
    out = _grouped_sdpa(q, k, v, mask, d ** -0.5)
    kk, vv = k.repeat_interleave(hq // hk, 1).float(), v.repeat_interleave(hq // hk, 1).float()
    s = (q.float() @ kk.transpose(-1, -2)) * d ** -0.5
    ref = (s.masked_fill(~mask, float("-inf")).softmax(-1) @ vv).transpose(1, 2)
    assert rel_norm(out.cpu(), ref.cpu()) < 2e-3


@pytest.mark.parametrize("lens", [[77, 0, 130, 1, 92], [300, 280, 296, 292, 112], [640, 5, 128, 64, 129]])
@pytest.mark.parametrize("dtype,autocast", [(torch.float16, False), (torch.float32, True), (torch.float32, False)])
def test_segment_attention_matches_the_masked_formula(dtype, autocast, lens, monkeypatch):
    """Causal attention inside the segments of a packed row (variable-length kernel, no mask)
    against softmax(mask(q k^T)) v in fp32: fp16 operands, fp32 operands under fp16 autocast (cast
    as SDPA casts them), and fp32 operands without autocast (the masked SDPA route). An empty
    segment and a segment of one token are among the rows."""
    from claudemaxing_b200 import attention as attention_mod
    from claudemaxing_b200.attention import mask_of_segments, segment_attention

    launches = []
    real_call = attention_mod._lib.call
    monkeypatch.setattr(attention_mod._lib, "call",
                        lambda name, *args: (launches.append(name), real_call(name, *args))[1])
    torch.manual_seed(0)
    n, hq, hk, d = sum(lens), 12, 2, 128
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    q = torch.randn(1, n, hq, d, device="cuda").to(dtype).transpose(1, 2).requires_grad_()
    k = torch.randn(1, n, hk, d, device="cuda").to(dtype).transpose(1, 2).requires_grad_()
    v = torch.randn(1, n, hk, d, device="cuda").to(dtype).transpose(1, 2).requires_grad_()
    go = torch.randn(1, n, hq, d, device="cuda")
    with torch.autocast("cuda", dtype=torch.float16, enabled=autocast):
        out = segment_attention(q, k, v, cu, max(lens), d ** -0.5)
    assert out.shape == (1, n, hq, d) and out.is_contiguous()
    assert out.dtype == (torch.float16 if autocast else dtype)
    # fp16 operands with adjacent heads: forward and backward are this library's kernels
    assert ("soup_attn_fwd" in launches) == (dtype == torch.float16)
    out.backward(go.to(out.dtype))
    assert ("soup_attn_bwd" in launches) == (dtype == torch.float16)
    got = [out.detach().float().cpu()] + [t.grad.float().cpu() for t in (q, k, v)]
    assert all(t.grad.dtype == dtype for t in (q, k, v))
    q2, k2, v2 = (t.detach().double().requires_grad_() for t in (q, k, v))
    mask = mask_of_segments(cu, n)
    s = (q2 @ k2.repeat_interleave(hq // hk, 1).transpose(-1, -2)) * d ** -0.5
    ref = (s.masked_fill(~mask, float("-inf")).softmax(-1) @ v2.repeat_interleave(hq // hk, 1)).transpose(1, 2)
    ref.backward(go.double())
    want = [ref.detach().float().cpu()] + [t.grad.float().cpu() for t in (q2, k2, v2)]
    for name, a, b in zip(("out", "dq", "dk", "dv"), got, want):
        assert rel_norm(a, b) < 3e-3, name


@pytest.mark.parametrize("resident_mb", [0, 4096])
def test_group_dequant_equals_per_weight_dequant(resident_mb, monkeypatch):
    """The shared pool of dequantised blocks returns each weight's own numbers whether a block is
    found resident or has been replaced (a pool of two blocks under three in turn), and a block
    that stays resident is dequantised once."""
    from claudemaxing_b200 import qlora
    from claudemaxing_b200.nf4 import dequantize_nf4

    monkeypatch.setattr(qlora.NF4Group, "resident_mb", resident_mb)
    monkeypatch.setattr(qlora.NF4Group, "_buffers", {})
    model, _ = qlora.build_qlora_model("cuda", dict(TINY, num_hidden_layers=3), seed=4)
    layers = model.model.layers
    fills = []
    real_fill = qlora.NF4Group._fill
    monkeypatch.setattr(qlora.NF4Group, "_fill",
                        lambda self, bufs, i, dtype: (fills.append(i), real_fill(self, bufs, i, dtype))[1])
    for layer in (layers[0], layers[1], layers[2], layers[0], layers[2], layers[1]):
        for mod in (layer.self_attn.o_proj, layer.mlp.down_proj, layer.self_attn.k_proj):
            got = mod.dequantized(torch.float16).clone()
            want = dequantize_nf4(mod.packed, mod.quant_state, torch.float16)
            assert torch.equal(got, want)
    # two buffers: 0 1 0(evicts block 0) then block 0 again into 1, block 2 resident, block 1 into 1
    assert fills == ([0, 1, 0, 1, 1] if resident_mb == 0 else [0, 1, 2])
    qlora.NF4Group.forget()
    assert layers[2].mlp.down_proj.dequantized(torch.float16) is not None and len(fills) == (6 if resident_mb == 0 else 4)


def test_captured_step_equals_the_eager_step_and_trains():
    """The CUDA-graph step on the padded packed bucket gives the eager step's loss (padding tokens
    are a segment of their own and carry ignore labels), leaves the adapters untouched by its own
    warm-up, and its replays train."""
    import claudemaxing_b200 as solution
    from claudemaxing_b200 import qlora

    solution.apply()
    model, lora = qlora.build_qlora_model("cuda", TINY, dropout=0.05, seed=3)
    batch = qlora.synthetic_batch(batch=4, min_len=16, max_len=96, vocab=TINY["vocab_size"], seed=9)
    dev_batch = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in batch.items()}
    eager_loss = float(qlora.qlora_step(model, dev_batch))      # B = 0: dropout cannot matter yet
    for p in lora:
        p.grad = None
    before = [p.detach().clone() for p in lora]
    opt = torch.optim.AdamW(lora, lr=2e-3, fused=True, capturable=True)
    step = qlora.CapturedStep(model, lora, opt, batch, loss_scale=1024.0)
    assert step.bucket % 128 == 0 and step.bucket >= batch["n_tokens"]
    assert all(torch.equal(a, b) for a, b in zip(before, lora))
    first = float(step.run())
    assert abs(first - eager_loss) < 2e-3 * abs(eager_loss)
    losses = [float(step.run()) for _ in range(12)]
    assert losses[-1] < first - 0.02
    assert any(not torch.equal(a, b) for a, b in zip(before, lora))
    # a different batch of at most the bucket's size goes through the same graphs
    other = qlora.synthetic_batch(batch=4, min_len=16, max_len=80, vocab=TINY["vocab_size"], seed=10)
    if other["n_tokens"] <= step.bucket:
        step.load(other)
        assert torch.isfinite(step.run()).item()
    # an eager step through the patched forward after the capture (it is what decides the tied
    # embedding's storage dtype on its first call) leaves everything the graphs read in place
    step.load(batch)
    before_eager = float(step.run())
    eager_now = float(qlora.qlora_step(model, dev_batch))
    after_eager = float(step.run())
    assert abs(eager_now - before_eager) < 0.05 * abs(before_eager)
    assert abs(after_eager - before_eager) < 0.05 * abs(before_eager)


@pytest.mark.parametrize("autocast_dtype", [torch.bfloat16, None])
def test_padded_batch_outside_fp16_keeps_the_packing_and_goes_through_the_logits(autocast_dtype):
    """A padded batch under bf16 autocast, or of an fp32 model without autocast, is still packed,
    but its head cannot be the fp16 tensor-core kernel: the loss and the per-token terms come
    from the logits of the packed row and match the installed forward on the padded batch."""
    import contextlib

    import claudemaxing_b200 as solution
    from claudemaxing_b200 import lm_head_loss, qlora
    from transformers import Qwen2Config, Qwen2ForCausalLM

    solution.apply()
    cfg = Qwen2Config(**dict(qlora.QWEN25_1P5B, **TINY))
    cfg._attn_implementation = "sdpa"
    torch.manual_seed(0)
    model = Qwen2ForCausalLM(cfg).float().cuda()
    for p in model.parameters():
        p.requires_grad_(False)
    model.model.layers[0].mlp.down_proj.weight.requires_grad_(True)   # something to train
    batch = qlora.synthetic_batch(batch=3, min_len=8, max_len=40, vocab=TINY["vocab_size"],
                                  seed=12, device="cuda")
    ctx = (torch.autocast("cuda", dtype=autocast_dtype) if autocast_dtype is not None
           else contextlib.nullcontext())
    kwargs = dict(input_ids=batch["input_ids"], attention_mask=batch["attention_mask"],
                  labels=batch["labels"], use_cache=False)
    with ctx:
        ref = model(**kwargs)                      # not flagged: the installed forward, padded
    ref.loss.backward()
    ref_grad = model.model.layers[0].mlp.down_proj.weight.grad.clone()
    model.zero_grad(set_to_none=True)
    fused_calls = []
    original = lm_head_loss.fused_head_loss
    lm_head_loss.fused_head_loss = lambda *a, **k: (fused_calls.append(1), original(*a, **k))[1]
    try:
        model.__dict__[lm_head_loss._REQUEST_ATTR] = True
        with ctx:
            out = model(**kwargs)
    finally:
        lm_head_loss.fused_head_loss = original
    assert out.logits is None and not fused_calls
    terms = model.__dict__.pop(lm_head_loss._STEP_ATTR)
    assert terms.token_loss.shape == batch["input_ids"].shape
    tol = 2e-2 if autocast_dtype is not None else 1e-4
    assert abs(out.loss.item() - ref.loss.item()) <= tol * abs(ref.loss.item())
    n_lab = int(terms.labelled)
    assert abs(terms.token_loss.sum().item() / n_lab - ref.loss.item()) <= tol * abs(ref.loss.item())
    out.loss.backward()
    assert rel_norm(model.model.layers[0].mlp.down_proj.weight.grad, ref_grad) < (5e-2 if autocast_dtype else 1e-3)
