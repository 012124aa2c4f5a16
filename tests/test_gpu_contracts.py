"""Host-side contracts of two ops the reference pins with tests of its own:

* MLPInputRecompute keeps nothing but the MLP input for backward, and its 4-bit fast path (one input
  cast, fp16 gate/up and gradients) equals the module-calling path bit for bit
  (tests_local/test_swiglu_recompute.py:225-327);
* shrink_tied_embedding stores the tied fp32 embedding/head weight in fp16 only when that changes
  no value, only for a plain frozen tied pair, and the lookup still returns the fp32 numbers
  (tests_local/test_embedding.py:37-87).

bitsandbytes is not installed, so the 4-bit projections are this package's NF4Linear, which follows
the same cast -> dequantise -> linear -> cast-back formula."""

import copy
import importlib

import pytest
import torch

from conftest import assert_close_rel_max

pytestmark = pytest.mark.gpu
F16, F32 = torch.float16, torch.float32


def _small_mlp(hidden=256, inter=704):
    from transformers.models.qwen2 import modeling_qwen2 as modeling

    torch.manual_seed(0)
    cfg = modeling.Qwen2Config(hidden_size=hidden, intermediate_size=inter, hidden_act="silu")
    return modeling, modeling.Qwen2MLP(cfg).cuda()


def _saved_pointers(fn):
    kept = []
    with torch.autograd.graph.saved_tensors_hooks(
            lambda t: (kept.append((t.data_ptr(), t.dtype, tuple(t.shape))), t)[1], lambda t: t):
        out = fn()
    return out, kept


@pytest.mark.parametrize("autocast", [False, True])
def test_frozen_mlp_recompute_keeps_only_its_input(autocast):
    mod = importlib.import_module("claudemaxing_b200.swiglu_recompute")

    modeling, mlp = _small_mlp()
    installed = modeling.Qwen2MLP.forward
    if getattr(installed, "_swiglu_recompute", False):
        pytest.skip("the class is already patched in this process; the installed forward is gone")
    mlp = mlp.float() if autocast else mlp.half()
    mlp.requires_grad_(False)
    ctx = (lambda: torch.autocast("cuda", dtype=F16)) if autocast else \
        (lambda: torch.autocast("cuda", enabled=False))
    x_dtype = F32 if autocast else F16
    x = (torch.randn(4, 96, 256, device="cuda") * 2).to(x_dtype)
    grad = torch.randn(4, 96, 256, device="cuda")
    x_ref = x.clone().requires_grad_()
    with ctx():
        out_ref = installed(mlp, x_ref)
    out_ref.backward(grad.to(out_ref.dtype))

    x_new = x.clone().requires_grad_()
    with ctx():
        out = mod._mlp_forward(mlp, x_new, installed)
    out.backward(grad.to(out.dtype))
    assert out.dtype == out_ref.dtype
    assert_close_rel_max(out, out_ref, 2e-3, "mlp output")
    assert_close_rel_max(x_new.grad, x_ref.grad, 2e-3, "mlp input gradient")

    x_hook = x.clone().requires_grad_()
    with ctx():
        _, kept = _saved_pointers(lambda: mod.MLPInputRecompute.apply(x_hook, mlp.gate_proj, mlp.up_proj))
    assert kept == [(x_hook.data_ptr(), x_dtype, tuple(x.shape))]


def _nf4_mlp():
    from claudemaxing_b200.qlora import NF4Linear

    modeling, mlp = _small_mlp()
    for name in ("gate_proj", "up_proj", "down_proj"):
        dense = getattr(mlp, name)
        setattr(mlp, name, NF4Linear.from_weight(dense.weight.data.half()).cuda())
    return modeling, mlp


@pytest.mark.parametrize("fused_gemm", [False, True])
@pytest.mark.parametrize("x_dtype", [F32, F16])
def test_nf4_mlp_fast_path_matches_the_module_path_bitwise(x_dtype, fused_gemm, monkeypatch):
    """With the two-step projections (dequantise, cuBLAS) the fast path equals the module-calling
    path bit for bit, as the reference's does. With the GEMM that dequantises in its prologue the
    outputs are still identical (same tiles, same order of accumulation), but the fast path sums
    the two input gradients in one accumulator where the module path rounds each to x's dtype
    first: equal to rounding, not to the bit."""
    mod = importlib.import_module("claudemaxing_b200.swiglu_recompute")
    from claudemaxing_b200.nf4 import dequantize_nf4
    from claudemaxing_b200.qlora import NF4Linear

    monkeypatch.setattr(NF4Linear, "fused_gemm", fused_gemm)

    modeling, mlp = _nf4_mlp()
    assert mod._four_bit_pair(mlp.gate_proj, mlp.up_proj, torch.zeros(1, device="cuda")) is not None
    installed = modeling.Qwen2MLP.forward
    x = (torch.randn(3, 80, 256, device="cuda") * 2).to(x_dtype)
    grad = torch.randn(3, 80, 256, device="cuda").to(x_dtype)

    def run(force_modules):
        real = mod._four_bit_pair
        if force_modules:
            mod._four_bit_pair = lambda *a: None
        try:
            xx = x.clone().requires_grad_()
            with torch.autocast("cuda", dtype=F16):
                out, kept = _saved_pointers(lambda: mod._mlp_forward(mlp, xx, installed))
            out.backward(grad.to(out.dtype))
            return out.detach(), xx.grad, kept
        finally:
            mod._four_bit_pair = real

    out, dx, kept = run(False)
    out_mod, dx_mod, _ = run(True)
    # the fast path hands the 4-bit down_proj its fp16 input directly, and NF4Linear casts its
    # output back to its input's dtype: fp16 out, the same numbers the module path returns after
    # its own cast back to x's dtype
    assert out_mod.dtype == x_dtype
    assert torch.equal(out.to(x_dtype), out_mod)
    if fused_gemm:
        assert_close_rel_max(dx, dx_mod, 2e-3, "input gradient, fast path against module path")
    else:
        assert torch.equal(dx, dx_mod)
    # nothing of size [rows, intermediate] survives forward: what is saved is x (as fp16) for
    # the recompute, and what down_proj's own matmul keeps is nothing (frozen 4-bit weight)
    rows = x.shape[0] * x.shape[1]
    assert all(shape[-1] != 704 for _, _, shape in kept), kept
    assert any(dtype == F16 and shape[-1] == 256 for _, dtype, shape in kept)
    assert sum(1 for _, _, shape in kept if len(shape) and torch.Size(shape).numel() >= rows * 256) <= 2
    # and it is the arithmetic of the plain formula on the dequantised weights
    w = {n: dequantize_nf4(getattr(mlp, n).packed, getattr(mlp, n).quant_state, F16).float()
         for n in ("gate_proj", "up_proj", "down_proj")}
    xf = x.float().half().float()
    ref = (torch.nn.functional.silu(xf @ w["gate_proj"].t()) * (xf @ w["up_proj"].t())) @ w["down_proj"].t()
    assert_close_rel_max(out, ref, 5e-3, "against the plain formula")


# --------------------------------------------------------------------------- tied embedding
def _tiny_lm(tied=True):
    from transformers import Qwen2Config, Qwen2ForCausalLM

    cfg = Qwen2Config(vocab_size=1000, hidden_size=64, intermediate_size=128, num_hidden_layers=1,
                      num_attention_heads=4, num_key_value_heads=2, tie_word_embeddings=tied)
    torch.manual_seed(0)
    model = Qwen2ForCausalLM(cfg).half().cuda()   # loaded in fp16 ...
    emb = model.get_input_embeddings()
    emb.weight.data = emb.weight.data.float()     # ... upcast and frozen, as k-bit preparation does
    if tied:
        model.lm_head.weight = emb.weight
    for p in model.parameters():
        p.requires_grad_(False)
    return model


def test_tied_embedding_shrinks_losslessly_and_lookups_keep_their_values():
    from claudemaxing_b200.embedding import shrink_tied_embedding

    model = _tiny_lm()
    emb, head = model.get_input_embeddings(), model.get_output_embeddings()
    assert head.weight is emb.weight and emb.weight.dtype == F32
    ref = emb.weight.detach().clone()
    ids = torch.randint(0, 1000, (2, 17), device="cuda")
    out_ref = emb(ids)
    seen = []
    emb.register_forward_hook(lambda m, i, o: seen.append(o.dtype))   # a peft-style hook still runs
    assert shrink_tied_embedding(model) is False          # outside fp16 autocast: not decided yet
    assert emb.weight.dtype == F32
    before = torch.cuda.memory_allocated()
    with torch.autocast("cuda", dtype=F16):
        assert shrink_tied_embedding(model) is True
    assert emb.weight.dtype == F16 and head.weight is emb.weight
    assert torch.equal(emb.weight.float(), ref)
    # the fp32 storage is gone: half of the weight's bytes were given back
    assert torch.cuda.memory_allocated() - before <= -(ref.numel() * 4) // 2 + 4096
    out = emb(ids)
    assert out.dtype == F32 and torch.equal(out, out_ref) and seen == [F32]
    assert shrink_tied_embedding(model) is True            # decided once
    with torch.autocast("cuda", dtype=F16):
        assert torch.equal(emb(ids), out_ref)
    assert torch.equal(copy.deepcopy(emb)(ids), out_ref)   # the fp32 lookup follows a deepcopy


def test_a_value_that_is_not_an_fp16_number_leaves_the_weight_alone():
    from claudemaxing_b200.embedding import shrink_tied_embedding

    model = _tiny_lm()
    w = model.get_input_embeddings().weight
    w.data[0, 0] = 1.0 + 2 ** -20
    with torch.autocast("cuda", dtype=F16):
        assert shrink_tied_embedding(model) is False
    assert w.dtype == F32 and w.data[0, 0].item() == 1.0 + 2 ** -20
    assert "forward" not in model.get_input_embeddings().__dict__


def test_untied_trainable_or_hooked_embeddings_are_left_alone():
    from claudemaxing_b200.embedding import shrink_tied_embedding

    with torch.autocast("cuda", dtype=F16):
        assert shrink_tied_embedding(_tiny_lm(tied=False)) is False
        model = _tiny_lm()
        model.get_input_embeddings().weight.requires_grad_(True)
        assert shrink_tied_embedding(model) is False
        model = _tiny_lm()
        model.get_input_embeddings().register_forward_pre_hook(lambda m, a: None)
        assert shrink_tied_embedding(model) is False
        assert model.get_input_embeddings().weight.dtype == F32
