"""Host-side logic that needs no GPU: the patch surface, label shifting, batch packing, the
compute-dtype rule, shard bounds, the quantiser against the oracle's."""

import torch

from claudemaxing_b200 import lm_head_loss as L
from claudemaxing_b200 import parallel, qlora


def test_apply_is_idempotent_and_class_level():
    import claudemaxing_b200 as solution
    from transformers.models.qwen2 import modeling_qwen2 as m

    solution.apply()
    first = (m.Qwen2RMSNorm.forward, m.Qwen2MLP.forward, m.apply_rotary_pos_emb,
             m.Qwen2ForCausalLM.forward)
    solution.apply()
    again = (m.Qwen2RMSNorm.forward, m.Qwen2MLP.forward, m.apply_rotary_pos_emb,
             m.Qwen2ForCausalLM.forward)
    assert all(a is b for a, b in zip(first, again))
    assert first[0]._fused_rmsnorm and first[1]._swiglu_recompute and first[2]._fused_rope
    assert first[3]._fused_head


def test_patched_modules_keep_original_behaviour_on_cpu():
    # the guards send CPU tensors to the installed implementation (third-party callers keep working)
    import claudemaxing_b200 as solution
    from transformers import Qwen2Config
    from transformers.models.qwen2 import modeling_qwen2 as m

    solution.apply()
    cfg = Qwen2Config(hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                      num_attention_heads=4, num_key_value_heads=2, vocab_size=50)
    norm = m.Qwen2RMSNorm(32)
    x = torch.randn(2, 5, 32)
    ref = norm.weight * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + norm.variance_epsilon))
    assert torch.allclose(norm(x), ref, atol=1e-6)
    mlp = m.Qwen2MLP(cfg)
    assert mlp(x).shape == x.shape
    q, k = torch.randn(1, 4, 5, 8), torch.randn(1, 2, 5, 8)
    cos, sin = torch.randn(1, 5, 8), torch.randn(1, 5, 8)
    oq, ok = m.apply_rotary_pos_emb(q, k, cos, sin)
    assert oq.shape == q.shape and ok.shape == k.shape


def test_shift_labels_left():
    labels = torch.tensor([[1, 2, 3], [4, -100, 6]])
    assert L.shift_labels_left(labels).tolist() == [[2, 3, -100], [-100, 6, -100]]


def test_head_compute_dtype_rule():
    h16, h32 = torch.zeros(1, dtype=torch.float16), torch.zeros(1)
    assert L.head_compute_dtype(h16, h16) == torch.float16
    assert L.head_compute_dtype(h32, h16) is None


def test_pack_tokens_layout():
    ids = torch.tensor([[5, 6, 7, 0], [8, 9, 0, 0]])
    mask = torch.tensor([[1, 1, 1, 0], [1, 1, 0, 0]])
    labels = ids.clone()
    p = L.pack_tokens(ids, mask, labels)
    assert p.ids.tolist() == [[5, 6, 7, 8, 9]] and p.pos.tolist() == [[0, 1, 2, 0, 1]]
    assert p.target.tolist() == [[6, 7, 0, 9, 0]]
    assert p.cu_rows.tolist() == [0, 3, 5] and p.cu_rows.dtype == torch.int32 and p.longest == 4
    allowed = p.mask[0, 0]   # the O(N^2) statement of the same segments, built on request
    assert allowed.shape == (5, 5) and allowed[2, :3].all() and not allowed[3, :3].any()
    assert allowed[4, 3] and not allowed[3, 4]
    assert L.pack_tokens(ids, torch.ones_like(mask), labels) is None  # nothing to drop
    assert L._chunk_tiles(None) == 0 and L._chunk_tiles(7) == 1 and L._chunk_tiles(8192) == 32


def test_segment_mask_is_the_row_and_column_rule_of_the_packed_batch():
    """`mask_of_segments` on the packed row's offsets is "same batch row and key column not after
    the query's" (the mask the reference's packing builds, solution/lm_head_loss.py:300-337), for
    ragged rows, left padding and a row without real tokens."""
    from claudemaxing_b200.attention import mask_of_segments, segment_arguments

    mask = torch.tensor([[1, 1, 1, 0, 0], [0, 0, 0, 0, 0], [0, 0, 1, 1, 1], [1, 0, 1, 0, 1]])
    ids = torch.arange(20).reshape(4, 5)
    p = L.pack_tokens(ids, mask, ids.clone())
    assert p.cu_rows.tolist() == [0, 3, 3, 6, 9]
    real = mask.reshape(-1).nonzero().reshape(-1)
    row, col = real // 5, real % 5
    want = (row[:, None] == row[None, :]) & (col[None, :] <= col[:, None])
    assert torch.equal(mask_of_segments(p.cu_rows, 9)[0, 0], want) and torch.equal(p.mask[0, 0], want)
    # without this package's attention function installed the decoder is given the mask itself
    from transformers.modeling_utils import AttentionInterface
    if not getattr(AttentionInterface._global_mapping.get("sdpa"), "_grouped_sdpa", False):
        args = segment_arguments(p.cu_rows, p.longest, 9)
        assert set(args) == {"attention_mask"} and torch.equal(args["attention_mask"][0, 0], want)


def test_shard_bounds_cover_the_vocabulary_in_whole_tiles():
    for vocab, world in ((151936, 8), (151936, 2), (5000, 4), (300, 4), (256, 1)):
        b = parallel.shard_bounds(vocab, world)
        assert b[0] == 0 and b[-1] == vocab and len(b) == world + 1
        assert all(x <= y for x, y in zip(b, b[1:]))
        assert all(x % 256 == 0 or x == vocab for x in b)
    sizes = [y - x for x, y in zip(*(lambda b: (b, b[1:]))(parallel.shard_bounds(151936, 8)))]
    assert max(sizes) - min(sizes) <= 512


def test_quantiser_and_tables_match_the_oracle():
    from oracle import nf4 as onf4

    assert torch.equal(qlora.normal_float4_levels(), onf4.nf4_code_table())
    assert torch.equal(qlora.absmax_levels(), onf4.dynamic_map())
    w = (torch.randn(64, 384, generator=torch.Generator().manual_seed(0)) * 0.02).half()
    for nested in (True, False):
        p1, s1 = qlora.quantize_nf4(w, nested=nested)
        p2, s2 = onf4.quantize_nf4(w, nested=nested)
        assert torch.equal(p1, p2) and torch.equal(s1.absmax, s2.absmax)
        if nested:
            assert torch.equal(s1.state2.absmax, s2.state2.absmax) and torch.equal(s1.offset, s2.offset)
        deq = onf4.dequantize_nf4(p1, s1)
        assert (deq.float() - w.float()).abs().max() < 0.2 * w.float().abs().max()


def test_nf4_supported_guard():
    from claudemaxing_b200.nf4 import _supported

    w = torch.zeros(4, 64, dtype=torch.float16)
    p, s = qlora.quantize_nf4(w)
    assert not _supported(p, s, torch.float16)  # CPU tensors are not for the kernel
    assert not _supported(p, None, torch.float16)


def test_fused_block_plan_accepts_this_package_s_layers_and_says_why_not_otherwise():
    """Host logic of decoder_block.py on a CPU model (no kernel runs): the structure check takes a
    block built by build_qlora_model, the q/k/v weights are adjacent in the group's buffer, and a
    call that is not the packed fp16-autocast training call is sent to the installed forward."""
    from claudemaxing_b200 import decoder_block as D
    from claudemaxing_b200 import qlora

    tiny = dict(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=2,
                num_key_value_heads=1, vocab_size=500, max_position_embeddings=128)
    model, lora = qlora.build_qlora_model("cpu", tiny, seed=0)
    layer = model.model.layers[0]
    plan = layer._soup_block
    assert plan.why_not == "" and plan.head_dim == 128 and plan.keep_products
    group = layer.self_attn.k_proj.group
    bases = [layer.self_attn.q_proj.base_layer, layer.self_attn.k_proj, layer.self_attn.v_proj.base_layer]
    assert group.stacked(bases, torch.float16, probe=True) is True
    assert group.stacked([bases[0], bases[2]], torch.float16, probe=True) is None     # not consecutive
    assert group.stacked([layer.mlp.up_proj, layer.mlp.down_proj], torch.float16, probe=True) is None   # other width
    casts = model.model.__dict__["_soup_adapter_casts"]
    assert len(casts.modules) == 2 * tiny["num_hidden_layers"] and not casts.armed
    casts.refresh()                      # CPU weights: nothing is cast, nothing is handed out
    assert not casts.armed and plan.adapter(layer.self_attn.k_proj, None) is None
    hidden = torch.zeros(1, 8, 256)
    cu = torch.tensor([0, 8], dtype=torch.int32)
    rope = (torch.zeros(1, 8, 128), torch.zeros(1, 8, 128))
    reason = D._why_not(plan, hidden, None, None, rope, {"cu_seq_lens_q": cu, "cu_seq_lens_k": cu})
    assert reason == "hidden states are not one contiguous fp32 CUDA row"
    assert "segment offsets" in D._why_not(plan, hidden, torch.ones(1, 1, 8, 8, dtype=torch.bool), None, rope, {})
    # a model whose blocks are not this package's layers is left alone
    from transformers import Qwen2Config, Qwen2ForCausalLM
    plain = Qwen2ForCausalLM(Qwen2Config(**tiny))
    assert D.install_fused_blocks(plain) == 0
    assert "NF4Linear" in D.BlockPlan(plain.model.layers[0]).why_not
    assert len(lora) == 4 * tiny["num_hidden_layers"]
