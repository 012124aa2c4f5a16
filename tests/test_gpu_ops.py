"""Parity of the memory-bound sm_100a kernels (through the C ABI) with the CPU oracle and with the
golden outputs of the reference's own kernels. NF4 and the dropout bits are compared bit for bit;
the floating-point ops use the reference's own tolerances (tests_local/ of the reference)."""

import pytest
import torch

from conftest import assert_close_rel_max, load_golden, rel_norm

pytestmark = pytest.mark.gpu

F16, F32, BF16 = torch.float16, torch.float32, torch.bfloat16
DEV = "cuda"


def _bits(t):
    return t.view(torch.int16) if t.element_size() == 2 else t.view(torch.int32)


# ----------------------------------------------------------------------------------- NF4
def _state_to_cuda(g):
    from oracle import nf4 as onf4

    nested = bool(g["nested"])
    inner = onf4.State(g["absmax2"], (g["absmax"].numel(),), g["code2"], g["blocksize2"],
                       F32) if nested else None
    return onf4.State(g["absmax"], tuple(g["shape"].tolist()), g["code"], g["blocksize"],
                      g["out"].dtype, offset=g["offset"] if nested else None, state2=inner)


@pytest.mark.parametrize("tag", ["a", "b", "c", "d"])
@pytest.mark.parametrize("dname", ["f16", "f32"])
def test_nf4_golden_bit_exact(tag, dname):
    from claudemaxing_b200.nf4 import dequantize_nf4

    g = load_golden(f"nf4_{tag}_{dname}")
    state = _state_to_cuda(g).to(DEV)
    out = dequantize_nf4(g["packed"].to(DEV), state)
    assert out.dtype == g["out"].dtype and out.shape == g["out"].shape
    assert torch.equal(_bits(out.cpu()), _bits(g["out"]))


@pytest.mark.parametrize("nested", [True, False])
@pytest.mark.parametrize("shape", [(1536, 1536), (256, 1536), (8960, 1536), (1536, 8960), (3, 64),
                                   (7, 34)])
def test_nf4_bit_exact_vs_oracle(shape, nested):
    # shapes of tests_local/test_nf4.py:27-29 plus one whose byte count is not a multiple of 16
    from claudemaxing_b200.nf4 import dequantize_nf4
    from oracle import nf4 as onf4

    gen = torch.Generator().manual_seed(shape[0] * 7 + nested)
    w = (torch.randn(*shape, generator=gen) * 0.05).half()
    w.view(-1)[:5] = torch.tensor([0.0, -0.0, 1e-7, 3.0, -2.5]).half()
    blocksize = 64 if shape != (7, 34) else 32
    packed, state = onf4.quantize_nf4(w, blocksize=blocksize, nested=nested)
    ref16 = onf4.dequantize_nf4(packed, state, F16)
    out16 = dequantize_nf4(packed.to(DEV), state.to(DEV))
    assert out16.dtype == F16 and out16.shape == ref16.shape
    assert torch.equal(_bits(out16.cpu()), _bits(ref16))
    out32 = dequantize_nf4(packed.to(DEV), state.to(DEV), F32)
    assert torch.equal(_bits(out32.cpu()), _bits(onf4.dequantize_nf4(packed, state, F32)))
    assert torch.equal(out32.half().cpu(), ref16)


def test_nf4_quantiser_matches_oracle_and_roundtrip_is_idempotent():
    from claudemaxing_b200 import qlora
    from claudemaxing_b200.nf4 import dequantize_nf4
    from oracle import nf4 as onf4

    w = (torch.randn(512, 1536, generator=torch.Generator().manual_seed(3)) * 0.02).half()
    p_dev, s_dev = qlora.quantize_nf4(w.to(DEV))
    p_cpu, s_cpu = onf4.quantize_nf4(w)
    assert torch.equal(p_dev.cpu(), p_cpu)
    # the nested codes depend on mean(absmax), whose summation order differs between CPU and GPU
    assert abs(s_dev.offset.item() - s_cpu.offset.item()) < 1e-6
    assert (s_dev.absmax.cpu() != s_cpu.absmax).float().mean().item() < 0.01
    deq = dequantize_nf4(p_dev, s_dev)
    # quantising the dequantised weight again reproduces the same codes (a fixed point)
    p_again, _ = qlora.quantize_nf4(deq, nested=False)
    p_first, _ = qlora.quantize_nf4(w.to(DEV), nested=False)
    assert (p_again != p_first).float().mean().item() < 0.02


def test_nf4_batched_launch_is_bit_identical_to_single_launches():
    from claudemaxing_b200.nf4 import dequantize_nf4, dequantize_nf4_batch
    from oracle import nf4 as onf4

    shapes = [(1536, 1536), (256, 1536), (256, 1536), (1536, 1536), (8960, 1536), (8960, 1536),
              (1536, 8960), (3, 64), (7, 34)]  # one decoder layer + two odd ones: two launches
    weights = []
    for i, shape in enumerate(shapes):
        w = (torch.randn(*shape, generator=torch.Generator().manual_seed(i)) * 0.02).half()
        packed, state = onf4.quantize_nf4(w, blocksize=64)
        weights.append((packed.to(DEV), state.to(DEV)))
    batched = dequantize_nf4_batch(weights)
    for (packed, state), got in zip(weights, batched):
        assert torch.equal(_bits(got), _bits(dequantize_nf4(packed, state)))


def test_nf4_rejects_bad_arguments():
    from claudemaxing_b200 import _lib

    x = torch.zeros(64, dtype=torch.uint8, device=DEV)
    with pytest.raises(RuntimeError, match="blocksize"):
        _lib.call("soup_nf4_dequant", x.data_ptr(), x.data_ptr(), x.data_ptr(), None, None, None,
                  x.data_ptr(), 128, 48, 1, 0, _lib.F16, 0)


# ----------------------------------------------------------------------------------- RMSNorm
@pytest.mark.parametrize("tag", ["f16f32", "f16f16", "f32f32"])
def test_rmsnorm_golden(tag):
    from claudemaxing_b200.rmsnorm import rmsnorm

    g = load_golden(f"rmsnorm_{tag}")
    x = g["x"].to(DEV).requires_grad_(True)
    w = g["w"].to(DEV).requires_grad_(True)
    out = rmsnorm(x, w, 1e-6)
    out.backward(g["dy"].to(DEV))
    tol = 2e-3 if F16 in (g["x"].dtype, g["w"].dtype) else 1e-4
    assert out.dtype == g["out"].dtype
    assert_close_rel_max(out.detach().cpu(), g["out"], tol, "out")
    assert_close_rel_max(x.grad.cpu(), g["dx"], tol, "dx")
    assert_close_rel_max(w.grad.cpu(), g["dw"], 5e-3, "dw")


@pytest.mark.parametrize("shape", [(4, 512, 1536), (3, 77, 1001), (2, 1, 4096), (1, 3, 16384),
                                   (2, 33, 1288), (5, 7, 2048), (1, 19, 64), (3, 11, 3072)])
@pytest.mark.parametrize("dtypes", [(F16, F32), (F16, F16), (F32, F32), (BF16, BF16)])
@pytest.mark.parametrize("train_w", [False, True])
def test_rmsnorm_vs_oracle(shape, dtypes, train_w):
    from claudemaxing_b200.rmsnorm import rmsnorm
    from oracle import elementwise as ew

    xdt, wdt = dtypes
    gen = torch.Generator().manual_seed(1)
    x = (3 * torch.randn(*shape, generator=gen)).to(xdt)
    w = (1 + 0.5 * torch.randn(shape[-1], generator=gen)).to(wdt)
    dy = torch.randn(*shape, generator=gen).to(torch.promote_types(xdt, wdt))
    ref_out, ref_dx, ref_dw = ew.rmsnorm_fwd_bwd(x, w, dy, weight_grad=train_w)
    xd = x.to(DEV).requires_grad_(True)
    wd = w.to(DEV).requires_grad_(train_w)
    out = rmsnorm(xd, wd, 1e-6)
    out.backward(dy.to(DEV))
    tol = 1e-4 if dtypes == (F32, F32) else (2e-3 if BF16 not in dtypes else 1.6e-2)
    assert out.dtype == ref_out.dtype and xd.grad.dtype == xdt
    assert_close_rel_max(out.detach().cpu(), ref_out, tol, "out")
    assert_close_rel_max(xd.grad.cpu(), ref_dx, tol, "dx")
    if train_w:
        assert_close_rel_max(wd.grad.cpu(), ref_dw, 5 * tol, "dw")
    else:
        assert wd.grad is None


def test_rmsnorm_fp16_copy_path_and_tiny_weights():
    # fp32 x, frozen fp32 w: forward leaves an fp16 copy for the next layers, backward uses it;
    # a 2e5 "massive activation" channel and tiny / zero weights (tests_local/test_rmsnorm.py:197-277)
    from claudemaxing_b200.rmsnorm import fp16_copy_of, rmsnorm
    from oracle import elementwise as ew

    gen = torch.Generator().manual_seed(2)
    x = torch.randn(2, 300, 1536, generator=gen)
    x[..., 7] = 2e5
    w = 1 + 0.5 * torch.randn(1536, generator=gen)
    w[3], w[50], w[900], w[1000] = 1e-5, -6.5e-6, 3e-4, 0.0
    dy = torch.randn(2, 300, 1536, generator=gen)
    x64, w64 = x.double().requires_grad_(True), w.double()
    ew.rmsnorm(x64, w64).backward(dy.double())
    xd = x.to(DEV).requires_grad_(True)
    wd = w.to(DEV)
    out = rmsnorm(xd, wd, 1e-6)
    low = fp16_copy_of(out)
    assert low is not None and low.dtype == F16 and torch.equal(low, out.detach().half())
    assert fp16_copy_of(out.detach().clone()) is None
    out.backward(dy.to(DEV))
    assert rel_norm(xd.grad.cpu(), x64.grad) < 1e-3
    out.detach().add_(1)  # a changed tensor (shared version counter) no longer has a copy
    assert fp16_copy_of(out) is None


# ----------------------------------------------------------------------------------- RoPE
@pytest.mark.parametrize("tag,tol", [("f16", 2e-3), ("f32", 1e-5)])
def test_rope_golden(tag, tol):
    from claudemaxing_b200.rope import rope

    g = load_golden(f"rope_{tag}")
    q = g["q"].to(DEV).requires_grad_(True)
    k = g["k"].to(DEV).requires_grad_(True)
    oq, ok = rope(q, k, g["cos"].to(DEV), g["sin"].to(DEV))
    torch.autograd.backward((oq, ok), (g["gq"].to(DEV), g["gk"].to(DEV)))
    for name, val in (("q_out", oq), ("k_out", ok), ("dq", q.grad), ("dk", k.grad)):
        assert_close_rel_max(val.detach().cpu(), g[name], tol, name)


@pytest.mark.parametrize("dims", [(4, 512, 12, 2, 128), (2, 37, 4, 4, 64), (1, 1, 2, 1, 128),
                                  (2, 5, 3, 1, 24)])
@pytest.mark.parametrize("dtype", [F32, F16])
@pytest.mark.parametrize("cos_batch_one", [False, True])
def test_rope_vs_oracle(dims, dtype, cos_batch_one):
    # shapes of tests_local/test_rope.py:28-31; q and k are transposed views, as in the model
    from claudemaxing_b200.rope import rope
    from oracle import elementwise as ew

    b, t, h, kv, d = dims
    gen = torch.Generator().manual_seed(0)
    q = torch.randn(b, t, h * d, generator=gen).to(dtype).view(b, t, h, d).transpose(1, 2)
    k = torch.randn(b, t, kv * d, generator=gen).to(dtype).view(b, t, kv, d).transpose(1, 2)
    cb = 1 if cos_batch_one else b
    pos = torch.arange(t, dtype=F32)[None].expand(cb, t)
    inv = 1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=F32) / d))
    emb = torch.cat((pos[..., None] * inv,) * 2, -1)
    cos, sin = emb.cos().to(dtype), emb.sin().to(dtype)
    gq, gk = torch.randn(b, h, t, d, generator=gen).to(dtype), torch.randn(b, kv, t, d, generator=gen).to(dtype)
    ref = ew.rope_fwd_bwd(q, k, cos, sin, gq, gk)
    qd = q.to(DEV).requires_grad_(True)
    kd = k.to(DEV).requires_grad_(True)
    oq, ok = rope(qd, kd, cos.to(DEV), sin.to(DEV))
    assert oq.is_contiguous() and oq.shape == (b, h, t, d) and oq.dtype == dtype
    torch.autograd.backward((oq, ok), (gq.to(DEV), gk.to(DEV)))
    tol = 2e-3 if dtype == F16 else 1e-5
    for name, val, r in zip(("q", "k", "dq", "dk"), (oq, ok, qd.grad, kd.grad), ref):
        assert_close_rel_max(val.detach().cpu(), r, tol, name)


def test_rope_packed_positions_restart_per_row():
    # benchmark config 3: one packed row of lengths {512,384,640,512}, positions restart at 0
    from claudemaxing_b200.rope import rope
    from oracle import elementwise as ew

    gen = torch.Generator().manual_seed(2)
    pos = torch.cat([torch.arange(n) for n in (512, 384, 640, 512)])
    cos, sin = ew.rope_tables(pos, 128, dtype=F16)
    q = torch.randn(1, 2048, 12 * 128, generator=gen).half().view(1, 2048, 12, 128).transpose(1, 2)
    k = torch.randn(1, 2048, 2 * 128, generator=gen).half().view(1, 2048, 2, 128).transpose(1, 2)
    rq, rk = ew.rope(q, k, cos, sin)
    oq, ok = rope(q.to(DEV), k.to(DEV), cos.to(DEV), sin.to(DEV))
    assert_close_rel_max(oq.cpu(), rq, 2e-3)
    assert_close_rel_max(ok.cpu(), rk, 2e-3)
    # rotation preserves the norm of every (x1, x2) pair up to rounding
    assert abs(oq.float().norm().item() / q.float().norm().item() - 1) < 1e-3


@pytest.mark.parametrize("dims", [(1280, 12, 2, 128), (37, 4, 4, 64), (5, 3, 1, 24)])
@pytest.mark.parametrize("with_term", [True, False])
def test_rope_of_a_sum_into_strided_outputs_is_the_chain_it_replaces(dims, with_term):
    """`rotate_into`: fp16 q (a column block of a wider projection output) + fp16 second term,
    fp32 tables, fp16 [tokens, heads, head_dim] outputs: bit-identical to what the per-op chain
    reaches (fp32 sum, rotation in fp32 through `rope`, one cast to fp16); and the transposed
    rotation written into column blocks of a wider gradient buffer."""
    from claudemaxing_b200.rope import rope, rotate_into

    t, h, kv, d = dims
    gen = torch.Generator().manual_seed(3)
    wide = torch.randn(t, (h + 2 * kv) * d, generator=gen).half().to(DEV)   # [q | k | v] columns
    term = torch.randn(1, t, h * d, generator=gen).half().to(DEV) if with_term else None
    pos = torch.arange(t, dtype=F32)[None]
    inv = 1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=F32) / d))
    emb = torch.cat((pos[..., None] * inv,) * 2, -1)
    cos, sin = emb.cos().to(DEV), emb.sin().to(DEV)

    def heads_first(x, heads):
        return x.unflatten(-1, (heads, d)).unsqueeze(0).transpose(1, 2)

    q_in, k_in = heads_first(wide[:, :h * d], h), heads_first(wide[:, h * d:(h + kv) * d], kv)
    q_out = torch.empty(t, h, d, dtype=F16, device=DEV)
    k_out = torch.empty(t, kv, d, dtype=F16, device=DEV)
    rotate_into(q_in, None if term is None else heads_first(term[0], h), k_in, cos, sin,
                q_out.unsqueeze(0).transpose(1, 2), k_out.unsqueeze(0).transpose(1, 2))
    q_sum = q_in.float() if term is None else q_in.float() + heads_first(term[0], h).float()
    want_q, want_k = rope(q_sum, k_in.float(), cos, sin)
    assert torch.equal(q_out, want_q.half().transpose(1, 2)[0])
    assert torch.equal(k_out, want_k.half().transpose(1, 2)[0])
    # backward: fp16 gradients in, fp16 column blocks out; the chain casts the fp32 result once
    gq = torch.randn(t, h, d, generator=gen).half().to(DEV)
    gk = torch.randn(t, kv, d, generator=gen).half().to(DEV)
    buf = torch.full((t, (h + 2 * kv) * d), 7.0, dtype=F16, device=DEV)
    rotate_into(gq.unsqueeze(0).transpose(1, 2), None, gk.unsqueeze(0).transpose(1, 2), cos, sin,
                heads_first(buf[:, :h * d], h), heads_first(buf[:, h * d:(h + kv) * d], kv), backward=True)
    q_leaf = q_sum.clone().requires_grad_()
    k_leaf = k_in.float().clone().requires_grad_()
    oq, ok = rope(q_leaf, k_leaf, cos, sin)
    torch.autograd.backward((oq, ok), (gq.float().unsqueeze(0).transpose(1, 2), gk.float().unsqueeze(0).transpose(1, 2)))
    assert torch.equal(buf[:, :h * d], q_leaf.grad.half().transpose(1, 2)[0].reshape(t, h * d))
    assert torch.equal(buf[:, h * d:(h + kv) * d], k_leaf.grad.half().transpose(1, 2)[0].reshape(t, kv * d))
    assert (buf[:, (h + kv) * d:] == 7.0).all()    # the v block is not this kernel's to write


@pytest.mark.parametrize("rows,cols", [(1280, 1536), (37, 256), (5, 4096)])
@pytest.mark.parametrize("with_residual", [True, False])
def test_rmsnorm_backward_with_the_residual_gradient_folded_in(rows, cols, with_residual):
    """`soup_rmsnorm_bwd_residual` = the saved-output RMSNorm backward, plus the residual branch's
    gradient, plus the fp16 copy of the sum: bit-identical to the backward kernel followed by
    torch's add and cast; and the autograd node `_NormResidual` gives the gradients of
    norm(h) and h + f(norm(h)) composed the plain way."""
    import importlib

    from claudemaxing_b200 import _lib

    rms = importlib.import_module("claudemaxing_b200.rmsnorm")
    block = importlib.import_module("claudemaxing_b200.decoder_block")
    gen = torch.Generator().manual_seed(8)
    h = torch.randn(1, rows, cols, generator=gen).to(DEV).requires_grad_()
    w = (torch.randn(cols, generator=gen) * 0.3 + 1.0).to(DEV)
    w[3] = 1e-5                                   # a tiny-|w| column goes through the side buffer
    dy = torch.randn(1, rows, cols, generator=gen).to(DEV)
    res = torch.randn(1, rows, cols, generator=gen).to(DEV) if with_residual else None
    out, rstd, low, slots, small = rms._forward_launch(h.detach().view(rows, cols), w, 1e-6, F32, True)
    plain = torch.empty(rows, cols, device=DEV)
    _lib.call("soup_rmsnorm_bwd", _lib.ptr(dy), _lib.ptr(low), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(plain),
              None, None, _lib.ptr(slots), _lib.ptr(small), small.shape[-1], rows, cols, _lib.F32,
              _lib.F16, _lib.F32, _lib.F32, 1, _lib.stream_of(dy))
    want = plain if res is None else plain + res.view(rows, cols)
    dx, dx16 = torch.empty(rows, cols, device=DEV), torch.empty(rows, cols, dtype=F16, device=DEV)
    try:
        _lib.call("soup_rmsnorm_bwd_residual", _lib.ptr(dy), _lib.ptr(low), _lib.ptr(w), _lib.ptr(rstd),
                  _lib.ptr(res), _lib.ptr(dx), _lib.ptr(dx16), _lib.ptr(slots), _lib.ptr(small),
                  small.shape[-1], rows, cols, _lib.stream_of(dy))
    except RuntimeError as err:     # rows too wide for the saved-output kernel: said so, not guessed
        assert cols > 1024 * 3 and "does not take the residual form" in str(err)
    else:
        assert cols <= 1024 * 3
        assert torch.equal(dx, want) and torch.equal(dx16, want.half())
    # the autograd node: y = norm(h) * 2 + h (a branch on the norm and the residual connection)
    x, h_res = block._NormResidual.apply(h, w, 1e-6)
    (x * 2.0 + h_res).backward(dy)
    h2 = h.detach().clone().requires_grad_()
    (rms.rmsnorm(h2, w, 1e-6) * 2.0 + h2).backward(dy)
    assert_close_rel_max(h.grad.cpu(), h2.grad.cpu(), 1e-5, "gradient through norm and residual")
    copy = block._GradCopies.take(h.grad)
    assert copy is None or torch.equal(copy.view_as(h.grad), h.grad.half())


# ----------------------------------------------------------------------------------- SwiGLU
@pytest.mark.parametrize("tag", ["f16", "f32", "mix", "noround"])
def test_swiglu_golden(tag):
    from claudemaxing_b200.swiglu_recompute import _silu_mul_bwd, _silu_mul_fwd

    g = load_golden(f"swiglu_{tag}")
    gate, up, dy = g["gate"].to(DEV), g["up"].to(DEV), g["dy"].to(DEV)
    out = torch.empty(gate.shape, dtype=g["out"].dtype, device=DEV)
    _silu_mul_fwd(gate, up, out, bool(g["round_silu"]))
    dg, du = torch.empty_like(gate), torch.empty_like(up)
    _silu_mul_bwd(dy, gate, up, dg, du, bool(g["round_silu"]))
    tol = 1e-4 if tag == "f32" else 2e-3
    assert_close_rel_max(out.cpu(), g["out"], tol, "out")
    assert_close_rel_max(dg.cpu(), g["dgate"], tol, "dgate")
    assert_close_rel_max(du.cpu(), g["dup"], tol, "dup")


@pytest.mark.parametrize("shape", [(4, 512, 8960), (3, 77, 1001), (1, 1, 8960), (5, 3)])
@pytest.mark.parametrize("dtypes", [(F16, F16), (F32, F32), (F16, F32), (F32, F16)])
@pytest.mark.parametrize("inplace", [False, True])
def test_swiglu_vs_oracle(shape, dtypes, inplace):
    from claudemaxing_b200.swiglu_recompute import swiglu_recompute
    from oracle import elementwise as ew

    gdt, udt = dtypes
    gen = torch.Generator().manual_seed(5)
    gate = torch.randn(*shape, generator=gen).to(gdt)
    up = torch.randn(*shape, generator=gen).to(udt)
    dy = torch.randn(*shape, generator=gen).to(torch.promote_types(gdt, udt))
    r_out, r_dg, r_du = ew.swiglu_fwd_bwd(gate, up, dy)
    g = gate.to(DEV).requires_grad_(True)
    u = up.to(DEV).requires_grad_(True)
    # inplace works on temporaries: feed clones whose storage backward may overwrite
    gi, ui = (g * 1, u * 1) if inplace else (g, u)
    out = swiglu_recompute(gi, ui, inplace)
    assert out.dtype == r_out.dtype
    out.backward(dy.to(DEV))
    tol = 1e-4 if dtypes == (F32, F32) else 2e-3
    assert_close_rel_max(out.detach().cpu(), r_out, tol, "out")
    assert_close_rel_max(g.grad.cpu(), r_dg, tol, "dgate")
    assert_close_rel_max(u.grad.cpu(), r_du, tol, "dup")
    if inplace:  # the gradients landed in the storage of the saved inputs
        assert gi.data_ptr() == g.grad.data_ptr() or torch.equal(gi.detach(), g.grad)
    else:
        assert torch.equal(g.detach().cpu(), gate) and torch.equal(u.detach().cpu(), up)


def test_swiglu_saves_exactly_gate_and_up_and_one_sided_grads():
    from claudemaxing_b200.swiglu_recompute import swiglu_recompute

    saved = []
    gate = torch.randn(64, 256, device=DEV, dtype=F16, requires_grad=True)
    up = torch.randn(64, 256, device=DEV, dtype=F16)
    with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(t) or t, lambda t: t):
        out = swiglu_recompute(gate, up)
    assert {t.data_ptr() for t in saved} == {gate.data_ptr(), up.data_ptr()}
    out.sum().backward()
    assert gate.grad is not None and up.grad is None


# ----------------------------------------------------------------------------------- dropout bits
def test_dropout_golden_bit_exact():
    from claudemaxing_b200.lora import _pack, _unpack

    g = load_golden("dropout")
    xd, bits = _pack(g["x"].to(DEV), g["mask"].to(DEV), g["scale"])
    assert torch.equal(bits.cpu(), g["bits"]) and torch.equal(_bits(xd.cpu()), _bits(g["xd"]))
    xd2, dx = _unpack(g["x16"].to(DEV), bits, g["g16"].to(DEV), g["scale"], F32)
    assert torch.equal(_bits(xd2.cpu()), _bits(g["xd2"])) and torch.equal(dx.cpu(), g["dx"])


@pytest.mark.parametrize("shape", [(3, 37, 64), (2048, 1536), (1, 8), (5, 24)])
@pytest.mark.parametrize("xdt", [F32, F16])
def test_dropout_bit_exact_vs_oracle(shape, xdt):
    from claudemaxing_b200.lora import _pack, _unpack
    from oracle import elementwise as ew

    gen = torch.Generator().manual_seed(9)
    x = torch.randn(*shape, generator=gen).to(xdt)
    mask = torch.rand(*shape, generator=gen) > 0.05
    scale = 1.0 / 0.95
    r_xd, r_bits = ew.dropout_pack(x, mask, scale)
    xd, bits = _pack(x.to(DEV), mask.to(DEV), scale)
    assert torch.equal(bits.cpu(), r_bits) and torch.equal(_bits(xd.cpu()), _bits(r_xd))
    g16 = torch.randn(*shape, generator=gen).half()
    r_xd2, r_dx = ew.dropout_unpack(x.half(), r_bits, g16, scale, F32)
    xd2, dx = _unpack(x.half().to(DEV), bits, g16.to(DEV), scale, F32)
    assert torch.equal(_bits(xd2.cpu()), _bits(r_xd2)) and torch.equal(dx.cpu(), r_dx)
    # pack -> unpack keeps the kept elements: unpacked bits give the mask back
    assert torch.equal((dx != 0).cpu() | (g16 == 0), mask | (g16 == 0))


def test_lora_branch_matches_plain_formula():
    # the branch against base-free peft math on the same dropout mask (same RNG stream)
    from claudemaxing_b200.lora import LoRABranch

    torch.manual_seed(0)
    x = torch.randn(4, 50, 256, device=DEV, requires_grad=True)
    a = torch.randn(16, 256, device=DEV, requires_grad=True) * 0.1
    b = torch.randn(64, 16, device=DEV, requires_grad=True) * 0.1
    a.retain_grad(), b.retain_grad()
    torch.manual_seed(123)
    out = LoRABranch.apply(x, x.detach().half(), a, b, 0.05, 2.0)
    g = torch.randn_like(out)
    out.backward(g)
    torch.manual_seed(123)
    x2 = x.detach().clone().requires_grad_(True)
    a2, b2 = a.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    xd = torch.nn.functional.dropout(x2, 0.05, True).half()
    ref = torch.nn.functional.linear(torch.nn.functional.linear(xd, a2.half()), b2.half()) * 2.0
    ref.backward(g)
    assert torch.equal(out, ref)
    assert rel_norm(x.grad.cpu(), x2.grad.cpu()) < 2e-3
    assert rel_norm(a.grad.cpu(), a2.grad.cpu()) < 5e-3
    assert rel_norm(b.grad.cpu(), b2.grad.cpu()) < 5e-3


@pytest.mark.parametrize("scaling", [2.0, 1.7])
def test_lora_branch_with_cast_scaled_weights_and_in_place_gradients(scaling, monkeypatch):
    """The branch given fp16 A and fp16(scaling * B) copies (no scaling pass over its output or
    the incoming gradient), adding its weight gradients into existing `.grad` tensors inside the
    GEMMs: the plain call's numbers (identical for a power-of-two scaling)."""
    from claudemaxing_b200.lora import LoRABranch

    torch.manual_seed(0)
    x = torch.randn(3, 40, 256, device=DEV)
    a = (torch.randn(16, 256, device=DEV) * 0.1).requires_grad_()
    b = (torch.randn(64, 16, device=DEV) * 0.1).requires_grad_()
    g = torch.randn(3, 40, 64, device=DEV).half()
    results = []
    for fast in (False, True):
        xx = x.clone().requires_grad_()
        a.grad, b.grad = torch.full_like(a, 0.5), torch.full_like(b, -0.25)   # something to add to
        kept = (a.grad, b.grad)
        monkeypatch.setattr(LoRABranch, "accumulate_in_place", fast)
        torch.manual_seed(7)
        extra = (a.detach().half(), (b.detach() * scaling).half(), True) if fast else ()
        out = LoRABranch.apply(xx, xx.detach().half(), a, b, 0.1, scaling, *extra)
        out.backward(g)
        assert (a.grad is kept[0] and b.grad is kept[1]) or not fast
        results.append((out.detach(), xx.grad, a.grad.clone(), b.grad.clone()))
    for name, plain, fast in zip(("out", "dx", "dA", "dB"), *results):
        if scaling == 2.0 and name in ("out", "dx"):
            assert torch.equal(plain, fast), name
        assert rel_norm(fast.float().cpu(), plain.float().cpu()) < 2e-3, name


def test_paired_lora_branches_are_the_two_single_branches():
    """LoRABranchPair (one packing launch, one batched product with A, one unpacking launch that
    sums the input gradients) against two LoRABranch calls with the same dropout draws: outputs
    and weight gradients per adapter and the summed input gradient, bit for bit."""
    from claudemaxing_b200.lora import LoRABranch, LoRABranchPair

    torch.manual_seed(0)
    x = torch.randn(1, 80, 256, device=DEV)
    weights = [(torch.randn(16, 256, device=DEV) * 0.1).requires_grad_(),
               (torch.randn(96, 16, device=DEV) * 0.1).requires_grad_(),
               (torch.randn(16, 256, device=DEV) * 0.1).requires_grad_(),
               (torch.randn(32, 16, device=DEV) * 0.1).requires_grad_()]
    g1, g2 = torch.randn(1, 80, 96, device=DEV).half(), torch.randn(1, 80, 32, device=DEV).half()
    a16 = torch.stack([weights[0].detach().half(), weights[2].detach().half()])
    b1, b2 = (weights[1].detach() * 2.0).half(), (weights[3].detach() * 2.0).half()
    results = []
    for paired in (False, True):
        xx = x.clone().requires_grad_()
        for w in weights:
            w.grad = None
        torch.manual_seed(5)
        if paired:
            o1, o2 = LoRABranchPair.apply(xx, xx.detach().half(), *weights, 0.1, 0.1, 2.0, 2.0, a16, b1, b2)
        else:
            o1 = LoRABranch.apply(xx, xx.detach().half(), weights[0], weights[1], 0.1, 2.0, a16[0], b1, True)
            o2 = LoRABranch.apply(xx, xx.detach().half(), weights[2], weights[3], 0.1, 2.0, a16[1], b2, True)
        torch.autograd.backward((o1, o2), (g1, g2))
        results.append([o1.detach(), o2.detach(), xx.grad] + [w.grad.clone() for w in weights])
    for name, single, pair in zip(("out1", "out2", "dx", "dA1", "dB1", "dA2", "dB2"), *results):
        assert torch.equal(single, pair), name


def test_ops_refuse_cpu_tensors():
    from claudemaxing_b200.rmsnorm import rmsnorm
    from claudemaxing_b200.swiglu_recompute import swiglu_recompute

    with pytest.raises(RuntimeError, match="CUDA"):
        rmsnorm(torch.randn(4, 64), torch.ones(64), 1e-6)
    with pytest.raises(RuntimeError, match="CUDA"):
        swiglu_recompute(torch.randn(4, 64), torch.randn(4, 64))


# ------------------------------------------------------------------------- bounded waits
def test_a_wait_that_nothing_completes_runs_out_and_reports():
    """Failure detection on the device: the kernels' waits give up after their limit, record a
    code and return; the context stays usable (no trap, no hang)."""
    import ctypes

    from claudemaxing_b200 import _lib

    gave_up, status = ctypes.c_int(-1), ctypes.c_int(-1)
    _lib.call("soup_wait_selftest", 2_000_000, ctypes.byref(gave_up), ctypes.byref(status),
              torch.cuda.current_stream().cuda_stream)
    assert gave_up.value == 1 and status.value == 99
    # the device still works
    x = torch.arange(8, device=DEV).sum().item()
    assert x == 28
    # the code reached the device's sticky status word, where the host-side check finds it: the
    # package raises instead of handing out results of a step whose kernels gave up
    row = ctypes.c_int(-1)
    _lib.call("soup_row_status", ctypes.byref(row), torch.cuda.current_stream().cuda_stream)
    assert row.value == 99
    with pytest.raises(RuntimeError, match="device status 99"):
        _lib.check_device_status()
    _lib.check_device_status()          # cleared by the failing check: healthy again
    assert _lib.device_status() == 0


def test_device_status_stays_clear_after_a_healthy_step():
    from claudemaxing_b200 import _lib, fused_head_loss

    _lib.device_status(clear=True)
    gen = torch.Generator().manual_seed(3)
    h = torch.randn(300, 256, generator=gen).half().to(DEV).requires_grad_(True)
    w = (torch.randn(5000, 256, generator=gen) * 0.05).half().to(DEV)
    t = torch.randint(0, 5000, (300,), generator=gen).to(DEV)
    loss, _ = fused_head_loss(h[None], w, None, target=t[None])
    loss.backward()
    _lib.check_device_status()
