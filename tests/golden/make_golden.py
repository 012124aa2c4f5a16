"""Generates tests/golden/*.npz by running the reference's own Triton kernels on the CPU.

Run in the authoring container only (it needs the reference checkout and Triton):

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference

Triton's interpreter executes `@triton.jit` functions with numpy on CPU tensors, so the stored
outputs are what the reference's kernels compute (fp32 arithmetic is unfused there, as in the
reference's NF4 launch with enable_fp_fusion=False). Inputs are seeded and stored next to the
outputs, so the tests need neither the reference nor Triton. One shim: kernels that call `.to()`
on a Python `range` index get a `range` that yields interpreter tensors; the kernels' source is
not touched.
"""

import os
import sys

import numpy as np
import torch

assert os.environ.get("TRITON_INTERPRET") == "1", "run with TRITON_INTERPRET=1"
if len(sys.argv) < 2:
    sys.exit("usage: TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference")
REF = sys.argv[1]
sys.path.insert(0, REF)
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
OUT = os.path.dirname(os.path.abspath(__file__))

import triton.language as tl  # noqa: E402

from oracle import nf4 as onf4  # noqa: E402  (only for the stand-in tables and the quantiser)


def _tensor_range(a, b=None, c=1):
    def val(v):
        return int(v.handle.data.item()) if hasattr(v, "handle") else int(v)

    if b is None:
        a, b = 0, a
    for i in range(val(a), val(b), val(c)):
        yield tl.program_id(0) * 0 + i


def npy(t):
    return t.detach().cpu().numpy()


def save(name, **arrays):
    path = os.path.join(OUT, name + ".npz")
    np.savez_compressed(path, **{k: (npy(v) if torch.is_tensor(v) else np.asarray(v))
                                 for k, v in arrays.items()})
    print("wrote", path, os.path.getsize(path), "bytes")


def golden_nf4():
    from solution import nf4 as ref

    for tag, shape, nested in (("a", (3, 64), True), ("b", (24, 256), True), ("c", (24, 256), False),
                               ("d", (5, 96), True)):
        torch.manual_seed(11)
        w = (torch.randn(*shape) * 0.05).half()
        w.view(-1)[:5] = torch.tensor([0.0, -0.0, 1e-7, 3.0, -2.5]).half()  # test_nf4.py:21
        blocksize = 32 if tag == "d" else 64
        packed, st = onf4.quantize_nf4(w, blocksize=blocksize, nested=nested)
        n = w.numel()
        for dtype, dname in ((torch.float16, "f16"), (torch.float32, "f32")):
            out = torch.empty(shape, dtype=dtype)
            s2 = st.state2
            ref.nf4_dequant_kernel[(-(-(n // 2) // ref.BLOCK),)](
                packed, st.absmax, st.code, s2.code if nested else st.code,
                s2.absmax if nested else st.absmax, st.offset if nested else st.absmax, out, n // 2,
                BLOCKSIZE=blocksize, BLOCKSIZE2=s2.blocksize if nested else 1, NESTED=nested,
                BLOCK=ref.BLOCK, num_warps=ref.WARPS)
            save(f"nf4_{tag}_{dname}", packed=packed, absmax=st.absmax, code=st.code,
                 code2=s2.code if nested else np.zeros(0, np.float32),
                 absmax2=s2.absmax if nested else np.zeros(0, np.float32),
                 offset=st.offset if nested else np.zeros(0, np.float32),
                 shape=np.array(shape), blocksize=blocksize, blocksize2=s2.blocksize if nested else 1,
                 nested=int(nested), out=out)


def golden_rmsnorm():
    from solution import rmsnorm as ref

    cases = (("f16f32", 7, 96, torch.float16, torch.float32, False),
             ("f16f16", 5, 1001, torch.float16, torch.float16, False),
             ("f32f32", 6, 160, torch.float32, torch.float32, False),
             ("low", 6, 160, torch.float32, torch.float32, True))
    for tag, rows, cols, xdt, wdt, low_path in cases:
        torch.manual_seed(5)
        x = (3 * torch.randn(rows, cols)).to(xdt)
        w = (1 + 0.5 * torch.randn(cols)).to(wdt)
        if low_path:
            w[3], w[17], w[40] = 1e-5, -6.5e-6, 3e-4  # tiny |w| columns, test_rmsnorm.py:263-277
        dy = torch.randn(rows, cols).to(torch.promote_types(xdt, wdt))
        out = torch.empty(rows, cols, dtype=torch.promote_types(xdt, wdt))
        rstd = torch.empty(rows, dtype=torch.float32)
        block, warps = ref._launch_shape(cols)
        if low_path:
            tiny = w.abs() < ref.MIN_ABS_WEIGHT
            n_small = int(tiny.sum())
            slots = torch.full((cols,), -1, dtype=torch.int32)
            slots[tiny] = torch.arange(n_small, dtype=torch.int32)
            low = torch.empty(rows, cols, dtype=torch.float16)
            small = torch.empty(rows, n_small, dtype=torch.float16)
        else:
            n_small, slots, low, small = 1, rstd, rstd, rstd
        ref.qwen_rmsnorm_fwd_kernel[(rows,)](x, w, out, rstd, low, slots, small, n_small, cols, 1e-6,
                                             BLOCK=block, SAVE_LOW=low_path, num_warps=warps)
        dx = torch.empty(rows, cols, dtype=xdt)
        programs = 3
        partial = torch.zeros(programs, cols, dtype=torch.float32)
        ref.qwen_rmsnorm_bwd_kernel[(programs,)](
            dy, low if low_path else x, w, rstd, dx, partial, slots, small, n_small, rows, cols,
            BLOCK=block, COMPUTE_DW=not low_path, SAVED_OUTPUT=low_path, num_warps=warps)
        extra = dict(low=low, small=small, slots=slots) if low_path else {}
        save(f"rmsnorm_{tag}", x=x, w=w, dy=dy, out=out, rstd=rstd, dx=dx,
             dw=partial.sum(0).to(wdt), low_path=int(low_path), **extra)


def golden_rope():
    from solution import rope as ref

    for tag, (b, t, h, kv, d), dt in (("f16", (2, 9, 4, 2, 64), torch.float16),
                                      ("f32", (1, 5, 3, 1, 128), torch.float32)):
        torch.manual_seed(7)
        q = torch.randn(b, t, h * d).to(dt).view(b, t, h, d).transpose(1, 2)
        k = torch.randn(b, t, kv * d).to(dt).view(b, t, kv, d).transpose(1, 2)
        pos = torch.arange(t, dtype=torch.float32)[None].expand(b, t)
        inv = 1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
        emb = torch.cat((pos[..., None] * inv,) * 2, -1)
        cos, sin = emb.cos().to(dt).contiguous(), emb.sin().to(dt).contiguous()
        gq, gk = torch.randn(b, h, t, d).to(dt), torch.randn(b, kv, t, d).to(dt)
        save(f"rope_{tag}", q=q.contiguous(), k=k.contiguous(), cos=cos, sin=sin, gq=gq, gk=gk,
             q_out=ref._rotate(q, cos, sin, dt, False), k_out=ref._rotate(k, cos, sin, dt, False),
             dq=ref._rotate(gq, cos, sin, dt, True), dk=ref._rotate(gk, cos, sin, dt, True))


def golden_swiglu():
    from solution import swiglu_recompute as ref

    ref.__dict__["range"] = _tensor_range
    for tag, gdt, udt, rnd in (("f16", torch.float16, torch.float16, True),
                               ("f32", torch.float32, torch.float32, True),
                               ("mix", torch.float16, torch.float32, True),
                               ("noround", torch.float16, torch.float16, False)):
        torch.manual_seed(3)
        n = 3 * 1001
        g, u = (2 * torch.randn(n)).to(gdt), torch.randn(n).to(udt)
        odt = torch.promote_types(gdt, udt) if rnd else torch.float32
        dy = torch.randn(n).to(odt)
        out = torch.empty(n, dtype=odt)
        ref.silu_mul_fwd_persistent[(2,)](g, u, out, n, BLOCK=ref.BLOCK, ROUND_SILU=rnd, num_warps=4)
        dg, du = torch.empty_like(g), torch.empty_like(u)
        ref.silu_mul_bwd_recompute[(2,)](dy, g, u, dg, du, n, BLOCK=ref.BLOCK, WANT_DGATE=True,
                                         WANT_DUP=True, ROUND_SILU=rnd, num_warps=4)
        save(f"swiglu_{tag}", gate=g, up=u, dy=dy, out=out, dgate=dg, dup=du, round_silu=int(rnd))
    del ref.__dict__["range"]


def golden_dropout():
    from solution import lora as ref

    torch.manual_seed(0)
    x = torch.randn(3, 37, 64)
    mask = torch.rand(3, 37, 64) > 0.3  # test_lora.py:24-33
    n = x.numel()
    xd = torch.empty(x.shape, dtype=torch.float16)
    bits = torch.empty(n // 8, dtype=torch.uint8)
    grid = (-(-(n // 8) // ref.PACK_BYTES),)
    ref.lora_dropout_pack_kernel[grid](x, mask, xd, bits, n // 8, 1.25, BLOCK=ref.PACK_BYTES, num_warps=4)
    x16, g16 = x.half(), torch.randn(3, 37, 64).half()
    xd2, dx = torch.empty_like(x16), torch.empty(x.shape, dtype=torch.float32)
    ref.lora_dropout_unpack_kernel[grid](x16, bits, g16, xd2, dx, n // 8, 1.25, BLOCK=ref.PACK_BYTES,
                                         num_warps=4)
    save("dropout", x=x, mask=mask, scale=1.25, xd=xd, bits=bits, x16=x16, g16=g16, xd2=xd2, dx=dx)


def golden_head():
    from solution import lm_head_loss as ref

    for tag, (n, hidden, vocab, chunk), sharp in (("a", (40, 64, 1000, 256), 0.0),
                                                   ("b", (24, 128, 37, 8192), 0.0),
                                                   ("sharp", (32, 64, 700, 256), 12.0)):
        torch.manual_seed(2)
        h = torch.randn(n, hidden).half()
        w = (torch.randn(vocab, hidden) * hidden ** -0.5).half()
        tgt = torch.randint(0, vocab, (n,))
        if sharp:  # confident labels, test_lm_head_loss.py:161-179
            h = (w[tgt].float() * sharp + 0.1 * torch.randn(n, hidden)).half()
        tgt[torch.rand(n) < 0.3] = -100
        tgt[:3] = -100
        hreq = h.clone().requires_grad_(True)
        denom = (tgt != -100).sum()
        loss, token_loss, entropy, correct = ref._FusedHeadLoss.apply(
            hreq, w, tgt, denom, torch.float16, chunk, True)
        loss.backward()
        logits = torch.mm(h, w.t())
        tl_, en_, co_ = (torch.empty(n), torch.empty(n), torch.empty(n, dtype=torch.int32))
        ref._rows(logits, tgt.contiguous(), tl_, en_, co_, False)
        save(f"head_{tag}", hidden=h, weight=w, target=tgt, chunk_cols=chunk, loss=loss.detach(),
             token_loss=token_loss, entropy=entropy, correct=correct, dhidden=hreq.grad,
             logits=logits, rows_loss=tl_, rows_entropy=en_, rows_correct=co_)


def golden_attention():
    """The reference's own (unused) Triton attention, solution/attention.py:27-246, on a padded
    batch: causal attention inside the valid keys of each batch row, grouped-query heads, fp16
    output and the gradients of q, k and v. The packed row of this repository is the same
    attention with the batch rows as segments."""
    from solution import attention as ref

    for tag, (B, H, KVH, T, D), lengths in (("a", (3, 6, 2, 40, 128), [40, 23, 1]),
                                            ("b", (2, 4, 4, 70, 128), [70, 33])):
        torch.manual_seed(5)
        q = torch.randn(B, T, H, D).transpose(1, 2).requires_grad_(True)
        k = torch.randn(B, T, KVH, D).transpose(1, 2).requires_grad_(True)
        v = torch.randn(B, T, KVH, D).transpose(1, 2).requires_grad_(True)
        pad = torch.arange(T)[None, :] < torch.tensor(lengths)[:, None]
        key_ok = pad.to(torch.int8).contiguous()
        g = torch.randn(B, T, H, D) * pad[:, :, None, None]
        out = ref.qwen_attention(q, k, v, key_ok, None, torch.float16)
        out.float().backward(g)
        save(f"attention_{tag}", q=q.detach(), k=k.detach(), v=v.detach(), lengths=torch.tensor(lengths),
             grad=g, out=out.detach(), dq=q.grad, dk=k.grad, dv=v.grad)


if __name__ == "__main__":
    if len(sys.argv) > 2 and sys.argv[2] == "attention":
        golden_attention()
        sys.exit(0)
    golden_nf4()
    golden_rmsnorm()
    golden_rope()
    golden_swiglu()
    golden_dropout()
    golden_head()
    golden_attention()
