"""Oracles of the memory-bound ops: plain torch, device-free, each following the reference function
the reference's own test compares against."""

import numpy as np
import torch
import torch.nn.functional as F


def rmsnorm(x, weight, eps=1e-6):
    """Qwen2RMSNorm.forward line for line (tests_local/test_rmsnorm.py:32-38)."""
    input_dtype = x.dtype
    h = x.to(torch.float32)
    variance = h.pow(2).mean(-1, keepdim=True)
    h = h * torch.rsqrt(variance + eps)
    return weight * h.to(input_dtype)


def rmsnorm_fwd_bwd(x, weight, dy, eps=1e-6, weight_grad=False):
    """(out, dx, dw or None) through autograd of `rmsnorm`."""
    x = x.detach().clone().requires_grad_(True)
    w = weight.detach().clone().requires_grad_(weight_grad)
    out = rmsnorm(x, w, eps)
    out.backward(dy.to(out.dtype))
    return out.detach(), x.grad, w.grad


def rmsnorm_rstd(x, eps=1e-6):
    return torch.rsqrt(x.float().pow(2).mean(-1) + eps)


def rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def rope(q, k, cos, sin):
    """transformers' apply_rotary_pos_emb with unsqueeze_dim=1, the function
    tests_local/test_rope.py:21-25 compares against (q*cos + rotate_half(q)*sin)."""
    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return q * cos + rotate_half(q) * sin, k * cos + rotate_half(k) * sin


def rope_fwd_bwd(q, k, cos, sin, gq, gk):
    q = q.detach().clone().requires_grad_(True)
    k = k.detach().clone().requires_grad_(True)
    oq, ok = rope(q, k, cos, sin)
    torch.autograd.backward((oq, ok), (gq.to(oq.dtype), gk.to(ok.dtype)))
    return oq.detach(), ok.detach(), q.grad, k.grad


def rope_tables(positions, head_dim, theta=1e6, dtype=torch.float32):
    """cos/sin [1, N, head_dim] for per-token positions (tests_local/test_rope.py:34-38 recipe)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    freqs = positions.float()[..., None] * inv
    emb = torch.cat((freqs, freqs), -1)
    return emb.cos().to(dtype)[None], emb.sin().to(dtype)[None]


def swiglu(gate, up):
    """F.silu(gate) * up on the real dtypes (tests_local/test_swiglu_recompute.py:33-34)."""
    return F.silu(gate) * up


def swiglu_fwd_bwd(gate, up, dy):
    g = gate.detach().clone().requires_grad_(True)
    u = up.detach().clone().requires_grad_(True)
    out = swiglu(g, u)
    out.backward(dy.to(out.dtype))
    return out.detach(), g.grad, u.grad


def swiglu_kernel_math(gate, up, dy=None, round_silu=True, out_dtype=None):
    """The kernels' own arithmetic (solution/swiglu_recompute.py:36-79) in fp32 torch: silu as
    g / (1 + 2^(-g log2 e)), optional rounding of silu and dy*up to the gate dtype."""
    g, u = gate.float(), up.float()
    denom = 1.0 + torch.exp2(g * -1.4426950408889634)
    sig = 1.0 / denom
    silu = g / denom
    if round_silu:
        silu = silu.to(gate.dtype).float()
    out_dtype = out_dtype or torch.promote_types(gate.dtype, up.dtype)
    out = (silu * u).to(out_dtype)
    if dy is None:
        return out
    d = dy.float()
    d_silu = d * u
    if round_silu:
        d_silu = d_silu.to(gate.dtype).float()
    d_up = (d * silu).to(up.dtype)
    d_gate = (d_silu * sig * (1.0 + g * (1.0 - sig))).to(gate.dtype)
    return out, d_gate, d_up


def dropout_pack(x, mask, scale):
    """(xd fp16, bits uint8): tests_local/test_lora.py:24-33 for the values,
    solution/lora.py:41 for the bit order (bit l of byte r = element 8r + l)."""
    s = torch.tensor(scale, dtype=torch.float32)
    xd = torch.where(mask, (x.float() * s).half(), torch.zeros((), dtype=torch.float16))
    bits = np.packbits(mask.reshape(-1).numpy().astype(np.uint8), bitorder="little")
    return xd, torch.from_numpy(bits)


def dropout_unpack(x16, bits, g16, scale, dx_dtype):
    """(xd fp16, dx): solution/lora.py:45-57."""
    n = x16.numel()
    mask = torch.from_numpy(np.unpackbits(bits.numpy(), bitorder="little")[:n].astype(bool)).view(x16.shape)
    s = torch.tensor(scale, dtype=torch.float32)
    xd = torch.where(mask, (x16.float() * s).half(), torch.zeros((), dtype=torch.float16))
    dx = torch.where(mask, g16.float() * s, torch.zeros(())).to(dx_dtype)
    return xd, dx
