"""One decoder block of the packed 4-bit LoRA training step as a short chain of fused steps.

The per-op patches keep transformers' block as it is: every 4-bit projection returns its fp16
product cast back to fp32, the adapter output is added in a kernel of its own, q and k are rotated
in fp32 and cast to fp16 again for the attention, the residual sums are separate mixed-dtype adds,
and backward mirrors each of those. At a few thousand packed tokens each of these elementwise
kernels costs a launch and a pass over [tokens, hidden]: about a quarter of the step on B200. This
module computes the same block with those passes folded into the kernels next to them:

* q, k and v come from one GEMM on the block's dequantised weights (adjacent in the buffer all of
  a block's projections are dequantised into) and stay fp16; `soup_rope_sum` adds the adapter
  output to q in fp32, rotates q and k and writes them as fp16 [tokens, heads, head_dim], which
  are exactly the values the reference chain reaches (fp32 sum, fp32 rotation, one rounding to
  fp16 at the attention's cast); v + adapter is one fp16 add (fp32 inside, one rounding);
* attention is causal attention inside the segments of the packed row (attention.py; for heads
  of 128 this library's kernels, called from the same autograd node as the projection);
* the block's two adapters are one node (lora.LoRABranchPair: both packed and unpacked by one
  launch each, one batched product with A), their weights cast once per decoder forward;
* o_proj and down_proj add the fp32 residual in the GEMM's epilogue and write fp32;
* backward rotates dq and dk straight into column blocks of one [tokens, q+k+v] fp16 buffer and
  forms the input gradient of the three projections in one GEMM with fp32 output; the MLP's two
  input gradients accumulate in one fp32 output as well;
* each norm and the residual connection that leaves the same tensor are one node (`_NormResidual`):
  its backward kernel adds the residual gradient and writes the fp16 copy the projection backward
  one block earlier wants.

Where a GEMM now writes its fp32 accumulator (+ residual) instead of rounding the product to fp16
first, results differ from the per-op chain by that rounding, within the tolerance the reference's
end-to-end test applies (tests_local/test_lm_head_trainer.py:186-188). The order of the dropout
draws is the per-op chain's (q_proj's adapter, then v_proj's).

It applies to blocks whose projections are this package's NF4Linear / LoRALinear layers sharing
one NF4Group (qlora.build_qlora_model), called in training under fp16 autocast with the packed
row's segment offsets; any other call runs the block's installed forward.
"""

import importlib
import os
import types

import torch

from . import _lib
from . import attention as attention_mod
from . import lora as lora_mod
from .attention import attention_gradients, segment_attention
from .rmsnorm import fp16_copy_of
from .rope import rotate_into
from .swiglu_recompute import _silu_mul_bwd, _silu_mul_fwd

F16, F32 = torch.float16, torch.float32
# the package exports a function of the same name as this module: fetch the module itself
rmsnorm_mod = importlib.import_module(__package__ + ".rmsnorm")


def _plain_precision(fn):
    """Runs `fn` with autocast off: its GEMMs take fp16 operands and state their output dtype
    themselves, and autocast would cast the fp32 residual of an `addmm` down to fp16."""
    import functools

    @functools.wraps(fn)
    def wrapped(*args, **kwargs):
        with torch.autocast("cuda", enabled=False):
            return fn(*args, **kwargs)

    return wrapped


def _base(module):
    return getattr(module, "base_layer", module)


class BlockPlan:
    """What `fused_block_forward` needs to know about one decoder block, checked once."""

    def __init__(self, layer):
        attn, mlp = layer.self_attn, layer.mlp
        self.layer = layer
        self.q, self.k, self.v, self.o = attn.q_proj, attn.k_proj, attn.v_proj, attn.o_proj
        self.gate, self.up, self.down = mlp.gate_proj, mlp.up_proj, mlp.down_proj
        self.head_dim = attn.head_dim
        self.why_not = self._structure()
        self._bias = None
        self.casts = None
        self.keep_products = os.environ.get("SOUP_MLP_RECOMPUTE", "0") != "1"

    def _structure(self):
        seven = (self.q, self.k, self.v, self.o, self.gate, self.up, self.down)
        bases = [_base(m) for m in seven]
        if not all(getattr(b, "_soup_nf4_linear", False) for b in bases):
            return "a projection is not an NF4Linear"
        group = bases[0].group
        if group is None or any(b.group is not group for b in bases):
            return "the projections do not share one NF4Group"
        if any(b.compute_dtype != F16 for b in bases):
            return "a projection computes in another dtype than fp16"
        if any(m is not b for m, b in zip(seven[3:], bases[3:])):
            return "an adapter on o_proj or the MLP"
        if bases[3].bias is not None or any(b.bias is not None for b in bases[4:]):
            return "a bias on o_proj or the MLP"
        if group.stacked(bases[:3], F16, probe=True) is None:
            return "q, k and v weights are not adjacent in the group's buffer"
        if getattr(getattr(self.layer.mlp, "config", None), "hidden_act", "silu") != "silu":
            return "another activation than silu"
        d = self.head_dim
        if d % 16 or d > 256 or any(b.out_features % d for b in bases[:3]):
            return "head dimension"
        if bases[1].out_features != bases[2].out_features:
            return "k and v widths differ"
        return ""

    def qkv_bias(self, device):
        """fp16 [q + k + v] bias of the stacked projection (zeros where a projection has none), or
        None when none of the three has one."""
        bases = [_base(m) for m in (self.q, self.k, self.v)]
        if all(b.bias is None for b in bases):
            return None
        if self._bias is None or self._bias.device != device:
            parts = [(b.bias.detach().to(device=device, dtype=F16) if b.bias is not None
                      else torch.zeros(b.out_features, dtype=F16, device=device)) for b in bases]
            self._bias = torch.cat(parts)
        return self._bias

    def adapter(self, module, x):
        """(A, B, p, scaling, A fp16, scaling * B fp16, True) of a LoRALinear whose adapter
        LoRABranch reproduces for this input (the copies None / False unless the model cast them
        for this forward); None
        for a bare projection; False when the adapter needs the module's own forward."""
        if module is _base(module):
            return None
        if not lora_mod.branch_covers(x, module.p, module.training):
            return False
        a16 = b16 = None
        if self.casts is not None and self.casts.armed:
            a16, b16 = self.casts.of(module)
        return (module.lora_A.weight, module.lora_B.weight, float(module.p), float(module.scaling),
                a16, b16, b16 is not None)


class AdapterCasts:
    """fp16 copies of the adapter weights of a model's fused blocks, refreshed by three
    multi-tensor launches at the start of every forward of the decoder (112 weights of 50 KB and
    less would otherwise be 112 launches): A as it is, B multiplied by its layer's scaling first
    (`LoRABranch`'s `b16_scaled`). The copies are handed out only while that forward runs
    (`armed`); a block called on its own casts its weights itself."""

    def __init__(self):
        self.modules, self.where = [], {}
        self.a16, self.b16 = [], []
        self.pairs, self.stacked = {}, {}
        self.armed = False

    def add(self, module):
        if id(module) not in self.where:
            self.where[id(module)] = len(self.modules)
            self.modules.append(module)

    def add_pair(self, first, second):
        """The two adapters of a block whose A weights have one shape: their fp16 copies are the
        two halves of one [2, r, in] tensor (`pair_of`), ready for a batched product."""
        self.add(first)
        self.add(second)
        if first.lora_A.weight.shape == second.lora_A.weight.shape:
            self.pairs[id(first)] = (self.where[id(first)], self.where[id(second)])

    def pair_of(self, first):
        at = self.pairs.get(id(first))
        return None if at is None or not self.stacked else self.stacked.get(at)

    def of(self, module):
        i = self.where[id(module)]
        return self.a16[i], self.b16[i]

    def refresh(self, *_):
        self.armed = False
        if not self.modules or not torch.is_grad_enabled():
            return
        a32 = [m.lora_A.weight.detach() for m in self.modules]
        b32 = [m.lora_B.weight.detach() for m in self.modules]
        if not all(w.is_cuda and w.dtype == F32 for w in a32 + b32):
            return
        if len(self.a16) != len(a32) or any(c.device != w.device or c.shape != w.shape
                                            for c, w in zip(self.a16 + self.b16, a32 + b32)):
            self.a16 = [torch.empty(w.shape, dtype=F16, device=w.device) for w in a32]
            self.b16 = [torch.empty(w.shape, dtype=F16, device=w.device) for w in b32]
            self.stacked = {}
            for i, j in self.pairs.values():     # the pair's two A copies as halves of one tensor
                both = torch.empty((2,) + tuple(a32[i].shape), dtype=F16, device=a32[i].device)
                self.a16[i], self.a16[j] = both[0], both[1]
                self.stacked[(i, j)] = both
        torch._foreach_copy_(self.a16, a32)
        torch._foreach_copy_(self.b16, torch._foreach_mul(b32, [float(m.scaling) for m in self.modules]))
        self.armed = True

    def disarm(self, *_):
        self.armed = False


class _GradCopies:
    """The fp16 copy of the hidden-state gradient `_NormResidual.backward` has just written, found
    again by the fp32 gradient's storage and version when the projection backward one block
    earlier receives that gradient."""

    key = copy = None

    @classmethod
    def record(cls, grad, copy):
        cls.key, cls.copy = (grad.data_ptr(), grad._version, tuple(grad.shape)), copy

    @classmethod
    def take(cls, grad):
        if cls.key != (grad.data_ptr(), grad._version, tuple(grad.shape)):
            return None
        copy, cls.key, cls.copy = cls.copy, None, None
        return copy


def _fp16_gradient_rows(grad):
    """[rows, hidden] fp16 of an fp32 hidden-state gradient: the copy the norm backward wrote
    beside it, else a cast."""
    copy = _GradCopies.take(grad)
    if copy is None:
        return grad.reshape(-1, grad.shape[-1]).to(F16)
    return copy.view(-1, grad.shape[-1])


class _NormResidual(torch.autograd.Function):
    """(RMSNorm(h), h): the norm of a block and the residual connection that leaves the same
    tensor, as one autograd node, so that backward sees the norm's output gradient and the
    residual gradient together: one kernel (`soup_rmsnorm_bwd_residual`) forms
    rmsnorm_backward(dy) + residual gradient and the fp16 copy of the sum, where autograd would
    launch the norm backward, an add and, in the projection backward that receives the sum, a
    cast. For the frozen fp32 norm weights of the 4-bit model (the forward's saved-output form)."""

    @staticmethod
    def forward(ctx, h, weight, eps):
        rows = h.view(-1, h.shape[-1])
        out, rstd, low, slots, small = rmsnorm_mod._forward_launch(rows, weight, eps, F32, True)
        ctx.save_for_backward(low, weight, rstd, slots, small)
        result = out.view(h.shape)
        rmsnorm_mod._LastCopy.record(result, low)
        return result, h

    @staticmethod
    def backward(ctx, dy, residual_grad):
        low, weight, rstd, slots, small = ctx.saved_tensors
        n, cols = low.shape
        if dy is None:
            return residual_grad, None, None
        dy = dy.contiguous()
        add = None if residual_grad is None else residual_grad.contiguous()
        dx = torch.empty(dy.shape, dtype=F32, device=dy.device)
        dx16 = torch.empty(dy.shape, dtype=F16, device=dy.device)
        try:
            _lib.call("soup_rmsnorm_bwd_residual", _lib.ptr(dy), _lib.ptr(low), _lib.ptr(weight),
                      _lib.ptr(rstd), _lib.ptr(add), _lib.ptr(dx), _lib.ptr(dx16), _lib.ptr(slots),
                      _lib.ptr(small), small.shape[-1], n, cols, _lib.stream_of(dy))
        except RuntimeError:   # a shape the residual form does not take: the three separate steps
            _lib.call("soup_rmsnorm_bwd", _lib.ptr(dy), _lib.ptr(low), _lib.ptr(weight), _lib.ptr(rstd),
                      _lib.ptr(dx), None, None, _lib.ptr(slots), _lib.ptr(small), small.shape[-1], n,
                      cols, _lib.F32, _lib.F16, _lib.F32, _lib.F32, 1, _lib.stream_of(dy))
            return (dx if add is None else dx + add), None, None
        _GradCopies.record(dx, dx16)
        return dx, None, None


def _norm_and_residual(norm, hidden):
    """(norm(hidden), hidden as the residual branch sees it) through `_NormResidual` when the norm
    is a frozen fp32 RMSNorm whose forward keeps the fp16 copy, else through the module."""
    weight = norm.weight
    if (hidden.requires_grad and weight.dtype == F32 and not weight.requires_grad and weight.is_cuda
            and weight.dim() == 1 and hidden.shape[-1] == weight.shape[0]
            and hidden.shape[-1] <= rmsnorm_mod.MAX_COLS and hidden.shape[-1] % 8 == 0
            and rmsnorm_mod._small_columns(weight) is not None):
        return _NormResidual.apply(hidden, weight, norm.variance_epsilon)
    return norm(hidden), hidden


class _QKVRope(torch.autograd.Function):
    """(x16 @ [Wq; Wk; Wv]^T + bias) split into q (+ adapter), k, v (+ adapter); q and k rotated;
    all three returned as fp16 [tokens, heads, head_dim]. With `cu_rows` (segment offsets of the
    packed row) the causal attention inside the segments runs here as well, on this library's
    kernels, and its output [tokens, heads, head_dim] is what is returned: backward then hands the
    attention kernel's fp32 dV straight to the copy into the projection's gradient buffer."""

    @staticmethod
    @_plain_precision
    def forward(ctx, x, x16, lora_q, lora_v, cos, sin, plan, cu_rows=None, scale=None):
        bases = [_base(m) for m in (plan.q, plan.k, plan.v)]
        n, d = x16.numel() // x16.shape[-1], plan.head_dim
        nq, nk = bases[0].out_features, bases[1].out_features
        rows = x16.reshape(n, x16.shape[-1])
        w = bases[0].group.stacked(bases, F16)
        bias = plan.qkv_bias(x16.device)
        qkv = torch.mm(rows, w.t()) if bias is None else torch.addmm(bias, rows, w.t())
        hq, hk = nq // d, nk // d
        q_out = torch.empty(n, hq, d, dtype=F16, device=x16.device)
        k_out = torch.empty(n, hk, d, dtype=F16, device=x16.device)

        def heads_first(t, h):   # [n, h*d] (any row stride) seen as [1, h, n, d]
            return t.unflatten(-1, (h, d)).unsqueeze(0).transpose(1, 2)

        rotate_into(heads_first(qkv[:, :nq], hq),
                    None if lora_q is None else heads_first(lora_q.reshape(n, nq), hq),
                    heads_first(qkv[:, nq:nq + nk], hk), cos, sin,
                    q_out.unsqueeze(0).transpose(1, 2), k_out.unsqueeze(0).transpose(1, 2))
        v_rows = qkv[:, nq + nk:]
        v_out = v_rows.contiguous() if lora_v is None else v_rows + lora_v.reshape(n, nk)
        ctx.plan, ctx.sizes, ctx.x_shape = plan, (n, d, nq, nk, hq, hk), x.shape
        ctx.lora_shapes = (None if lora_q is None else lora_q.shape, None if lora_v is None else lora_v.shape)
        ctx.attends = cu_rows is not None
        v_out = v_out.view(n, hk, d)
        if not ctx.attends:
            ctx.save_for_backward(cos, sin)
            return q_out, k_out, v_out
        attended = torch.empty(n, hq, d, dtype=F16, device=x16.device)
        lse = torch.empty(hq, n, dtype=F32, device=x16.device)
        _lib.call("soup_attn_fwd", _lib.ptr(q_out), _lib.ptr(k_out), _lib.ptr(v_out), _lib.ptr(cu_rows),
                  _lib.ptr(attended), _lib.ptr(lse), n, cu_rows.numel() - 1, hq, hk, d,
                  q_out.stride(0), k_out.stride(0), v_out.stride(0), float(scale), _lib.stream_of(q_out))
        ctx.save_for_backward(cos, sin, q_out, k_out, v_out, attended, lse, cu_rows)
        ctx.scale = float(scale)
        return attended

    @staticmethod
    @_plain_precision
    def backward(ctx, *grads):
        plan, (n, d, nq, nk, hq, hk) = ctx.plan, ctx.sizes
        if ctx.attends:
            cos, sin, q_out, k_out, v_out, attended, lse, cu_rows = ctx.saved_tensors
            dq, dk, dv = attention_gradients(q_out, k_out, v_out, attended, lse,
                                             grads[0].reshape(n, hq, d), cu_rows, ctx.scale)
            dk = dk.to(F16)   # the pipelined rotation wants q and k of one element size
        else:
            cos, sin = ctx.saved_tensors
            dq, dk, dv = grads
        dq, dk = (g if g.stride(-1) == 1 else g.contiguous() for g in (dq, dk))
        dqkv = torch.empty(n, nq + 2 * nk, dtype=F16, device=dq.device)

        def heads_first(t, h):
            return t.unflatten(-1, (h, d)).unsqueeze(0).transpose(1, 2)

        rotate_into(dq.unsqueeze(0).transpose(1, 2), None, dk.unsqueeze(0).transpose(1, 2), cos, sin,
                    heads_first(dqkv[:, :nq], hq), heads_first(dqkv[:, nq:nq + nk], hk), backward=True)
        dqkv[:, nq + nk:].copy_(dv.reshape(n, nk))
        dx = None
        if ctx.needs_input_grad[0]:
            bases = [_base(m) for m in (plan.q, plan.k, plan.v)]
            w = bases[0].group.stacked(bases, F16)
            dx = torch.mm(dqkv, w, out_dtype=F32).view(ctx.x_shape)
        q_shape, v_shape = ctx.lora_shapes
        return (dx, None,
                None if q_shape is None else dqkv[:, :nq].view(q_shape),
                None if v_shape is None else dqkv[:, nq + nk:].view(v_shape),
                None, None, None, None, None)


class _ProjectAddResidual(torch.autograd.Function):
    """residual + y @ W^T with the sum formed in the GEMM's fp32 epilogue (y fp16 [n, k], residual
    fp32 [..., h], W the dequantised weight of a frozen bias-free NF4Linear)."""

    @staticmethod
    @_plain_precision
    def forward(ctx, y, residual, linear):
        w = linear.dequantized(F16)
        h = residual.shape[-1]
        out = torch.addmm(residual.reshape(-1, h), y, w.t(), out_dtype=F32).view(residual.shape)
        ctx.linear, ctx.y_shape = linear, y.shape
        return out

    @staticmethod
    @_plain_precision
    def backward(ctx, grad):
        dy = None
        if ctx.needs_input_grad[0]:
            g16 = _fp16_gradient_rows(grad)
            dy = torch.mm(g16, ctx.linear.dequantized(F16)).view(ctx.y_shape)
        return dy, (grad if ctx.needs_input_grad[1] else None), None


class _GatedMLPAddResidual(torch.autograd.Function):
    """residual + down(silu(gate(x)) * up(x)) for frozen 4-bit projections, with the residual sum
    in down_proj's epilogue and the two input gradients in one fp32 accumulator. silu(gate) * up
    is never kept: backward rebuilds it from gate and up inside the gradient kernel, as
    SwiGLURecompute does (solution/swiglu_recompute.py:60-100). What is kept besides depends on
    `BlockPlan.keep_products`: the two fp16 products gate and up (the default here: 2 x tokens x
    intermediate x 2 bytes per block, 1.3 GB for the whole Qwen2.5-1.5B step at 1280 tokens, on a
    180 GB part), or only the fp16 input, the two projections being run again in backward (the
    reference's MLPInputRecompute, solution/swiglu_recompute.py:138-215, made for a 16 GB part)."""

    @staticmethod
    @_plain_precision
    def forward(ctx, x, x16, residual, plan):
        rows = x16.reshape(-1, x16.shape[-1])
        gate = torch.mm(rows, plan.gate.dequantized(F16).t())
        up = torch.mm(rows, plan.up.dequantized(F16).t())
        act = torch.empty_like(gate)
        _silu_mul_fwd(gate, up, act, False)   # fp32 input, fp16 products: silu is not rounded first
        h = residual.shape[-1]
        out = torch.addmm(residual.reshape(-1, h), act, plan.down.dequantized(F16).t(),
                          out_dtype=F32).view(residual.shape)
        ctx.kept = plan.keep_products
        if ctx.kept:
            ctx.save_for_backward(gate, up)
        else:
            ctx.save_for_backward(x16)
        ctx.plan, ctx.x_shape = plan, x.shape
        return out

    @staticmethod
    @_plain_precision
    def backward(ctx, grad):
        plan = ctx.plan
        dx = None
        if ctx.needs_input_grad[0]:
            g16 = _fp16_gradient_rows(grad)
            d_act = torch.mm(g16, plan.down.dequantized(F16))
            w_gate, w_up = plan.gate.dequantized(F16), plan.up.dequantized(F16)
            if ctx.kept:
                gate, up = ctx.saved_tensors
                d_gate, d_up = torch.empty_like(gate), torch.empty_like(up)
                _silu_mul_bwd(d_act, gate, up, d_gate, d_up, False)
            else:
                (x16,) = ctx.saved_tensors
                rows = x16.reshape(-1, x16.shape[-1])
                d_gate, d_up = torch.mm(rows, w_gate.t()), torch.mm(rows, w_up.t())
                _silu_mul_bwd(d_act, d_gate, d_up, d_gate, d_up, False)   # over the recomputed pair
            dx = torch.mm(d_gate, w_gate, out_dtype=F32)
            dx = torch.addmm(dx, d_up, w_up, out_dtype=F32).view(ctx.x_shape)
        return dx, None, (grad if ctx.needs_input_grad[2] else None), None


def _why_not(plan, hidden, attention_mask, past_key_values, position_embeddings, kwargs):
    """Why this call runs the block's installed forward ("" when the fused chain covers it)."""
    if plan.why_not:
        return plan.why_not
    if type(_base(plan.q)).fused_gemm:
        return "the projections are set to run on the GEMM that dequantises in its prologue"
    cu = kwargs.get("cu_seq_lens_q")
    if attention_mask is not None or not isinstance(cu, torch.Tensor) or kwargs.get("cu_seq_lens_k") is not cu:
        return "not a packed row given as segment offsets"
    if past_key_values is not None or position_embeddings is None:
        return "a cache, or no rotary tables"
    if not (isinstance(hidden, torch.Tensor) and hidden.is_cuda and hidden.dtype == F32
            and hidden.dim() == 3 and hidden.shape[0] == 1 and hidden.is_contiguous()):
        return "hidden states are not one contiguous fp32 CUDA row"
    if not (plan.layer.training and torch.is_grad_enabled() and lora_mod._autocast_fp16()):
        return "not a training call under fp16 autocast"
    attn = plan.layer.self_attn
    if getattr(attn, "sliding_window", None) is not None or (attn.training and attn.attention_dropout):
        return "sliding window or attention dropout"
    if kwargs.get("output_attentions", False):
        return "attention weights are wanted"
    cos, sin = position_embeddings
    if cos.dim() != 3 or cos.shape[0] != 1 or cos.shape[-1] != plan.head_dim or cos.requires_grad:
        return "rotary tables of another shape"
    return ""


def fused_block_forward(layer, hidden_states, attention_mask=None, position_ids=None,
                        past_key_values=None, use_cache=False, position_embeddings=None, **kwargs):
    """Qwen2DecoderLayer.forward for the covered case (see the module docstring); same arguments,
    same return value."""
    plan = layer._soup_block
    if _why_not(plan, hidden_states, attention_mask, past_key_values, position_embeddings, kwargs):
        return plan.installed(hidden_states, attention_mask=attention_mask, position_ids=position_ids,
                              past_key_values=past_key_values, use_cache=use_cache,
                              position_embeddings=position_embeddings, **kwargs)
    x, residual = _norm_and_residual(layer.input_layernorm, hidden_states)
    adapters = [plan.adapter(m, x) for m in (plan.q, plan.k, plan.v)]
    if adapters[1] is not None or any(a is False for a in adapters):
        # an adapter on k_proj, or one LoRABranch does not reproduce: the installed forward (the
        # norm runs again there; nothing else has happened yet)
        return plan.installed(hidden_states, attention_mask=attention_mask, position_ids=position_ids,
                              past_key_values=past_key_values, use_cache=use_cache,
                              position_embeddings=position_embeddings, **kwargs)
    x16 = fp16_copy_of(x)
    if x16 is None:
        x16 = x.detach().to(F16)
    pair = plan.casts.pair_of(plan.q) if (plan.casts is not None and plan.casts.armed) else None
    if (pair is not None and adapters[0] is not None and adapters[2] is not None
            and lora_mod.pair_covers(x, x16, plan.q, plan.v)):
        (a_q, b_q, p_q, s_q, _, bq16, _), (a_v, b_v, p_v, s_v, _, bv16, _) = adapters[0], adapters[2]
        out_q, out_v = lora_mod.LoRABranchPair.apply(x, x16, a_q, b_q, a_v, b_v, p_q, p_v, s_q, s_v,
                                                     pair, bq16, bv16)
        branches = [out_q, None, out_v]
    else:
        branches = [None if a is None else lora_mod.LoRABranch.apply(x, x16, *a) for a in adapters]
    cos, sin = position_embeddings
    cu = kwargs["cu_seq_lens_q"]
    scale = layer.self_attn.scaling
    if (plan.head_dim == 128 and attention_mod.OWN_FORWARD and attention_mod.OWN_BACKWARD
            and cu.dtype == torch.int32 and cu.is_cuda):
        attended = _QKVRope.apply(x, x16, branches[0], branches[2], cos.contiguous(), sin.contiguous(),
                                  plan, cu, plan.head_dim ** -0.5 if scale is None else scale)
        n = attended.shape[0]
    else:
        q, k, v = _QKVRope.apply(x, x16, branches[0], branches[2], cos.contiguous(), sin.contiguous(), plan)
        n = q.shape[0]
        attended = segment_attention(q.unsqueeze(0).transpose(1, 2), k.unsqueeze(0).transpose(1, 2),
                                     v.unsqueeze(0).transpose(1, 2), cu, kwargs.get("max_length_q", n),
                                     scale)
    hidden_states = _ProjectAddResidual.apply(attended.reshape(n, -1), residual, plan.o)
    x, residual = _norm_and_residual(layer.post_attention_layernorm, hidden_states)
    x16 = fp16_copy_of(x)
    if x16 is None:
        x16 = x.detach().to(F16)
    return _GatedMLPAddResidual.apply(x, x16, residual, plan)


def install_fused_blocks(model):
    """Gives every decoder block of `model` whose structure the fused chain covers the fused
    forward (on the instance: other models keep transformers' class). Returns the number of
    blocks taken."""
    taken = 0
    decoder = model.model
    casts = decoder.__dict__.get("_soup_adapter_casts")
    if casts is None:
        casts = AdapterCasts()
        decoder.__dict__["_soup_adapter_casts"] = casts
        decoder.register_forward_pre_hook(casts.refresh)
        decoder.register_forward_hook(casts.disarm, always_call=True)
    for layer in decoder.layers:
        if getattr(layer, "_soup_block", None) is not None:
            taken += 1
            continue
        plan = BlockPlan(layer)
        if plan.why_not:
            continue
        plan.installed = layer.forward
        plan.casts = casts
        if plan.q is not _base(plan.q) and plan.v is not _base(plan.v):
            casts.add_pair(plan.q, plan.v)
        for module in (plan.q, plan.k, plan.v):
            if module is not _base(module):
                casts.add(module)
        layer.__dict__["_soup_block"] = plan
        layer.forward = types.MethodType(fused_block_forward, layer)
        taken += 1
    return taken
