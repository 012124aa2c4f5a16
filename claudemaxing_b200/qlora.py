"""Self-contained 4-bit linear and LoRA layers for running the hot path without bitsandbytes/peft.

The reference reaches its kernels through bitsandbytes' `Linear4bit` and peft's LoRA `Linear4bit`
(call sites solution/nf4.py:102-130 and solution/lora.py:137-160). Those packages are optional
here: `NF4Linear` and `LoRALinear` follow the same formulas

    base:  x.to(compute) -> dequantise W -> F.linear -> cast back to x.dtype   (dequantised again
           in backward for the input gradient, as bitsandbytes' MatMul4Bit does)
    lora:  base(x) + lora_B(lora_A(dropout(x))) * scaling

and route through this package's kernels (`dequantize_nf4`, `LoRABranch`). `quantize_nf4` builds
the packed weight and its double-quantised statistics in the bitsandbytes layout with plain torch
ops on whatever device the weight is on; it is set-up code, not part of the step.
"""

import math
import os
import weakref
from types import SimpleNamespace

import torch
import torch.nn.functional as F

from .lora import LoRABranch, _shared_fp16, branch_covers
from .nf4 import dequantize_nf4, gemm_supported, nf4_linear, nf4_linear_dx
from .rmsnorm import fp16_copy_of


class QuantState:
    """The fields of bitsandbytes' QuantState that `dequantize_nf4` reads."""

    def __init__(self, absmax, shape, code, blocksize, dtype, offset=None, state2=None):
        self.absmax, self.shape, self.code = absmax, torch.Size(shape), code
        self.blocksize, self.dtype, self.offset, self.state2 = blocksize, dtype, offset, state2
        self.quant_type = "nf4"
        self.nested = state2 is not None

    def to(self, device):
        s2 = self.state2.to(device) if self.state2 is not None else None
        off = self.offset.to(device) if self.offset is not None else None
        return QuantState(self.absmax.to(device), self.shape, self.code.to(device), self.blocksize,
                          self.dtype, off, s2)


def normal_float4_levels():
    """16 quantisation levels in [-1, 1] with an exact zero: 8 + 1 quantiles of N(0,1) on the
    positive side and 7 + 1 on the negative side (the NormalFloat construction of the QLoRA
    paper), computed with torch's inverse error function."""
    edge = 0.5 * ((1 - 1 / 32) + (1 - 1 / 30))
    icdf = lambda p: math.sqrt(2.0) * torch.erfinv(2 * p - 1)  # noqa: E731
    pos = icdf(torch.linspace(edge, 0.5, 9, dtype=torch.float64)[:-1])
    neg = -icdf(torch.linspace(edge, 0.5, 8, dtype=torch.float64)[:-1])
    levels = torch.cat([neg, torch.zeros(1, dtype=torch.float64), pos]).sort().values
    return (levels / levels.abs().max()).float()


def absmax_levels():
    """256 sorted levels in [-1, 1] for the 8-bit quantisation of the absmax: signed
    fraction * 10^-e over seven decades, denser towards zero."""
    vals = {0.0, 1.0, -1.0}
    for e in range(7):
        for j in range(18):
            f = (0.1 + 0.9 * (j + 0.5) / 18) * 10.0 ** -e
            vals.add(f)
            vals.add(-f)
    vals.add(5e-8)
    out = torch.tensor(sorted(vals), dtype=torch.float64)
    return out[:256].float() if out.numel() >= 256 else F.pad(out, (0, 256 - out.numel()), value=1.0).float()


def _nearest(levels, x):
    return torch.bucketize(x, (levels[1:] + levels[:-1]) / 2)


def quantize_nf4(w, blocksize=64, nested=True, blocksize2=256, code=None, code2=None):
    """(packed uint8 [n/2, 1], QuantState) of a 2-D weight: blocks of `blocksize` along the
    row-major flattening, fp32 absmax, nearest level of w/absmax, element 2i in the high nibble of
    byte i; nested: (absmax - mean) quantised to 8 bits per block of `blocksize2`."""
    dev = w.device
    code = (normal_float4_levels() if code is None else code).to(dev)
    flat = w.detach().float().reshape(-1)
    n = flat.numel()
    if n % 2:
        raise ValueError("NF4 packing needs an even number of elements")
    blocks = F.pad(flat, (0, (-n) % blocksize)).view(-1, blocksize)
    absmax = blocks.abs().amax(1)
    idx = _nearest(code, blocks / absmax.clamp(min=1e-30)[:, None]).reshape(-1)[:n].to(torch.uint8)
    packed = ((idx[0::2] << 4) | idx[1::2]).reshape(-1, 1).contiguous()
    if not nested:
        return packed, QuantState(absmax, w.shape, code, blocksize, w.dtype)
    code2 = (absmax_levels() if code2 is None else code2).to(dev)
    offset = absmax.mean()
    centred = absmax - offset
    b2 = F.pad(centred, (0, (-centred.numel()) % blocksize2)).view(-1, blocksize2)
    absmax2 = b2.abs().amax(1)
    q8 = _nearest(code2, b2 / absmax2.clamp(min=1e-30)[:, None]).reshape(-1)[:centred.numel()]
    inner = QuantState(absmax2, (absmax.numel(),), code2, blocksize2, torch.float32)
    return packed, QuantState(q8.to(torch.uint8), w.shape, code, blocksize, w.dtype,
                              offset=offset.reshape(1).clone(), state2=inner)


class _MatMul4Bit(torch.autograd.Function):
    """x @ dequant(W)^T; the weight is dequantised again in backward instead of being kept. With
    `NF4Linear.fused_gemm` both products run on the tcgen05 GEMM that dequantises inside its
    operand prologue, so the fp16 weight is never written to memory; otherwise (the default) the
    weight is dequantised into a buffer and cuBLAS multiplies (the reference's two steps,
    solution/nf4.py:122)."""

    @staticmethod
    def forward(ctx, x, layer, x_low=None):
        """`x_low`, when given, is x already cast to the compute dtype (no autograd history of its
        own): the product is formed from it and the gradient goes to x in x's dtype. The layer's
        bias (frozen) is added by the GEMM's epilogue."""
        ctx.layer, ctx.x_dtype = layer, x.dtype
        src = x if x_low is None else x_low
        bias = layer.bias
        if layer.takes_fused_gemm(src):
            return nf4_linear(src, [(layer.packed, layer.quant_state)], [bias])[0]
        if bias is not None and bias.dtype != src.dtype:
            bias = bias.to(src.dtype)
        return F.linear(src, layer.dequantized(src.dtype), bias)

    @staticmethod
    def backward(ctx, grad):
        if not ctx.needs_input_grad[0]:
            return None, None, None
        layer = ctx.layer
        if layer.takes_fused_gemm(grad) and layer.out_features % 64 == 0:
            direct = ctx.x_dtype if ctx.x_dtype in (torch.float16, torch.float32) else torch.float16
            dx = nf4_linear_dx([grad], [(layer.packed, layer.quant_state)], direct)
            return dx.to(ctx.x_dtype), None, None
        dx = torch.matmul(grad, layer.dequantized(grad.dtype))
        return dx.to(ctx.x_dtype), None, None


class _DequantBuffers:
    """The fp16 weight buffers of one (device, dtype) that all groups of a model share, each the
    size of the largest block, kept in order of last use."""

    def __init__(self, numel, dtype, device):
        self.numel, self.dtype, self.device = numel, dtype, device
        self.flat = []                 # allocated on demand, up to NF4Group.resident_blocks(numel)
        self.owner = []                # weakref to the group whose weights the buffer holds
        self.key = []
        self.order = []                # buffer indices, least recently used first

    def holds(self, group, key):
        for i, owner in enumerate(self.owner):
            if owner is not None and owner() is group and self.key[i] == key:
                return i
        return None

    def touch(self, i):
        if i in self.order:
            self.order.remove(i)
        self.order.append(i)

    def take(self, limit):
        """Index of a buffer to overwrite: one whose contents are unknown, a new one while fewer
        than `limit` exist, else the one used longest ago."""
        for i, owner in enumerate(self.owner):
            if owner is None:
                return i
        if len(self.flat) < limit:
            self.flat.append(torch.empty(self.numel, dtype=self.dtype, device=self.device))
            self.owner.append(None)
            self.key.append(None)
            return len(self.flat) - 1
        return self.order[0]


class NF4Group:
    """The 4-bit projections of one decoder block, dequantised together.

    A block's seven weights are used right after one another (q, k, v, o, gate, up, down forward;
    the reverse in backward), each too small to fill the GPU with its own launch. One batched
    launch writes all of them into a buffer of a small pool that every group of the model shares
    (the largest block's fp16 weights each, 94 MB for Qwen2.5-1.5B). The pool holds as many blocks
    as fit `SOUP_NF4_RESIDENT_MB` (default 4096, at least two blocks), replaced in order of last
    use: on a 180 GB part the 2.6 GB of a whole Qwen2.5-1.5B stay resident from forward to
    backward, so a training step dequantises every block once instead of twice; a larger model
    keeps the blocks backward reaches first. Any order of use stays correct: a block that is not
    in a buffer is dequantised on the spot. The returned weight is a view that a later block may
    overwrite: use it on the current stream at once and do not keep it.

    Dequantising the next block ahead on a side stream was tried and removed: on the
    Qwen2.5-1.5B step it was slower (24.2 ms against 22.5 ms per captured step), the dequant CTAs
    taking SM slots and HBM bandwidth from the GEMMs for longer than the 26 us they cost in line.
    """

    _buffers = {}  # (device, dtype) -> _DequantBuffers
    resident_mb = int(os.environ.get("SOUP_NF4_RESIDENT_MB", "4096"))

    @classmethod
    def resident_blocks(cls, numel, dtype):
        per_block = numel * torch.empty((), dtype=dtype).element_size()
        return max(2, (cls.resident_mb << 20) // max(per_block, 1))

    @classmethod
    def forget(cls):
        """Declares every buffer's contents unknown. A CUDA graph must not start from weights that
        happen to be resident at capture time, and what a capture "ran" never ran."""
        for bufs in cls._buffers.values():
            bufs.owner = [None] * len(bufs.flat)
            bufs.key = [None] * len(bufs.flat)

    def __init__(self, layers):
        self.layers = list(layers)
        self.sizes = [l.in_features * l.out_features for l in self.layers]
        self.offsets = [0]
        for n in self.sizes:
            self.offsets.append(self.offsets[-1] + (n + 127) // 128 * 128)  # 256-byte aligned slices
        self.next = self.prev = None   # neighbours in forward order (set by `chain`)
        for l in self.layers:
            l.group = self

    @staticmethod
    def chain(groups):
        """Tells every group its neighbours in forward order."""
        for before, after in zip(groups, groups[1:]):
            before.next, after.prev = after, before

    def _key(self):
        return tuple(l.packed._version for l in self.layers) + tuple(l.packed.data_ptr() for l in self.layers)

    def _views(self, flat):
        return [flat[o:o + n].view(l.out_features, l.in_features)
                for l, o, n in zip(self.layers, self.offsets, self.sizes)]

    def _fill(self, bufs, i, dtype):
        from .nf4 import dequantize_nf4_batch

        dequantize_nf4_batch([(l.packed, l.quant_state) for l in self.layers], dtype,
                             outs=self._views(bufs.flat[i]))
        bufs.owner[i], bufs.key[i] = weakref.ref(self), self._key()

    def stacked(self, layers, dtype, probe=False):
        """The dequantised weights of consecutive `layers` of this group as one
        [sum of out_features, in_features] matrix (they are adjacent in the buffer when each one's
        element count is a multiple of 128), or None when they are not adjacent or differ in
        in_features. With `probe` only the answer to that question (True / None): nothing is
        dequantised."""
        index = [self.layers.index(l) for l in layers]
        adjacent = all(j == i + 1 and self.offsets[j] == self.offsets[i] + self.sizes[i]
                       for i, j in zip(index, index[1:]))
        if not adjacent or len({l.in_features for l in layers}) != 1:
            return None
        if probe:
            return True
        first = self.weight(layers[0], dtype)
        flat = first.reshape(-1)
        total = sum(l.out_features for l in layers)
        return torch.as_strided(flat, (total, layers[0].in_features), (layers[0].in_features, 1))

    def weight(self, layer, dtype):
        device = layer.packed.device
        bufs = NF4Group._buffers.get((device, dtype))
        if bufs is None or bufs.numel < self.offsets[-1]:
            bufs = _DequantBuffers(self.offsets[-1], dtype, device)
            NF4Group._buffers[(device, dtype)] = bufs
        i = bufs.holds(self, self._key())
        if i is None:
            i = bufs.take(self.resident_blocks(bufs.numel, dtype))
            self._fill(bufs, i, dtype)
        bufs.touch(i)
        return self._views(bufs.flat[i])[self.layers.index(layer)]


class NF4Linear(torch.nn.Module):
    """Frozen, bias-free linear with an NF4 double-quantised weight."""

    _soup_nf4_linear = True
    # SOUP_NF4_GEMM=1 routes the projections through the tcgen05 GEMM that dequantises in its
    # operand prologue. It is off by default: measured on B200 at the training step's shapes
    # (1280 rows) it takes 94 us for gate+up against 75 us for this library's dequant kernel plus
    # cuBLAS, and the 1536 x 1536 / 256 x 1536 projections are bound by its ~13 us of fixed cost.
    fused_gemm = os.environ.get("SOUP_NF4_GEMM", "0") == "1"

    def __init__(self, in_features, out_features, packed, quant_state, compute_dtype=torch.float16,
                 bias=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("packed", packed, persistent=False)
        self.quant_state = quant_state
        self.compute_dtype = compute_dtype
        self.group = None   # an NF4Group when the block's weights are dequantised together
        self.bias = None
        if bias is not None:
            self.bias = torch.nn.Parameter(bias.detach().clone(), requires_grad=False)

    @classmethod
    def from_weight(cls, weight, compute_dtype=torch.float16, blocksize=64, bias=None):
        packed, state = quantize_nf4(weight.to(torch.float16), blocksize=blocksize, nested=True)
        return cls(weight.shape[1], weight.shape[0], packed, state, compute_dtype, bias)

    def _apply(self, fn, *args, **kwargs):
        super()._apply(fn, *args, **kwargs)
        self.quant_state = self.quant_state.to(self.packed.device)
        return self

    def dequantized(self, dtype):
        """The [out, in] weight in `dtype`: a fresh tensor, or a short-lived view of the group's
        buffer."""
        if self.group is not None:
            return self.group.weight(self, dtype)
        return dequantize_nf4(self.packed, self.quant_state, dtype)

    def takes_fused_gemm(self, operand):
        """Whether a product with `operand` (fp16, CUDA) runs on the GEMM that dequantises in its
        prologue."""
        return (NF4Linear.fused_gemm and operand.dtype == torch.float16 and operand.is_cuda
                and gemm_supported(self.quant_state, self.in_features))

    def matmul_4bit(self, x_low):
        return _MatMul4Bit.apply(x_low, self)

    def forward(self, x):
        x_low = None
        if self.compute_dtype == torch.float16 and x.dtype == torch.float32:
            x_low = fp16_copy_of(x)   # the copy the RMSNorm before this layer wrote, if any
        if x_low is not None:
            out = _MatMul4Bit.apply(x, self, x_low)
        else:
            out = self.matmul_4bit(x.to(self.compute_dtype))
        return out.to(x.dtype)


class LoRALinear(torch.nn.Module):
    """base(x) + lora_B(lora_A(dropout(x))) * scaling with fp32 adapter weights (peft's layout:
    A Kaiming-uniform, B zero)."""

    def __init__(self, base_layer, r=16, alpha=32, dropout=0.05):
        super().__init__()
        self.base_layer = base_layer
        self.lora_A = torch.nn.Linear(base_layer.in_features, r, bias=False, dtype=torch.float32)
        self.lora_B = torch.nn.Linear(r, base_layer.out_features, bias=False, dtype=torch.float32)
        torch.nn.init.kaiming_uniform_(self.lora_A.weight, a=math.sqrt(5))
        torch.nn.init.zeros_(self.lora_B.weight)
        self.p = float(dropout)
        self.scaling = alpha / r

    def forward(self, x):
        result = self.base_layer(x)
        if branch_covers(x, self.p, self.training):
            lora = LoRABranch.apply(x, _shared_fp16(x), self.lora_A.weight, self.lora_B.weight,
                                    self.p, float(self.scaling))
            return result + lora
        xa = F.dropout(x.to(self.lora_A.weight.dtype), self.p, self.training)
        return result + self.lora_B(self.lora_A(xa)) * self.scaling


QWEN25_1P5B = dict(hidden_size=1536, intermediate_size=8960, num_hidden_layers=28,
                   num_attention_heads=12, num_key_value_heads=2, vocab_size=151936,
                   max_position_embeddings=32768, rms_norm_eps=1e-6, rope_theta=1e6,
                   tie_word_embeddings=True)


def build_qlora_model(device, config=None, lora_targets=("q_proj", "v_proj"), r=16, alpha=32,
                      dropout=0.05, seed=0, group_dequant=True, fused_blocks=True):
    """A Qwen2 causal LM prepared the way the reference's run prepares it, without its packages:
    random fp16 weights of the given architecture (default Qwen2.5-1.5B), every decoder
    projection NF4-quantised (blocksize 64, double-quantised absmax), norms and the tied
    embedding/head in fp32 and frozen, LoRA (fp32 A Kaiming-uniform, B zero) on q_proj and v_proj.
    With `group_dequant` each block's seven weights are dequantised by one launch (NF4Group);
    with `fused_blocks` as well, the packed training call runs each block as the fused chain of
    decoder_block.py. Returns (model, list of trainable LoRA parameters)."""
    from transformers import Qwen2Config, Qwen2ForCausalLM

    cfg = dict(QWEN25_1P5B)
    cfg.update(config or {})
    hf_cfg = Qwen2Config(**cfg)
    hf_cfg._attn_implementation = "sdpa"
    torch.manual_seed(seed)
    with torch.device(device):
        model = Qwen2ForCausalLM(hf_cfg).to(torch.float16)
    for p in model.parameters():
        p.requires_grad_(False)
    groups = []
    for layer in model.model.layers:
        for parent, names in ((layer.self_attn, ("q_proj", "k_proj", "v_proj", "o_proj")),
                              (layer.mlp, ("gate_proj", "up_proj", "down_proj"))):
            for name in names:
                lin = getattr(parent, name)
                q = NF4Linear.from_weight(lin.weight.data, bias=lin.bias)
                if name in lora_targets:
                    q = LoRALinear(q, r=r, alpha=alpha, dropout=dropout).to(device)
                setattr(parent, name, q)
                del lin
        if group_dequant:
            groups.append(NF4Group(
                [getattr(parent, name).base_layer if isinstance(getattr(parent, name), LoRALinear)
                 else getattr(parent, name)
                 for parent, names in ((layer.self_attn, ("q_proj", "k_proj", "v_proj", "o_proj")),
                                       (layer.mlp, ("gate_proj", "up_proj", "down_proj")))
                 for name in names]))
    NF4Group.chain(groups)
    # what prepare_model_for_kbit_training leaves: fp32 norms and fp32 (tied) embedding
    for module in model.modules():
        if type(module).__name__ == "Qwen2RMSNorm":
            module.weight.data = module.weight.data.float()
    model.model.embed_tokens.weight.data = model.model.embed_tokens.weight.data.float()
    if hf_cfg.tie_word_embeddings:
        model.lm_head.weight = model.model.embed_tokens.weight
    lora_params = [p for n, p in model.named_parameters() if "lora_" in n]
    for p in lora_params:
        p.requires_grad_(True)
    if group_dequant and fused_blocks:
        from .decoder_block import install_fused_blocks

        install_fused_blocks(model)
    torch.cuda.empty_cache() if torch.cuda.is_available() else None
    return model, lora_params


def synthetic_batch(batch=4, min_len=64, max_len=512, vocab=151936, seed=3, device="cpu"):
    """Right-padded batch of random token ids with lengths uniform in [min_len, max_len];
    labels = inputs, -100 on the padding (the loss shifts them)."""
    gen = torch.Generator().manual_seed(seed)
    lengths = torch.randint(min_len, max_len + 1, (batch,), generator=gen)
    width = int(lengths.max())
    ids = torch.randint(0, vocab, (batch, width), generator=gen)
    mask = (torch.arange(width)[None, :] < lengths[:, None]).long()
    labels = torch.where(mask.bool(), ids, torch.full_like(ids, -100))
    ids = ids * mask
    return dict(input_ids=ids.to(device), attention_mask=mask.to(device), labels=labels.to(device),
                n_tokens=int(lengths.sum()))


def qlora_step(model, batch, optimizer=None, scaler=None, num_items=None):
    """One training step under fp16 autocast through the patched forward (packed real tokens,
    fused head): loss, backward, optional optimizer step. Returns the detached loss."""
    from .lm_head_loss import _REQUEST_ATTR

    model.train()
    model.__dict__[_REQUEST_ATTR] = True  # what the patched SFTTrainer.compute_loss sets
    with torch.autocast("cuda", dtype=torch.float16):
        out = model(input_ids=batch["input_ids"], attention_mask=batch["attention_mask"],
                    labels=batch["labels"], use_cache=False,
                    **({"num_items_in_batch": num_items} if num_items is not None else {}))
    loss = out.loss
    (scaler.scale(loss) if scaler is not None else loss).backward()
    if optimizer is not None:
        if scaler is not None:
            scaler.step(optimizer)
            scaler.update()
        else:
            optimizer.step()
        optimizer.zero_grad(set_to_none=True)
    return loss.detach()


class CapturedStep:
    """One QLoRA training step replayed from CUDA graphs instead of ~3000 eager launches.

    The packed real tokens of a batch are padded up to `bucket_tokens` (the padding tokens are
    an attention segment of their own and carry ignore labels, so loss and gradients are those of
    the real tokens) and copied into fixed device buffers, with the offsets of the batch rows in
    the packed row for the attention (a later batch may have at most as many rows as the one the
    step was captured on). Forward, backward and the loss-scaled gradient
    clean-up are one graph; the optimizer step is a second one, so a data-parallel job can
    all-reduce the LoRA gradients (one flat fp32 buffer that every `.grad` is a view of) between
    the two. The eager launch sequence it replaces is the trainer's compute_loss → backward →
    optimizer.step of the reference (solution/lm_head_loss.py:375-430 wraps the first).

    `load()` takes a host or device batch and moves 3 × bucket_tokens int64 values and the row offsets; `run()` replays
    and returns the (device) loss of the step. Construction runs `warmup` eager steps and the
    capture on `batch`, then puts the parameters, the optimizer state and the loss scale back to
    what they were, so the first `run()` is the first training step. The optimizer must be built
    with `capturable=True`; `bucket_tokens` defaults to the real tokens of `batch` rounded up to a
    multiple of 128.
    """

    def __init__(self, model, params, optimizer, batch, bucket_tokens=None, scaler=None,
                 loss_scale=1024.0, group=None, warmup=3):
        from . import lm_head_loss as L

        self._L = L
        self.model, self.params, self.optimizer, self.scaler = model, list(params), optimizer, scaler
        self.loss_scale = float(loss_scale)
        self.group = group
        self.world = 1
        if group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()):
            self.world = torch.distributed.get_world_size(group)
        dev = self.params[0].device
        real = int((batch["attention_mask"] != 0).sum())
        n = int(bucket_tokens) if bucket_tokens else -(-real // 128) * 128
        self.bucket = n
        self.ids = torch.zeros(1, n, dtype=torch.int64, device=dev)
        self.col = torch.zeros(1, n, dtype=torch.int64, device=dev)
        # segment offsets of the packed row: the batch rows, then the padding tokens as one segment
        self.max_rows = int(batch["input_ids"].shape[0])
        self.cu_rows = torch.zeros(self.max_rows + 2, dtype=torch.int32, device=dev)
        self.target = torch.full((1, n), -100, dtype=torch.int64, device=dev)
        self.index = torch.arange(n, dtype=torch.int64, device=dev)
        # divisor of the loss: the labelled tokens of the whole job divided by the ranks, so that
        # the mean of the ranks' gradients is the gradient of the job's mean token loss (what the
        # reference's trainer gets from a global num_items_in_batch)
        self.denominator = torch.ones((), dtype=torch.float32, device=dev)
        # every LoRA gradient is a view of one flat buffer: one all-reduce, no gather/scatter
        total = sum(p.numel() for p in self.params)
        self.flat_grad = torch.zeros(total, dtype=self.params[0].dtype, device=dev)
        offset = 0
        for p in self.params:
            p.grad = self.flat_grad[offset:offset + p.numel()].view_as(p)
            offset += p.numel()
        self.loss = None
        self.load(batch)
        self._capture(warmup)

    # ------------------------------------------------------------------ host side of a step
    def load(self, batch):
        """Packs `batch` (input_ids, attention_mask, labels of shape [B, T], host or device) and
        copies ids / positions / shifted labels / row offsets into the graph's buffers."""
        L = self._L
        ids, mask, labels = batch["input_ids"], batch["attention_mask"], batch["labels"]
        B, T = ids.shape
        keep = (mask.reshape(-1) != 0).nonzero().squeeze(1)
        n = keep.numel()
        if n > self.bucket:
            raise ValueError(f"batch has {n} real tokens, the captured step holds {self.bucket}")
        if B > self.max_rows:
            raise ValueError(f"batch has {B} rows, the captured step holds {self.max_rows}")
        target = L.shift_labels_left(labels).reshape(-1)[keep]
        stage = torch.empty(3, self.bucket, dtype=torch.int64, device=ids.device,
                            pin_memory=not ids.is_cuda)
        stage[0, :n] = ids.reshape(-1)[keep]
        stage[1, :n] = keep % T
        stage[2, :n] = target
        stage[0:2, n:] = 0
        stage[2, n:] = -100
        ends = torch.bincount(keep // T, minlength=B).cumsum(0)
        cu = torch.full((self.max_rows + 2,), n, dtype=torch.int32, device=ids.device)
        cu[0] = 0
        cu[1:B + 1] = ends
        cu[-1] = self.bucket
        self.ids.copy_(stage[0:1], non_blocking=True)
        self.col.copy_(stage[1:2], non_blocking=True)
        self.target.copy_(stage[2:3], non_blocking=True)
        self.cu_rows.copy_(cu.pin_memory() if not cu.is_cuda else cu, non_blocking=True)
        labelled = (self.target != -100).sum().to(torch.float32)
        if self.world > 1:
            torch.distributed.all_reduce(labelled, group=self.group)
            labelled = labelled / self.world
        self.denominator.copy_(labelled.clamp(min=1.0))
        return n

    def run(self):
        self.graph_fb.replay()
        NF4Group.forget()           # the replay rewrote the shared weight buffers behind Python's back
        if self.world > 1:
            torch.distributed.all_reduce(self.flat_grad, group=self.group)
            self.flat_grad.div_(self.world)
        self.graph_opt.replay()
        return self.loss

    # ------------------------------------------------------------------ captured bodies
    def _forward_backward(self):
        L = self._L
        packed = SimpleNamespace(B=1, T=self.bucket, index=self.index, ids=self.ids, pos=self.col,
                                 target=self.target, cu_rows=self.cu_rows, longest=self.bucket)
        self.flat_grad.zero_()
        # every adapter gradient is a view of the zeroed flat buffer: the GEMMs that form them add
        # into it directly (no hooks hang on these parameters here)
        was, LoRABranch.accumulate_in_place = LoRABranch.accumulate_in_place, True
        try:
            with torch.autocast("cuda", dtype=torch.float16):
                out = L._packed_forward(self.model, {"use_cache": False,
                                                     "num_items_in_batch": self.denominator}, packed)
            scaled = self.scaler.scale(out.loss) if self.scaler is not None else out.loss * self.loss_scale
            scaled.backward()
        finally:
            LoRABranch.accumulate_in_place = was
        return out.loss.detach()

    def _optimizer_step(self):
        if self.scaler is not None:
            self.scaler.step(self.optimizer)
            self.scaler.update()
        else:
            self.flat_grad.div_(self.loss_scale)
            self.optimizer.step()

    def _snapshot(self):
        state = {}
        for p in self.params:
            for key, value in self.optimizer.state.get(p, {}).items():
                if torch.is_tensor(value):
                    state[(p, key)] = value.clone()
        scaler = self.scaler.state_dict() if self.scaler is not None else None
        return [p.detach().clone() for p in self.params], state, scaler

    def _restore(self, snapshot):
        values, state, scaler = snapshot
        with torch.no_grad():
            for p, v in zip(self.params, values):
                p.copy_(v)
            for p in self.params:
                for key, value in self.optimizer.state.get(p, {}).items():
                    if torch.is_tensor(value):  # in place: the graphs hold these addresses
                        old = state.get((p, key))
                        value.copy_(old) if old is not None else value.zero_()
            self.flat_grad.zero_()
        if scaler is not None and scaler:
            self.scaler.load_state_dict(scaler)

    def _capture(self, warmup):
        from .embedding import shrink_tied_embedding

        self.model.train()
        # what the patched forward does on its first training call: decided here, before the
        # capture, because it replaces the tied weight's storage (a graph captured on the fp32
        # storage would read freed memory once an eager step shrank it)
        with torch.autocast("cuda", dtype=torch.float16):
            shrink_tied_embedding(self.model)
        snapshot = self._snapshot()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                self._forward_backward()
                self._optimizer_step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        NF4Group.forget()           # the graph dequantises its first block itself
        self.graph_fb = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph_fb):
            self.loss = self._forward_backward()
        NF4Group.forget()           # nothing the capture recorded has run
        self.graph_opt = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph_opt, pool=self.graph_fb.pool()):
            self._optimizer_step()
        self._restore(snapshot)
        torch.cuda.synchronize()
