"""NF4 weight dequantisation (bitsandbytes 4-bit layout, double-quantised absmax) in one kernel.

Drop-in for the reference's solution/nf4.py: `dequantize_nf4(packed, state, dtype=None, out=None)`
takes anything that looks like a bitsandbytes QuantState (`.absmax .code .blocksize .shape .dtype
.nested .offset .state2{.absmax .code .blocksize} .quant_type`) and returns the [N, K] weight.
Layout: byte i holds elements 2i (high nibble) and 2i+1 (low nibble); element j belongs to absmax
block j // blocksize; nested: absmax[b] = code2[absmax8[b]] * absmax2[b // blocksize2] + offset.
The code tables are inputs, so the result is bit-identical to the unfused fp32 reference for any
tables (csrc/nf4.cu). `patch_bnb_nf4_dequant` routes bitsandbytes through it when that package is
installed and is a no-op otherwise.
"""

import torch

from . import _lib

_BLOCKSIZES = (32, 64, 128, 256, 512, 1024, 2048, 4096)


def _supported(packed, state, dtype):
    if state is None or not packed.is_cuda or packed.dtype != torch.uint8:
        return False
    if getattr(state, "quant_type", None) != "nf4" or dtype not in (torch.float16, torch.float32):
        return False
    code = getattr(state, "code", None)
    if code is None or code.numel() != 16 or code.dtype != torch.float32 or not code.is_cuda:
        return False
    if not state.absmax.is_cuda or len(state.shape) != 2 or not packed.is_contiguous():
        return False
    if state.blocksize not in _BLOCKSIZES or (state.shape[0] * state.shape[1]) % 2:
        return False
    if state.nested:
        s2 = state.state2
        return (s2.blocksize > 0 and (s2.blocksize & (s2.blocksize - 1)) == 0
                and s2.code.dtype == torch.float32 and s2.absmax.dtype == torch.float32
                and state.absmax.dtype == torch.uint8)
    return state.absmax.dtype == torch.float32


def _offset_tensor(offset, device):
    """The offset of the nested statistics as a one-element fp32 tensor on `device` (bitsandbytes
    keeps a 0-d tensor; a Python number is accepted too). No host round trip for a tensor."""
    return torch.as_tensor(offset, dtype=torch.float32, device=device).reshape(1)


def dequantize_nf4(packed, state, dtype=None, out=None):
    """The [N, K] weight of an NF4 QuantState in `dtype` (default: state.dtype)."""
    dtype = dtype or state.dtype
    _lib.require_cuda(packed)
    n = state.shape[0] * state.shape[1]
    if out is None:
        out = torch.empty(tuple(state.shape), dtype=dtype, device=packed.device)
    if n == 0:
        return out
    nested = bool(state.nested)
    if nested:
        s2 = state.state2
        code2, absmax2 = s2.code.contiguous(), s2.absmax.contiguous()
        offset = _offset_tensor(state.offset, packed.device)  # stays on the GPU: no sync
        bs2 = int(s2.blocksize)
    else:
        code2 = absmax2 = offset = None
        bs2 = 1
    _lib.call("soup_nf4_dequant", _lib.ptr(packed), _lib.ptr(state.absmax.contiguous()),
              _lib.ptr(state.code), _lib.ptr(code2), _lib.ptr(absmax2), _lib.ptr(offset),
              _lib.ptr(out), n, int(state.blocksize), bs2, int(nested),
              _lib.dtype_code(out.dtype), _lib.stream_of(packed))
    return out


def dequantize_nf4_batch(weights, dtype=None, outs=None):
    """Dequantises several NF4 weights with one launch per eight tensors. `weights` is a list of
    (packed, state) with a common blocksize / nesting; returns the list of [N, K] tensors
    (`outs`, when given, are filled instead of allocating)."""
    import ctypes

    if not weights:
        return []
    first = weights[0][1]
    dtype = dtype or first.dtype
    nested = bool(first.nested)
    items = (_lib.Nf4Item * len(weights))()
    results = []
    keep = []  # tensors whose pointers are in `items` must outlive the launch call
    for i, (packed, st) in enumerate(weights):
        _lib.require_cuda(packed)
        if (bool(st.nested) != nested or st.blocksize != first.blocksize
                or (nested and st.state2.blocksize != first.state2.blocksize)):
            raise ValueError("a batch shares blocksize and nesting")
        out = outs[i] if outs is not None else torch.empty(tuple(st.shape), dtype=dtype,
                                                           device=packed.device)
        results.append(out)
        absmax = st.absmax.contiguous()
        keep.append(absmax)
        items[i].packed, items[i].absmax, items[i].out = packed.data_ptr(), absmax.data_ptr(), out.data_ptr()
        items[i].n_elems = st.shape[0] * st.shape[1]
        if nested:
            code2, absmax2 = st.state2.code.contiguous(), st.state2.absmax.contiguous()
            offset = _offset_tensor(st.offset, packed.device)
            keep += [code2, absmax2, offset]
            items[i].code2, items[i].absmax2, items[i].offset = (code2.data_ptr(), absmax2.data_ptr(),
                                                                 offset.data_ptr())
    _lib.call("soup_nf4_dequant_batch", ctypes.cast(items, ctypes.c_void_p), len(weights),
              _lib.ptr(first.code), int(first.blocksize),
              int(first.state2.blocksize) if nested else 1, int(nested),
              _lib.dtype_code(results[0].dtype), _lib.stream_of(weights[0][0]))
    return results


# ------------------------------------------------------------------ GEMMs on the packed weight
def gemm_supported(state, k=None):
    """Whether the tcgen05 GEMM with the dequantisation in its prologue takes this weight: NF4 with
    blocksize 64 (one block = one 128-byte row of the operand tile), rows a multiple of 64 long,
    fp32 tables, plain or double-quantised absmax."""
    if getattr(state, "quant_type", None) != "nf4" or state.blocksize != 64 or len(state.shape) != 2:
        return False
    if state.shape[1] % 64 or state.shape[0] % 8 or (k is not None and state.shape[1] != k):
        return False
    code = getattr(state, "code", None)
    if code is None or code.numel() != 16 or code.dtype != torch.float32 or not code.is_cuda:
        return False
    if state.nested:
        s2 = state.state2
        return (s2.blocksize > 0 and (s2.blocksize & (s2.blocksize - 1)) == 0
                and s2.code.dtype == torch.float32 and s2.code.numel() == 256
                and s2.absmax.dtype == torch.float32 and state.absmax.dtype == torch.uint8)
    return state.absmax.dtype == torch.float32


def _gemm_items(weights, keep):
    import ctypes

    items = (_lib.Nf4GemmItem * len(weights))()
    first = weights[0][1]
    for i, (packed, st) in enumerate(weights):
        _lib.require_cuda(packed)
        if (bool(st.nested) != bool(first.nested)
                or (st.nested and st.state2.blocksize != first.state2.blocksize)):
            raise ValueError("the weights of one launch share their nesting")
        absmax = st.absmax.contiguous()
        keep.append(absmax)
        items[i].packed, items[i].absmax = packed.data_ptr(), absmax.data_ptr()
        items[i].n_out = st.shape[0]
        if st.nested:
            code2, absmax2 = st.state2.code.contiguous(), st.state2.absmax.contiguous()
            offset = _offset_tensor(st.offset, packed.device)
            keep += [code2, absmax2, offset]
            items[i].code2, items[i].absmax2, items[i].offset = (code2.data_ptr(), absmax2.data_ptr(),
                                                                 offset.data_ptr())
    return items, ctypes.cast(items, ctypes.c_void_p)


# contractions at least this long may be split over CTA pairs (needs an fp32 buffer; the result is
# then summed with atomics and not bit-reproducible)
SPLIT_MIN_K = 4096


def nf4_linear(x, weights, biases=None):
    """[x @ dequant(W_i)^T (+ bias_i)] for up to four NF4 weights that share the input, in one
    launch, without the fp16 weights in memory. `x` fp16 [..., k]; `weights` a list of
    (packed, state); returns a list of fp16 [..., n_i]."""
    if x.dtype != torch.float16:
        raise TypeError("the NF4 GEMM computes in float16")
    k = x.shape[-1]
    rows = x.reshape(-1, k).contiguous()
    m = rows.shape[0]
    keep = []
    items, items_ptr = _gemm_items(weights, keep)
    outs = []
    for i, (packed, st) in enumerate(weights):
        if not gemm_supported(st, k):
            raise ValueError(f"weight {i} ({tuple(st.shape)}, blocksize {st.blocksize}) is not one "
                             "the NF4 GEMM takes")
        out = torch.empty((m, st.shape[0]), dtype=torch.float16, device=x.device)
        outs.append(out)
        items[i].out = out.data_ptr()
        bias = None if biases is None else biases[i]
        if bias is not None:
            bias = bias.to(torch.float16).contiguous()
            keep.append(bias)
            items[i].bias = bias.data_ptr()
    first = weights[0][1]
    workspace, nbytes = None, 0
    if len(weights) == 1 and k >= SPLIT_MIN_K and m:
        nbytes = _lib.lib().soup_nf4_gemm_workspace_bytes(m, first.shape[0])
        workspace = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    _lib.call("soup_nf4_linear_fwd", _lib.ptr(rows), items_ptr, len(weights), _lib.ptr(first.code), m, k,
              int(bool(first.nested)), int(first.blocksize),
              int(first.state2.blocksize) if first.nested else 1, _lib.ptr(workspace), nbytes,
              _lib.stream_of(rows))
    return [o.view(*x.shape[:-1], o.shape[-1]) for o in outs]


def nf4_linear_dx(grads, weights, dx_dtype=torch.float16):
    """sum_i grads[i] @ dequant(W_i): the input gradient of `nf4_linear` for one or two weights,
    the sum formed in the accumulator. `grads[i]` fp16 [..., n_i]; returns `dx_dtype` (fp16 or
    fp32) [..., k]."""
    first = weights[0][1]
    k = first.shape[1]
    keep = []
    items, items_ptr = _gemm_items(weights, keep)
    lead = grads[0].shape[:-1]
    m = grads[0].reshape(-1, grads[0].shape[-1]).shape[0]
    for i, ((packed, st), g) in enumerate(zip(weights, grads)):
        if g.dtype != torch.float16:
            raise TypeError("the NF4 GEMM computes in float16")
        if not gemm_supported(st, k) or st.shape[0] % 64 or g.shape[-1] != st.shape[0]:
            raise ValueError(f"weight {i} ({tuple(st.shape)}) is not one the NF4 GEMM takes")
        g2 = g.reshape(-1, st.shape[0]).contiguous()
        keep.append(g2)
        items[i].dy = g2.data_ptr()
    dx = torch.empty((m, k), dtype=dx_dtype, device=grads[0].device)
    workspace, nbytes = None, 0
    if dx_dtype != torch.float32 and sum(st.shape[0] for _, st in weights) >= SPLIT_MIN_K and m:
        nbytes = _lib.lib().soup_nf4_gemm_workspace_bytes(m, k)
        workspace = torch.empty(nbytes, dtype=torch.uint8, device=dx.device)
    _lib.call("soup_nf4_linear_dx", items_ptr, len(weights), _lib.ptr(first.code), _lib.ptr(dx),
              _lib.dtype_code(dx_dtype), m, k, int(bool(first.nested)), int(first.blocksize),
              int(first.state2.blocksize) if first.nested else 1, _lib.ptr(workspace), nbytes,
              _lib.stream_of(dx))
    return dx.view(*lead, k)


ORIGINALS = {}    # "fallback" / "dequant": bitsandbytes' own functions, kept for everything we leave alone
_CODE = {}


def _nf4_code(device):
    """bitsandbytes' own NF4 code table on `device` (needs bitsandbytes)."""
    if device not in _CODE:
        import bitsandbytes.functional as bnbF

        _CODE[device] = bnbF.get_4bit_type("nf4", device=device).float()
    return _CODE[device]


# Why a gemm_4bit fallback call stays with bitsandbytes: (reason, predicate over the call's
# arguments). The first that holds wins; `explain_fallback_route` returns its reason.
_FALLBACK_RULES = (
    ("not nf4", lambda a: a["quant_type"] != "nf4"),
    ("activation dtype other than fp16/fp32", lambda a: a["A"].dtype not in (torch.float16, torch.float32)),
    ("activation not on a CUDA device", lambda a: not a["A"].is_cuda),
    ("nested statistics incomplete",
     lambda a: a["absmax_8bit"] is not None and (a["absmax_code"] is None or a["absmax_offset"] is None)),
)


def explain_fallback_route(**call):
    """"" when `_dequant_linear_fallback(**call)` can use this package's kernel, else the reason."""
    for reason, holds in _FALLBACK_RULES:
        if holds(call):
            return reason
    return ""


def _state_of_call(state_cls, call, code):
    """The QuantState a gemm_4bit fallback call describes. bitsandbytes hands the pieces over
    separately; with double quantisation `absmax` is the inner (fp32, per 256 blocks) statistic and
    `absmax_8bit` the per-block codes."""
    common = dict(shape=torch.Size(call["shapeB"]), code=code, blocksize=call["blocksize"],
                  quant_type="nf4", dtype=call["A"].dtype)
    if call["absmax_8bit"] is None:
        return state_cls(absmax=call["absmax"], **common)
    inner = state_cls(absmax=call["absmax"], code=call["absmax_code"], blocksize=256,
                      dtype=torch.float32)
    return state_cls(absmax=call["absmax_8bit"], offset=call["absmax_offset"], state2=inner, **common)


def patch_bnb_nf4_dequant():
    """Routes the two places where bitsandbytes dequantises an NF4 weight through
    `dequantize_nf4`: the dequant + F.linear fallback of gemm_4bit (forward of Linear4bit for more
    than one row) and functional.dequantize_4bit (the input gradient of MatMul4Bit.backward).
    Everything the kernel does not cover (fp4, bf16, CPU tensors, an `out=` buffer, layouts
    `_supported` refuses) is handed to bitsandbytes' own function unchanged. Idempotent; without
    bitsandbytes there is nothing to patch and the call returns (the reference's patch raises
    there, solution/nf4.py:94-96)."""
    if ORIGINALS:
        return
    try:
        import bitsandbytes.functional as bnbF
        from bitsandbytes.backends.cuda import ops as cuda_ops
    except Exception:  # noqa: BLE001
        return
    state_cls = bnbF.QuantState
    theirs_linear, theirs_dequant = cuda_ops._dequant_linear_fallback, bnbF.dequantize_4bit
    ORIGINALS.update(fallback=theirs_linear, dequant=theirs_dequant)

    def _dequant_linear_fallback(A, B, shapeB, absmax, blocksize, quant_type, bias=None,
                                 absmax_8bit=None, absmax_code=None, absmax_offset=None):
        call = dict(A=A, B=B, shapeB=shapeB, absmax=absmax, blocksize=blocksize,
                    quant_type=quant_type, absmax_8bit=absmax_8bit, absmax_code=absmax_code,
                    absmax_offset=absmax_offset)
        state = None
        if not explain_fallback_route(**call):
            state = _state_of_call(state_cls, call, _nf4_code(A.device))
        if state is None or not _supported(B, state, A.dtype):
            return theirs_linear(A, B, shapeB, absmax, blocksize, quant_type, bias,
                                 absmax_8bit=absmax_8bit, absmax_code=absmax_code,
                                 absmax_offset=absmax_offset)
        return torch.nn.functional.linear(A, dequantize_nf4(B, state, A.dtype), bias)

    def dequantize_4bit(A, quant_state=None, absmax=None, out=None, blocksize=None,
                        quant_type="fp4"):
        ours = out is None and quant_state is not None and _supported(A, quant_state, quant_state.dtype)
        if not ours:
            return theirs_dequant(A, quant_state, absmax, out, blocksize, quant_type)
        weight = dequantize_nf4(A, quant_state)
        # a weight packed as one row [1, X] is stored transposed by bitsandbytes
        return weight.t() if A.shape[0] == 1 else weight

    cuda_ops._dequant_linear_fallback = _dequant_linear_fallback
    bnbF.dequantize_4bit = dequantize_4bit
