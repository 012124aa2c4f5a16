"""NF4 oracle: dequantiser restated from solution/nf4.py:31-46, plus stand-in tables/quantiser.

bitsandbytes 0.50.2 (pinned by the reference's kaggle_run.sh:10-11) owns the literal 16-entry NF4
table, the 256-entry dynamic map and the quantiser; none of them is in the reference tree. The
stand-ins below follow the published description of NF4 (QLoRA, Dettmers et al. 2023, appendix:
2^(k-1)+1 quantiles of N(0,1) for the positive half and 2^(k-1) for the negative half, an exact
zero, normalised to [-1, 1]) and blockwise absmax quantisation with double quantisation of the
absmax (blocksize 256, mean offset). They define the test inputs; parity of the dequantiser does
not depend on their values because it reads every table from memory.
"""

import numpy as np
import torch


def nf4_code_table():
    """16 levels: quantiles of N(0,1) normalised to [-1, 1], asymmetric with an exact zero."""
    from scipy.stats import norm

    edge = 0.5 * (1 - 1 / 32 + 1 - 1 / 30)  # tail probability between the two half-grids
    pos = norm.ppf(np.linspace(edge, 0.5, 9)[:-1])
    neg = -norm.ppf(np.linspace(edge, 0.5, 8)[:-1])
    levels = np.sort(np.concatenate([neg, [0.0], pos]))
    levels = levels / np.abs(levels).max()
    return torch.tensor(levels, dtype=torch.float32)


def dynamic_map():
    """256-entry signed map in [-1, 1], monotone, denser near zero: sign * 10^(-e) * fraction with
    7 exponent decades. Stands in for bitsandbytes' dynamic 8-bit code."""
    values = [0.0, 1.0]
    per_decade = 18
    for e in range(7):
        frac = np.linspace(0.1, 1.0, per_decade + 1)[:-1] + 0.9 / per_decade / 2
        for f in frac:
            values += [f * 10.0 ** -e, -f * 10.0 ** -e]
    values += [-1.0, 5e-8]
    arr = np.array(sorted(set(values)), dtype=np.float64)
    assert arr.size >= 254, arr.size
    while arr.size < 256:
        arr = np.sort(np.append(arr, -arr[arr > 0][arr.size - 254] * 0.5))
    return torch.tensor(arr[:256], dtype=torch.float32)


def _nearest(table, x):
    """Index of the nearest table entry (table sorted ascending) for every element of x."""
    mid = (table[1:] + table[:-1]) / 2
    return torch.bucketize(x, mid)


class State:
    """Duck-type of bitsandbytes' QuantState, as solution/nf4.py:49-61 reads it."""

    def __init__(self, absmax, shape, code, blocksize, dtype, offset=None, state2=None):
        self.absmax, self.shape, self.code, self.blocksize = absmax, torch.Size(shape), code, blocksize
        self.dtype, self.offset, self.state2 = dtype, offset, state2
        self.quant_type = "nf4"
        self.nested = state2 is not None

    def to(self, device):
        s2 = self.state2
        if s2 is not None:
            s2 = State(s2.absmax.to(device), s2.shape, s2.code.to(device), s2.blocksize, s2.dtype)
        return State(self.absmax.to(device), self.shape, self.code.to(device), self.blocksize,
                     self.dtype, None if self.offset is None else self.offset.to(device), s2)


def quantize_nf4(w, blocksize=64, nested=True, blocksize2=256, code=None, code2=None):
    """Blockwise NF4 quantisation of a 2-D weight (row-major flattening): per block absmax in fp32,
    nearest code of w/absmax, two codes per byte high nibble first; nested: absmax minus its mean
    quantised to 8 bits per block of 256 with its own fp32 absmax. Returns (packed uint8 [n/2, 1],
    State)."""
    code = nf4_code_table() if code is None else code
    code2 = dynamic_map() if code2 is None else code2
    flat = w.detach().float().reshape(-1)
    n = flat.numel()
    assert n % 2 == 0
    pad = (-n) % blocksize
    blocks = torch.nn.functional.pad(flat, (0, pad)).view(-1, blocksize)
    absmax = blocks.abs().amax(1)
    scaled = blocks / absmax.clamp(min=1e-30)[:, None]
    idx = _nearest(code, scaled).reshape(-1)[:n].to(torch.uint8)
    packed = ((idx[0::2] << 4) | idx[1::2]).reshape(-1, 1)
    if not nested:
        return packed, State(absmax, w.shape, code, blocksize, w.dtype)
    offset = absmax.mean()
    centred = absmax - offset
    pad2 = (-centred.numel()) % blocksize2
    b2 = torch.nn.functional.pad(centred, (0, pad2)).view(-1, blocksize2)
    absmax2 = b2.abs().amax(1)
    q8 = _nearest(code2, (b2 / absmax2.clamp(min=1e-30)[:, None])).reshape(-1)[:centred.numel()]
    inner = State(absmax2, (absmax.numel(),), code2, blocksize2, torch.float32)
    return packed, State(q8.to(torch.uint8), w.shape, code, blocksize, w.dtype,
                         offset=offset.reshape(1).clone(), state2=inner)


def dequantize_nf4(packed, state, dtype=None):
    """solution/nf4.py:31-46 step by step in unfused fp32 torch ops: scale = code2[q8] * absmax2
    (one multiply), + offset (one add), value = code[nibble] * scale (one multiply), cast."""
    dtype = dtype or state.dtype
    byte = packed.reshape(-1).to(torch.int64)
    n = state.shape[0] * state.shape[1]
    elem = torch.arange(n // 2, dtype=torch.int64) * 2
    blk = elem // state.blocksize
    if state.nested:
        s2 = state.state2
        scale = s2.code[state.absmax.to(torch.int64)[blk]] * s2.absmax[blk // s2.blocksize]
        scale = scale + state.offset.reshape(())
    else:
        scale = state.absmax[blk]
    hi = state.code[byte >> 4] * scale
    lo = state.code[byte & 0xF] * scale
    return torch.stack((hi, lo), 1).reshape(tuple(state.shape)).to(dtype)
