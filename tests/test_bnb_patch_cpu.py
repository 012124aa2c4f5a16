"""Routing of patch_bnb_nf4_dequant on CPU with a stand-in `bitsandbytes` package (three modules,
the attributes the patch touches). The reference tests this against the real package on a GPU
(tests_local/test_nf4.py:40-89: both patched functions must reach the kernel, anything unsupported
must reach bitsandbytes' own code unchanged); bitsandbytes is not installed here, so what is
checked is which function each call ends up in and what it is given."""

import sys
import types

import pytest
import torch

from claudemaxing_b200 import nf4


class _QuantState:
    def __init__(self, absmax, shape=None, code=None, blocksize=None, quant_type=None, dtype=None,
                 offset=None, state2=None):
        self.absmax, self.shape, self.code, self.blocksize = absmax, shape, code, blocksize
        self.quant_type, self.dtype, self.offset, self.state2 = quant_type, dtype, offset, state2
        self.nested = state2 is not None


@pytest.fixture
def fake_bnb(monkeypatch):
    calls = {"fallback": [], "dequant": []}
    functional = types.ModuleType("bitsandbytes.functional")
    functional.QuantState = _QuantState
    functional.get_4bit_type = lambda kind, device=None: torch.linspace(-1, 1, 16)

    def dequantize_4bit(A, quant_state=None, absmax=None, out=None, blocksize=None, quant_type="fp4"):
        calls["dequant"].append((A, quant_state, absmax, out, blocksize, quant_type))
        return "theirs-dequant"

    functional.dequantize_4bit = dequantize_4bit
    ops = types.ModuleType("bitsandbytes.backends.cuda.ops")

    def _dequant_linear_fallback(A, B, shapeB, absmax, blocksize, quant_type, bias=None,
                                 absmax_8bit=None, absmax_code=None, absmax_offset=None):
        calls["fallback"].append(dict(A=A, B=B, shapeB=shapeB, absmax=absmax, blocksize=blocksize,
                                      quant_type=quant_type, bias=bias, absmax_8bit=absmax_8bit,
                                      absmax_code=absmax_code, absmax_offset=absmax_offset))
        return "theirs-linear"

    ops._dequant_linear_fallback = _dequant_linear_fallback
    root = types.ModuleType("bitsandbytes")
    backends = types.ModuleType("bitsandbytes.backends")
    cuda = types.ModuleType("bitsandbytes.backends.cuda")
    root.functional, root.backends, backends.cuda, cuda.ops = functional, backends, cuda, ops
    for name, mod in (("bitsandbytes", root), ("bitsandbytes.functional", functional),
                      ("bitsandbytes.backends", backends), ("bitsandbytes.backends.cuda", cuda),
                      ("bitsandbytes.backends.cuda.ops", ops)):
        monkeypatch.setitem(sys.modules, name, mod)
    monkeypatch.setattr(nf4, "ORIGINALS", {})
    monkeypatch.setattr(nf4, "_CODE", {})
    yield types.SimpleNamespace(functional=functional, ops=ops, calls=calls)


def test_patch_installs_once_and_keeps_the_originals(fake_bnb):
    theirs_linear, theirs_dequant = fake_bnb.ops._dequant_linear_fallback, fake_bnb.functional.dequantize_4bit
    nf4.patch_bnb_nf4_dequant()
    assert nf4.ORIGINALS == {"fallback": theirs_linear, "dequant": theirs_dequant}
    installed = (fake_bnb.ops._dequant_linear_fallback, fake_bnb.functional.dequantize_4bit)
    assert installed[0] is not theirs_linear and installed[1] is not theirs_dequant
    nf4.patch_bnb_nf4_dequant()        # a second call changes nothing
    assert (fake_bnb.ops._dequant_linear_fallback, fake_bnb.functional.dequantize_4bit) == installed


def test_without_bitsandbytes_the_patch_is_a_no_op(monkeypatch):
    monkeypatch.setattr(nf4, "ORIGINALS", {})
    monkeypatch.setitem(sys.modules, "bitsandbytes", None)      # import raises ImportError
    monkeypatch.setitem(sys.modules, "bitsandbytes.functional", None)
    nf4.patch_bnb_nf4_dequant()
    assert nf4.ORIGINALS == {}


def test_fallback_route_rules_name_the_reason():
    a16 = torch.zeros(2, 64, dtype=torch.float16)
    base = dict(A=a16, B=None, shapeB=(4, 64), absmax=None, blocksize=64, quant_type="nf4",
                absmax_8bit=None, absmax_code=None, absmax_offset=None)
    assert nf4.explain_fallback_route(**dict(base, quant_type="fp4")) == "not nf4"
    assert "dtype" in nf4.explain_fallback_route(**dict(base, A=a16.bfloat16()))
    assert "CUDA" in nf4.explain_fallback_route(**base)          # a CPU activation
    assert "nested" in nf4.explain_fallback_route(
        **dict(base, A=types.SimpleNamespace(dtype=torch.float16, is_cuda=True),
               absmax_8bit=torch.zeros(4, dtype=torch.uint8)))
    assert nf4.explain_fallback_route(
        **dict(base, A=types.SimpleNamespace(dtype=torch.float32, is_cuda=True))) == ""


def test_unsupported_calls_reach_bitsandbytes_unchanged(fake_bnb):
    nf4.patch_bnb_nf4_dequant()
    a = torch.zeros(2, 64, dtype=torch.float16)
    packed = torch.zeros(128, 1, dtype=torch.uint8)
    absmax, bias = torch.ones(4), torch.ones(4)
    out = fake_bnb.ops._dequant_linear_fallback(a, packed, (4, 64), absmax, 64, "fp4", bias)
    assert out == "theirs-linear"
    seen = fake_bnb.calls["fallback"][-1]
    assert seen["A"] is a and seen["B"] is packed and seen["bias"] is bias and seen["quant_type"] == "fp4"
    # nf4, but on the CPU: still theirs, nested arguments passed through by keyword
    a8, code2, off = torch.zeros(4, dtype=torch.uint8), torch.zeros(256), torch.zeros(())
    out = fake_bnb.ops._dequant_linear_fallback(a, packed, (4, 64), absmax, 64, "nf4", None,
                                                absmax_8bit=a8, absmax_code=code2, absmax_offset=off)
    seen = fake_bnb.calls["fallback"][-1]
    assert out == "theirs-linear" and seen["absmax_8bit"] is a8 and seen["absmax_code"] is code2
    assert seen["absmax_offset"] is off
    # dequantize_4bit: an out= buffer, a missing state, or an unsupported state keep their code
    state = _QuantState(absmax, (4, 64), torch.zeros(16), 64, "nf4", torch.float16)
    for kwargs in (dict(quant_state=state, out=torch.empty(4, 64)), dict(quant_state=None),
                   dict(quant_state=state)):
        assert fake_bnb.functional.dequantize_4bit(packed, **kwargs) == "theirs-dequant"
    assert len(fake_bnb.calls["dequant"]) == 3


def test_supported_calls_reach_the_kernel_with_the_state_the_call_describes(fake_bnb, monkeypatch):
    nf4.patch_bnb_nf4_dequant()
    seen = []

    def kernel(packed, state, dtype=None, out=None):
        seen.append((packed, state, dtype))
        shape = tuple(state.shape)
        return torch.arange(shape[0] * shape[1], dtype=torch.float32).view(shape).to(dtype or state.dtype)

    monkeypatch.setattr(nf4, "dequantize_nf4", kernel)
    monkeypatch.setattr(nf4, "_supported", lambda packed, state, dtype: True)
    monkeypatch.setattr(nf4, "_FALLBACK_RULES",
                        tuple(r for r in nf4._FALLBACK_RULES if "CUDA" not in r[0]))
    a = torch.ones(2, 8, dtype=torch.float32)
    packed = torch.zeros(12, 1, dtype=torch.uint8)
    inner_absmax, a8 = torch.ones(1), torch.zeros(1, dtype=torch.uint8)
    code2, off, bias = torch.zeros(256), torch.tensor(0.5), torch.ones(3)
    out = fake_bnb.ops._dequant_linear_fallback(a, packed, (3, 8), inner_absmax, 64, "nf4", bias,
                                                absmax_8bit=a8, absmax_code=code2, absmax_offset=off)
    got_packed, state, dtype = seen[-1]
    assert got_packed is packed and dtype == torch.float32 and not fake_bnb.calls["fallback"]
    assert state.absmax is a8 and state.offset is off and state.blocksize == 64 and state.nested
    assert state.state2.absmax is inner_absmax and state.state2.code is code2 and state.state2.blocksize == 256
    assert tuple(state.shape) == (3, 8) and state.quant_type == "nf4" and state.code.numel() == 16
    want = torch.nn.functional.linear(a, torch.arange(24, dtype=torch.float32).view(3, 8), bias)
    assert torch.equal(out, want)
    # without double quantisation `absmax` is the per-block statistic itself
    fake_bnb.ops._dequant_linear_fallback(a, packed, (3, 8), inner_absmax, 64, "nf4")
    assert seen[-1][1].absmax is inner_absmax and not seen[-1][1].nested
    # dequantize_4bit: [n/2, 1] packing gives [N, K]; a one-row packing [1, n/2] gives its transpose
    state = _QuantState(inner_absmax, (3, 8), torch.zeros(16), 64, "nf4", torch.float16)
    w = fake_bnb.functional.dequantize_4bit(packed, state)
    assert w.shape == (3, 8) and w.dtype == torch.float16
    wt = fake_bnb.functional.dequantize_4bit(packed.t(), state)
    assert wt.shape == (8, 3) and torch.equal(wt, w.t()) and not fake_bnb.calls["dequant"]
