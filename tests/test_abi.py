"""The C-ABI library loads on a machine without a GPU and exports every symbol that
include/soup_b200.h declares, with the argument counts the ctypes binding uses; argument checks
that run before any CUDA call answer with an error code and a message (never abort)."""

import os
import re

import pytest

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "soup_b200.h")


def declared():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = {}
    for m in re.finditer(r"^(?:int|int64_t|const char\*)\s+(soup_\w+)\((.*?)\);", text, re.M | re.S):
        args = m.group(2).strip()
        out[m.group(1)] = 0 if args == "void" else len(args.split(","))
    return out


def test_header_symbols_exported_and_bound():
    from claudemaxing_b200 import _lib

    lib = _lib.lib()
    decl = declared()
    assert len(decl) >= 18
    for name, n_args in decl.items():
        assert hasattr(lib, name), f"{name} is declared but not exported"
        if name in ("soup_version", "soup_last_error_string"):
            continue
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
        assert len(_lib.SIGNATURES[name]) == n_args, f"{name}: header has {n_args} arguments"
    assert lib.soup_version() >= 1
    assert set(_lib.SIGNATURES) <= set(decl)


def test_argument_errors_are_reported_not_fatal():
    from claudemaxing_b200 import _lib

    with pytest.raises(RuntimeError, match="n_elems must be even"):
        _lib.call("soup_nf4_dequant", 16, 16, 16, None, None, None, 16, 3, 64, 1, 0, _lib.F16, None)
    with pytest.raises(RuntimeError, match="multiple of 8"):
        _lib.call("soup_dropout_pack", 16, 16, 16, 16, 12, 1.0, _lib.F32, None)
    with pytest.raises(RuntimeError, match="n_cols"):
        _lib.call("soup_rmsnorm_fwd", 16, 16, 16, 16, None, None, None, 1, 4, 20000, 1e-6, 0, 0, 0, None)
    with pytest.raises(RuntimeError, match="head_dim must be even"):
        _lib.call("soup_rope", 16, None, 16, 16, 16, None, 1, 1, 0, 4, 7, 0, 0, 0, 0, 0, 0, 0, 0,
                  0, 0, 0, 0, 0, 0, None)
    # zero-sized work is a no-op that needs no device
    assert _lib.call("soup_silu_mul_fwd", None, None, None, 0, 0, 0, 0, 1, None) == 0
    assert _lib.lib().soup_last_error_string() is not None


def test_no_cpu_fallback():
    import torch

    from claudemaxing_b200.lora import _pack
    from claudemaxing_b200.nf4 import dequantize_nf4
    from claudemaxing_b200.rmsnorm import rmsnorm

    with pytest.raises(RuntimeError, match="no CPU fallback"):
        rmsnorm(torch.randn(2, 8), torch.ones(8), 1e-6)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _pack(torch.randn(16), torch.ones(16, dtype=torch.bool), 1.0)

    class S:
        shape, dtype = (2, 8), torch.float16

    with pytest.raises(RuntimeError, match="no CPU fallback"):
        dequantize_nf4(torch.zeros(8, dtype=torch.uint8), S())
