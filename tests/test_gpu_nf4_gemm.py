"""The tcgen05 GEMM with the NF4 dequantisation in its operand prologue (forward and input
gradient) through the C ABI.

* The operand must be bit-identical to dequantize_nf4's fp16 output (the reference's contract for
  the weight, tests_local/test_nf4.py:27-37): multiplying with an identity matrix returns the
  operand itself, exactly, through the real kernel path (one non-zero product per sum).
* The products must match F.linear on the dequantised weight (what the reference computes,
  solution/nf4.py:122) to fp16 rounding, and the fp32 CPU product within 1e-2 of the largest value,
  for the seven projection shapes of Qwen2.5-1.5B at the row counts of the training step, with and
  without bias, with ragged row counts, for one weight and for two weights in one launch."""

import pytest
import torch

from conftest import assert_close_rel_max

pytestmark = pytest.mark.gpu
DEV = "cuda"
F16, F32 = torch.float16, torch.float32

SHAPES = {"q": (1536, 1536), "kv": (256, 1536), "gate": (8960, 1536), "down": (1536, 8960)}


def quantised(shape, seed=0, nested=True):
    from claudemaxing_b200 import qlora

    gen = torch.Generator().manual_seed(seed)
    w = (torch.randn(*shape, generator=gen) * 0.02).half().to(DEV)
    packed, state = qlora.quantize_nf4(w, nested=nested)
    return packed, state


@pytest.mark.parametrize("name", ["kv", "q", "gate", "down"])
@pytest.mark.parametrize("nested", [True, False])
def test_forward_operand_is_bit_identical_to_the_dequant_kernel(name, nested):
    from claudemaxing_b200.nf4 import dequantize_nf4, nf4_linear

    n, k = SHAPES[name]
    packed, state = quantised((n, k), seed=1, nested=nested)
    want = dequantize_nf4(packed, state, F16)
    eye = torch.eye(k, dtype=F16, device=DEV)
    (got,) = nf4_linear(eye, [(packed, state)])          # got[i, j] = W[j, i]
    assert got.shape == (k, n)
    assert torch.equal(got.t().contiguous().view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("name", ["kv", "q", "gate", "down"])
def test_backward_operand_is_bit_identical_to_the_dequant_kernel(name):
    from claudemaxing_b200.nf4 import dequantize_nf4, nf4_linear_dx

    n, k = SHAPES[name]
    packed, state = quantised((n, k), seed=2)
    want = dequantize_nf4(packed, state, F16)
    eye = torch.eye(n, dtype=F16, device=DEV)
    for dtype in (F16, F32):
        got = nf4_linear_dx([eye], [(packed, state)], dtype)  # got = W
        assert got.shape == (n, k) and got.dtype == dtype
        assert torch.equal(got.to(F16).view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("name", ["kv", "q", "gate", "down"])
@pytest.mark.parametrize("rows", [1168, 1280, 2048, 77])
def test_forward_matches_linear_on_the_dequantised_weight(name, rows):
    from claudemaxing_b200.nf4 import dequantize_nf4, nf4_linear

    n, k = SHAPES[name]
    packed, state = quantised((n, k), seed=3)
    w = dequantize_nf4(packed, state, F16)
    gen = torch.Generator().manual_seed(rows)
    x = torch.randn(1, rows, k, generator=gen).half().to(DEV)
    bias = (torch.randn(n, generator=gen) * 0.1).half().to(DEV) if name in ("q", "kv") else None
    (got,) = nf4_linear(x, [(packed, state)], [bias])
    assert got.shape == (1, rows, n) and got.dtype == F16
    lib = torch.nn.functional.linear(x, w, bias)
    assert_close_rel_max(got, lib, 2e-3, "against F.linear on the dequantised weight")
    ref = torch.nn.functional.linear(x.float().cpu(), w.float().cpu(), None if bias is None else bias.float().cpu())
    assert_close_rel_max(got.cpu(), ref, 1e-2, "against the fp32 CPU product")


@pytest.mark.parametrize("name", ["kv", "q", "gate", "down"])
@pytest.mark.parametrize("rows", [1280, 300])
@pytest.mark.parametrize("dx_dtype", [F16, F32])
def test_input_gradient_matches_matmul_with_the_dequantised_weight(name, rows, dx_dtype):
    from claudemaxing_b200.nf4 import dequantize_nf4, nf4_linear_dx

    n, k = SHAPES[name]
    packed, state = quantised((n, k), seed=4)
    w = dequantize_nf4(packed, state, F16)
    g = torch.randn(rows, n, generator=torch.Generator().manual_seed(5)).half().to(DEV)
    got = nf4_linear_dx([g], [(packed, state)], dx_dtype)
    assert got.shape == (rows, k) and got.dtype == dx_dtype
    ref = g.float().cpu() @ w.float().cpu()
    assert_close_rel_max(got.cpu(), ref, 2e-3 if dx_dtype == F32 else 4e-3, "against the fp32 CPU product")


def test_gate_and_up_in_one_launch_and_their_summed_input_gradient():
    from claudemaxing_b200.nf4 import dequantize_nf4, nf4_linear, nf4_linear_dx

    weights = [quantised(SHAPES["gate"], seed=6), quantised(SHAPES["gate"], seed=7)]
    x = torch.randn(1168, 1536, generator=torch.Generator().manual_seed(8)).half().to(DEV)
    gate, up = nf4_linear(x, weights)
    singles = [nf4_linear(x, [w])[0] for w in weights]
    # the same tiles, the same order of accumulation: identical to the one-weight launches
    assert torch.equal(gate, singles[0]) and torch.equal(up, singles[1])
    dg = torch.randn(1168, 8960, generator=torch.Generator().manual_seed(9)).half().to(DEV)
    du = torch.randn(1168, 8960, generator=torch.Generator().manual_seed(10)).half().to(DEV)
    dx = nf4_linear_dx([dg, du], weights, F32)
    dense = [dequantize_nf4(p, s, F16).float().cpu() for p, s in weights]
    ref = dg.float().cpu() @ dense[0] + du.float().cpu() @ dense[1]
    assert_close_rel_max(dx.cpu(), ref, 2e-3, "summed input gradient")


def test_unsupported_layouts_are_refused_with_a_message():
    from claudemaxing_b200 import qlora
    from claudemaxing_b200.nf4 import gemm_supported, nf4_linear

    w = (torch.randn(128, 256, generator=torch.Generator().manual_seed(0)) * 0.02).half().to(DEV)
    packed, state = qlora.quantize_nf4(w, blocksize=128)
    assert not gemm_supported(state)
    with pytest.raises(ValueError, match="not one the NF4 GEMM takes"):
        nf4_linear(torch.zeros(4, 256, dtype=F16, device=DEV), [(packed, state)])
    packed, state = qlora.quantize_nf4(w)
    with pytest.raises(TypeError):
        nf4_linear(torch.zeros(4, 256, device=DEV), [(packed, state)])
    from claudemaxing_b200 import _lib

    _lib.check_device_status()
