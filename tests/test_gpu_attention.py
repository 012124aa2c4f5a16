"""The packed row's attention kernels (csrc/attention.cu) through the C ABI: forward output and
log-sum-exp, and the three gradients, against the float64 oracle (oracle/attention.py), on the
reference's golden vectors, at the shapes of the reference's own attention test with its
criterion (tests_local/test_attention.py:45-50, :85-97: the error against fp32 must stay within
three times the error of torch's fp16 SDPA on the same inputs), and on the edge cases of the
packed layout (empty and one-token segments, segments that end inside a tile, strided q/k/v)."""

import pytest
import torch

from conftest import assert_close_rel_max, rel_norm

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cu(lens):
    return torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)


def _run(q, k, v, cu, grad, scale=None):
    """(out, lse, dq, dk, dv) of the kernels on [N, h, 128] fp16 views (any row pitch)."""
    from claudemaxing_b200 import _lib
    from claudemaxing_b200.attention import attention_gradients

    n, hq, d = q.shape
    scale = d ** -0.5 if scale is None else scale
    out = torch.full((n, hq, d), float("nan"), dtype=torch.float16, device=DEV)
    lse = torch.full((hq, n), float("nan"), dtype=torch.float32, device=DEV)
    cu = cu.to(DEV)
    _lib.call("soup_attn_fwd", _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(cu), _lib.ptr(out),
              _lib.ptr(lse), n, cu.numel() - 1, hq, k.shape[1], d, q.stride(0), k.stride(0),
              v.stride(0), float(scale), _lib.stream_of(q))
    dq, dk, dv = attention_gradients(q, k, v, out, lse, grad, cu, scale)
    _lib.check_device_status()
    return out, lse, dq, dk, dv


@pytest.mark.parametrize("tag", ["a", "b"])
def test_attention_kernels_on_the_reference_kernels_golden_vectors(tag):
    from test_oracle_golden import _packed_attention_case

    _, q, k, v, cu, grad, want = _packed_attention_case(tag)
    out, _, dq, dk, dv = _run(q.to(DEV), k.to(DEV), v.to(DEV), cu, grad.to(DEV))
    for name, got in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
        assert_close_rel_max(got.float().cpu(), want[name].float(), 4e-3, name)


@pytest.mark.parametrize("hq,hk,lens", [
    (12, 2, [128, 128]),
    (12, 2, [200, 150, 77, 1]),
    (12, 2, [512, 300, 129]),
    (4, 4, [70]),
    (12, 2, [300, 0, 280, 296, 292, 112]),
    (6, 1, [1000, 3]),
    (4, 2, [40] * 100 + [3]),        # more than 64 segments: the plain tile order
    (2, 1, [2500]),                  # twenty key tiles: many turns of every barrier
])
def test_attention_kernels_against_fp32_with_the_fp16_sdpa_error_as_the_bar(hq, hk, lens):
    from oracle import attention as oat

    from claudemaxing_b200.attention import mask_of_segments

    torch.manual_seed(0)
    n, d = sum(lens), 128
    cu = _cu(lens)
    q, k, v = (torch.randn(n, h, d, device=DEV).half() for h in (hq, hk, hk))
    grad = torch.randn(n, hq, d, device=DEV).half()
    out, lse, dq, dk, dv = _run(q, k, v, cu, grad)
    want_out, want_lse = oat.segment_attention(q.cpu(), k.cpu(), v.cpu(), cu)
    want = (want_out,) + oat.segment_attention_backward(q.cpu(), k.cpu(), v.cpu(), cu, grad.cpu())
    # the bar: torch's fp16 SDPA with the mask on the same inputs
    leaves = [t.clone().requires_grad_() for t in (q, k, v)]
    ref = torch.nn.functional.scaled_dot_product_attention(
        leaves[0].transpose(0, 1)[None], leaves[1].transpose(0, 1)[None], leaves[2].transpose(0, 1)[None],
        attn_mask=mask_of_segments(cu.to(DEV), n), enable_gqa=hq != hk)[0].transpose(0, 1)
    ref.backward(grad)
    bar = (ref.detach(),) + tuple(t.grad for t in leaves)
    for name, got, exact, lib in zip(("out", "dq", "dk", "dv"), (out, dq, dk, dv), want, bar):
        assert torch.isfinite(got).all(), name
        err, allowed = rel_norm(got.float().cpu(), exact.float()), rel_norm(lib.float().cpu(), exact.float())
        assert err <= 3 * allowed + 1e-4, (name, err, allowed)
    assert dk.dtype == dv.dtype == torch.float32 and dq.dtype == torch.float16
    assert (lse.double().cpu() - want_lse).abs().max() < 2e-3


def test_attention_kernels_read_q_k_v_as_column_blocks_and_leave_other_rows_alone():
    """q, k and v as column blocks of one wider matrix (row pitch larger than heads x 128), and
    segments that do not cover the last tokens: those rows of out / dq are not written."""
    from oracle import attention as oat

    torch.manual_seed(1)
    lens, spare = [130, 61], 9
    n_seg, hq, hk, d = sum(lens), 4, 2, 128
    n = n_seg + spare
    wide = torch.randn(n, (hq + 2 * hk) * d, device=DEV).half()
    q = wide[:, :hq * d].unflatten(-1, (hq, d))
    k = wide[:, hq * d:(hq + hk) * d].unflatten(-1, (hk, d))
    v = wide[:, (hq + hk) * d:].unflatten(-1, (hk, d))
    grad = torch.randn(n, hq, d, device=DEV).half()
    out, _, dq, dk, dv = _run(q, k, v, _cu(lens), grad, scale=0.11)
    want_out, _ = oat.segment_attention(q.cpu(), k.cpu(), v.cpu(), _cu(lens), 0.11)
    want = oat.segment_attention_backward(q.cpu(), k.cpu(), v.cpu(), _cu(lens), grad.cpu(), 0.11)
    assert_close_rel_max(out[:n_seg].float().cpu(), want_out[:n_seg].float(), 4e-3, "out")
    for name, got, exact in zip(("dq", "dk", "dv"), (dq[:n_seg], dk[:n_seg], dv[:n_seg]), want):
        assert_close_rel_max(got.float().cpu(), exact[:n_seg].float(), 4e-3, name)
    assert torch.isnan(out[n_seg:].float()).all()             # never touched
    assert (dk[n_seg:] == 0).all() and (dv[n_seg:] == 0).all()  # cleared, nothing added


def test_attention_kernels_refuse_what_they_do_not_cover():
    from claudemaxing_b200 import _lib

    q = torch.zeros(8, 2, 64, dtype=torch.float16, device=DEV)
    cu = torch.tensor([0, 8], dtype=torch.int32, device=DEV)
    out, lse = torch.empty_like(q), torch.empty(2, 8, device=DEV)
    with pytest.raises(RuntimeError, match="head_dim must be 128"):
        _lib.call("soup_attn_fwd", _lib.ptr(q), _lib.ptr(q), _lib.ptr(q), _lib.ptr(cu), _lib.ptr(out),
                  _lib.ptr(lse), 8, 1, 2, 2, 64, 128, 128, 128, 0.125, _lib.stream_of(q))
    q = torch.zeros(8, 3, 128, dtype=torch.float16, device=DEV)
    with pytest.raises(RuntimeError, match="multiple of key heads"):
        _lib.call("soup_attn_fwd", _lib.ptr(q), _lib.ptr(q), _lib.ptr(q), _lib.ptr(cu), _lib.ptr(q),
                  _lib.ptr(lse), 8, 1, 3, 2, 128, 384, 384, 384, 0.1, _lib.stream_of(q))
