"""soup_rmsnorm_bwd_noalloc: the RMSNorm backward whose dw workspace is a fixed array inside the
library, for hosts that cannot allocate device memory during a step. It must give what
soup_rmsnorm_bwd gives with a caller-provided workspace, call after call (the built-in array keeps
the previous call's contents), and refuse shapes beyond its fixed size. Collected last on purpose:
a failure here must not hide the results of the other GPU tests in a stop-at-first-failure run."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _run(entry, dy, x, w, rstd, n_rows, n_cols, with_workspace):
    from claudemaxing_b200 import _lib

    dx = torch.empty_like(x)
    dw = torch.empty_like(w)
    code = _lib.dtype_code
    common = (None, None, 1, n_rows, n_cols, code(dy.dtype), code(x.dtype), code(w.dtype),
              code(x.dtype), 0, _lib.stream_of(x))
    if with_workspace:
        parts = _lib.lib().soup_rmsnorm_bwd_partials(n_rows, n_cols)
        partial = torch.empty(parts, n_cols, dtype=torch.float32, device=DEV)
        _lib.call(entry, dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                  partial.data_ptr(), dw.data_ptr(), *common)
    else:
        _lib.call(entry, dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                  dw.data_ptr(), *common)
    torch.cuda.synchronize()
    return dx, dw


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_noalloc_matches_workspace_entry_on_two_calls_in_a_row(dtype):
    gen = torch.Generator().manual_seed(0)
    results = []
    for n_rows, n_cols in ((700, 1536), (300, 1000)):  # second call: fewer rows, other width
        x = (3 * torch.randn(n_rows, n_cols, generator=gen)).to(dtype).to(DEV)
        w = (1 + 0.5 * torch.randn(n_cols, generator=gen)).to(dtype).to(DEV)
        dy = torch.randn(n_rows, n_cols, generator=gen).to(dtype).to(DEV)
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
        ref_dx, ref_dw = _run("soup_rmsnorm_bwd", dy, x, w, rstd, n_rows, n_cols, True)
        got_dx, got_dw = _run("soup_rmsnorm_bwd_noalloc", dy, x, w, rstd, n_rows, n_cols, False)
        # same kernels, same fixed-order reduction: identical, well inside the 2e-3 the other
        # RMSNorm tests allow
        assert torch.equal(got_dx, ref_dx)
        assert torch.equal(got_dw, ref_dw)
        scale = ref_dw.float().abs().max().item()
        assert (got_dw.float() - ref_dw.float()).abs().max().item() <= 2e-3 * scale
        # and against the CPU oracle (autograd of Qwen2RMSNorm.forward), so that the check does not
        # rest on the sibling entry alone; tolerances of the other RMSNorm tests
        from conftest import assert_close_rel_max
        from oracle import elementwise as ew

        _, o_dx, o_dw = ew.rmsnorm_fwd_bwd(x.cpu(), w.cpu(), dy.cpu(), weight_grad=True)
        tol = 2e-3 if dtype == torch.float16 else 1e-4
        assert_close_rel_max(got_dx.cpu(), o_dx, tol, "dx against the oracle")
        assert_close_rel_max(got_dw.cpu(), o_dw, 5 * tol, "dw against the oracle")
        results.append(got_dw)
    assert results[0].shape != results[1].shape


def test_noalloc_refuses_rows_wider_than_its_workspace():
    from claudemaxing_b200 import _lib

    x = torch.zeros(4, 8192, device=DEV, dtype=torch.float16)
    w = torch.ones(8192, device=DEV, dtype=torch.float16)
    rstd = torch.ones(4, device=DEV)
    with pytest.raises(RuntimeError, match="exceeds the built-in workspace"):
        _run("soup_rmsnorm_bwd_noalloc", x, x, w, rstd, 4, 8192, False)
