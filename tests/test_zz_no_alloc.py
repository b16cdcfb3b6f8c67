"""The allocation-free RMSNorm backward (fluxb_rms_norm_bwd_static) against the ordinary entry
point (fluxb_rms_norm_bwd + a sum over its partial rows), called straight through the C ABI.

It exists for callers that cannot allocate device memory — e.g. a host with a frozen memory
plan that only hands the library a stream and ready-made buffers — so its scratch is a fixed
array inside the library.  Two calls in a row (the second smaller, so it reuses a region the
first one filled) check that nothing one call leaves in that array reaches the next.
This file sorts last so that a run stopping at the first failure has already run everything else.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, _lib, rows, cols, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g).to(dtype).cuda()
    dy = torch.randn(rows, cols, generator=g).to(dtype).cuda()
    w = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype).cuda()
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6).contiguous()
    code = _lib.dtype_code(x)
    st = _lib.stream_handle()
    # existing entry point: caller-allocated scratch, caller-side reduction
    parts = lib.fluxb_rms_norm_bwd_partial_rows(rows)
    dx_ref = torch.empty_like(x)
    partial = torch.empty(parts, cols, dtype=torch.float32, device="cuda")
    _lib.check(lib.fluxb_rms_norm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx_ref.data_ptr(),
                                      partial.data_ptr(), rows, cols, code, st))
    dw_ref = partial.sum(0)
    # new entry point: only inputs and outputs
    dx = torch.empty_like(x)
    dw = torch.full((cols,), float("nan"), dtype=torch.float32, device="cuda")
    _lib.check(lib.fluxb_rms_norm_bwd_static(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                             dw.data_ptr(), rows, cols, code, st))
    torch.cuda.synchronize()
    return dx, dw, dx_ref, dw_ref


def test_static_scratch_backward_matches_on_two_calls_in_a_row(lib):
    from triton_kernels_b200 import _lib

    for rows, cols, dtype, seed in [(24 * 300, 128, torch.float32, 31), (1000, 128, torch.float32, 32),
                                    (700, 3072, torch.bfloat16, 33)]:
        dx, dw, dx_ref, dw_ref = _both(lib, _lib, rows, cols, dtype, seed)
        assert torch.equal(dx, dx_ref)  # same kernel, same inputs
        torch.testing.assert_close(dw, dw_ref, atol=1e-3, rtol=1e-4)


def test_static_scratch_backward_rejects_oversized_problems(lib):
    from triton_kernels_b200 import _lib

    limit = lib.fluxb_rms_norm_bwd_static_max_floats()
    assert limit == 1 << 20
    rows, cols = 64 * 400, 3072  # 400 partial rows x 3072 > 1 Mi floats
    t = torch.zeros(8, device="cuda")
    rc = lib.fluxb_rms_norm_bwd_static(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(),
                                       t.data_ptr(), rows, cols, _lib.F32, _lib.stream_handle())
    assert rc == _lib.ERR_UNSUPPORTED
    assert b"built-in array" in lib.fluxb_last_error()
