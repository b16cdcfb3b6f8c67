"""`layer_norm_modulation` and `rms_norm` (reference: triton_kernels/kernels/normalization.py)."""
from __future__ import annotations

import torch

from triton_kernels_b200 import _lib


def _vec(t: torch.Tensor) -> int:
    return 8 if t.dtype == torch.bfloat16 else 4


def layer_norm_modulation_into(x2d, scale2d, shift2d, y2d, rows_per_batch: int, eps: float) -> None:
    """x2d/y2d: [rows, C] views (row stride free); scale2d/shift2d: [B, C] views with a common
    batch stride (chunks of the packed modulation tensor are fine)."""
    rows, C = x2d.shape
    assert scale2d.stride(0) == shift2d.stride(0) or scale2d.shape[0] == 1
    _lib.check(
        _lib.load().fluxb_layer_norm_modulation(
            _lib.ptr(x2d), _lib.ptr(scale2d), _lib.ptr(shift2d), _lib.ptr(y2d), rows, C, rows_per_batch,
            x2d.stride(0), y2d.stride(0), scale2d.stride(0) if scale2d.shape[0] > 1 else 0, eps,
            _lib.dtype_code(x2d), _lib.stream_handle(),
        )
    )


def layer_norm_modulation(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """LayerNorm(x) without affine, then `* (1 + weight) + bias` with weight/bias of shape
    [B, 1, C] broadcast over the sequence (reference :47-77; its default eps 1e-5 is kept).
    Statistics are fp32 whatever the storage dtype (rows of 2-24 KB: sum and sum of squares in
    one pass, fp32 rows shifted by their first element; other widths: mean, then centred variance)."""
    assert x.shape[0] == weight.shape[0] == bias.shape[0]
    assert x.shape[-1] == weight.shape[-1] == bias.shape[-1]
    _lib.require_cuda(x, weight, bias)
    B, C = x.shape[0], x.shape[-1]
    x = x.contiguous()
    v = _vec(x)
    w2 = weight.reshape(B, C).to(x.dtype)
    b2 = bias.reshape(B, C).to(x.dtype)

    def ok(t):
        return t.stride(1) == 1 and t.stride(0) % v == 0 and t.data_ptr() % 16 == 0

    if not (ok(w2) and ok(b2) and (B == 1 or w2.stride(0) == b2.stride(0))):
        w2, b2 = w2.contiguous(), b2.contiguous()
    y = torch.empty_like(x)
    x2 = x.reshape(-1, C)
    layer_norm_modulation_into(x2, w2, b2, y.reshape(-1, C), x2.shape[0] // B, eps)
    return y


class _rms_norm(torch.autograd.Function):
    """Forward and backward of RMSNorm over the last dim (reference :142-190)."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, scale: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
        assert x.shape[-1] == scale.shape[-1]
        _lib.require_cuda(x, scale)
        N = x.shape[-1]
        v = _vec(x)
        # Up to 3 leading dims are addressed through strides (head-split views need no copy).
        lead = x.shape[:-1]
        strided_ok = (
            x.dim() <= 4 and x.stride(-1) == 1 and all(s % v == 0 for s in x.stride()[:-1]) and x.data_ptr() % 16 == 0
        )
        if not strided_ok:
            x = x.contiguous()
        dims = [1] * (3 - len(lead)) + list(lead)
        strides = [0] * (3 - len(lead)) + list(x.stride()[:-1])
        # decided on the caller's tensors: the cast copy of `scale` below never requires grad
        need_grad = any(ctx.needs_input_grad[:2])
        ctx.scale_dtype = scale.dtype
        scale = scale.to(x.dtype).contiguous()
        y = torch.empty(x.shape, device=x.device, dtype=x.dtype)
        M = y.numel() // N
        rstd = torch.empty((M,), dtype=torch.float32, device=x.device) if need_grad else None
        _lib.check(
            _lib.load().fluxb_rms_norm(
                _lib.ptr(x), _lib.ptr(scale), _lib.ptr(y), _lib.ptr(rstd), dims[0], dims[1], dims[2], N,
                strides[0], strides[1], strides[2], eps, _lib.dtype_code(x), _lib.stream_handle(),
            )
        )
        if need_grad:
            ctx.save_for_backward(x, scale, rstd)
        return y

    @staticmethod
    def backward(ctx, dy: torch.Tensor):
        x, w, rstd = ctx.saved_tensors
        N = x.shape[-1]
        xc = x.contiguous().reshape(-1, N)
        dyc = dy.contiguous().reshape(-1, N).to(x.dtype)
        M = xc.shape[0]
        lib = _lib.load()
        dx = torch.empty_like(xc)
        parts = lib.fluxb_rms_norm_bwd_partial_rows(M)
        dw_partial = torch.empty((parts, N), dtype=torch.float32, device=x.device)
        _lib.check(
            lib.fluxb_rms_norm_bwd(
                _lib.ptr(dyc), _lib.ptr(xc), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(dx), _lib.ptr(dw_partial),
                M, N, _lib.dtype_code(xc), _lib.stream_handle(),
            )
        )
        dw = dw_partial.sum(dim=0).to(ctx.scale_dtype)
        return dx.reshape(x.shape), dw, None


rms_norm = _rms_norm.apply
