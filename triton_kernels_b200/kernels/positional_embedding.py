"""`apply_rope(xq, xk, freqs_cis)` (reference: triton_kernels/kernels/positional_embedding.py:55-82)."""
from __future__ import annotations

import torch

from triton_kernels_b200 import _lib


def apply_rope(xq: torch.Tensor, xk: torch.Tensor, freqs_cis: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Applies the per-position 2x2 transforms in `freqs_cis` ([1,1,L,D/2,2,2], fp32) to every
    (even, odd) pair of q and k ([B,H,L,D]).  The table may be any 2x2 matrices, not only
    rotations.  A table with a batch or head dimension other than 1 is rejected (the reference
    kernel silently ignores those dims)."""
    _lib.require_cuda(xq, xk, freqs_cis)
    assert xq.shape == xk.shape and xq.dtype == xk.dtype
    b, h, s, d = xq.shape
    if freqs_cis.numel() != s * (d // 2) * 4:
        raise ValueError(f"freqs_cis must hold one [L, D/2, 2, 2] table, got shape {tuple(freqs_cis.shape)}")
    xq, xk = xq.contiguous(), xk.contiguous()
    f = freqs_cis.to(torch.float32).contiguous()
    xq_out = torch.empty_like(xq)
    xk_out = torch.empty_like(xk)
    _lib.check(
        _lib.load().fluxb_rope(
            _lib.ptr(xq), _lib.ptr(xk), _lib.ptr(f), _lib.ptr(xq_out), _lib.ptr(xk_out), b * h, s, d,
            _lib.dtype_code(xq), _lib.stream_handle(),
        )
    )
    return xq_out, xk_out
