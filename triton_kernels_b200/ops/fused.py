"""Stand-alone callables for the small fused ops around the block GEMMs.

Each corresponds to one raw kernel of the reference's triton_kernels/ops/ directory (which has
no launchers): linear.py (mm + bias), modulation.py (scale/shift and gate*proj + residual),
qkv_concat.py (txt/img split + head-major concat) and silu.py.  In the fused blocks most of
these run as GEMM epilogues or inside `qkv_prepare`; the stand-alone forms exist for API parity
and microbenchmarks.
"""
from __future__ import annotations

import torch

from triton_kernels_b200 import _lib
from triton_kernels_b200.kernels.linear import linear


def linear_bias(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """out = a @ w.T + c (reference ops/linear.py:5-71: mm template with a row-broadcast bias)."""
    return linear(a, w, c)


def _vec(t):
    return 8 if t.dtype == torch.bfloat16 else 4


def modulation_scale_shift(x: torch.Tensor, modulation: torch.Tensor, is_mod1: bool = True) -> torch.Tensor:
    """(1 + scale) * x + shift with (shift, scale) = chunks (0,1) [mod1] or (3,4) [mod2] of the
    packed modulation tensor [B, n*C] (reference ops/modulation.py:5-27).  x: [B, L, C]."""
    _lib.require_cuda(x, modulation)
    B, L, C = x.shape
    x = x.contiguous()
    modulation = modulation.reshape(B, -1).to(x.dtype).contiguous()
    out = torch.empty_like(x)
    _lib.check(
        _lib.load().fluxb_modulation_scale_shift(
            _lib.ptr(x), _lib.ptr(modulation), _lib.ptr(out), B, L, C, modulation.stride(0), int(is_mod1),
            _lib.dtype_code(x), _lib.stream_handle(),
        )
    )
    return out


def modulation_gate_proj(img: torch.Tensor, modulation: torch.Tensor, proj: torch.Tensor, gate_chunk: int = 2) -> torch.Tensor:
    """img + gate * proj with gate = chunk `gate_chunk` of the packed modulation tensor
    (reference ops/modulation.py:29-44 uses chunk 2 = mod1.gate; chunk 5 is mod2.gate)."""
    _lib.require_cuda(img, modulation, proj)
    B, L, C = img.shape
    img, proj = img.contiguous(), proj.contiguous()
    modulation = modulation.reshape(B, -1).to(img.dtype).contiguous()
    out = torch.empty_like(img)
    _lib.check(
        _lib.load().fluxb_modulation_gate_proj(
            _lib.ptr(img), _lib.ptr(modulation), _lib.ptr(proj), _lib.ptr(out), B, L, C, modulation.stride(0),
            gate_chunk, _lib.dtype_code(img), _lib.stream_handle(),
        )
    )
    return out


def silu(x: torch.Tensor) -> torch.Tensor:
    """x * sigmoid(x) (reference ops/silu.py:5-13)."""
    _lib.require_cuda(x)
    x = x.contiguous()
    out = torch.empty_like(x)
    _lib.check(_lib.load().fluxb_silu(_lib.ptr(x), _lib.ptr(out), x.numel(), _lib.dtype_code(x), _lib.stream_handle()))
    return out


def modulation_silu_linear(vec: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None) -> torch.Tensor:
    """silu(vec) @ w.T + b for a small batch: the adaLN modulation projection
    (reference modules/blocks.py:61-62).  bf16; weights are streamed exactly once."""
    _lib.require_cuda(vec, w, b)
    if vec.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise NotImplementedError("modulation_silu_linear takes bfloat16 tensors")
    B, K = vec.shape
    N = w.shape[0]
    vec, w = vec.contiguous(), w.contiguous()
    if b is not None:
        b = b.to(torch.bfloat16).contiguous()
    out = torch.empty((B, N), device=vec.device, dtype=vec.dtype)
    _lib.check(
        _lib.load().fluxb_modulation_gemv(
            _lib.ptr(vec), _lib.ptr(w), _lib.ptr(b), _lib.ptr(out), B, N, K, 1, _lib.stream_handle()
        )
    )
    return out


def modulation_silu_linear_rows(vec: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None, out: torch.Tensor,
                                row0: int, row1: int, light: bool = False) -> None:
    """Columns [row0, row1) of `out` [B, N] = silu(vec) @ w[row0:row1].T + b[row0:row1]: the
    modulation projection filled in pieces.  `light` launches a form small enough to be resident
    beside a GEMM, for a piece whose result is needed later."""
    B, K = vec.shape
    assert out.shape == (B, w.shape[0]) and out.stride(1) == 1 and 0 <= row0 <= row1 <= w.shape[0]
    assert vec.is_contiguous() and w.is_contiguous() and vec.dtype == w.dtype == out.dtype == torch.bfloat16
    bias = None if b is None else b[row0:row1]
    assert bias is None or (bias.dtype == torch.bfloat16 and bias.is_contiguous())
    _lib.check(
        _lib.load().fluxb_modulation_gemv_rows(
            _lib.ptr(vec), _lib.ptr(w[row0:row1]), _lib.ptr(bias), _lib.ptr(out[:, row0:row1]), B, row1 - row0, K,
            out.stride(0), 1, int(light), _lib.stream_handle()
        )
    )


def qkv_prepare_into(
    streams: list[tuple[torch.Tensor, torch.Tensor | None, torch.Tensor | None]],
    pe: torch.Tensor | None,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    num_heads: int,
    eps: float = 1e-6,
    out_layout: tuple[int, int, int, int, int] | None = None,
    head_dim: int | None = None,
) -> None:
    """streams: one or two (src [B, L_s, >=3*H*D] with unit column stride, q_scale, k_scale);
    q,k,v: outputs with L = sum L_s rows per (batch, head).  By default they are contiguous
    [B,H,L,D]; `out_layout` = (heads_per_group, batch stride, group stride, head stride, row
    stride) in elements addresses them as b*sb + (h // hpg)*sg + (h % hpg)*sh + l*sl instead."""
    assert 1 <= len(streams) <= 2
    B = streams[0][0].shape[0]
    D = head_dim if head_dim is not None else q.shape[-1]
    args = []
    for src, qs, ks in streams:
        assert src.stride(2) == 1 and (src.shape[0] == 1 or src.stride(0) == src.shape[1] * src.stride(1))
        args += [_lib.ptr(src), src.shape[1], src.stride(1), _lib.ptr(qs), _lib.ptr(ks)]
    if len(streams) == 1:
        args += [None, 0, 0, None, None]
    pe_c = None
    if pe is not None:
        pe_c = pe if (pe.dtype == torch.float32 and pe.is_contiguous()) else pe.to(torch.float32).contiguous()
    layout = out_layout if out_layout is not None else (0, 0, 0, 0, 0)
    _lib.check(
        _lib.load().fluxb_qkv_prep(
            *args, _lib.ptr(pe_c), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), B, num_heads, D, *layout, eps,
            _lib.stream_handle()
        )
    )


def qkv_prepare_scatter(
    streams: list[tuple[torch.Tensor, torch.Tensor | None, torch.Tensor | None]],
    pe: torch.Tensor | None,
    group_bases,
    n_groups: int,
    k_off: int,
    v_off: int,
    num_heads: int,
    head_dim: int,
    strides: tuple[int, int, int],
    eps: float = 1e-6,
) -> None:
    """qkv_prepare_into with one output base address per head group (a ctypes array of
    `n_groups` device pointers, possibly into other GPUs' memory): q of head h, token l, batch b
    lands at group_bases[h // hpg] + b*sb + (h % hpg)*sh + l*sl with (sb, sh, sl) = `strides` in
    elements and hpg = num_heads // n_groups; k and v lie k_off / v_off elements further."""
    assert 1 <= len(streams) <= 2
    B = streams[0][0].shape[0]
    args = []
    for src, qs, ks in streams:
        assert src.stride(2) == 1 and (src.shape[0] == 1 or src.stride(0) == src.shape[1] * src.stride(1))
        args += [_lib.ptr(src), src.shape[1], src.stride(1), _lib.ptr(qs), _lib.ptr(ks)]
    if len(streams) == 1:
        args += [None, 0, 0, None, None]
    pe_c = None
    if pe is not None:
        pe_c = pe if (pe.dtype == torch.float32 and pe.is_contiguous()) else pe.to(torch.float32).contiguous()
    sb, sh, sl = strides
    _lib.check(
        _lib.load().fluxb_qkv_prep_scatter(
            *args, _lib.ptr(pe_c), group_bases, n_groups, k_off, v_off, B, num_heads, head_dim,
            num_heads // n_groups, sb, sh, sl, eps, _lib.stream_handle()
        )
    )


def qkv_prepare(
    qkv_streams: list[torch.Tensor],
    num_heads: int,
    q_scales: list[torch.Tensor] | None = None,
    k_scales: list[torch.Tensor] | None = None,
    pe: torch.Tensor | None = None,
    eps: float = 1e-6,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Split packed q|k|v projections of one or two token streams (first stream's tokens first),
    RMS-normalise q and k per head with the per-stream scales, apply RoPE with `pe`, and return
    q, k, v as [B, H, L, D].  With no scales and no pe this is exactly the reference's
    ops/qkv_concat.py:5-60; with them it also covers QKNorm + apply_rope of
    modules/blocks.py:113-119,148-162."""
    _lib.require_cuda(*qkv_streams)
    B = qkv_streams[0].shape[0]
    HD3 = qkv_streams[0].shape[-1]
    D = HD3 // (3 * num_heads)
    L = sum(t.shape[1] for t in qkv_streams)
    dev, dt = qkv_streams[0].device, qkv_streams[0].dtype
    if dt != torch.bfloat16:
        raise NotImplementedError("qkv_prepare takes bfloat16 tensors")
    q = torch.empty((B, num_heads, L, D), device=dev, dtype=dt)
    k = torch.empty_like(q)
    v = torch.empty_like(q)
    streams = []
    for i, t in enumerate(qkv_streams):
        qs = q_scales[i].to(dt).contiguous() if q_scales is not None else None
        ks = k_scales[i].to(dt).contiguous() if k_scales is not None else None
        streams.append((t.contiguous(), qs, ks))
    qkv_prepare_into(streams, pe, q, k, v, num_heads, eps)
    return q, k, v


def qkv_concat(txt_qkv: torch.Tensor, img_qkv: torch.Tensor, num_heads: int):
    """Reference ops/qkv_concat.py:5-60: q,k,v = cat((txt, img), dim=L) in head-major layout."""
    return qkv_prepare([txt_qkv, img_qkv], num_heads)
