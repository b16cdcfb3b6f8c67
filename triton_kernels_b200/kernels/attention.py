"""`scaled_dot_product_attention(q, k, v, sm_scale)` on the tcgen05 flash kernel
(reference: triton_kernels/kernels/attention.py:173-221)."""
from __future__ import annotations

import math

import torch

from triton_kernels_b200 import _lib


def attention_into(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, sm_scale: float,
                   k_splits: int = 1) -> None:
    """q,k,v,o are 4-D [B,H,L,D] *views* (any batch/head/row strides, unit stride on D).
    k_splits > 1: the keys run as that many ranges in separate CTAs plus a merge pass."""
    B, H, Lq, D = q.shape
    Lk = k.shape[2]
    for t in (q, k, v, o):
        assert t.stride(3) == 1
    if k_splits > 1:
        part_o = torch.empty((k_splits, B, H, Lq, D), device=q.device, dtype=torch.float32)
        part_lse = torch.empty((k_splits, B, H, Lq), device=q.device, dtype=torch.float32)
        _lib.check(
            _lib.load().fluxb_attention_split(
                _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), None, 0, 0, B, H, Lq, Lk, D,
                q.stride(0), q.stride(1), q.stride(2),
                k.stride(0), k.stride(1), k.stride(2),
                v.stride(0), v.stride(1), v.stride(2),
                o.stride(0), o.stride(1), o.stride(2),
                float(sm_scale), k_splits, _lib.ptr(part_o), _lib.ptr(part_lse), _lib.stream_handle(),
            )
        )
        return
    _lib.check(
        _lib.load().fluxb_attention(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), B, H, Lq, Lk, D,
            q.stride(0), q.stride(1), q.stride(2),
            k.stride(0), k.stride(1), k.stride(2),
            v.stride(0), v.stride(1), v.stride(2),
            o.stride(0), o.stride(1), o.stride(2),
            float(sm_scale), _lib.stream_handle(),
        )
    )


def key_splits_for(B: int, H: int, Lq: int, Lk: int, D: int = 128, sm_count: int | None = None) -> int:
    """1 or 2: whether cutting the keys in two pays.  A CTA owns 256 query rows of one head; when
    the last wave of B*H*ceil(Lq/256) CTAs leaves most SMs idle (3 heads x 66 query blocks = 198
    CTAs on 148 SMs run as two waves) twice as many half-length CTAs finish sooner, three
    half-waves.  Against that stand a second CTA prologue / output pass per query block and the
    merge pass over fp32 partial rows, so the estimate is in microseconds (measured on B200:
    1.85 us per key tile, 5.5 us per CTA outside the key loop, partial rows written and read once
    at about 5 TB/s) and the split must win by 5 %.  It does for 3 local heads at 16896 tokens
    (eight-way sequence parallelism) and does not for 6 or 12."""
    if sm_count is None:
        sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    ctas = B * H * ((Lq + 255) // 256)
    key_tiles = (Lk + 127) // 128
    if key_tiles < 8:
        return 1
    t1 = math.ceil(ctas / sm_count) * (key_tiles * 1.85 + 5.5)
    merge_us = 2 * 2 * B * H * Lq * D * 4 / 5e12 * 1e6 + 5.0
    t2 = math.ceil(2 * ctas / sm_count) * (math.ceil(key_tiles / 2) * 1.85 + 7.5) + merge_us
    return 2 if t2 < 0.95 * t1 else 1


def attention_scatter_into(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o_bases, n_ranks: int, rows_per_rank: int,
    o_strides: tuple[int, int, int], sm_scale: float, k_splits: int | None = None,
) -> None:
    """attention_into whose output rows go to one base address per owner of query rows (a ctypes
    array of `n_ranks` device pointers, possibly into other GPUs' memory): row r of head h, batch
    b lands at o_bases[r // rows_per_rank] + b*sb + h*sh + (r % rows_per_rank)*sl, with
    (sb, sh, sl) = `o_strides` in elements.  `k_splits` (default: key_splits_for) > 1 runs the
    keys as that many ranges in separate CTAs with a merge pass (fluxb_attention_split)."""
    B, H, Lq, D = q.shape
    Lk = k.shape[2]
    for t in (q, k, v):
        assert t.stride(3) == 1
    if k_splits is None:
        k_splits = key_splits_for(B, H, Lq, Lk, D)
    if k_splits > 1:
        part_o = torch.empty((k_splits, B, H, Lq, D), device=q.device, dtype=torch.float32)
        part_lse = torch.empty((k_splits, B, H, Lq), device=q.device, dtype=torch.float32)
        _lib.check(
            _lib.load().fluxb_attention_split(
                _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), None, o_bases, n_ranks, rows_per_rank, B, H, Lq, Lk, D,
                q.stride(0), q.stride(1), q.stride(2),
                k.stride(0), k.stride(1), k.stride(2),
                v.stride(0), v.stride(1), v.stride(2),
                *o_strides, float(sm_scale), k_splits, _lib.ptr(part_o), _lib.ptr(part_lse), _lib.stream_handle(),
            )
        )
        return
    _lib.check(
        _lib.load().fluxb_attention_scatter(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), o_bases, n_ranks, rows_per_rank, B, H, Lq, Lk, D,
            q.stride(0), q.stride(1), q.stride(2),
            k.stride(0), k.stride(1), k.stride(2),
            v.stride(0), v.stride(1), v.stride(2),
            *o_strides, float(sm_scale), _lib.stream_handle(),
        )
    )


def scaled_dot_product_attention(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, sm_scale: float | None = None
) -> torch.Tensor:
    """Non-causal softmax(q k^T * sm_scale) v for [B,H,L,D] bf16 tensors; returns [B,H,L,D].

    Unlike the reference kernel, L need not be a multiple of the tile size (tails are masked).
    """
    HEAD_DIM_Q, HEAD_DIM_K, HEAD_DIM_V = q.shape[-1], k.shape[-1], v.shape[-1]
    assert HEAD_DIM_Q == HEAD_DIM_K == HEAD_DIM_V
    assert HEAD_DIM_K in {16, 32, 64, 128, 256}
    _lib.require_cuda(q, k, v)
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise NotImplementedError("attention runs in bfloat16 only (the reference casts P to bf16 as well)")
    if HEAD_DIM_K not in (64, 128):
        raise NotImplementedError(f"attention is built for head_dim 64 and 128 (Flux uses 128); got {HEAD_DIM_K}")

    def usable(t):
        return t.stride(3) == 1 and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0

    q, k, v = (t if usable(t) else t.contiguous() for t in (q, k, v))
    if sm_scale is None:
        sm_scale = 1 / math.sqrt(HEAD_DIM_K)
    o = torch.empty(q.shape, device=q.device, dtype=q.dtype)
    attention_into(q, k, v, o, sm_scale)
    return o
