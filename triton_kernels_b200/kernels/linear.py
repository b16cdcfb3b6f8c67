"""`linear(x, w, b, activation)` on the tcgen05 GEMM (reference: triton_kernels/kernels/linear.py:104-151)."""
from __future__ import annotations

import torch

from triton_kernels_b200 import _lib


class UnsupportedDtype(KeyError, TypeError):
    """Raised for non-bf16 inputs.  The reference raises KeyError here (its tile-config table
    has a bfloat16 entry only, triton_kernels/kernels/linear.py:105-114,142); this is also a
    TypeError so callers can catch either."""


def linear_into(
    x2d: torch.Tensor,
    w: torch.Tensor,
    b: torch.Tensor | None,
    y: torch.Tensor,
    *,
    epi: int = _lib.EPI_NONE,
    y2: torch.Tensor | None = None,
    split: int | None = None,
    epi2: int = _lib.EPI_NONE,
    resid: torch.Tensor | None = None,
    gate: torch.Tensor | None = None,
    gate_stride: int = 0,
    rows_per_batch: int = 1,
    round_before_act: bool = False,
) -> None:
    """Lowest-level launch: x2d [M,K] (row stride free), w [N,K], outputs caller-allocated 2-D
    views (row stride free, unit column stride).  See fluxb_linear in include/fluxb200.h."""
    M, K = x2d.shape
    N = w.shape[0]
    assert x2d.stride(1) == 1 and w.stride(1) == 1 and y.stride(1) == 1
    if split is None:
        split = N
    _lib.check(
        _lib.load().fluxb_linear(
            _lib.ptr(x2d), _lib.ptr(w), _lib.ptr(b), _lib.ptr(y), M, N, K,
            x2d.stride(0), w.stride(0), y.stride(0), epi,
            _lib.ptr(y2), y2.stride(0) if y2 is not None else 0, split, epi2,
            _lib.ptr(resid), resid.stride(0) if resid is not None else 0,
            _lib.ptr(gate), gate_stride, rows_per_batch, int(round_before_act),
            _lib.stream_handle(),
        )
    )


def linear_grouped_into(
    problems: list[dict],
    *,
    epi: int = _lib.EPI_NONE,
    split: int | None = None,
    epi2: int = _lib.EPI_NONE,
    round_before_act: bool = False,
) -> None:
    """Several linears with the same N, K and epilogue in ONE launch (fluxb_linear_grouped).
    Each problem is a dict with the keyword names of `linear_into`: x2d, w, b, y and optionally
    y2, resid, gate, gate_stride, rows_per_batch.  At most four problems per launch; longer
    lists are cut into launches of four."""
    if not problems:
        return
    N, K = problems[0]["w"].shape
    if split is None:
        split = N
    for lo in range(0, len(problems), 4):
        chunk = problems[lo : lo + 4]
        arr = (_lib.LinearProblem * len(chunk))()
        for slot, pr in zip(arr, chunk):
            x2d, w, y = pr["x2d"], pr["w"], pr["y"]
            assert tuple(w.shape) == (N, K) and x2d.shape[1] == K
            assert x2d.stride(1) == 1 and w.stride(1) == 1 and y.stride(1) == 1
            y2, resid, gate = pr.get("y2"), pr.get("resid"), pr.get("gate")
            slot.x, slot.w, slot.bias, slot.y = _lib.ptr(x2d), _lib.ptr(w), _lib.ptr(pr.get("b")), _lib.ptr(y)
            slot.M, slot.ldx, slot.ldw, slot.ldy = x2d.shape[0], x2d.stride(0), w.stride(0), y.stride(0)
            slot.y2, slot.ldy2 = _lib.ptr(y2), (y2.stride(0) if y2 is not None else 0)
            slot.resid, slot.ldr = _lib.ptr(resid), (resid.stride(0) if resid is not None else 0)
            slot.gate, slot.gate_stride = _lib.ptr(gate), pr.get("gate_stride", 0)
            slot.rows_per_batch = pr.get("rows_per_batch", 1)
        _lib.check(
            _lib.load().fluxb_linear_grouped(arr, len(chunk), N, K, epi, split, epi2, int(round_before_act), _lib.stream_handle())
        )


def qkv_projection_supported(stream_lengths, head_dim: int, num_heads: int) -> bool:
    """Whether linear_qkv_grouped_into takes these streams (see its docstring).  The head count
    must be even: an output tile is 256 columns = two heads and is treated as a whole as q, k or v."""
    import os

    if os.environ.get("FLUXB_GEMM_PAIR", "1") == "0":  # the single-CTA kernel has no such epilogue
        return False
    return (head_dim == 128 and num_heads % 2 == 0 and 1 <= len(stream_lengths) <= 4
            and all(L > 0 and L % 128 == 0 for L in stream_lengths))


def qkv_projection_scatter_supported(stream_lengths, head_dim: int, num_heads: int, batch: int) -> bool:
    """Whether linear_qkv_grouped_into takes these streams in its scatter form (one output base per
    head group, rows masked one by one): with one batch item any stream lengths will do."""
    import os

    if os.environ.get("FLUXB_GEMM_PAIR", "1") == "0":
        return False
    return (head_dim == 128 and num_heads % 2 == 0 and 1 <= len(stream_lengths) <= 4
            and all(L > 0 and (batch == 1 or L % 128 == 0) for L in stream_lengths))


def linear_qkv_grouped_into(streams: list[dict], pe: torch.Tensor | None, qkv_out: torch.Tensor | None, eps: float = 1e-6,
                            epi2: int = _lib.EPI_NONE, round_before_act: bool = False, scatter: dict | None = None) -> None:
    """q|k|v projections of up to four token streams with the whole path to attention in the GEMM
    epilogue (fluxb_linear_qkv_grouped): per-head RMS norm of q and k, rotation with `pe`,
    head-major layout, streams concatenated in list order.

    streams[i]: dict(x [B, L_i, K] contiguous, w [3*H*D, K], b or None, q_scale [D] or None,
    k_scale [D] or None); every L_i a multiple of 128.  pe: fp32 [1, 1, L, D/2, 2, 2] over the joint
    sequence or None.  qkv_out: bf16 [3, B, H, L, D] contiguous with L = sum L_i, D = 128.
    A stream may carry `y2` ([B*L_i, N2] view, unit column stride): then w (and b) have N2 more rows
    after the q|k|v ones and those columns go to y2 with epilogue `epi2` (none or GELU).

    Scatter form (fluxb_linear_qkv_grouped_scatter; qkv_out = None): `scatter` = dict(bases = ctypes
    array of n_groups device pointers, n_groups, k_off, v_off, strides = (batch, head, token) in
    elements, num_heads, head_dim): head h of q, token l, lands at bases[h // (H/n_groups)] +
    b*sb + (h % (H/n_groups))*sh + l*sl, k and v k_off / v_off elements further; the bases may lie
    in other GPUs' memory.  Stream lengths are free when B == 1."""
    if scatter is None:
        three, B, H, L, D = qkv_out.shape
        assert three == 3 and qkv_out.is_contiguous() and qkv_out.dtype == torch.bfloat16
    else:
        assert qkv_out is None
        B, H, D = streams[0]["x"].shape[0], scatter["num_heads"], scatter["head_dim"]
        L = sum(s["x"].shape[1] for s in streams)
    assert sum(s["x"].shape[1] for s in streams) == L
    pe_c = None
    if pe is not None:
        pe_c = pe if (pe.dtype == torch.float32 and pe.is_contiguous()) else pe.to(torch.float32).contiguous()
    K = streams[0]["w"].shape[1]
    N2 = streams[0]["y2"].shape[1] if streams[0].get("y2") is not None else 0
    arr = (_lib.LinearProblem * len(streams))()
    desc = (_lib.QkvStream * len(streams))()
    keep = []
    row = 0
    for slot, d, st in zip(arr, desc, streams):
        x, w = st["x"], st["w"]
        y2 = st.get("y2")
        n2 = y2.shape[1] if y2 is not None else 0
        assert x.is_contiguous() and x.shape[0] == B and x.shape[2] == K and tuple(w.shape) == (3 * H * D + n2, K) and w.stride(1) == 1
        assert n2 == N2
        slot.y2, slot.ldy2 = _lib.ptr(y2), (y2.stride(0) if y2 is not None else 0)
        qs, ks = st.get("q_scale"), st.get("k_scale")
        if qs is not None:
            qs, ks = qs.to(torch.bfloat16), ks.to(torch.bfloat16)
            keep += [qs, ks]
        slot.x, slot.w, slot.bias, slot.y = _lib.ptr(x), _lib.ptr(w), _lib.ptr(st.get("b")), None
        slot.M, slot.ldx, slot.ldw, slot.ldy = B * x.shape[1], K, w.stride(0), 0
        slot.rows_per_batch = x.shape[1]
        d.pe, d.q_scale, d.k_scale, d.row_offset = _lib.ptr(pe_c), _lib.ptr(qs), _lib.ptr(ks), row
        row += x.shape[1]
    if scatter is not None:
        sb, sh, sl = scatter["strides"]
        _lib.check(
            _lib.load().fluxb_linear_qkv_grouped_scatter(
                arr, desc, len(streams), B, H, D, L, K, scatter["bases"], scatter["n_groups"], scatter["k_off"],
                scatter["v_off"], sb, sh, sl, eps, N2, epi2, int(round_before_act), _lib.stream_handle())
        )
        return
    _lib.check(
        _lib.load().fluxb_linear_qkv_grouped(arr, desc, len(streams), B, H, D, L, K, _lib.ptr(qkv_out), eps, N2, epi2,
                                             int(round_before_act), _lib.stream_handle())
    )


def _as_2d(x: torch.Tensor, K: int) -> torch.Tensor:
    x2d = x.reshape(-1, K)
    if x2d.stride(1) != 1 or x2d.stride(0) % 8 or x2d.data_ptr() % 16:
        x2d = x2d.contiguous()
    return x2d


def linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None, activation: str = "") -> torch.Tensor:
    """y = x @ w.T (+ b), optionally followed by tanh-GELU; bf16 in/out, fp32 accumulation.

    Same contract as the reference launcher: `w` is [N, K] (nn.Linear layout), any leading
    dims on `x`, a fresh output tensor.  Bias add and GELU run in fp32 on the accumulator.
    """
    assert x.shape[-1] == w.shape[-1], "Incompatible dimensions"
    assert x.dtype == w.dtype, "Incompatible dtypes"
    assert activation in ("", "GELU"), f"unknown activation {activation!r}"
    _lib.require_cuda(x, w, b)
    if x.dtype != torch.bfloat16:
        raise UnsupportedDtype(x.dtype)
    N, K = w.shape
    lead = x.shape[:-1]
    x2d = _as_2d(x, K)
    M = x2d.shape[0]
    if w.stride(1) != 1 or w.stride(0) % 8:
        w = w.contiguous()
    if b is not None:
        b = b.to(torch.bfloat16).contiguous()
    y = torch.empty((M, N), device=x.device, dtype=x.dtype)
    if M <= 8 and K <= 12288 and K % 8 == 0 and x2d.is_contiguous() and w.is_contiguous() and not activation:
        # Skinny problems (the modulation projection, M = batch) are pure weight streaming.
        _lib.check(
            _lib.load().fluxb_modulation_gemv(
                _lib.ptr(x2d), _lib.ptr(w), _lib.ptr(b), _lib.ptr(y), M, N, K, 0, _lib.stream_handle()
            )
        )
    else:
        linear_into(x2d, w, b, y, epi=_lib.EPI_GELU if activation == "GELU" else _lib.EPI_NONE)
    return y.reshape(*lead, N)
