"""Flux double- and single-stream blocks on the fused sm_100a kernels.

Constructor arguments, forward signatures and state-dict keys are those of the reference's
triton_kernels/modules/blocks.py:78-172 (and therefore of triton_kernels/flux/layers.py), so
`load_state_dict` works across the three.  The forward passes differ in how the work is cut:

  reference (per stream)                         here
  silu, linear (M = batch)                       one weight-streaming GEMV with SiLU prologue
  layer_norm_modulation                          same kernel, reads the packed modulation in place
  linear -> rearrange -> rms_norm x2 -> cat x3   GEMM, then ONE q/k/v assembly kernel doing the
    -> apply_rope                                  split, QK-RMSNorm, RoPE and txt|img concat
  attention -> rearrange (copy)                  attention writes [B, L, H*D] directly
  linear ; gate * y ; x + ...                    GEMM with the gate/residual epilogue
  linear1 -> split ; GELU ; cat ; linear2        GEMM with a column-split epilogue that writes
                                                   GELU(mlp) next to where attention writes

13 launches per double-stream block (5 per single-stream block) instead of about 40, and no
elementwise pass over [L, C] outside a GEMM epilogue.  LayerNorm uses eps 1e-6 like the PyTorch blocks of
triton_kernels/flux/layers.py:162,165,247 (the reference kernel blocks pass 1e-5; the
difference is far below bf16 resolution).
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
from torch import Tensor, nn

from triton_kernels_b200 import _lib
from triton_kernels_b200.kernels.attention import (
    attention_into,
    attention_scatter_into,
    key_splits_for,
    scaled_dot_product_attention,
)
from triton_kernels_b200.kernels.linear import (
    linear,
    linear_grouped_into,
    linear_into,
    linear_qkv_grouped_into,
    qkv_projection_scatter_supported,
    qkv_projection_supported,
)
from triton_kernels_b200.kernels.normalization import layer_norm_modulation_into
from triton_kernels_b200.kernels.positional_embedding import apply_rope
from triton_kernels_b200.modules.normalization import QKNorm
from triton_kernels_b200.ops.fused import (
    modulation_silu_linear,
    modulation_silu_linear_rows,
    qkv_prepare_into,
    qkv_prepare_scatter,
)

LN_EPS = 1e-6


def attention(q: Tensor, k: Tensor, v: Tensor, pe: Tensor) -> Tensor:
    """RoPE on q,k then attention, returned as [B, L, H*D] (reference :11-15)."""
    q, k = apply_rope(q, k, pe)
    B, H, L, D = q.shape
    out = torch.empty((B, L, H * D), device=q.device, dtype=q.dtype)
    attention_into(q, k, v.contiguous(), out.view(B, L, H, D).permute(0, 2, 1, 3), D**-0.5)
    return out


class Linear(nn.Linear):
    def forward(self, input: Tensor) -> Tensor:
        return linear(input, self.weight, self.bias)


class LinearGELU(nn.Linear):
    def forward(self, input: Tensor) -> Tensor:
        return linear(input, self.weight, self.bias, activation="GELU")


def MLP(hidden_size: int, mlp_hidden_dim: int, bias: bool = True) -> nn.Sequential:
    """Keys `0.*` (up-projection + GELU) and `2.*` (down-projection), as in the reference."""
    return nn.Sequential(
        LinearGELU(hidden_size, mlp_hidden_dim, bias=bias),
        nn.Identity(),
        Linear(mlp_hidden_dim, hidden_size, bias=bias),
    )


class SelfAttention(nn.Module):
    def __init__(self, dim: int, num_heads: int = 8, qkv_bias: bool = False):
        super().__init__()
        self.num_heads = num_heads
        self.qkv = Linear(dim, dim * 3, bias=qkv_bias)
        self.norm = QKNorm(dim // num_heads)
        self.proj = Linear(dim, dim)

    def forward(self, x: Tensor, pe: Tensor) -> Tensor:
        B, L, C = x.shape
        qkv = self.qkv(x)
        attn = torch.empty((B, L, C), device=x.device, dtype=x.dtype)
        _joint_attention([(qkv, self.norm)], pe, self.num_heads, (C // self.num_heads) ** -0.5, attn)
        return self.proj(attn)


@dataclass
class ModulationOut:
    shift: Tensor
    scale: Tensor
    gate: Tensor


class Modulation(nn.Module):
    def __init__(self, dim: int, double: bool):
        super().__init__()
        self.is_double = double
        self.multiplier = 6 if double else 3
        self.lin = Linear(dim, self.multiplier * dim, bias=True)

    def packed(self, vec: Tensor) -> Tensor:
        """[B, multiplier*dim]: shift | scale | gate (| shift2 | scale2 | gate2)."""
        return modulation_silu_linear(vec, self.lin.weight, self.lin.bias)

    def packed_rows(self, vec: Tensor, out: Tensor, first_half: bool, light: bool = False) -> None:
        """Fills one half of the packed [B, 6*dim] tensor of a double modulation: shift | scale |
        gate (needed before attention) or shift2 | scale2 | gate2 (needed after it)."""
        n = self.lin.weight.shape[0] // 2
        r0, r1 = (0, n) if first_half else (n, 2 * n)
        bias = self.lin.bias
        if bias is not None and bias.dtype != torch.bfloat16:
            bias = bias.to(torch.bfloat16)
        modulation_silu_linear_rows(vec.contiguous(), self.lin.weight, bias, out, r0, r1, light)

    def forward(self, vec: Tensor) -> tuple[ModulationOut, ModulationOut | None]:
        out = self.packed(vec)[:, None, :].chunk(self.multiplier, dim=-1)
        return ModulationOut(*out[:3]), ModulationOut(*out[3:]) if self.is_double else None


def _check_inputs(*tensors: Tensor) -> None:
    _lib.require_cuda(*tensors)
    for t in tensors:
        if t.dtype != torch.bfloat16:
            raise NotImplementedError(f"the fused Flux blocks run in bfloat16; got {t.dtype}")


def _assemble_qkv(streams, pe: Tensor, num_heads: int):
    """streams: [(packed projection [B, L_s, >= 3C], QKNorm module)], first stream's tokens first."""
    B = streams[0][0].shape[0]
    L = sum(s.shape[1] for s, _ in streams)
    D = streams[0][1].query_norm.scale.shape[0]
    dev, dt = streams[0][0].device, streams[0][0].dtype
    q = torch.empty((B, num_heads, L, D), device=dev, dtype=dt)
    k = torch.empty_like(q)
    v = torch.empty_like(q)
    args = [(s, n.query_norm.scale.to(dt), n.key_norm.scale.to(dt)) for s, n in streams]
    qkv_prepare_into(args, pe, q, k, v, num_heads, eps=1e-6)
    return q, k, v


def _joint_attention(streams, pe: Tensor, num_heads: int, scale: float, out: Tensor | None, sp=None) -> Tensor:
    """q/k/v assembly (split, QK-RMSNorm, RoPE, stream concat) + attention.  The result is
    written into `out`, a [B, L, C] view with unit stride on the last dim (it may be a column
    range of a wider buffer), or, with out=None, into a buffer of the callee's choice; the
    tensor holding it is returned.  With a SequenceParallel handle the local tokens are
    exchanged for the local heads before attention and back after it
    (triton_kernels_b200/parallel/ulysses.py)."""
    if sp is None or sp.world == 1:
        q, k, v = _assemble_qkv(streams, pe, num_heads)
        B, H, L, D = q.shape
        if out is None:
            out = torch.empty((B, L, H * D), device=q.device, dtype=q.dtype)
        attention_into(q, k, v, out.unflatten(2, (H, D)).permute(0, 2, 1, 3), scale)
        return out
    B = streams[0][0].shape[0]
    L_loc = sum(s.shape[1] for s, _ in streams)
    D = streams[0][1].query_norm.scale.shape[0]
    dev, dt = streams[0][0].device, streams[0][0].dtype
    if sp.exchange == "peer":
        # Both exchanges happen inside the producing kernels, as stores into the peers' arenas.
        pb = sp.peer_buffers(B, L_loc, num_heads, D, dt)
        args = [(s, n.query_norm.scale.to(dt), n.key_norm.scale.to(dt)) for s, n in streams]
        qkv_prepare_scatter(args, pe, pb.q_bases, pb.P, pb.k_off, pb.v_off, num_heads, D, pb.qkv_strides,
                            eps=1e-6)
        return _peer_attention(pb, L_loc, scale, out)
    if out is None:
        out = torch.empty((B, L_loc, num_heads * D), device=dev, dtype=dt)
    shape, layout = sp.send_layout(B, L_loc, num_heads, D)
    Hp = layout[0]
    send = torch.empty(shape, device=dev, dtype=dt)
    flat = send.view(-1)
    args = [(s, n.query_norm.scale.to(dt), n.key_norm.scale.to(dt)) for s, n in streams]
    qkv_prepare_into(args, pe, flat, flat[Hp * D :], flat[2 * Hp * D :], num_heads, eps=1e-6, out_layout=layout,
                     head_dim=D)
    full = sp.tokens_to_heads(send)  # [B, L, 3, Hp, D]
    L = full.shape[1]
    o = torch.empty((B, L, Hp * D), device=dev, dtype=dt)
    qv, kv, vv = (full[:, :, i].permute(0, 2, 1, 3) for i in range(3))  # [B, Hp, L, D] views
    attention_into(qv, kv, vv, o.view(B, L, Hp, D).permute(0, 2, 1, 3), scale, k_splits=key_splits_for(B, Hp, L, L, D))
    sp.heads_to_tokens(o, out)
    return out


def _peer_attention(pb, L_loc: int, scale: float, out: Tensor | None) -> Tensor:
    """Attention over the q/k/v that all ranks have stored into this rank's arena, for the local
    heads, with the output rows stored straight into their owners' arenas.  Barrier 0: all q/k/v
    have arrived; barrier 1: all outputs have arrived, and the peers may overwrite this rank's
    receive buffer again."""
    pb.arena.signal(0)
    pb.arena.wait(0)
    qv, kv, vv = (pb.recv[:, :, i].permute(0, 2, 1, 3) for i in range(3))  # [B, Hp, L, D] views
    attention_scatter_into(qv, kv, vv, pb.o_bases, pb.P, L_loc, pb.o_strides, scale)
    pb.arena.signal(1)
    pb.arena.wait(1)
    if out is None:
        return pb.out  # valid until this rank's next attention with the same shape
    out.copy_(pb.out)
    return out


def _scatter_target(pb, num_heads: int, head_dim: int) -> dict:
    """Where the scatter form of the q|k|v projection writes: the peers' receive buffers."""
    return dict(bases=pb.q_bases, n_groups=pb.P, k_off=pb.k_off, v_off=pb.v_off, strides=pb.qkv_strides,
                num_heads=num_heads, head_dim=head_dim)


def _ln_mod(x: Tensor, packed_mod: Tensor, chunk_shift: int) -> Tensor:
    """LayerNorm + modulation reading (shift, scale) = chunks (chunk_shift, chunk_shift+1)."""
    B, L, C = x.shape
    y = torch.empty_like(x)
    layer_norm_modulation_into(
        x.view(B * L, C),
        packed_mod[:, (chunk_shift + 1) * C : (chunk_shift + 2) * C],
        packed_mod[:, chunk_shift * C : (chunk_shift + 1) * C],
        y.view(B * L, C),
        L,
        LN_EPS,
    )
    return y


def _gated_linear(a2d: Tensor, lin: nn.Linear, resid2d: Tensor, gate: Tensor, rows_per_batch: int, out2d: Tensor):
    """out = resid + gate[batch] * (a @ W^T + b) in one GEMM."""
    linear_into(
        a2d, lin.weight, lin.bias, out2d, epi=_lib.EPI_GATE_RESID, resid=resid2d, gate=gate,
        gate_stride=gate.stride(0) if gate.shape[0] > 1 else 0, rows_per_batch=rows_per_batch,
    )


class SingleStreamBlock(nn.Module):
    """Parallel attention + MLP block (https://arxiv.org/abs/2302.05442) with adaLN modulation."""

    def __init__(self, hidden_size: int, num_heads: int, mlp_ratio: float = 4.0, qk_scale: float | None = None):
        super().__init__()
        self.hidden_dim = hidden_size
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        head_dim = hidden_size // num_heads
        self.scale = qk_scale or head_dim**-0.5
        self.mlp_hidden_dim = int(hidden_size * mlp_ratio)
        self.linear1 = Linear(hidden_size, hidden_size * 3 + self.mlp_hidden_dim)  # qkv | mlp_in
        self.linear2 = Linear(hidden_size + self.mlp_hidden_dim, hidden_size)  # proj | mlp_out
        self.norm = QKNorm(head_dim)
        self.mlp_act = nn.GELU(approximate="tanh")
        self.modulation = Modulation(hidden_size, double=False)
        self.sequence_parallel = None  # set to a parallel.SequenceParallel to shard tokens over ranks
        # QK norm + RoPE + head-major layout in linear1's epilogue when shapes allow (FLUXB_FUSE_QKV=0: off)
        self.fuse_qkv_epilogue = os.environ.get("FLUXB_FUSE_QKV", "1") != "0"

    def forward(self, x: Tensor, vec: Tensor, pe: Tensor, modulation: Tensor | None = None) -> Tensor:
        """`modulation` may carry the packed [B, 3C] output of `self.modulation.packed(vec)`
        computed ahead of time (it depends on `vec` only); by default it is computed here."""
        _check_inputs(x, vec)
        x = x.contiguous()
        B, L, C = x.shape
        H, M = self.num_heads, self.mlp_hidden_dim
        D = C // H
        mod = modulation if modulation is not None else self.modulation.packed(vec)  # [B, 3C] = shift | scale | gate
        x_mod = _ln_mod(x, mod, 0)

        # linear1: columns [0, 3C) -> qkv, columns [3C, 3C+M) -> GELU -> cat[:, :, C:]
        cat = torch.empty((B, L, C + M), device=x.device, dtype=x.dtype)  # attn | gelu(mlp)
        sp = self.sequence_parallel
        if ((sp is None or sp.world == 1) and self.fuse_qkv_epilogue and qkv_projection_supported((L,), D, H)
                and (3 * C) % 256 == 0 and M % 8 == 0):
            # one GEMM: the q|k|v columns leave normalised, rotated and head-major, the MLP columns
            # through GELU into the concat buffer
            qkv_heads = torch.empty((3, B, H, L, D), device=x.device, dtype=x.dtype)
            linear_qkv_grouped_into(
                [dict(x=x_mod, w=self.linear1.weight, b=self.linear1.bias, q_scale=self.norm.query_norm.scale,
                      k_scale=self.norm.key_norm.scale, y2=cat.view(B * L, C + M)[:, C:])],
                pe, qkv_heads, eps=1e-6, epi2=_lib.EPI_GELU)
            attention_into(qkv_heads[0], qkv_heads[1], qkv_heads[2],
                           cat[:, :, :C].unflatten(2, (H, D)).permute(0, 2, 1, 3), self.scale)
            out = torch.empty_like(x)
            _gated_linear(cat.view(B * L, C + M), self.linear2, x.view(B * L, C), mod[:, 2 * C : 3 * C], L, out.view(B * L, C))
            return out
        if (sp is not None and sp.world > 1 and sp.scatter_from_projection and self.fuse_qkv_epilogue
                and qkv_projection_scatter_supported((L,), D, H, B) and (3 * C) % 256 == 0 and M % 8 == 0):
            # sequence parallel: the q|k|v columns leave linear1 normalised and rotated, each head
            # group straight into the arena of the rank that attends over it
            pb = sp.peer_buffers(B, L, H, D, x.dtype)
            linear_qkv_grouped_into(
                [dict(x=x_mod, w=self.linear1.weight, b=self.linear1.bias, q_scale=self.norm.query_norm.scale,
                      k_scale=self.norm.key_norm.scale, y2=cat.view(B * L, C + M)[:, C:])],
                pe, None, eps=1e-6, epi2=_lib.EPI_GELU, scatter=_scatter_target(pb, H, D))
            _peer_attention(pb, L, self.scale, cat[:, :, :C])
            out = torch.empty_like(x)
            _gated_linear(cat.view(B * L, C + M), self.linear2, x.view(B * L, C), mod[:, 2 * C : 3 * C], L, out.view(B * L, C))
            return out
        qkv = torch.empty((B, L, 3 * C), device=x.device, dtype=x.dtype)
        if (3 * C) % 256 == 0:
            linear_into(
                x_mod.view(B * L, C), self.linear1.weight, self.linear1.bias, qkv.view(B * L, 3 * C),
                y2=cat.view(B * L, C + M)[:, C:], split=3 * C, epi2=_lib.EPI_GELU,
            )
        else:  # narrow models whose qkv width is not a whole number of column tiles
            w, b = self.linear1.weight, self.linear1.bias
            linear_into(x_mod.view(B * L, C), w[: 3 * C], b[: 3 * C], qkv.view(B * L, 3 * C))
            linear_into(x_mod.view(B * L, C), w[3 * C :], b[3 * C :], cat.view(B * L, C + M)[:, C:], epi=_lib.EPI_GELU)

        _joint_attention([(qkv, self.norm)], pe, H, self.scale, cat[:, :, :C], self.sequence_parallel)

        out = torch.empty_like(x)
        _gated_linear(cat.view(B * L, C + M), self.linear2, x.view(B * L, C), mod[:, 2 * C : 3 * C], L, out.view(B * L, C))
        return out


class DoubleStreamBlock(nn.Module):
    """Separate image / text streams with their own modulation, projections and MLPs, joined
    by one attention over the concatenated (text first, then image) tokens."""

    def __init__(self, hidden_size: int, num_heads: int, mlp_ratio: float, qkv_bias: bool = False):
        super().__init__()
        mlp_hidden_dim = int(hidden_size * mlp_ratio)
        self.num_heads = num_heads
        self.hidden_size = hidden_size
        self.img_mod = Modulation(hidden_size, double=True)
        self.img_attn = SelfAttention(dim=hidden_size, num_heads=num_heads, qkv_bias=qkv_bias)
        self.img_mlp = MLP(hidden_size, mlp_hidden_dim)
        self.txt_mod = Modulation(hidden_size, double=True)
        self.txt_attn = SelfAttention(dim=hidden_size, num_heads=num_heads, qkv_bias=qkv_bias)
        self.txt_mlp = MLP(hidden_size, mlp_hidden_dim)
        self.sequence_parallel = None  # set to a parallel.SequenceParallel to shard tokens over ranks
        # QK norm + RoPE + head-major layout in the qkv GEMM's epilogue when shapes allow (FLUXB_FUSE_QKV=0: off)
        self.fuse_qkv_epilogue = os.environ.get("FLUXB_FUSE_QKV", "1") != "0"
        self._side_stream = None  # created on first use
        self._mod_stream = None

    def forward(self, img: Tensor, txt: Tensor, vec: Tensor, pe: Tensor,
                modulation: tuple[Tensor, Tensor] | None = None) -> tuple[Tensor, Tensor]:
        """`modulation` may carry (txt, img) packed [B, 6C] modulation tensors computed ahead of
        time from `vec`; by default they are computed here."""
        _check_inputs(img, txt, vec)
        img, txt = img.contiguous(), txt.contiguous()
        B, Li, C = img.shape
        Lt = txt.shape[1]
        H = self.num_heads
        D = C // H
        dev, dt = img.device, img.dtype
        # stream order everywhere below: (txt, img), the order of the joint sequence
        xs = (txt, img)
        Ls = (Lt, Li)
        attns = (self.txt_attn, self.img_attn)
        mlps = (self.txt_mlp, self.img_mlp)
        # The block opens with bandwidth-bound work only (two weight-streaming modulation
        # projections, two LayerNorms); the text stream's half runs on a side stream next to the
        # image stream's so that the two together keep HBM busy.
        main = torch.cuda.current_stream()
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream()
        side = self._side_stream
        # Only shift | scale | gate are needed before attention: the other half of each projection
        # (56 MB of weights per stream) is launched afterwards in a form that fits on the SMs beside
        # the q|k|v GEMM and streams its weights while that GEMM computes.  (Deferring gate as well, 75 MB
        # per stream, measured slower: 1.043 against 1.038 ms per step without any deferral, where
        # the halves give 1.010 against 1.015 ms.)
        split_mod = modulation is None and vec.dtype == torch.bfloat16 and self.img_mod.lin.weight.dtype == torch.bfloat16
        if split_mod:
            txt_mod = torch.empty((B, 6 * C), device=dev, dtype=dt)
            img_mod = torch.empty((B, 6 * C), device=dev, dtype=dt)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            if split_mod:
                self.txt_mod.packed_rows(vec, txt_mod, True)
            else:
                txt_mod = modulation[0] if modulation is not None else self.txt_mod.packed(vec)
            h_txt = _ln_mod(txt, txt_mod, 0)
        if split_mod:
            self.img_mod.packed_rows(vec, img_mod, True)
        else:
            img_mod = modulation[1] if modulation is not None else self.img_mod.packed(vec)
        h_img = _ln_mod(img, img_mod, 0)
        main.wait_stream(side)
        for t_ in (txt_mod, h_txt):
            t_.record_stream(main)
        if split_mod:
            if self._mod_stream is None:
                self._mod_stream = torch.cuda.Stream()
            later = self._mod_stream  # a stream of its own: `side` is needed again before attention
            later.wait_stream(main)
            with torch.cuda.stream(later):
                self.txt_mod.packed_rows(vec, txt_mod, False, light=True)
                self.img_mod.packed_rows(vec, img_mod, False, light=True)
        mods = (txt_mod, img_mod)  # [B, 6C] each

        def gate_of(mod, chunk, b=None):
            g = mod[:, chunk * C : (chunk + 1) * C]
            return (g, g.stride(0) if B > 1 else 0) if b is None else (g[b : b + 1], 0)

        h1 = [h_txt, h_img]
        sp = self.sequence_parallel
        if (sp is None or sp.world == 1) and self.fuse_qkv_epilogue and qkv_projection_supported(Ls, D, H):
            # both streams' qkv projections in one launch whose epilogue also does the QK norm, the
            # rotation and the head-major text|image layout attention reads
            qkv_heads = torch.empty((3, B, H, Lt + Li, D), device=dev, dtype=dt)
            linear_qkv_grouped_into([
                dict(x=h, w=a.qkv.weight, b=a.qkv.bias, q_scale=a.norm.query_norm.scale, k_scale=a.norm.key_norm.scale)
                for h, a in zip(h1, attns)], pe, qkv_heads, eps=1e-6)
            attn = torch.empty((B, Lt + Li, C), device=dev, dtype=dt)
            attention_into(qkv_heads[0], qkv_heads[1], qkv_heads[2], attn.unflatten(2, (H, D)).permute(0, 2, 1, 3), D**-0.5)
        elif (sp is not None and sp.world > 1 and sp.scatter_from_projection and self.fuse_qkv_epilogue
              and qkv_projection_scatter_supported(Ls, D, H, B)):
            # sequence parallel: the same epilogue, storing every head group straight into the arena
            # of the rank that attends over it
            pb = sp.peer_buffers(B, Lt + Li, H, D, dt)
            linear_qkv_grouped_into([
                dict(x=h, w=a.qkv.weight, b=a.qkv.bias, q_scale=a.norm.query_norm.scale, k_scale=a.norm.key_norm.scale)
                for h, a in zip(h1, attns)], pe, None, eps=1e-6, scatter=_scatter_target(pb, H, D))
            attn = _peer_attention(pb, Lt + Li, D**-0.5, None)
        elif (sp is not None and sp.world > 1 and sp.exchange == "peer" and sp.pipeline_exchange and B == 1
              and Li >= 512):
            # sequence parallel, peer exchange: project and scatter the image tokens in pieces so that
            # one piece's stores into the peers' arenas (NVLink-bound, few issue slots) run beside
            # the next piece's projection instead of after the whole projection
            pb = sp.peer_buffers(B, Lt + Li, H, D, dt)
            from triton_kernels_b200.parallel.ulysses import exchange_pieces

            # two pieces: three and four measured slower (1.83 / 1.85 against 1.81 ms on four GPUs)
            pieces = exchange_pieces(Li, 2)
            qkvs = [torch.empty((B, L, 3 * C), device=dev, dtype=dt) for L in Ls]
            x_img, y_img = h1[1].view(Li, C), qkvs[1].view(Li, 3 * C)
            a_t, a_i = attns
            norms = [(a.norm.query_norm.scale.to(dt), a.norm.key_norm.scale.to(dt)) for a in attns]
            pe_rows = pe.reshape(-1, D // 2, 2, 2)
            scat = (pb.P, pb.k_off, pb.v_off, H, D, pb.qkv_strides)
            for i, (r0, r1) in enumerate(pieces):
                last = r1 == Li
                probs = [dict(x2d=x_img[r0:r1], w=a_i.qkv.weight, b=a_i.qkv.bias, y=y_img[r0:r1])]
                if i == 0:
                    probs.insert(0, dict(x2d=h1[0].view(Lt, C), w=a_t.qkv.weight, b=a_t.qkv.bias, y=qkvs[0].view(Lt, 3 * C)))
                linear_grouped_into(probs)
                srcs = [(qkvs[1][:, r0:r1], *norms[1])]
                if i == 0:
                    srcs.insert(0, (qkvs[0], *norms[0]))
                first_row = 0 if i == 0 else Lt + r0
                if last:  # nothing left to hide it behind: on the main stream
                    qkv_prepare_scatter(srcs, pe_rows[first_row : Lt + r1], pb.q_bases_from_row(first_row), *scat, eps=1e-6)
                else:
                    side.wait_stream(main)
                    with torch.cuda.stream(side):
                        qkv_prepare_scatter(srcs, pe_rows[first_row : Lt + r1], pb.q_bases_from_row(first_row), *scat,
                                            eps=1e-6)
            main.wait_stream(side)
            attn = _peer_attention(pb, Lt + Li, D**-0.5, None)
        else:
            # both streams' qkv projections in one launch, then the assembly kernel
            qkvs = [torch.empty((B, L, 3 * C), device=dev, dtype=dt) for L in Ls]
            linear_grouped_into([
                dict(x2d=h.view(B * L, C), w=a.qkv.weight, b=a.qkv.bias, y=o.view(B * L, 3 * C))
                for h, a, o, L in zip(h1, attns, qkvs, Ls)])
            attn = _joint_attention([(qkvs[0], self.txt_attn.norm), (qkvs[1], self.img_attn.norm)], pe, H, D**-0.5,
                                    None, sp)

        # proj + gate/residual: the rows of one stream of one batch item are one strided 2-D block
        x1 = [torch.empty_like(x) for x in xs]
        row0 = (0, Lt)
        probs = []
        for s_ in range(2):
            for b in range(B):
                g, gs = gate_of(mods[s_], 2, b)
                probs.append(dict(x2d=attn[b, row0[s_] : row0[s_] + Ls[s_]], w=attns[s_].proj.weight, b=attns[s_].proj.bias,
                                  y=x1[s_][b], resid=xs[s_][b], gate=g, gate_stride=gs, rows_per_batch=Ls[s_]))
        linear_grouped_into(probs, epi=_lib.EPI_GATE_RESID)

        # MLP: LN+mod2, up-projection with GELU, down-projection with gate/residual
        # (the text stream's LayerNorm is 512 rows, a launch that is all latency: beside the image
        # stream's on the second stream, not before it: 3 us per step)
        if split_mod:
            main.wait_stream(self._mod_stream)  # shift2 | scale2 | gate2 are complete
        side.wait_stream(main)
        with torch.cuda.stream(side):
            h2_txt = _ln_mod(x1[0], mods[0], 3)
        h2 = [h2_txt, _ln_mod(x1[1], mods[1], 3)]
        main.wait_stream(side)
        h2_txt.record_stream(main)
        ups = [torch.empty((B * L, mlp[0].out_features), device=dev, dtype=dt) for L, mlp in zip(Ls, mlps)]
        linear_grouped_into([
            dict(x2d=h.view(B * L, C), w=mlp[0].weight, b=mlp[0].bias, y=u) for h, mlp, u, L in zip(h2, mlps, ups, Ls)],
            epi=_lib.EPI_GELU)
        outs = [torch.empty_like(x) for x in xs]
        probs = []
        for s_ in range(2):
            g, gs = gate_of(mods[s_], 5)
            probs.append(dict(x2d=ups[s_], w=mlps[s_][2].weight, b=mlps[s_][2].bias, y=outs[s_].view(B * Ls[s_], C),
                              resid=x1[s_].view(B * Ls[s_], C), gate=g, gate_stride=gs, rows_per_batch=Ls[s_]))
        linear_grouped_into(probs, epi=_lib.EPI_GATE_RESID)
        return outs[1], outs[0]
