"""Full Flux DiT denoising forward assembled from the fused blocks.

The reference ships the parts — `EmbedND`, `timestep_embedding`, `MLPEmbedder`, `LastLayer`
(triton_kernels/flux/layers.py:38-85, 267-278) and the two block types — but no model class.
This module wires them the way the benchmark's full-forward config describes: img_in 64 -> C,
txt_in 4096 -> C, timestep and guidance embedders (sinusoidal 256 -> MLP) summed into `vec`,
`depth` double-stream blocks, concat (txt, img), `depth_single` single-stream blocks, drop the
text rows, final adaLN + linear C -> 64.  Parameter names follow the Flux layer naming so a
state-dict written for those layers loads here.

Everything that touches [L, C] activations runs in the sm_100a kernels; the only PyTorch math is
the sinusoid of the scalar timestep/guidance and the (cached) RoPE table.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
from torch import Tensor, nn

from triton_kernels_b200 import _lib
from triton_kernels_b200.kernels.linear import linear, linear_into
from triton_kernels_b200.kernels.normalization import layer_norm_modulation_into
from triton_kernels_b200.modules.blocks import DoubleStreamBlock, SingleStreamBlock
from triton_kernels_b200.ops.fused import modulation_silu_linear


def rope_table(pos: Tensor, dim: int, theta: int) -> Tensor:
    """[..., dim/2, 2, 2] table of [[cos, -sin], [sin, cos]]; frequencies in float64
    (triton_kernels/flux/layers.py:20-27)."""
    assert dim % 2 == 0
    exponent = torch.arange(0, dim, 2, dtype=torch.float64, device=pos.device) / dim
    angles = pos.to(torch.float64).unsqueeze(-1) / (theta**exponent)
    c, s = torch.cos(angles), torch.sin(angles)
    return torch.stack((c, -s, s, c), dim=-1).unflatten(-1, (2, 2)).float()


class EmbedND(nn.Module):
    """Per-axis RoPE tables concatenated over the frequency dim, with a broadcast head dim:
    ids [B, L, n_axes] -> [B, 1, L, sum(axes_dim)/2, 2, 2] (triton_kernels/flux/layers.py:38-52)."""

    def __init__(self, dim: int, theta: int, axes_dim: list[int]):
        super().__init__()
        self.dim, self.theta, self.axes_dim = dim, theta, list(axes_dim)

    def forward(self, ids: Tensor) -> Tensor:
        tables = [rope_table(ids[..., a], self.axes_dim[a], self.theta) for a in range(ids.shape[-1])]
        return torch.cat(tables, dim=-3).unsqueeze(1)


def flux_position_ids(txt_len: int, grid_h: int, grid_w: int, device=None) -> Tensor:
    """[1, txt_len + h*w, 3]: text rows (0,0,0) first, then image rows (0, y, x)."""
    img = torch.zeros(grid_h, grid_w, 3, device=device)
    img[..., 1] = torch.arange(grid_h, device=device)[:, None]
    img[..., 2] = torch.arange(grid_w, device=device)[None, :]
    return torch.cat((torch.zeros(txt_len, 3, device=device), img.reshape(-1, 3)), dim=0)[None]


def timestep_embedding(t: Tensor, dim: int, max_period: int = 10000, time_factor: float = 1000.0) -> Tensor:
    """[N] -> [N, dim] sinusoidal embedding, cos half then sin half
    (triton_kernels/flux/layers.py:55-74)."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = (time_factor * t)[:, None].float() * freqs[None]
    emb = torch.cat((torch.cos(args), torch.sin(args)), dim=-1)
    if dim % 2:
        emb = torch.cat((emb, torch.zeros_like(emb[:, :1])), dim=-1)
    return emb.to(t.dtype) if torch.is_floating_point(t) else emb


class MLPEmbedder(nn.Module):
    """out_layer(silu(in_layer(x))) on a handful of rows (triton_kernels/flux/layers.py:77-85):
    two weight-streaming GEMV launches, the second with the SiLU prologue."""

    def __init__(self, in_dim: int, hidden_dim: int):
        super().__init__()
        self.in_layer = nn.Linear(in_dim, hidden_dim, bias=True)
        self.silu = nn.SiLU()
        self.out_layer = nn.Linear(hidden_dim, hidden_dim, bias=True)

    def forward(self, x: Tensor) -> Tensor:
        h = linear(x, self.in_layer.weight, self.in_layer.bias)
        return modulation_silu_linear(h, self.out_layer.weight, self.out_layer.bias)


class LastLayer(nn.Module):
    """adaLN (shift, scale) from vec, LayerNorm(eps 1e-6) with that modulation, linear to
    patch_size^2 * out_channels (triton_kernels/flux/layers.py:267-278)."""

    def __init__(self, hidden_size: int, patch_size: int, out_channels: int):
        super().__init__()
        self.norm_final = nn.LayerNorm(hidden_size, elementwise_affine=False, eps=1e-6)
        self.linear = nn.Linear(hidden_size, patch_size * patch_size * out_channels, bias=True)
        self.adaLN_modulation = nn.Sequential(nn.SiLU(), nn.Linear(hidden_size, 2 * hidden_size, bias=True))

    def forward(self, x: Tensor, vec: Tensor) -> Tensor:
        B, L, C = x.shape
        lin = self.adaLN_modulation[1]
        mod = modulation_silu_linear(vec, lin.weight, lin.bias)  # [B, 2C] = shift | scale
        x = x.contiguous()
        h = torch.empty_like(x)
        layer_norm_modulation_into(x.view(B * L, C), mod[:, C:], mod[:, :C], h.view(B * L, C), L, 1e-6)
        return linear(h, self.linear.weight, self.linear.bias)


@dataclass
class FluxParams:
    in_channels: int = 64
    context_in_dim: int = 4096
    hidden_size: int = 3072
    mlp_ratio: float = 4.0
    num_heads: int = 24
    depth: int = 19
    depth_single_blocks: int = 38
    axes_dim: list[int] = field(default_factory=lambda: [16, 56, 56])
    theta: int = 10_000
    guidance_embed: bool = True


class FluxDiT(nn.Module):
    """img [B, L_img, in_channels], txt [B, L_txt, context_in_dim], ids [B, L, 3], timesteps and
    guidance [B] -> [B, L_img, in_channels]."""

    def __init__(self, params: FluxParams = FluxParams()):
        super().__init__()
        p = self.params = params
        assert p.hidden_size % p.num_heads == 0 and sum(p.axes_dim) == p.hidden_size // p.num_heads
        self.pe_embedder = EmbedND(p.hidden_size // p.num_heads, p.theta, p.axes_dim)
        self.img_in = nn.Linear(p.in_channels, p.hidden_size, bias=True)
        self.time_in = MLPEmbedder(256, p.hidden_size)
        self.guidance_in = MLPEmbedder(256, p.hidden_size) if p.guidance_embed else None
        self.txt_in = nn.Linear(p.context_in_dim, p.hidden_size, bias=True)
        self.double_blocks = nn.ModuleList(
            [DoubleStreamBlock(p.hidden_size, p.num_heads, p.mlp_ratio) for _ in range(p.depth)])
        self.single_blocks = nn.ModuleList(
            [SingleStreamBlock(p.hidden_size, p.num_heads, p.mlp_ratio) for _ in range(p.depth_single_blocks)])
        self.final_layer = LastLayer(p.hidden_size, 1, p.in_channels)
        self._mod_stream = None  # side stream for the modulation projections, created on first use

    def set_sequence_parallel(self, sp) -> None:
        """Shard tokens over the ranks of `sp` (a parallel.SequenceParallel, or None to undo):
        callers then pass each rank its slice of img, txt and of the RoPE table
        (parallel.shard_joint_sequence) and get that rank's slice of the output."""
        for blk in list(self.double_blocks) + list(self.single_blocks):
            blk.sequence_parallel = sp

    def forward(self, img: Tensor, txt: Tensor, timesteps: Tensor, guidance: Tensor | None, pe: Tensor) -> Tensor:
        """`pe` is the RoPE table of the joint (text first, then image) sequence, e.g.
        `self.pe_embedder(torch.cat((txt_ids, img_ids), 1))`; it does not change between
        denoising steps, so callers compute it once."""
        _lib.require_cuda(img, txt, timesteps, pe)
        dt = self.img_in.weight.dtype
        img = linear(img.to(dt), self.img_in.weight, self.img_in.bias)
        vec = self.time_in(timestep_embedding(timesteps, 256).to(dt))
        if self.guidance_in is not None:
            if guidance is None:
                raise ValueError("this model was built with a guidance embedder: pass guidance")
            vec = vec + self.guidance_in(timestep_embedding(guidance, 256).to(dt))
        # Every block's adaLN modulation depends on `vec` only.  They are pure weight streaming
        # (6.5 GB over the 57 blocks), so all of them are issued on a side stream right away and
        # run underneath the compute-bound GEMMs; each block waits only for its own.
        main = torch.cuda.current_stream()
        if self._mod_stream is None:
            self._mod_stream = torch.cuda.Stream()
        side = self._mod_stream
        side.wait_stream(main)
        mods, ready = [], []
        with torch.cuda.stream(side):
            for blk in self.double_blocks:
                mods.append((blk.txt_mod.packed(vec), blk.img_mod.packed(vec)))
                ready.append(torch.cuda.Event())
                ready[-1].record(side)
            for blk in self.single_blocks:
                mods.append(blk.modulation.packed(vec))
                ready.append(torch.cuda.Event())
                ready[-1].record(side)
        txt = linear(txt.to(dt), self.txt_in.weight, self.txt_in.bias)
        n_double = len(self.double_blocks)
        for i, blk in enumerate(self.double_blocks):
            main.wait_event(ready[i])
            img, txt = blk(img, txt, vec, pe, modulation=mods[i])
        x = torch.cat((txt, img), dim=1)
        for i, blk in enumerate(self.single_blocks):
            main.wait_event(ready[n_double + i])
            x = blk(x, vec, pe, modulation=mods[n_double + i])
        for m in mods:  # the side stream allocated these; the main stream used them
            for t in (m if isinstance(m, tuple) else (m,)):
                t.record_stream(main)
        return self.final_layer(x[:, txt.shape[1]:], vec)


class GraphedForward:
    """Captures one forward of `fn(*static_inputs)` in a CUDA graph and replays it.

    The model launches ~10 kernels per block and 57 blocks per step; replaying a graph removes
    the per-launch host work (argument marshalling, tensor-map encoding, allocator calls) from
    the step.  Inputs are copied into the captured buffers before each replay; the returned
    tensors are the captured outputs (overwritten by the next replay)."""

    def __init__(self, fn, example_inputs: tuple, warmup: int = 2):
        self.fn = fn
        self.static_inputs = tuple(t.clone() if isinstance(t, Tensor) else t for t in example_inputs)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(warmup):  # first calls set function attributes, status word, caches
                fn(*self.static_inputs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.static_outputs = fn(*self.static_inputs)

    def __call__(self, *inputs):
        for dst, src in zip(self.static_inputs, inputs):
            if isinstance(dst, Tensor) and src is not dst:
                dst.copy_(src, non_blocking=True)
        self.graph.replay()
        return self.static_outputs
