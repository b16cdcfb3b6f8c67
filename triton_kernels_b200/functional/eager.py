"""Plain-PyTorch LayerNorm+modulation, RMSNorm and RoPE.

Counterparts of triton_kernels/functional/normalization.py:6-33 and
triton_kernels/functional/positional_embedding.py:5-19.  The reference also exports
`*_torch_compile` twins wrapped in torch.compile; this build has no tracing compiler on any
path, so the twins here are the same eager functions under the second name.
"""
from __future__ import annotations

import torch
from torch import Tensor


def layer_norm_modulation_torch(x: Tensor, scale: Tensor, shift: Tensor) -> Tensor:
    """LayerNorm over the last dim (no affine, eps 1e-5 = F.layer_norm default), then
    x * (1 + scale) + shift."""
    mu = x.mean(dim=-1, keepdim=True)
    var = x.var(dim=-1, keepdim=True, unbiased=False)
    normed = (x - mu) * torch.rsqrt(var + 1e-5)
    return normed * (1 + scale) + shift


def rms_norm_torch(x: Tensor, scale: Tensor) -> Tensor:
    """x / rms(x) in fp32 (eps 1e-6), cast back to x's dtype, then times scale."""
    xf = x.to(torch.float32)
    inv = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + 1e-6)
    return (xf * inv).to(x.dtype) * scale


def apply_rope_torch(xq: Tensor, xk: Tensor, freqs_cis: Tensor) -> tuple[Tensor, Tensor]:
    """out[..., 2i+j] = f[..., i, j, 0] * x[..., 2i] + f[..., i, j, 1] * x[..., 2i+1], in fp32."""

    def one(x: Tensor) -> Tensor:
        pairs = x.to(torch.float32).unflatten(-1, (-1, 2))  # [..., D/2, 2]
        out = freqs_cis[..., 0] * pairs[..., 0:1] + freqs_cis[..., 1] * pairs[..., 1:2]
        return out.flatten(-2).to(x.dtype)

    return one(xq), one(xk)


layer_norm_modulation_torch_compile = layer_norm_modulation_torch
rms_norm_torch_compile = rms_norm_torch
apply_rope_torch_compile = apply_rope_torch
