"""CPU oracle for the Flux DiT block forward path — TEST INFRASTRUCTURE, not product code.

A plain-PyTorch restatement (CPU, any float dtype; tests use float32/float64) of what
ai-compiler-study/triton-kernels computes on this path.  Only tests/, the smoke check and the
benchmark's CPU-baseline leg may import it; the package under triton_kernels_b200/ never does.

Every function cites the reference lines it restates (paths relative to the reference's root).
Blocks are written as functions over a state-dict (`params`) with the reference's parameter
names, so weights move freely between this oracle, the reference modules and the CUDA modules.

Pinned against the reference itself: tests/golden/*.pt hold outputs produced by importing the
reference's own PyTorch path (triton_kernels/flux/layers.py, triton_kernels/functional/*) with
tests/golden/make_golden.py; tests/test_oracle.py checks this file against them.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import Tensor

# --------------------------------------------------------------------------------------
# Per-kernel oracles
# --------------------------------------------------------------------------------------


def gelu_tanh(x: Tensor) -> Tensor:
    """0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) — triton_kernels/kernels/linear.py:22-28,
    the same formula as nn.GELU(approximate="tanh") used at triton_kernels/flux/layers.py:168,249."""
    c = math.sqrt(2.0 / math.pi)
    return 0.5 * x * (1.0 + torch.tanh(c * (x + 0.044715 * x * x * x)))


def linear(x: Tensor, w: Tensor, b: Tensor | None = None, activation: str = "") -> Tensor:
    """y = x w^T + b, optional tanh-GELU — triton_kernels/kernels/linear.py:104-151 (`linear`);
    the torch form is F.linear / nn.Linear at triton_kernels/flux/layers.py:116-118,166-170."""
    y = x @ w.transpose(-1, -2)
    if b is not None:
        y = y + b
    if activation == "GELU":
        y = gelu_tanh(y)
    return y


def layer_norm_modulation(x: Tensor, scale: Tensor, shift: Tensor, eps: float = 1e-5) -> Tensor:
    """LayerNorm without affine over the last dim, then x (1 + scale) + shift —
    triton_kernels/kernels/normalization.py:8-44 (default eps 1e-5 at :47) and
    triton_kernels/functional/normalization.py:6-13.  The flux blocks use eps 1e-6
    (triton_kernels/flux/layers.py:162,165,247)."""
    mean = x.mean(dim=-1, keepdim=True)
    var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * (1 + scale) + shift


def rms_norm(x: Tensor, scale: Tensor, eps: float = 1e-6) -> Tensor:
    """x rsqrt(mean(x^2) + eps) scale — triton_kernels/kernels/normalization.py:80-106 and
    triton_kernels/flux/layers.py:88-97 (which casts x*rrms back to x.dtype before the scale)."""
    xf = x.float() if x.dtype in (torch.bfloat16, torch.float16) else x
    rrms = torch.rsqrt((xf * xf).mean(dim=-1, keepdim=True) + eps)
    return (xf * rrms).to(x.dtype) * scale


def rms_norm_backward(dy: Tensor, x: Tensor, scale: Tensor, eps: float = 1e-6) -> tuple[Tensor, Tensor]:
    """dx = rstd (dy w) - rstd^3/N sum(dy w x) x ; dw = sum_rows dy x rstd —
    triton_kernels/kernels/normalization.py:109-139,171-190."""
    n = x.shape[-1]
    rstd = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    m = dy * scale
    dx = rstd * m - (rstd**3 / n) * (m * x).sum(dim=-1, keepdim=True) * x
    dw = (dy * x * rstd).reshape(-1, n).sum(dim=0)
    return dx, dw


def apply_rope(xq: Tensor, xk: Tensor, freqs_cis: Tensor) -> tuple[Tensor, Tensor]:
    """out[2i+j] = f[i,j,0] x[2i] + f[i,j,1] x[2i+1] —
    triton_kernels/kernels/positional_embedding.py:9-52, triton_kernels/flux/layers.py:30-35,
    triton_kernels/functional/positional_embedding.py:5-10.  Math in fp32, result in x.dtype."""

    def one(x: Tensor) -> Tensor:
        xf = x.float() if x.dtype != torch.float64 else x
        even, odd = xf[..., 0::2], xf[..., 1::2]  # [..., D/2]
        f = freqs_cis.to(xf.dtype)
        o0 = f[..., 0, 0] * even + f[..., 0, 1] * odd
        o1 = f[..., 1, 0] * even + f[..., 1, 1] * odd
        return torch.stack((o0, o1), dim=-1).flatten(-2).to(x.dtype)

    return one(xq), one(xk)


def scaled_dot_product_attention(q: Tensor, k: Tensor, v: Tensor, sm_scale: float | None = None) -> Tensor:
    """softmax(q k^T sm_scale) v, non-causal, default scale 1/sqrt(D) —
    triton_kernels/kernels/attention.py:173-221 and F.scaled_dot_product_attention at
    triton_kernels/flux/layers.py:14."""
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    s = (q @ k.transpose(-1, -2)) * sm_scale
    return torch.softmax(s, dim=-1) @ v


def silu(x: Tensor) -> Tensor:
    """x sigmoid(x) — triton_kernels/ops/silu.py:5-13."""
    return x * torch.sigmoid(x)


def modulation_scale_shift(x: Tensor, mod: Tensor, is_mod1: bool) -> Tensor:
    """(scale + 1) x + shift from the packed [B, 6C] modulation, chunks (0,1) or (3,4) —
    triton_kernels/ops/modulation.py:5-27."""
    C = x.shape[-1]
    i = 0 if is_mod1 else 3
    shift = mod[:, None, i * C : (i + 1) * C]
    scale = mod[:, None, (i + 1) * C : (i + 2) * C]
    return (scale + 1.0) * x + shift


def modulation_gate_proj(img: Tensor, mod: Tensor, proj: Tensor, gate_chunk: int = 2) -> Tensor:
    """img + gate proj, gate = chunk 2 of the packed modulation — triton_kernels/ops/modulation.py:29-44."""
    C = img.shape[-1]
    return img + mod[:, None, gate_chunk * C : (gate_chunk + 1) * C] * proj


def split_heads(qkv: Tensor, num_heads: int) -> tuple[Tensor, Tensor, Tensor]:
    """rearrange "B L (K H D) -> K B H L D", K=3 — triton_kernels/modules/blocks.py:40,115,148."""
    B, L, _ = qkv.shape
    t = qkv.reshape(B, L, 3, num_heads, -1).permute(2, 0, 3, 1, 4)
    return t[0], t[1], t[2]


def qkv_concat(txt_qkv: Tensor, img_qkv: Tensor, num_heads: int) -> tuple[Tensor, Tensor, Tensor]:
    """Head-major split of both streams and concat along L, text first —
    triton_kernels/ops/qkv_concat.py:5-60; triton_kernels/modules/blocks.py:148-160."""
    tq, tk, tv = split_heads(txt_qkv, num_heads)
    iq, ik, iv = split_heads(img_qkv, num_heads)
    return torch.cat((tq, iq), 2), torch.cat((tk, ik), 2), torch.cat((tv, iv), 2)


# --------------------------------------------------------------------------------------
# Positional table and embedders (triton_kernels/flux/layers.py:20-85)
# --------------------------------------------------------------------------------------


def rope_table(pos: Tensor, dim: int, theta: int) -> Tensor:
    """[[cos, -sin], [sin, cos]] per (position, frequency), omega in float64 —
    triton_kernels/flux/layers.py:20-27."""
    assert dim % 2 == 0
    omega = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
    ang = pos.to(torch.float64)[..., None] * omega
    out = torch.stack((torch.cos(ang), -torch.sin(ang), torch.sin(ang), torch.cos(ang)), dim=-1)
    return out.reshape(*ang.shape, 2, 2).float()


def embed_nd(ids: Tensor, axes_dim: list[int], theta: int = 10000) -> Tensor:
    """Per-axis tables concatenated over frequency, plus a head dim: [B, 1, L, D/2, 2, 2] —
    triton_kernels/flux/layers.py:38-52."""
    emb = torch.cat([rope_table(ids[..., i], axes_dim[i], theta) for i in range(ids.shape[-1])], dim=-3)
    return emb.unsqueeze(1)


def flux_position_ids(txt_len: int, grid_h: int, grid_w: int) -> Tensor:
    """ids [1, txt_len + h*w, 3]: text rows (0,0,0) first, then image rows (0, y, x)."""
    img = torch.zeros(grid_h, grid_w, 3)
    img[..., 1] = torch.arange(grid_h)[:, None]
    img[..., 2] = torch.arange(grid_w)[None, :]
    return torch.cat((torch.zeros(txt_len, 3), img.reshape(-1, 3)), dim=0)[None]


def timestep_embedding(t: Tensor, dim: int, max_period: int = 10000, time_factor: float = 1000.0) -> Tensor:
    """Sinusoidal embedding [cos | sin] of time_factor * t — triton_kernels/flux/layers.py:55-74."""
    t = time_factor * t
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32) / half)
    args = t[:, None].float() * freqs[None]
    emb = torch.cat((torch.cos(args), torch.sin(args)), dim=-1)
    if dim % 2:
        emb = torch.cat((emb, torch.zeros_like(emb[:, :1])), dim=-1)
    return emb.to(t.dtype) if torch.is_floating_point(t) else emb


def mlp_embedder(x: Tensor, params: dict, prefix: str) -> Tensor:
    """out_layer(silu(in_layer(x))) — triton_kernels/flux/layers.py:77-85."""
    h = linear(x, params[prefix + "in_layer.weight"], params[prefix + "in_layer.bias"])
    return linear(silu(h), params[prefix + "out_layer.weight"], params[prefix + "out_layer.bias"])


# --------------------------------------------------------------------------------------
# Blocks (triton_kernels/flux/layers.py:124-264; kernel-based twins at
# triton_kernels/modules/blocks.py:55-172)
# --------------------------------------------------------------------------------------


def modulation(vec: Tensor, params: dict, prefix: str, double: bool) -> list[Tensor]:
    """lin(silu(vec))[:, None, :].chunk(6 or 3): shift, scale, gate (x2 if double) —
    triton_kernels/flux/layers.py:131-146."""
    out = linear(silu(vec), params[prefix + "lin.weight"], params[prefix + "lin.bias"])
    return list(out[:, None, :].chunk(6 if double else 3, dim=-1))


def _attention(q: Tensor, k: Tensor, v: Tensor, pe: Tensor) -> Tensor:
    """rope + attention + "B H L D -> B L (H D)" — triton_kernels/flux/layers.py:11-17."""
    q, k = apply_rope(q, k, pe)
    x = scaled_dot_product_attention(q, k, v)
    B, H, L, D = x.shape
    return x.permute(0, 2, 1, 3).reshape(B, L, H * D)


def _qk_norm(q: Tensor, k: Tensor, v: Tensor, params: dict, prefix: str) -> tuple[Tensor, Tensor]:
    """triton_kernels/flux/layers.py:100-109."""
    q = rms_norm(q, params[prefix + "query_norm.scale"])
    k = rms_norm(k, params[prefix + "key_norm.scale"])
    return q.to(v.dtype), k.to(v.dtype)


def single_stream_block(x: Tensor, vec: Tensor, pe: Tensor, params: dict, num_heads: int, ln_eps: float = 1e-6) -> Tensor:
    """triton_kernels/flux/layers.py:252-264 (kernel twin: triton_kernels/modules/blocks.py:110-123)."""
    C = x.shape[-1]
    shift, scale, gate = modulation(vec, params, "modulation.", double=False)
    x_mod = layer_norm_modulation(x, scale, shift, eps=ln_eps)
    lin1 = linear(x_mod, params["linear1.weight"], params["linear1.bias"])
    qkv, mlp = lin1[..., : 3 * C], lin1[..., 3 * C :]
    q, k, v = split_heads(qkv, num_heads)
    q, k = _qk_norm(q, k, v, params, "norm.")
    attn = _attention(q, k, v, pe)
    out = linear(torch.cat((attn, gelu_tanh(mlp)), dim=2), params["linear2.weight"], params["linear2.bias"])
    return x + gate * out


def double_stream_block(
    img: Tensor, txt: Tensor, vec: Tensor, pe: Tensor, params: dict, num_heads: int, ln_eps: float = 1e-6
) -> tuple[Tensor, Tensor]:
    """triton_kernels/flux/layers.py:183-216 (kernel twin: triton_kernels/modules/blocks.py:141-172)."""
    im = modulation(vec, params, "img_mod.", double=True)
    tm = modulation(vec, params, "txt_mod.", double=True)

    def pre(x, m, name):
        xm = layer_norm_modulation(x, m[1], m[0], eps=ln_eps)
        qkv = linear(xm, params[f"{name}_attn.qkv.weight"], params.get(f"{name}_attn.qkv.bias"))
        q, k, v = split_heads(qkv, num_heads)
        q, k = _qk_norm(q, k, v, params, f"{name}_attn.norm.")
        return q, k, v

    iq, ik, iv = pre(img, im, "img")
    tq, tk, tv = pre(txt, tm, "txt")
    attn = _attention(torch.cat((tq, iq), 2), torch.cat((tk, ik), 2), torch.cat((tv, iv), 2), pe)
    Lt = txt.shape[1]
    txt_attn, img_attn = attn[:, :Lt], attn[:, Lt:]

    def post(x, a, m, name):
        x = x + m[2] * linear(a, params[f"{name}_attn.proj.weight"], params[f"{name}_attn.proj.bias"])
        h = layer_norm_modulation(x, m[4], m[3], eps=ln_eps)
        h = linear(h, params[f"{name}_mlp.0.weight"], params[f"{name}_mlp.0.bias"], activation="GELU")
        h = linear(h, params[f"{name}_mlp.2.weight"], params[f"{name}_mlp.2.bias"])
        return x + m[5] * h

    return post(img, img_attn, im, "img"), post(txt, txt_attn, tm, "txt")


def last_layer(x: Tensor, vec: Tensor, params: dict, prefix: str = "final_layer.") -> Tensor:
    """adaLN (shift, scale) + LayerNorm(eps 1e-6) + linear — triton_kernels/flux/layers.py:267-278."""
    mod = linear(silu(vec), params[prefix + "adaLN_modulation.1.weight"], params[prefix + "adaLN_modulation.1.bias"])
    shift, scale = mod.chunk(2, dim=1)
    x = layer_norm_modulation(x, scale[:, None, :], shift[:, None, :], eps=1e-6)
    return linear(x, params[prefix + "linear.weight"], params[prefix + "linear.bias"])


# --------------------------------------------------------------------------------------
# Full DiT forward.  The reference ships the parts (triton_kernels/flux/layers.py:38-85,
# 183-278) but no model class; this wiring follows the architecture the benchmark names:
# img_in, txt_in, time/guidance embedders summed into vec, `depth` double blocks, concat
# (txt, img), `depth_single` single blocks, drop the text rows, final adaLN layer.
# --------------------------------------------------------------------------------------


def sub_params(params: dict, prefix: str) -> dict:
    # entries are read through params[k] so that a mapping which converts on access (the
    # full-depth test keeps the weights in bf16 and upcasts one block at a time) works here too
    n = len(prefix)
    return {k[n:]: params[k] for k in params if k.startswith(prefix)}


def flux_dit_forward(
    img: Tensor,
    txt: Tensor,
    timesteps: Tensor,
    guidance: Tensor | None,
    pe: Tensor,
    params: dict,
    num_heads: int,
    depth: int,
    depth_single: int,
) -> Tensor:
    img = linear(img, params["img_in.weight"], params["img_in.bias"])
    vec = mlp_embedder(timestep_embedding(timesteps, 256).to(img.dtype), params, "time_in.")
    if guidance is not None:
        vec = vec + mlp_embedder(timestep_embedding(guidance, 256).to(img.dtype), params, "guidance_in.")
    txt = linear(txt, params["txt_in.weight"], params["txt_in.bias"])
    for i in range(depth):
        img, txt = double_stream_block(img, txt, vec, pe, sub_params(params, f"double_blocks.{i}."), num_heads)
    x = torch.cat((txt, img), dim=1)
    for i in range(depth_single):
        x = single_stream_block(x, vec, pe, sub_params(params, f"single_blocks.{i}."), num_heads)
    x = x[:, txt.shape[1] :]
    return last_layer(x, vec, params)


# --------------------------------------------------------------------------------------
# Seeded synthetic parameters / inputs shared by tests, smoke and bench
# --------------------------------------------------------------------------------------


def single_block_shapes(C: int, mlp_ratio: float = 4.0, head_dim: int = 128) -> dict:
    M = int(C * mlp_ratio)
    return {
        "linear1.weight": (3 * C + M, C),
        "linear1.bias": (3 * C + M,),
        "linear2.weight": (C, C + M),
        "linear2.bias": (C,),
        "norm.query_norm.scale": (head_dim,),
        "norm.key_norm.scale": (head_dim,),
        "modulation.lin.weight": (3 * C, C),
        "modulation.lin.bias": (3 * C,),
    }


def double_block_shapes(C: int, mlp_ratio: float = 4.0, head_dim: int = 128) -> dict:
    M = int(C * mlp_ratio)
    out = {}
    for s in ("img", "txt"):
        out.update(
            {
                f"{s}_mod.lin.weight": (6 * C, C),
                f"{s}_mod.lin.bias": (6 * C,),
                f"{s}_attn.qkv.weight": (3 * C, C),
                f"{s}_attn.norm.query_norm.scale": (head_dim,),
                f"{s}_attn.norm.key_norm.scale": (head_dim,),
                f"{s}_attn.proj.weight": (C, C),
                f"{s}_attn.proj.bias": (C,),
                f"{s}_mlp.0.weight": (M, C),
                f"{s}_mlp.0.bias": (M,),
                f"{s}_mlp.2.weight": (C, M),
                f"{s}_mlp.2.bias": (C,),
            }
        )
    return out


def dit_shapes(C: int, in_ch: int, ctx_dim: int, depth: int, depth_single: int, guidance: bool = True) -> dict:
    out = {"img_in.weight": (C, in_ch), "img_in.bias": (C,), "txt_in.weight": (C, ctx_dim), "txt_in.bias": (C,)}
    for name in ["time_in."] + (["guidance_in."] if guidance else []):
        out.update(
            {
                name + "in_layer.weight": (C, 256),
                name + "in_layer.bias": (C,),
                name + "out_layer.weight": (C, C),
                name + "out_layer.bias": (C,),
            }
        )
    for i in range(depth):
        out.update({f"double_blocks.{i}.{k}": v for k, v in double_block_shapes(C).items()})
    for i in range(depth_single):
        out.update({f"single_blocks.{i}.{k}": v for k, v in single_block_shapes(C).items()})
    out.update(
        {
            "final_layer.adaLN_modulation.1.weight": (2 * C, C),
            "final_layer.adaLN_modulation.1.bias": (2 * C,),
            "final_layer.linear.weight": (in_ch, C),
            "final_layer.linear.bias": (in_ch,),
        }
    )
    return out


def init_params(shapes: dict, gen: torch.Generator, bias_std: float = 0.0, scale_jitter: float = 0.0) -> dict:
    """Weights N(0, 0.02); biases N(0, bias_std) (0 = zeros, as the benchmark configs say);
    QK-norm scales 1 + N(0, scale_jitter).  Drawn in dict order from one generator."""
    params = {}
    for name, shape in shapes.items():
        if name.endswith(".scale"):
            params[name] = torch.ones(shape) + scale_jitter * torch.randn(shape, generator=gen)
        elif name.endswith(".bias"):
            params[name] = bias_std * torch.randn(shape, generator=gen) if bias_std else torch.zeros(shape)
        else:
            params[name] = 0.02 * torch.randn(shape, generator=gen)
    return params
