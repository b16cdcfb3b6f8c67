"""The caller side of the DiT forward: patchify, the timestep schedule, the Euler denoising
loop and state-dict loading.

The reference has no sampler or model loop (it ends at the block modules); these are the steps
either side of the hot path, kept to what exercises it: every step of the loop is one
CUDA-graph replay of `FluxDiT.forward`, and the Euler update is a single fused `add` on the
[B, L, 64] latent tokens.
"""
from __future__ import annotations

import math

import torch
from torch import Tensor

from triton_kernels_b200.flux.model import FluxDiT, GraphedForward


def patchify(latent: Tensor, patch: int = 2) -> Tensor:
    """[B, C, H, W] -> [B, (H/p)*(W/p), C*p*p] tokens, channel-major inside a token
    (the "b c (h ph) (w pw) -> b (h w) (c ph pw)" packing Flux uses)."""
    B, C, H, W = latent.shape
    assert H % patch == 0 and W % patch == 0
    x = latent.reshape(B, C, H // patch, patch, W // patch, patch)
    return x.permute(0, 2, 4, 1, 3, 5).reshape(B, (H // patch) * (W // patch), C * patch * patch)


def unpatchify(tokens: Tensor, height: int, width: int, patch: int = 2) -> Tensor:
    """Inverse of `patchify` for a latent of height x width."""
    B, L, CPP = tokens.shape
    C = CPP // (patch * patch)
    h, w = height // patch, width // patch
    assert L == h * w
    x = tokens.reshape(B, h, w, C, patch, patch)
    return x.permute(0, 3, 1, 4, 2, 5).reshape(B, C, height, width)


def time_shift(mu: float, sigma: float, t: Tensor) -> Tensor:
    return math.exp(mu) / (math.exp(mu) + (1 / t - 1) ** sigma)


def get_schedule(num_steps: int, image_seq_len: int, base_shift: float = 0.5, max_shift: float = 1.15,
                 shift: bool = True) -> list[float]:
    """num_steps + 1 times from 1 to 0; with `shift` the schedule is warped towards high noise
    for long sequences (linear in the sequence length between 256 and 4096 tokens)."""
    t = torch.linspace(1, 0, num_steps + 1)
    if shift:
        m = (max_shift - base_shift) / (4096 - 256)
        mu = m * image_seq_len + (base_shift - m * 256)
        t = time_shift(mu, 1.0, t)
    return t.tolist()


@torch.no_grad()
def denoise(model: FluxDiT, img: Tensor, txt: Tensor, pe: Tensor, timesteps: list[float], guidance: float = 3.5,
            use_graph: bool = True) -> Tensor:
    """Euler integration of the flow: img <- img + (t_next - t_cur) * model(img, txt, t_cur).

    img [B, L_img, 64] latent tokens, txt [B, L_txt, context_in_dim]; `pe` the joint RoPE table.
    With `use_graph` the forward is captured once and replayed for every step (the step's only
    changing inputs are the tokens and the scalar time)."""
    B = img.shape[0]
    dev = img.device
    t_vec = torch.full((B,), timesteps[0], device=dev, dtype=torch.float32)
    g_vec = torch.full((B,), guidance, device=dev, dtype=torch.float32)
    img = img.clone()
    fwd = lambda i, x, t, g: model(i, x, t, g, pe)  # noqa: E731
    step = GraphedForward(fwd, (img, txt, t_vec, g_vec)) if use_graph else fwd
    for t_cur, t_next in zip(timesteps[:-1], timesteps[1:]):
        t_vec.fill_(t_cur)
        pred = step(img, txt, t_vec, g_vec)
        img.add_(pred.to(img.dtype), alpha=t_next - t_cur)
    return img


def load_flux_state_dict(model: FluxDiT, state_dict: dict, dtype: torch.dtype = torch.bfloat16) -> None:
    """Loads a state-dict written for the Flux layer classes (keys `img_in.*`, `time_in.*`,
    `double_blocks.N.*`, `single_blocks.N.*`, `final_layer.*`, ...) into the fused model.

    Parameter names are identical, so this is `load_state_dict` plus the checks that matter on
    this path: every tensor is cast to `dtype`, keys that the fused model does not have (e.g. a
    `vector_in` embedder of checkpoints with pooled text conditioning) are reported rather than
    silently dropped, and missing keys are an error."""
    own = set(model.state_dict().keys())
    extra = sorted(k for k in state_dict if k not in own)
    missing = sorted(k for k in own if k not in state_dict)
    if missing:
        raise KeyError(f"state-dict lacks {len(missing)} parameters of the model, e.g. {missing[:3]}")
    if extra:
        import warnings

        warnings.warn(f"ignoring {len(extra)} state-dict entries the model has no use for, e.g. {extra[:3]}")
    model.load_state_dict({k: v.to(dtype) for k, v in state_dict.items() if k in own})
