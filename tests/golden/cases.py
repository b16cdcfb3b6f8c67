"""Seeded inputs of the golden cases, shared by make_golden.py (which runs the reference on
them) and by the tests (which run the oracle and the CUDA kernels on the same tensors).

All draws come from one CPU torch.Generator per case, in the order written here.
"""
from __future__ import annotations

import torch

HEAD_DIM = 128


def _gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def randn(g, *shape, std=1.0):
    return std * torch.randn(*shape, generator=g)


def init_like(shapes: dict, g: torch.Generator, bias_std: float, scale_jitter: float) -> dict:
    """Weights N(0,0.02), biases N(0,bias_std), norm scales 1 + N(0,scale_jitter)."""
    out = {}
    for name, shape in shapes.items():
        if name.endswith(".scale"):
            out[name] = torch.ones(shape) + scale_jitter * torch.randn(shape, generator=g)
        elif name.endswith(".bias"):
            out[name] = bias_std * torch.randn(shape, generator=g)
        else:
            out[name] = 0.02 * torch.randn(shape, generator=g)
    return out


def flux_ids(txt_len: int, gh: int, gw: int) -> torch.Tensor:
    img = torch.zeros(gh, gw, 3)
    img[..., 1] = torch.arange(gh)[:, None]
    img[..., 2] = torch.arange(gw)[None, :]
    return torch.cat((torch.zeros(txt_len, 3), img.reshape(-1, 3)), dim=0)[None]


def case_rms_norm():
    g = _gen(101)
    return {"x": randn(g, 2, 3, 40, 128), "scale": 1 + randn(g, 128, std=0.1)}


def case_layer_norm_modulation():
    g = _gen(102)
    return {"x": randn(g, 2, 24, 256) * 2 + 0.5, "scale": randn(g, 2, 1, 256), "shift": randn(g, 2, 1, 256)}


def case_rope_random_table():
    g = _gen(103)
    return {"q": randn(g, 2, 3, 24, 128), "k": randn(g, 2, 3, 24, 128), "pe": randn(g, 1, 1, 24, 64, 2, 2)}


def case_embed_nd():
    return {"ids": flux_ids(8, 4, 6), "axes_dim": [16, 56, 56], "theta": 10000}


def case_timestep_embedding():
    return {"t": torch.tensor([0.5, 0.03125, 1.0]), "dim": 256}


def single_block_shapes(C: int, M: int) -> dict:
    return {
        "linear1.weight": (3 * C + M, C),
        "linear1.bias": (3 * C + M,),
        "linear2.weight": (C, C + M),
        "linear2.bias": (C,),
        "norm.query_norm.scale": (HEAD_DIM,),
        "norm.key_norm.scale": (HEAD_DIM,),
        "modulation.lin.weight": (3 * C, C),
        "modulation.lin.bias": (3 * C,),
    }


def double_block_shapes(C: int, M: int) -> dict:
    out = {}
    for s in ("img", "txt"):
        out.update(
            {
                f"{s}_mod.lin.weight": (6 * C, C),
                f"{s}_mod.lin.bias": (6 * C,),
                f"{s}_attn.qkv.weight": (3 * C, C),
                f"{s}_attn.norm.query_norm.scale": (HEAD_DIM,),
                f"{s}_attn.norm.key_norm.scale": (HEAD_DIM,),
                f"{s}_attn.proj.weight": (C, C),
                f"{s}_attn.proj.bias": (C,),
                f"{s}_mlp.0.weight": (M, C),
                f"{s}_mlp.0.bias": (M,),
                f"{s}_mlp.2.weight": (C, M),
                f"{s}_mlp.2.bias": (C,),
            }
        )
    return out


def case_single_block_small():
    """hidden 256 = 2 heads x 128, 8 text + 4x6 image tokens, non-trivial biases and norm scales."""
    g = _gen(104)
    C, M, H = 256, 1024, 2
    params = init_like(single_block_shapes(C, M), g, bias_std=0.02, scale_jitter=0.1)
    return {"params": params, "x": randn(g, 2, 32, C), "vec": randn(g, 2, C), "ids": flux_ids(8, 4, 6),
            "hidden": C, "heads": H}


def case_double_block_small():
    g = _gen(105)
    C, M, H = 256, 1024, 2
    params = init_like(double_block_shapes(C, M), g, bias_std=0.02, scale_jitter=0.1)
    return {"params": params, "img": randn(g, 2, 24, C), "txt": randn(g, 2, 8, C), "vec": randn(g, 2, C),
            "ids": flux_ids(8, 4, 6), "hidden": C, "heads": H}


def case_single_block_config1():
    """Benchmark config 1: hidden 3072 = 24 x 128, 64 text + 16x16 image tokens, weights
    N(0,0.02), biases 0, norm scales 1, activations and vec N(0,1), seed 0."""
    g = _gen(0)
    C, M, H = 3072, 12288, 24
    params = init_like(single_block_shapes(C, M), g, bias_std=0.0, scale_jitter=0.0)
    return {"params": params, "x": randn(g, 1, 320, C), "vec": randn(g, 1, C), "ids": flux_ids(64, 16, 16),
            "hidden": C, "heads": H}


def case_last_layer():
    g = _gen(106)
    C, out = 256, 64
    params = {
        "adaLN_modulation.1.weight": randn(g, 2 * C, C, std=0.02),
        "adaLN_modulation.1.bias": randn(g, 2 * C, std=0.02),
        "linear.weight": randn(g, out, C, std=0.02),
        "linear.bias": randn(g, out, std=0.02),
    }
    return {"params": params, "x": randn(g, 2, 24, C), "vec": randn(g, 2, C), "hidden": C, "out": out}


def case_mlp_embedder():
    g = _gen(107)
    params = {
        "in_layer.weight": randn(g, 256, 256, std=0.02),
        "in_layer.bias": randn(g, 256, std=0.02),
        "out_layer.weight": randn(g, 256, 256, std=0.02),
        "out_layer.bias": randn(g, 256, std=0.02),
    }
    return {"params": params, "x": randn(g, 3, 256)}


def fingerprint(t: torch.Tensor) -> list[float]:
    """Cheap check that a regenerated input equals the one the golden output was made from."""
    t = t.double().flatten()
    return [float(t.sum()), float(t.abs().sum()), float(t[:: max(1, t.numel() // 7)].sum())]
