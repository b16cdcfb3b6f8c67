"""Launchable forms of the reference's un-launched triton_kernels/ops/* kernels."""
from triton_kernels_b200.ops.fused import (
    linear_bias,
    modulation_gate_proj,
    modulation_scale_shift,
    modulation_silu_linear,
    qkv_concat,
    qkv_prepare,
    silu,
)

__all__ = [
    "linear_bias",
    "modulation_gate_proj",
    "modulation_scale_shift",
    "modulation_silu_linear",
    "qkv_concat",
    "qkv_prepare",
    "silu",
]
