"""Flux block modules (same names as the reference's triton_kernels/modules/__init__.py:1-2)."""
from triton_kernels_b200.modules.blocks import (
    MLP,
    DoubleStreamBlock,
    Linear,
    LinearGELU,
    Modulation,
    ModulationOut,
    SelfAttention,
    SingleStreamBlock,
    attention,
)
from triton_kernels_b200.modules.normalization import QKNorm, RMSNorm

__all__ = [
    "MLP", "DoubleStreamBlock", "Linear", "LinearGELU", "Modulation", "ModulationOut", "SelfAttention",
    "SingleStreamBlock", "attention", "QKNorm", "RMSNorm",
]
