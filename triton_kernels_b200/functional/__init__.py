"""Eager-PyTorch forms of the norm / RoPE ops (same names as the reference's
triton_kernels/functional/__init__.py:1-7).  They are API surface, not a fallback: the CUDA
kernels in `kernels/` never route through them."""
from triton_kernels_b200.functional.eager import (
    apply_rope_torch,
    apply_rope_torch_compile,
    layer_norm_modulation_torch,
    layer_norm_modulation_torch_compile,
    rms_norm_torch,
    rms_norm_torch_compile,
)

__all__ = [
    "apply_rope_torch",
    "apply_rope_torch_compile",
    "layer_norm_modulation_torch",
    "layer_norm_modulation_torch_compile",
    "rms_norm_torch",
    "rms_norm_torch_compile",
]
