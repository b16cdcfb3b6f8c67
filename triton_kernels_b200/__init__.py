"""B200-native kernels and blocks for the Flux DiT block forward path.

The flat namespace mirrors the reference's triton_kernels/__init__.py:1-10, so
`import triton_kernels_b200 as tk` gives `tk.linear`, `tk.rms_norm_torch`,
`tk.SingleStreamBlock`, ... with the same call signatures.  Every kernel-backed name runs a
hand-written sm_100a kernel from libfluxb200.so through its C ABI (include/fluxb200.h);
nothing here falls back to PyTorch or to the CPU.
"""
from triton_kernels_b200.functional import (
    apply_rope_torch,
    apply_rope_torch_compile,
    layer_norm_modulation_torch,
    layer_norm_modulation_torch_compile,
    rms_norm_torch,
    rms_norm_torch_compile,
)
from triton_kernels_b200.kernels import apply_rope, layer_norm_modulation, linear, rms_norm, scaled_dot_product_attention
from triton_kernels_b200.modules import DoubleStreamBlock, QKNorm, RMSNorm, SingleStreamBlock

__all__ = [
    "apply_rope_torch", "apply_rope_torch_compile", "layer_norm_modulation_torch",
    "layer_norm_modulation_torch_compile", "rms_norm_torch", "rms_norm_torch_compile",
    "apply_rope", "layer_norm_modulation", "linear", "rms_norm", "scaled_dot_product_attention",
    "DoubleStreamBlock", "QKNorm", "RMSNorm", "SingleStreamBlock",
]
