"""Operator API of the path: same names and call signatures as the reference's
triton_kernels/kernels/__init__.py:1-4, each backed by one C-ABI entry point."""
from triton_kernels_b200.kernels.attention import scaled_dot_product_attention
from triton_kernels_b200.kernels.linear import linear
from triton_kernels_b200.kernels.normalization import layer_norm_modulation, rms_norm
from triton_kernels_b200.kernels.positional_embedding import apply_rope

__all__ = ["scaled_dot_product_attention", "linear", "layer_norm_modulation", "rms_norm", "apply_rope"]
