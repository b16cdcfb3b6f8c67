"""Flux DiT assembly on the fused blocks: positional tables, embedders, final layer and the
19 + 38 block model the benchmark's full-forward config names."""
from triton_kernels_b200.flux.model import (
    EmbedND,
    FluxDiT,
    FluxParams,
    GraphedForward,
    LastLayer,
    MLPEmbedder,
    flux_position_ids,
    rope_table,
    timestep_embedding,
)

from triton_kernels_b200.flux.sampling import denoise, get_schedule, load_flux_state_dict, patchify, unpatchify

__all__ = [
    "denoise", "get_schedule", "load_flux_state_dict", "patchify", "unpatchify",
    "EmbedND", "FluxDiT", "FluxParams", "GraphedForward", "LastLayer", "MLPEmbedder", "flux_position_ids",
    "rope_table", "timestep_embedding",
]
