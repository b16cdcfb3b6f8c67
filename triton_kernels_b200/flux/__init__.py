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

__all__ = [
    "EmbedND", "FluxDiT", "FluxParams", "GraphedForward", "LastLayer", "MLPEmbedder", "flux_position_ids",
    "rope_table", "timestep_embedding",
]
