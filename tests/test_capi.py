"""The C-ABI library builds, loads without a GPU, and exports exactly what the header declares."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def declared_functions() -> list[str]:
    text = (ROOT / "include" / "fluxb200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fluxb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_functions()
    for must in ("fluxb_linear", "fluxb_attention", "fluxb_layer_norm_modulation", "fluxb_rms_norm", "fluxb_rope",
                 "fluxb_qkv_prep", "fluxb_modulation_gemv", "fluxb_silu"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in include/fluxb200.h but not exported"


def test_binding_table_matches_header(lib):
    from triton_kernels_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_header_arity_matches_binding():
    from triton_kernels_b200 import _lib

    text = (ROOT / "include" / "fluxb200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    for name, (_, argtypes) in _lib.SIGNATURES.items():
        m = re.search(r"\b" + name + r"\s*\(([^;]*?)\)\s*;", text, flags=re.S)
        assert m, name
        args = m.group(1).strip()
        n = 0 if args in ("", "void") else len(args.split(","))
        assert n == len(argtypes), f"{name}: header has {n} parameters, binding has {len(argtypes)}"


def test_version_and_error_text_without_gpu(lib):
    assert lib.fluxb_version() >= 100
    assert isinstance(lib.fluxb_last_error(), bytes)


def test_argument_validation_needs_no_gpu(lib):
    """Bad arguments are rejected on the host before anything is launched."""
    from triton_kernels_b200 import _lib

    rc = lib.fluxb_attention(None, None, None, None, 1, 1, 128, 128, 32, *([128] * 12), 1.0, None)
    assert rc == _lib.ERR_UNSUPPORTED and b"head_dim" in lib.fluxb_last_error()
    rc = lib.fluxb_linear(None, None, None, None, 128, 256, 64, 64, 64, 256, 0, None, 0, 256, 0, None, 0, None, 0, 1, 0, None)
    assert rc == _lib.ERR_BAD_ARG
    rc = lib.fluxb_rope(None, None, None, None, None, 1, 1, 12, _lib.BF16, None)
    assert rc == _lib.ERR_BAD_ARG
    rc = lib.fluxb_silu(None, None, 16, 7, None)
    assert rc == _lib.ERR_UNSUPPORTED
    assert lib.fluxb_silu(None, None, 0, _lib.BF16, None) == 0  # empty input is a no-op
    assert lib.fluxb_rms_norm_bwd_partial_rows(1000) == 16
    # modulation projection over a row range: the output row stride cannot be shorter than the range
    rc = lib.fluxb_modulation_gemv_rows(None, None, None, None, 1, 512, 3072, 256, 1, 0, None)
    assert rc == _lib.ERR_BAD_ARG
    assert lib.fluxb_modulation_gemv_rows(None, None, None, None, 1, 0, 3072, 0, 1, 1, None) == 0  # empty range
    assert lib.fluxb_layer_norm_modulation(None, None, None, None, 0, 3072, 16, 3072, 3072, 0, 1e-6, _lib.BF16, None) == 0


def test_python_wrappers_reject_cpu_tensors():
    """No CPU fallback: the operator API raises on non-CUDA tensors."""
    import triton_kernels_b200 as tk

    x = torch.randn(2, 8, 256)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        tk.layer_norm_modulation(x, torch.zeros(2, 1, 256), torch.zeros(2, 1, 256))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        tk.linear(x.bfloat16(), torch.randn(64, 256).bfloat16(), None)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        tk.SingleStreamBlock(256, 2)(x.bfloat16(), torch.randn(2, 256).bfloat16(), torch.randn(1, 1, 8, 64, 2, 2))


def test_state_dict_keys_match_reference_layout():
    """Key names/shapes the reference blocks use (so load_state_dict works across them)."""
    import cases

    import triton_kernels_b200 as tk

    s = tk.SingleStreamBlock(256, 2, 4.0)
    assert {k: tuple(v.shape) for k, v in s.state_dict().items()} == cases.single_block_shapes(256, 1024)
    d = tk.DoubleStreamBlock(256, 2, 4.0)
    assert {k: tuple(v.shape) for k, v in d.state_dict().items()} == cases.double_block_shapes(256, 1024)
    s.load_state_dict(cases.case_single_block_small()["params"])
    d.load_state_dict(cases.case_double_block_small()["params"])


def test_package_embedders_match_reference_golden(golden):
    """The PyTorch-side pieces of the DiT assembly (RoPE table, timestep embedding) against the
    reference's own outputs; they run on any device."""
    import cases

    from triton_kernels_b200.flux import EmbedND, flux_position_ids, timestep_embedding

    c = cases.case_embed_nd()
    pe = EmbedND(128, c["theta"], c["axes_dim"])(c["ids"])
    torch.testing.assert_close(pe, golden["embed_nd"]["pe"], atol=1e-6, rtol=0)
    torch.testing.assert_close(flux_position_ids(8, 4, 6), c["ids"], atol=0, rtol=0)
    t = cases.case_timestep_embedding()
    torch.testing.assert_close(timestep_embedding(t["t"], t["dim"]), golden["timestep_embedding"]["emb"], atol=1e-6, rtol=0)


def test_dit_state_dict_keys_match_oracle_layout():
    from oracle import flux_oracle as O
    from triton_kernels_b200.flux import FluxDiT, FluxParams

    m = FluxDiT(FluxParams(hidden_size=256, num_heads=2, depth=1, depth_single_blocks=2, context_in_dim=96))
    assert {k: tuple(v.shape) for k, v in m.state_dict().items()} == O.dit_shapes(256, 64, 96, 1, 2)


def test_patchify_round_trip_and_schedule():
    from triton_kernels_b200.flux import get_schedule, patchify, unpatchify

    x = torch.arange(2 * 16 * 8 * 12, dtype=torch.float32).reshape(2, 16, 8, 12)
    tok = patchify(x)
    assert tok.shape == (2, 24, 64)
    # token (h, w) holds channel-major 2x2 patches
    torch.testing.assert_close(tok[0, 1 * 6 + 2].reshape(16, 2, 2), x[0, :, 2:4, 4:6])
    torch.testing.assert_close(unpatchify(tok, 8, 12), x)
    ts = get_schedule(4, 4096)
    assert len(ts) == 5 and ts[0] == 1.0 and ts[-1] == 0.0 and all(a > b for a, b in zip(ts, ts[1:]))
    assert get_schedule(4, 4096, shift=False) == [1.0, 0.75, 0.5, 0.25, 0.0]
    assert ts[2] > 0.5  # shifted towards high noise for long sequences


def test_state_dict_loader_reports_missing_and_extra_keys():
    from oracle import flux_oracle as O
    from triton_kernels_b200.flux import FluxDiT, FluxParams, load_flux_state_dict

    m = FluxDiT(FluxParams(hidden_size=256, num_heads=2, depth=1, depth_single_blocks=1, context_in_dim=96))
    g = torch.Generator().manual_seed(3)
    sd = O.init_params(O.dit_shapes(256, 64, 96, 1, 1), g, bias_std=0.02)
    sd["vector_in.in_layer.weight"] = torch.zeros(4, 4)
    with pytest.warns(UserWarning, match="ignoring 1"):
        load_flux_state_dict(m, sd, dtype=torch.float32)
    torch.testing.assert_close(m.single_blocks[0].linear1.weight.detach(), sd["single_blocks.0.linear1.weight"])
    del sd["img_in.bias"]
    with pytest.raises(KeyError, match="lacks 1"):
        load_flux_state_dict(m, sd)
