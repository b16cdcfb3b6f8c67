"""The CPU oracle against vectors produced by the reference's own PyTorch path
(tests/golden/reference_vectors.pt, made by tests/golden/make_golden.py)."""
import cases
import pytest
import torch

from oracle import flux_oracle as O

ATOL = 2e-5  # float32 CPU math on both sides; differences are summation order only


def _check_inputs(case: dict, fps: dict):
    for name, fp in fps.items():
        t = case[name] if name in case else case["params"]["linear1.weight" if name == "w" and "linear1.weight" in case["params"] else "img_mlp.0.weight"]
        got = cases.fingerprint(t)
        assert got == pytest.approx(fp, rel=1e-9, abs=1e-9), f"seeded input {name} differs from the one the golden was made from"


def test_rms_norm(golden):
    c = cases.case_rms_norm()
    _check_inputs(c, golden["rms_norm"]["fp"])
    y = O.rms_norm(c["x"], c["scale"])
    torch.testing.assert_close(y, golden["rms_norm"]["y"], atol=ATOL, rtol=0)
    torch.testing.assert_close(y, golden["rms_norm"]["y_module"], atol=ATOL, rtol=0)


def test_rms_norm_backward_matches_autograd():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(6, 40, 128, generator=g, dtype=torch.float64, requires_grad=True)
    w = (1 + 0.1 * torch.randn(128, generator=g, dtype=torch.float64)).requires_grad_()
    dy = torch.randn(6, 40, 128, generator=g, dtype=torch.float64)
    O.rms_norm(x, w).backward(dy)
    dx, dw = O.rms_norm_backward(dy, x.detach(), w.detach())
    torch.testing.assert_close(dx, x.grad, atol=1e-10, rtol=0)
    torch.testing.assert_close(dw, w.grad, atol=1e-10, rtol=0)


def test_layer_norm_modulation(golden):
    c = cases.case_layer_norm_modulation()
    _check_inputs(c, golden["layer_norm_modulation"]["fp"])
    y = O.layer_norm_modulation(c["x"], c["scale"], c["shift"], eps=1e-5)
    torch.testing.assert_close(y, golden["layer_norm_modulation"]["y"], atol=ATOL, rtol=0)


def test_rope_random_table(golden):
    c = cases.case_rope_random_table()
    q, k = O.apply_rope(c["q"], c["k"], c["pe"])
    torch.testing.assert_close(q, golden["rope_random_table"]["q"], atol=ATOL, rtol=0)
    torch.testing.assert_close(k, golden["rope_random_table"]["k"], atol=ATOL, rtol=0)


def test_embed_nd(golden):
    c = cases.case_embed_nd()
    pe = O.embed_nd(c["ids"], c["axes_dim"], c["theta"])
    assert pe.shape == golden["embed_nd"]["pe"].shape == (1, 1, 32, 64, 2, 2)
    torch.testing.assert_close(pe, golden["embed_nd"]["pe"], atol=1e-6, rtol=0)
    torch.testing.assert_close(O.flux_position_ids(8, 4, 6), c["ids"], atol=0, rtol=0)


def test_timestep_embedding(golden):
    c = cases.case_timestep_embedding()
    torch.testing.assert_close(O.timestep_embedding(c["t"], c["dim"]), golden["timestep_embedding"]["emb"], atol=1e-6, rtol=0)


def test_mlp_embedder(golden):
    c = cases.case_mlp_embedder()
    torch.testing.assert_close(O.mlp_embedder(c["x"], c["params"], ""), golden["mlp_embedder"]["y"], atol=ATOL, rtol=0)


def test_single_block_small(golden):
    c = cases.case_single_block_small()
    pe = O.embed_nd(c["ids"], [16, 56, 56])
    y = O.single_stream_block(c["x"], c["vec"], pe, c["params"], c["heads"])
    torch.testing.assert_close(y, golden["single_block_small"]["y"], atol=ATOL, rtol=0)


def test_double_block_small(golden):
    c = cases.case_double_block_small()
    pe = O.embed_nd(c["ids"], [16, 56, 56])
    img, txt = O.double_stream_block(c["img"], c["txt"], c["vec"], pe, c["params"], c["heads"])
    torch.testing.assert_close(img, golden["double_block_small"]["img"], atol=ATOL, rtol=0)
    torch.testing.assert_close(txt, golden["double_block_small"]["txt"], atol=ATOL, rtol=0)


def test_last_layer(golden):
    c = cases.case_last_layer()
    y = O.last_layer(c["x"], c["vec"], c["params"], prefix="")
    torch.testing.assert_close(y, golden["last_layer"]["y"], atol=ATOL, rtol=0)


def test_single_block_config1(golden):
    """Benchmark config 1 at full size (hidden 3072, 320 tokens, seed 0)."""
    c = cases.case_single_block_config1()
    g = golden["single_block_config1"]
    _check_inputs(c, g["fp"])
    pe = O.embed_nd(c["ids"], [16, 56, 56])
    y = O.single_stream_block(c["x"], c["vec"], pe, c["params"], c["heads"])
    torch.testing.assert_close(y[0, ::16, ::48], g["sample"], atol=1e-4, rtol=0)
    stats = torch.tensor([float(y.mean()), float(y.std()), float(y.abs().max())])
    torch.testing.assert_close(stats, g["stats"], atol=1e-4, rtol=0)


def test_fused_op_restatements_agree_with_block_expressions():
    """ops/* have no reference tests; pin their oracle forms to the block expressions they replace."""
    g = torch.Generator().manual_seed(9)
    B, L, C, H = 2, 6, 256, 2
    x = torch.randn(B, L, C, generator=g)
    mod = torch.randn(B, 6 * C, generator=g)
    ch = mod[:, None, :].chunk(6, dim=-1)
    torch.testing.assert_close(O.modulation_scale_shift(x, mod, True), (1 + ch[1]) * x + ch[0])
    torch.testing.assert_close(O.modulation_scale_shift(x, mod, False), (1 + ch[4]) * x + ch[3])
    proj = torch.randn(B, L, C, generator=g)
    torch.testing.assert_close(O.modulation_gate_proj(x, mod, proj), x + ch[2] * proj)
    txt = torch.randn(B, 3, 3 * C, generator=g)
    img = torch.randn(B, 5, 3 * C, generator=g)
    q, k, v = O.qkv_concat(txt, img, H)
    assert q.shape == (B, H, 8, 128)
    torch.testing.assert_close(q[:, 1, 4], img[:, 1, 128:256])
    torch.testing.assert_close(v[:, 0, 2], txt[:, 2, 2 * C : 2 * C + 128])


def test_dit_forward_runs_and_uses_every_part():
    g = torch.Generator().manual_seed(11)
    C, H = 256, 2
    shapes = O.dit_shapes(C, in_ch=64, ctx_dim=96, depth=1, depth_single=2)
    params = O.init_params(shapes, g, bias_std=0.02, scale_jitter=0.1)
    img = torch.randn(1, 24, 64, generator=g)
    txt = torch.randn(1, 8, 96, generator=g)
    pe = O.embed_nd(O.flux_position_ids(8, 4, 6), [16, 56, 56])
    y = O.flux_dit_forward(img, txt, torch.tensor([0.5]), torch.tensor([3.5]), pe, params, H, 1, 2)
    assert y.shape == (1, 24, 64) and torch.isfinite(y).all()
    # dropping guidance changes vec and therefore the output
    y2 = O.flux_dit_forward(img, txt, torch.tensor([0.5]), None, pe, params, H, 1, 2)
    assert (y - y2).abs().max() > 1e-4
