"""Per-kernel parity on a B200: every C-ABI kernel against the CPU oracle on identical seeded
inputs.  Tolerances: fp32 I/O kernels 1e-5 absolute (the reference's own test tolerance);
bf16 kernels atol = rtol = 2e-2 (the per-kernel tolerance of the benchmark spec)."""
import math

import pytest
import torch

from oracle import flux_oracle as O

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def gen(seed):
    return torch.Generator().manual_seed(seed)


def close_bf16(got, want, atol=2e-2, rtol=2e-2):
    torch.testing.assert_close(got.float().cpu(), want.float(), atol=atol, rtol=rtol)


def rel_l2(got, want):
    got, want = got.float().cpu(), want.float()
    return float((got - want).norm() / want.norm())


@pytest.fixture(scope="module")
def tk(lib):
    import triton_kernels_b200 as tk

    assert torch.cuda.is_available()
    return tk


# ------------------------------------------------------------------ LayerNorm + modulation
@pytest.mark.parametrize("B,L,N", [(1, 256, 1024), (2, 512, 2048), (16, 256, 3072), (3, 37, 3072), (2, 5, 72), (1, 9, 4096)])
def test_layer_norm_modulation_fp32(tk, B, L, N):
    g = gen(1)
    x = torch.randn(B, L, N, generator=g) * 1.7 + 0.3
    sc, sh = torch.randn(B, 1, N, generator=g), torch.randn(B, 1, N, generator=g)
    y = tk.layer_norm_modulation(x.cuda(), sc.cuda(), sh.cuda())
    torch.testing.assert_close(y.cpu(), O.layer_norm_modulation(x, sc, sh, eps=1e-5), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("B,L,N,eps", [(1, 4608, 3072, 1e-6), (2, 300, 3072, 1e-5), (4, 33, 256, 1e-6), (1, 7, 1000, 1e-6)])
def test_layer_norm_modulation_bf16(tk, B, L, N, eps):
    g = gen(2)
    x = (torch.randn(B, L, N, generator=g) * 2 + 0.5).to(BF)
    sc = (0.1 * torch.randn(B, 1, N, generator=g)).to(BF)
    sh = (0.1 * torch.randn(B, 1, N, generator=g)).to(BF)
    y = tk.layer_norm_modulation(x.cuda(), sc.cuda(), sh.cuda(), eps=eps)
    assert y.dtype == BF
    close_bf16(y, O.layer_norm_modulation(x.float(), sc.float(), sh.float(), eps=eps))


@pytest.mark.parametrize("mean", [50.0, -200.0])
def test_layer_norm_modulation_rows_far_from_zero(tk, mean):
    """The wide-row kernel takes its statistics in one pass (sum and sum of squares).  Rows whose
    mean is many standard deviations from zero are where that form cancels: fp32 rows are shifted
    by their first element, 16-bit rows rely on their own quantisation being the larger error."""
    g = gen(21)
    B, L, N = 1, 64, 3072
    sc, sh = 0.1 * torch.randn(B, 1, N, generator=g), 0.1 * torch.randn(B, 1, N, generator=g)
    x = torch.randn(B, L, N, generator=g) + mean
    y = tk.layer_norm_modulation(x.cuda(), sc.cuda(), sh.cuda(), eps=1e-6)
    torch.testing.assert_close(y.cpu(), O.layer_norm_modulation(x, sc, sh, eps=1e-6), atol=2e-4, rtol=2e-4)
    xb, scb, shb = x.to(BF), sc.to(BF), sh.to(BF)
    yb = tk.layer_norm_modulation(xb.cuda(), scb.cuda(), shb.cuda(), eps=1e-6)
    close_bf16(yb, O.layer_norm_modulation(xb.float(), scb.float(), shb.float(), eps=1e-6))


def test_layer_norm_modulation_reads_packed_chunks_in_place(tk):
    """scale/shift given as chunk views of a packed [B, 6C] tensor (no copies needed)."""
    g = gen(3)
    B, L, C = 2, 64, 3072
    x = torch.randn(B, L, C, generator=g).to(BF)
    mod = (0.2 * torch.randn(B, 6 * C, generator=g)).to(BF)
    ch = mod[:, None, :].chunk(6, dim=-1)
    mc = mod.cuda()
    cc = mc[:, None, :].chunk(6, dim=-1)
    y = tk.layer_norm_modulation(x.cuda(), cc[4], cc[3], eps=1e-6)
    close_bf16(y, O.layer_norm_modulation(x.float(), ch[4].float(), ch[3].float(), eps=1e-6))


# ------------------------------------------------------------------ RMSNorm
@pytest.mark.parametrize("shape", [(1, 2, 256, 128), (2, 24, 512, 128), (8, 4, 77, 256), (1, 3, 50, 512), (2, 2, 9, 3072), (3, 1, 5, 96)])
def test_rms_norm_fp32(tk, shape):
    g = gen(4)
    x = torch.randn(*shape, generator=g)
    w = 1 + 0.1 * torch.randn(shape[-1], generator=g)
    y = tk.rms_norm(x.cuda(), w.cuda())
    torch.testing.assert_close(y.cpu(), O.rms_norm(x, w), atol=1e-5, rtol=1e-5)


def test_rms_norm_bf16_on_head_split_view(tk):
    """The block's use: q is a strided [B,H,L,D] view of the packed projection."""
    g = gen(5)
    B, L, H, D = 2, 333, 24, 128
    qkv = torch.randn(B, L, 3 * H * D, generator=g).to(BF)
    w = (1 + 0.1 * torch.randn(D, generator=g)).to(BF)
    q_view = qkv.cuda().view(B, L, 3, H, D).permute(2, 0, 3, 1, 4)[1]
    y = tk.rms_norm(q_view, w.cuda())
    want = O.rms_norm(qkv.view(B, L, 3, H, D).permute(2, 0, 3, 1, 4)[1].float(), w.float())
    assert y.shape == (B, H, L, D) and y.is_contiguous()
    close_bf16(y, want)


def test_rms_norm_3072_wide_bf16(tk):
    g = gen(6)
    x = torch.randn(1, 4608, 3072, generator=g).to(BF)
    w = (1 + 0.1 * torch.randn(3072, generator=g)).to(BF)
    close_bf16(tk.rms_norm(x.cuda(), w.cuda()), O.rms_norm(x.float(), w.float()))


@pytest.mark.parametrize("shape", [(2, 4, 256, 128), (1, 24, 100, 128), (3, 2, 65, 256)])
def test_rms_norm_backward_fp32(tk, shape):
    g = gen(7)
    x = torch.randn(*shape, generator=g)
    w = 1 + 0.1 * torch.randn(shape[-1], generator=g)
    dy = torch.randn(*shape, generator=g)
    xc, wc = x.cuda().requires_grad_(), w.cuda().requires_grad_()
    tk.rms_norm(xc, wc).backward(dy.cuda())
    dx, dw = O.rms_norm_backward(dy.double(), x.double(), w.double())
    torch.testing.assert_close(xc.grad.cpu().double(), dx, atol=1e-3, rtol=0)
    torch.testing.assert_close(wc.grad.cpu().double(), dw, atol=1e-3, rtol=1e-4)


# ------------------------------------------------------------------ RoPE
@pytest.mark.parametrize("B,H,L,D", [(1, 2, 256, 128), (2, 24, 100, 128), (8, 3, 33, 256), (1, 5, 7, 64)])
def test_rope_fp32_random_table(tk, B, H, L, D):
    g = gen(8)
    q, k = torch.randn(B, H, L, D, generator=g), torch.randn(B, H, L, D, generator=g)
    pe = torch.randn(1, 1, L, D // 2, 2, 2, generator=g)
    oq, ok = tk.apply_rope(q.cuda(), k.cuda(), pe.cuda())
    wq, wk = O.apply_rope(q, k, pe)
    torch.testing.assert_close(oq.cpu(), wq, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(ok.cpu(), wk, atol=1e-5, rtol=1e-5)


def test_rope_bf16_flux_table(tk):
    g = gen(9)
    q, k = torch.randn(1, 24, 576, 128, generator=g).to(BF), torch.randn(1, 24, 576, 128, generator=g).to(BF)
    pe = O.embed_nd(O.flux_position_ids(64, 16, 32), [16, 56, 56])
    oq, ok = tk.apply_rope(q.cuda(), k.cuda(), pe.cuda())
    wq, wk = O.apply_rope(q, k, pe)
    # same fp32 math and one rounding on both sides: bit-exact up to fma contraction
    close_bf16(oq, wq, atol=1e-2, rtol=1e-2)
    close_bf16(ok, wk, atol=1e-2, rtol=1e-2)
    assert (oq.cpu() != wq).float().mean() < 0.01


def test_rope_rejects_batched_table(tk):
    q = torch.randn(2, 2, 8, 128, device="cuda")
    with pytest.raises(ValueError):
        tk.apply_rope(q, q, torch.randn(2, 1, 8, 64, 2, 2, device="cuda"))


# ------------------------------------------------------------------ q/k/v assembly, modulation ops, SiLU, GEMV
def test_qkv_concat_is_a_pure_permutation(tk):
    from triton_kernels_b200 import ops

    g = gen(10)
    B, H, D, Lt, Li = 2, 24, 128, 37, 150
    txt = torch.randn(B, Lt, 3 * H * D, generator=g).to(BF)
    img = torch.randn(B, Li, 3 * H * D, generator=g).to(BF)
    q, k, v = ops.qkv_concat(txt.cuda(), img.cuda(), H)
    wq, wk, wv = O.qkv_concat(txt, img, H)
    assert torch.equal(q.cpu(), wq) and torch.equal(k.cpu(), wk) and torch.equal(v.cpu(), wv)


def test_qkv_prepare_with_norm_and_rope(tk):
    from triton_kernels_b200 import ops

    g = gen(11)
    B, H, D, Lt, Li = 1, 24, 128, 64, 16 * 24
    txt = torch.randn(B, Lt, 3 * H * D, generator=g).to(BF)
    img = torch.randn(B, Li, 3 * H * D, generator=g).to(BF)
    scales = [(1 + 0.1 * torch.randn(D, generator=g)).to(BF) for _ in range(4)]
    pe = O.embed_nd(O.flux_position_ids(Lt, 16, 24), [16, 56, 56])
    q, k, v = ops.qkv_prepare([txt.cuda(), img.cuda()], H, [scales[0].cuda(), scales[2].cuda()],
                              [scales[1].cuda(), scales[3].cuda()], pe.cuda())
    tq, tk_, tv = O.split_heads(txt.float(), H)
    iq, ik, iv = O.split_heads(img.float(), H)
    wq = torch.cat((O.rms_norm(tq, scales[0].float()), O.rms_norm(iq, scales[2].float())), 2)
    wk = torch.cat((O.rms_norm(tk_, scales[1].float()), O.rms_norm(ik, scales[3].float())), 2)
    wq, wk = O.apply_rope(wq, wk, pe)
    close_bf16(q, wq)
    close_bf16(k, wk)
    assert torch.equal(v.cpu().float(), torch.cat((tv, iv), 2))


@pytest.mark.parametrize("dtype", [torch.float32, BF])
def test_modulation_ops_and_silu(tk, dtype):
    from triton_kernels_b200 import ops

    g = gen(12)
    B, L, C = 2, 50, 3072
    x = torch.randn(B, L, C, generator=g).to(dtype)
    proj = torch.randn(B, L, C, generator=g).to(dtype)
    mod = torch.randn(B, 6 * C, generator=g).to(dtype)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    for is1 in (True, False):
        got = ops.modulation_scale_shift(x.cuda(), mod.cuda(), is1)
        torch.testing.assert_close(got.float().cpu(), O.modulation_scale_shift(x.float(), mod.float(), is1), **tol)
    for chunk in (2, 5):
        got = ops.modulation_gate_proj(x.cuda(), mod.cuda(), proj.cuda(), chunk)
        torch.testing.assert_close(got.float().cpu(), O.modulation_gate_proj(x.float(), mod.float(), proj.float(), chunk), **tol)
    v = torch.randn(3, 1001, generator=g).to(dtype) * 3
    torch.testing.assert_close(ops.silu(v.cuda()).float().cpu(), O.silu(v.float()), **tol)


@pytest.mark.parametrize("B,N,K", [(1, 18432, 3072), (2, 9216, 3072), (5, 1000, 256), (8, 64, 3072),
                                   (3, 500, 1536), (1, 301, 4608)])  # one and three chunks per row, ragged N
def test_modulation_projection(tk, B, N, K):
    from triton_kernels_b200 import ops

    g = gen(13)
    vec = torch.randn(B, K, generator=g).to(BF)
    w = (0.02 * torch.randn(N, K, generator=g)).to(BF)
    b = (0.02 * torch.randn(N, generator=g)).to(BF)
    got = ops.modulation_silu_linear(vec.cuda(), w.cuda(), b.cuda())
    want = O.linear(O.silu(vec.float()), w.float(), b.float())
    close_bf16(got, want)


@pytest.mark.parametrize("B,light", [(1, False), (1, True), (2, True), (3, False)])
def test_modulation_projection_filled_in_row_ranges(tk, B, light):
    """The packed [B, 6C] modulation tensor filled by two calls over row ranges (the block computes
    the half that is needed after attention later, in the light launch form)."""
    from triton_kernels_b200.ops.fused import modulation_silu_linear_rows

    g = gen(22)
    K, N = 3072, 6 * 512
    vec = torch.randn(B, K, generator=g).to(BF)
    w = (0.02 * torch.randn(N, K, generator=g)).to(BF)
    b = (0.02 * torch.randn(N, generator=g)).to(BF)
    out = torch.full((B, N), float("nan"), dtype=BF).cuda()
    vc, wc, bc = vec.cuda(), w.cuda(), b.cuda()
    modulation_silu_linear_rows(vc, wc, bc, out, 0, N // 2, False)
    assert torch.isnan(out[:, N // 2 :].float()).all()  # the other half is untouched
    modulation_silu_linear_rows(vc, wc, bc, out, N // 2, N, light)
    close_bf16(out, O.linear(O.silu(vec.float()), w.float(), b.float()))
    # a ragged range in the light form
    out2 = torch.zeros((B, N), dtype=BF).cuda()
    modulation_silu_linear_rows(vc, wc, bc, out2, 5, 1006, True)
    want = O.linear(O.silu(vec.float()), w.float(), b.float())
    close_bf16(out2[:, 5:1006], want[:, 5:1006])
    assert float(out2[:, :5].abs().max()) == 0 and float(out2[:, 1006:].abs().max()) == 0


# ------------------------------------------------------------------ linear (tcgen05 GEMM)
@pytest.mark.parametrize(
    "M,K,N,act,bias",
    [
        (128, 64, 256, "", False),       # exactly one tile, one k-block
        (128, 256, 256, "", True),       # ring wraps once
        (256, 1024, 1024, "", True),
        (1024, 512, 3072, "GELU", True),
        (300, 328, 1000, "", True),      # ragged M, K, N
        (77, 64, 64, "GELU", True),      # smaller than one tile in every dim
        (4608, 3072, 3072, "", True),    # multiple tiles per CTA (persistent loop + both accumulators)
    ],
)
def test_linear(tk, M, K, N, act, bias):
    g = gen(14)
    x = torch.randn(M, K, generator=g).to(BF)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(BF)
    b = (0.5 * torch.randn(N, generator=g)).to(BF) if bias else None
    y = tk.linear(x.cuda(), w.cuda(), b.cuda() if bias else None, activation=act)
    want = O.linear(x.double(), w.double(), b.double() if bias else None, act)
    close_bf16(y, want)
    assert rel_l2(y, want) < 4e-3


def test_linear_batched_input_and_small_m(tk):
    g = gen(15)
    x = torch.randn(2, 3, 50, 256, generator=g).to(BF)
    w = (0.05 * torch.randn(512, 256, generator=g)).to(BF)
    y = tk.linear(x.cuda(), w.cuda(), None)
    assert y.shape == (2, 3, 50, 512)
    close_bf16(y, O.linear(x.float(), w.float()))
    v = torch.randn(2, 3072, generator=g).to(BF)
    w2 = (0.02 * torch.randn(1024, 3072, generator=g)).to(BF)
    close_bf16(tk.linear(v.cuda(), w2.cuda(), None), O.linear(v.float(), w2.float()))


def test_linear_rejects_fp32_like_the_reference(tk):
    with pytest.raises(KeyError):
        tk.linear(torch.randn(8, 64, device="cuda"), torch.randn(64, 64, device="cuda"), None)


def test_linear_epilogues(tk):
    """Column-split output with GELU on the second part, and the gate/residual epilogue."""
    from triton_kernels_b200 import _lib
    from triton_kernels_b200.kernels.linear import linear_into

    g = gen(16)
    M, K, N, split = 200, 256, 768, 512
    x = torch.randn(M, K, generator=g).to(BF)
    w = (torch.randn(N, K, generator=g) / 16).to(BF)
    b = (0.1 * torch.randn(N, generator=g)).to(BF)
    y1 = torch.zeros(M, split, dtype=BF, device="cuda")
    wide = torch.zeros(M, 64 + (N - split), dtype=BF, device="cuda")
    linear_into(x.cuda(), w.cuda(), b.cuda(), y1, y2=wide[:, 64:], split=split, epi2=_lib.EPI_GELU)
    ref = O.linear(x.float(), w.float(), b.float())
    close_bf16(y1, ref[:, :split])
    close_bf16(wide[:, 64:], O.gelu_tanh(ref[:, split:]))
    assert float(wide[:, :64].abs().max()) == 0.0  # untouched columns

    B, L = 2, 100
    resid = torch.randn(B * L, N, generator=g).to(BF)
    gate = torch.randn(B, N, generator=g).to(BF)
    out = torch.empty(B * L, N, dtype=BF, device="cuda")
    gc = gate.cuda()
    linear_into(x.cuda(), w.cuda(), b.cuda(), out, epi=_lib.EPI_GATE_RESID, resid=resid.cuda(), gate=gc,
                gate_stride=gc.stride(0), rows_per_batch=L)
    want = resid.float() + gate.float().repeat_interleave(L, 0) * ref
    close_bf16(out, want)


# ------------------------------------------------------------------ attention
@pytest.mark.parametrize("B,H,L", [(1, 2, 256), (2, 4, 512), (1, 24, 1024), (1, 3, 128), (2, 2, 200), (1, 2, 77), (1, 1, 1), (1, 2, 641)])
def test_attention(tk, B, H, L):
    g = gen(17)
    q, k, v = (torch.randn(B, H, L, 128, generator=g).to(BF) for _ in range(3))
    o = tk.scaled_dot_product_attention(q.cuda(), k.cuda(), v.cuda())
    want = O.scaled_dot_product_attention(q.float(), k.float(), v.float())
    torch.testing.assert_close(o.float().cpu(), want, atol=1e-2, rtol=2e-2)
    assert rel_l2(o, want) < 1e-2


@pytest.mark.parametrize("B,H,L", [(2, 4, 256), (1, 8, 512), (4, 2, 1024), (1, 24, 300), (1, 3, 65)])
def test_attention_head_dim_64(tk, B, H, L):
    """The reference's attention test also sweeps head_dim 64 (tests/test_attention.py:9)."""
    g = gen(27)
    q, k, v = (torch.randn(B, H, L, 64, generator=g).to(BF) for _ in range(3))
    o = tk.scaled_dot_product_attention(q.cuda(), k.cuda(), v.cuda())
    want = O.scaled_dot_product_attention(q.float(), k.float(), v.float())
    torch.testing.assert_close(o.float().cpu(), want, atol=1e-2, rtol=2e-2)
    assert rel_l2(o, want) < 1e-2


@pytest.mark.parametrize("B,L,K,N", [(1, 256, 256, 1024), (2, 512, 512, 2048), (4, 1024, 1024, 3072), (4, 256, 1024, 2048)])
@pytest.mark.parametrize("act", ["", "GELU"])
def test_linear_reference_grid(tk, B, L, K, N, act):
    """Corners of the reference's own grid (tests/test_linear.py:7-12): batched [B, L, K] inputs
    and, like there, N(0,1) weights; its tolerances are 1e-5 / 0.02 absolute against a bf16
    F.linear, here the comparison is against float64 with the bf16 tolerance."""
    g = gen(28)
    x = torch.randn(B, L, K, generator=g).to(BF)
    w = torch.randn(N, K, generator=g).to(BF)
    b = torch.randn(N, generator=g).to(BF)
    y = tk.linear(x.cuda(), w.cuda(), b.cuda(), activation=act)
    want = O.linear(x.double(), w.double(), b.double(), act)
    assert y.shape == (B, L, N)
    assert rel_l2(y, want) < 4e-3
    torch.testing.assert_close(y.float().cpu(), want.float(), atol=0.02 * K**0.5, rtol=2e-2)


def test_attention_sharp_softmax_and_custom_scale(tk):
    """Large logits make the running maximum jump, exercising the lazy-rescale path."""
    g = gen(18)
    B, H, L = 1, 2, 1152
    q = (4 * torch.randn(B, H, L, 128, generator=g)).to(BF)
    k = (4 * torch.randn(B, H, L, 128, generator=g)).to(BF)
    v = torch.randn(B, H, L, 128, generator=g).to(BF)
    for scale in (None, 0.3):
        o = tk.scaled_dot_product_attention(q.cuda(), k.cuda(), v.cuda(), sm_scale=scale)
        want = O.scaled_dot_product_attention(q.float(), k.float(), v.float(), scale)
        torch.testing.assert_close(o.float().cpu(), want, atol=2e-2, rtol=2e-2)


def test_attention_different_kv_length_and_strided_output(tk):
    from triton_kernels_b200.kernels.attention import attention_into

    g = gen(19)
    B, H, Lq, Lk, D = 2, 3, 300, 450, 128
    q = torch.randn(B, H, Lq, D, generator=g).to(BF)
    k = torch.randn(B, H, Lk, D, generator=g).to(BF)
    v = torch.randn(B, H, Lk, D, generator=g).to(BF)
    out = torch.zeros(B, Lq, H * D + 256, dtype=BF, device="cuda")  # wider buffer, like the single block's
    o_view = out[:, :, : H * D].unflatten(2, (H, D)).permute(0, 2, 1, 3)
    attention_into(q.cuda(), k.cuda(), v.cuda(), o_view, D**-0.5)
    want = O.scaled_dot_product_attention(q.float(), k.float(), v.float()).permute(0, 2, 1, 3).reshape(B, Lq, H * D)
    torch.testing.assert_close(out[:, :, : H * D].float().cpu(), want, atol=1e-2, rtol=2e-2)
    assert float(out[:, :, H * D :].abs().max()) == 0.0


@pytest.mark.parametrize("B,H,Lq,Lk,D,splits", [(1, 3, 1024, 2048, 128, 2), (2, 2, 300, 1100, 128, 3), (1, 4, 512, 1024, 64, 2)])
def test_attention_key_splits(tk, B, H, Lq, Lk, D, splits):
    """The keys cut into ranges that run as separate CTAs, merged by their log-sum-exp: same
    result as the one-pass kernel up to the merge's rounding."""
    from triton_kernels_b200.kernels.attention import attention_into, key_splits_for

    g = gen(29)
    q = torch.randn(B, H, Lq, D, generator=g).to(BF)
    k = (2 * torch.randn(B, H, Lk, D, generator=g)).to(BF)
    v = torch.randn(B, H, Lk, D, generator=g).to(BF)
    o1 = torch.zeros(B, H, Lq, D, dtype=BF, device="cuda")
    o2 = torch.zeros_like(o1)
    attention_into(q.cuda(), k.cuda(), v.cuda(), o1, D**-0.5)
    attention_into(q.cuda(), k.cuda(), v.cuda(), o2, D**-0.5, k_splits=splits)
    want = O.scaled_dot_product_attention(q.float(), k.float(), v.float())
    torch.testing.assert_close(o2.float().cpu(), want, atol=1e-2, rtol=2e-2)
    assert rel_l2(o2, want) < 1e-2
    assert rel_l2(o2, o1.float().cpu()) < 4e-3
    # 3 heads x 66 query blocks: two waves of whole CTAs or three half-waves
    assert key_splits_for(1, 3, 16896, 16896, 128, 148) == 2
    assert [key_splits_for(1, h, 16896, 16896, 128, 148) for h in (6, 12, 24)] == [1, 1, 1]
    assert key_splits_for(1, 24, 4608, 4608, 128, 148) == 1


def test_empty_inputs_are_no_ops(tk):
    """Zero tokens: every operator returns an empty tensor of the right shape and launches
    nothing that could fault (the reference's launchers would start a grid of zero programs)."""
    from triton_kernels_b200 import ops

    dev = "cuda"
    w = torch.randn(256, 128, device=dev).to(BF)
    b = torch.zeros(256, device=dev, dtype=BF)
    assert tk.linear(torch.empty(2, 0, 128, device=dev, dtype=BF), w, b).shape == (2, 0, 256)
    assert tk.linear(torch.empty(0, 128, device=dev, dtype=BF), w, None, activation="GELU").shape == (0, 256)
    q = torch.empty(1, 2, 0, 128, device=dev, dtype=BF)
    assert tk.scaled_dot_product_attention(q, q, q).shape == (1, 2, 0, 128)
    x = torch.empty(2, 0, 256, device=dev)
    sc = torch.zeros(2, 1, 256, device=dev)
    assert tk.layer_norm_modulation(x, sc, sc).shape == (2, 0, 256)
    assert tk.rms_norm(torch.empty(1, 3, 0, 128, device=dev), torch.ones(128, device=dev)).shape == (1, 3, 0, 128)
    oq, ok = tk.apply_rope(q, q, torch.empty(1, 1, 0, 64, 2, 2, device=dev))
    assert oq.shape == ok.shape == (1, 2, 0, 128)
    assert ops.silu(torch.empty(0, device=dev)).shape == (0,)
    torch.cuda.synchronize()
    from triton_kernels_b200 import _lib

    assert _lib.device_status() == (0, 0)


def test_device_status_is_clean(tk):
    from triton_kernels_b200 import _lib

    assert _lib.device_status() == (0, 0)


@pytest.mark.parametrize("B,Lt,Li,bias", [(1, 128, 384, False), (2, 256, 128, True)])
def test_linear_qkv_grouped_matches_projection_plus_assembly(tk, B, Lt, Li, bias):
    """The q|k|v projection with norm, rotation and head-major layout in its epilogue against the
    plain projection followed by the assembly kernel."""
    from triton_kernels_b200 import ops
    from triton_kernels_b200.kernels.linear import linear_qkv_grouped_into

    g = gen(61)
    H, D, K = 4, 128, 512
    C3 = 3 * H * D
    xs = [torch.randn(B, L, K, generator=g).to(BF).cuda() for L in (Lt, Li)]
    ws = [(torch.randn(C3, K, generator=g) * 0.05).to(BF).cuda() for _ in range(2)]
    bs = [(torch.randn(C3, generator=g) * 0.1).to(BF).cuda() if bias else None for _ in range(2)]
    qs = [(1 + 0.1 * torch.randn(D, generator=g)).to(BF).cuda() for _ in range(2)]
    ks = [(1 + 0.1 * torch.randn(D, generator=g)).to(BF).cuda() for _ in range(2)]
    L = Lt + Li
    pe = torch.randn(1, 1, L, D // 2, 2, 2, generator=g).cuda()
    out = torch.zeros(3, B, H, L, D, dtype=BF, device="cuda")
    linear_qkv_grouped_into([dict(x=x, w=w, b=b, q_scale=q_, k_scale=k_) for x, w, b, q_, k_ in zip(xs, ws, bs, qs, ks)],
                            pe, out)
    qkvs = [tk.linear(x, w, b) for x, w, b in zip(xs, ws, bs)]
    q, k, v = ops.qkv_prepare(qkvs, H, qs, ks, pe)
    torch.cuda.synchronize()
    assert torch.equal(out[2], v)
    torch.testing.assert_close(out[0].float(), q.float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(out[1].float(), k.float(), atol=2e-2, rtol=2e-2)
    # without scales and table it is the projection re-laid out
    out2 = torch.zeros_like(out)
    linear_qkv_grouped_into([dict(x=x, w=w, b=b) for x, w, b in zip(xs, ws, bs)], None, out2)
    q2, k2, v2 = ops.qkv_prepare(qkvs, H)
    torch.cuda.synchronize()
    assert torch.equal(out2[0], q2) and torch.equal(out2[1], k2) and torch.equal(out2[2], v2)


def test_double_block_fused_qkv_epilogue_matches_unfused(tk):
    g = gen(62)
    C, H, Lt, Li = 512, 4, 128, 256
    blk = tk.DoubleStreamBlock(C, H, 4.0).to(BF).cuda()
    with torch.no_grad():
        for name, p in blk.named_parameters():
            p.copy_((torch.randn(p.shape, generator=g) * (0.1 if name.endswith("scale") else 0.03)
                     + (1.0 if name.endswith("scale") else 0.0)).to(BF))
    img = torch.randn(1, Li, C, generator=g).to(BF).cuda()
    txt = torch.randn(1, Lt, C, generator=g).to(BF).cuda()
    vec = torch.randn(1, C, generator=g).to(BF).cuda()
    pe = torch.randn(1, 1, Lt + Li, C // H // 2, 2, 2, generator=g).cuda()
    with torch.no_grad():
        blk.fuse_qkv_epilogue = True
        a_img, a_txt = blk(img, txt, vec, pe)
        blk.fuse_qkv_epilogue = False
        b_img, b_txt = blk(img, txt, vec, pe)
    torch.cuda.synchronize()
    for a, b in ((a_img, b_img), (a_txt, b_txt)):
        rel = float((a.float() - b.float()).norm() / b.float().norm())
        assert rel < 3e-3, rel


def test_single_block_fused_qkv_epilogue_matches_unfused(tk):
    g = gen(63)
    C, H, L = 512, 4, 384
    blk = tk.SingleStreamBlock(C, H, 4.0).to(BF).cuda()
    with torch.no_grad():
        for name, p in blk.named_parameters():
            p.copy_((torch.randn(p.shape, generator=g) * (0.1 if name.endswith("scale") else 0.03)
                     + (1.0 if name.endswith("scale") else 0.0)).to(BF))
    x = torch.randn(2, L, C, generator=g).to(BF).cuda()
    vec = torch.randn(2, C, generator=g).to(BF).cuda()
    pe = torch.randn(1, 1, L, C // H // 2, 2, 2, generator=g).cuda()
    with torch.no_grad():
        blk.fuse_qkv_epilogue = True
        a = blk(x, vec, pe)
        blk.fuse_qkv_epilogue = False
        b = blk(x, vec, pe)
    torch.cuda.synchronize()
    rel = float((a.float() - b.float()).norm() / b.float().norm())
    assert rel < 3e-3, rel
