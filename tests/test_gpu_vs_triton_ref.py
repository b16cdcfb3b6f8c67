"""Head to head with the reference's own Triton kernels on the same GPU: identical seeded bf16
inputs through `triton_kernels.*` (the copy staged by oracle/make_ref.py) and through this
library, compared with each other at atol = rtol = 2e-2 per kernel and relative L2 per block,
and both against the fp32 CPU oracle.  Skipped when the staged copy is absent.

Only aligned shapes are given to the reference: its attention kernel builds block pointers
without boundary checks (triton_kernels/kernels/attention.py:109-146) and its RMSNorm launcher
drops the last rows % 8 rows (triton_kernels/kernels/normalization.py:152-154)."""
import pytest
import torch

from oracle import flux_oracle as O
from oracle import make_ref

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
C, H, D = 3072, 24, 128
L_IMG, L_TXT, GRID = 4096, 512, 64
L = L_IMG + L_TXT


@pytest.fixture(scope="module")
def ref():
    mod = make_ref.import_reference()
    if mod is None:
        pytest.skip("the reference package is not staged under oracle/_ref (python oracle/make_ref.py <checkout>)")
    return mod


@pytest.fixture(scope="module")
def tk(lib):
    import triton_kernels_b200 as tk

    return tk


def rel_l2(got, want):
    got, want = got.float().cpu(), want.float().cpu()
    return float((got - want).norm() / want.norm())


def report(name, ours, theirs, want):
    e_ours, e_ref, e_between = rel_l2(ours, want), rel_l2(theirs, want), rel_l2(ours, theirs)
    print(f"{name}: rel-L2 vs fp32 oracle: ours {e_ours:.2e}, reference Triton {e_ref:.2e}; ours vs reference {e_between:.2e}")
    return e_ours, e_ref, e_between


def close(ours, theirs):
    torch.testing.assert_close(ours.float().cpu(), theirs.float().cpu(), atol=2e-2, rtol=2e-2)


def test_rms_norm(tk, ref):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(1, H, L, D, generator=g).to(BF)
    w = (1 + 0.1 * torch.randn(D, generator=g)).to(BF)
    ours, theirs = tk.rms_norm(x.cuda(), w.cuda()), ref.rms_norm(x.cuda(), w.cuda())
    close(ours, theirs)
    e_ours, e_ref, _ = report("rms_norm [1,24,4608,128]", ours, theirs, O.rms_norm(x.float(), w.float()))
    assert e_ours <= 1.5 * e_ref + 1e-3  # fp32 statistics here, bf16 reductions there


def test_layer_norm_modulation(tk, ref):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(1, L, C, generator=g).to(BF)
    sc, sh = ((0.1 * torch.randn(1, 1, C, generator=g)).to(BF) for _ in range(2))
    ours = tk.layer_norm_modulation(x.cuda(), sc.cuda(), sh.cuda(), eps=1e-6)
    theirs = ref.layer_norm_modulation(x.cuda(), sc.cuda(), sh.cuda(), eps=1e-6)
    close(ours, theirs)
    e_ours, e_ref, _ = report("layer_norm_modulation [1,4608,3072]", ours, theirs,
                              O.layer_norm_modulation(x.float(), sc.float(), sh.float(), eps=1e-6))
    assert e_ours <= 1.5 * e_ref + 1e-3


def test_apply_rope(tk, ref):
    g = torch.Generator().manual_seed(1)
    q, k = (torch.randn(1, H, L, D, generator=g).to(BF) for _ in range(2))
    pe = O.embed_nd(O.flux_position_ids(L_TXT, GRID, GRID), [16, 56, 56])
    oq, ok = tk.apply_rope(q.cuda(), k.cuda(), pe.cuda())
    rq, rk = ref.apply_rope(q.cuda(), k.cuda(), pe.cuda())
    close(oq, rq)
    close(ok, rk)
    wq, _ = O.apply_rope(q.float(), k.float(), pe)
    report("apply_rope [1,24,4608,128]", oq, rq, wq)


@pytest.mark.parametrize("act", ["", "GELU"])
def test_linear(tk, ref, act):
    g = torch.Generator().manual_seed(1)
    M, K, N = L, C, 4 * C
    x = torch.randn(M, K, generator=g).to(BF)
    w = (0.02 * torch.randn(N, K, generator=g)).to(BF)
    b = (0.02 * torch.randn(N, generator=g)).to(BF)
    ours = tk.linear(x.cuda(), w.cuda(), b.cuda(), activation=act)
    theirs = ref.linear(x.cuda(), w.cuda(), b.cuda(), activation=act)
    close(ours, theirs)
    e_ours, e_ref, _ = report(f"linear{'+GELU' if act else ''} M4608 K3072 N12288", ours, theirs,
                              O.linear(x.float(), w.float(), b.float(), act))
    assert e_ours <= 1.5 * e_ref + 1e-3


def test_attention(tk, ref):
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(1, H, L, D, generator=g).to(BF) for _ in range(3))
    ours = tk.scaled_dot_product_attention(q.cuda(), k.cuda(), v.cuda())
    theirs = ref.scaled_dot_product_attention(q.cuda(), k.cuda(), v.cuda())
    close(ours, theirs)
    report("attention [1,24,4608,128]", ours, theirs, O.scaled_dot_product_attention(q.float(), k.float(), v.float()))


def test_single_stream_block(tk, ref):
    g = torch.Generator().manual_seed(81)
    pb = {k: v.to(BF) for k, v in O.init_params(O.single_block_shapes(C), g, bias_std=0.02, scale_jitter=0.1).items()}
    x = torch.randn(1, L, C, generator=g).to(BF)
    vec = torch.randn(1, C, generator=g).to(BF)
    pe = O.embed_nd(O.flux_position_ids(L_TXT, GRID, GRID), [16, 56, 56])
    outs = []
    for pkg in (tk, ref):
        blk = pkg.SingleStreamBlock(C, H, 4.0).to(BF)
        blk.load_state_dict(pb)
        blk = blk.cuda()
        with torch.no_grad():
            outs.append(blk(x.cuda(), vec.cuda(), pe.cuda()))
        del blk
    with torch.no_grad():
        want = O.single_stream_block(x.float(), vec.float(), pe, {k: v.float() for k, v in pb.items()}, H)
    e_ours, e_ref, e_between = report("SingleStreamBlock 4608 tokens", outs[0], outs[1], want)
    assert e_ours < 1e-2 and e_between < 2e-2
    torch.testing.assert_close(outs[0].float().cpu(), outs[1].float().cpu(), atol=0.1, rtol=2e-2)  # the reference's own block bound


def test_double_stream_block(tk, ref):
    import bench

    params, img, txt, vec, pe = bench.make_inputs(bench.SEED)
    pb = {k: v.to(BF) for k, v in params.items()}
    outs = []
    for pkg in (tk, ref):
        blk = pkg.DoubleStreamBlock(C, H, 4.0).to(BF)
        blk.load_state_dict(pb)
        blk = blk.cuda()
        with torch.no_grad():
            outs.append(blk(img.to(BF).cuda(), txt.to(BF).cuda(), vec.to(BF).cuda(), pe.cuda()))
        del blk
    with torch.no_grad():
        wi, wt = O.double_stream_block(img.to(BF).float(), txt.to(BF).float(), vec.to(BF).float(), pe,
                                       {k: v.float() for k, v in pb.items()}, H)
    for name, i, want in (("img", 0, wi), ("txt", 1, wt)):
        e_ours, e_ref, e_between = report(f"DoubleStreamBlock 4096+512 tokens ({name})", outs[0][i], outs[1][i], want)
        assert e_ours < 1e-2 and e_between < 2e-2
        torch.testing.assert_close(outs[0][i].float().cpu(), outs[1][i].float().cpu(), atol=0.1, rtol=2e-2)
