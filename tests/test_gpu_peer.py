"""Single-GPU checks of the peer-exchange entry points: the scatter forms of the q/k/v assembly
and attention kernels against their plain forms (with every "peer" base in local memory), and
the signal / wait kernels, including a wait that nobody satisfies: it must give up after its
limit, report FLUXB_ERR_TIMEOUT in the device status word and leave the context usable."""
import ctypes
from ctypes import c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def gen(seed):
    return torch.Generator().manual_seed(seed)


def test_qkv_prep_scatter_matches_group_layout(lib):
    from triton_kernels_b200.ops.fused import qkv_prepare_into, qkv_prepare_scatter

    g = gen(71)
    B, H, D, Lt, Li, P = 1, 8, 128, 24, 72, 4
    Hp, L = H // P, Lt + Li
    txt = torch.randn(B, Lt, 3 * H * D, generator=g).to(BF).cuda()
    img = torch.randn(B, Li, 3 * H * D, generator=g).to(BF).cuda()
    scales = [(1 + 0.1 * torch.randn(D, generator=g)).to(BF).cuda() for _ in range(4)]
    pe = torch.randn(1, 1, L, D // 2, 2, 2, generator=g).cuda()
    streams = [(txt, scales[0], scales[1]), (img, scales[2], scales[3])]
    row = 3 * Hp * D
    # plain form: send layout [P, B, L, 3, Hp, D]
    send = torch.zeros(P, B, L, 3, Hp, D, dtype=BF, device="cuda")
    flat = send.view(-1)
    qkv_prepare_into(streams, pe, flat, flat[Hp * D:], flat[2 * Hp * D:], H, eps=1e-6,
                     out_layout=(Hp, L * row, B * L * row, D, row), head_dim=D)
    # scatter form: every group into a buffer of its own
    bufs = [torch.zeros(B, L, 3, Hp, D, dtype=BF, device="cuda") for _ in range(P)]
    bases = (c_void_p * P)(*[b.data_ptr() for b in bufs])
    qkv_prepare_scatter(streams, pe, bases, P, Hp * D, 2 * Hp * D, H, D, (L * row, D, row), eps=1e-6)
    torch.cuda.synchronize()
    for gi in range(P):
        assert torch.equal(bufs[gi], send[gi])


@pytest.mark.parametrize("Lt,Li,P,n2", [(128, 256, 2, 0), (32, 136, 4, 0), (64, 2048, 8, 0), (0, 200, 2, 512)])
def test_linear_qkv_grouped_scatter_matches_head_major_form(lib, Lt, Li, P, n2):
    """The q|k|v projection whose epilogue stores every head group into a buffer of its own (the
    sequence-parallel form, here with all "peers" in local memory) against the head-major form:
    same kernel up to the stores, so the bits must agree.  Stream lengths that are not multiples
    of 128 exist only in the scatter form; they are checked against the assembly kernel."""
    from triton_kernels_b200 import _lib, ops
    from triton_kernels_b200.kernels.linear import linear, linear_qkv_grouped_into

    g = gen(73)
    B, H, D, K = 1, 8, 128, 256
    Hp, L = H // P, Lt + Li
    C3 = 3 * H * D
    lens = [n for n in (Lt, Li) if n > 0]
    xs = [torch.randn(B, n, K, generator=g).to(BF).cuda() for n in lens]
    ws = [(0.05 * torch.randn(C3 + n2, K, generator=g)).to(BF).cuda() for _ in lens]
    bs = [(0.1 * torch.randn(C3 + n2, generator=g)).to(BF).cuda() for _ in lens]
    qs = [(1 + 0.1 * torch.randn(D, generator=g)).to(BF).cuda() for _ in lens]
    ks = [(1 + 0.1 * torch.randn(D, generator=g)).to(BF).cuda() for _ in lens]
    pe = torch.randn(1, 1, L, D // 2, 2, 2, generator=g).cuda()
    y2s = [torch.zeros(B * n, n2, dtype=BF, device="cuda") if n2 else None for n in lens]
    row = 3 * Hp * D
    bufs = [torch.zeros(B, L, 3, Hp, D, dtype=BF, device="cuda") for _ in range(P)]
    bases = (c_void_p * P)(*[b.data_ptr() for b in bufs])
    streams = [dict(x=x, w=w, b=b, q_scale=q_, k_scale=k_, y2=y2) for x, w, b, q_, k_, y2 in zip(xs, ws, bs, qs, ks, y2s)]
    linear_qkv_grouped_into(streams, pe, None, eps=1e-6, epi2=_lib.EPI_GELU,
                            scatter=dict(bases=bases, n_groups=P, k_off=Hp * D, v_off=2 * Hp * D,
                                         strides=(L * row, D, row), num_heads=H, head_dim=D))
    torch.cuda.synchronize()
    got = torch.stack(bufs, 0)  # [P, B, L, 3, Hp, D]
    got = got.permute(3, 1, 0, 4, 2, 5).reshape(3, B, H, L, D)
    if all(n % 128 == 0 for n in lens):
        want = torch.zeros(3, B, H, L, D, dtype=BF, device="cuda")
        y2w = [torch.zeros_like(y) if y is not None else None for y in y2s]
        linear_qkv_grouped_into([dict(s_, y2=y) for s_, y in zip(streams, y2w)], pe, want, eps=1e-6, epi2=_lib.EPI_GELU)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    else:
        qkvs = [linear(x, w[:C3], b[:C3]) for x, w, b in zip(xs, ws, bs)]
        q, k, v = ops.qkv_prepare(qkvs, H, qs, ks, pe)
        torch.cuda.synchronize()
        assert torch.equal(got[2], v)
        torch.testing.assert_close(got[0].float(), q.float(), atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(got[1].float(), k.float(), atol=2e-2, rtol=2e-2)
    if n2:
        for x, w, b, y2 in zip(xs, ws, bs, y2s):
            ref = linear(x, w[C3:], b[C3:], activation="GELU").view(-1, n2)
            torch.testing.assert_close(y2.float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_attention_scatter_matches_plain(lib):
    from triton_kernels_b200.kernels.attention import attention_into, attention_scatter_into

    g = gen(72)
    B, H, L, D, P = 1, 3, 600, 128, 4
    L_loc = L // P
    q, k, v = (torch.randn(B, H, L, D, generator=g).to(BF).cuda() for _ in range(3))
    want = torch.zeros(B, L, H * D, dtype=BF, device="cuda")
    attention_into(q, k, v, want.view(B, L, H, D).permute(0, 2, 1, 3), D**-0.5)
    outs = [torch.zeros(B, L_loc, H * D, dtype=BF, device="cuda") for _ in range(P)]
    bases = (c_void_p * P)(*[o.data_ptr() for o in outs])
    attention_scatter_into(q, k, v, bases, P, L_loc, (L_loc * H * D, D, H * D), D**-0.5)
    torch.cuda.synchronize()
    for r in range(P):
        assert torch.equal(outs[r], want[:, r * L_loc:(r + 1) * L_loc])
    # the key-split form of the same launch: the merge pass does the scatter
    outs2 = [torch.zeros(B, L_loc, H * D, dtype=BF, device="cuda") for _ in range(P)]
    bases2 = (c_void_p * P)(*[o.data_ptr() for o in outs2])
    attention_scatter_into(q, k, v, bases2, P, L_loc, (L_loc * H * D, D, H * D), D**-0.5, k_splits=2)
    torch.cuda.synchronize()
    for r in range(P):
        torch.testing.assert_close(outs2[r].float(), outs[r].float(), atol=1e-2, rtol=2e-2)


def test_scatter_argument_validation(lib):
    bad = (c_void_p * 2)(None, None)
    rc = lib.fluxb_attention_scatter(None, None, None, bad, 2, 16, 1, 1, 32, 32, 128, *([128] * 12), 1.0, None)
    assert rc == -1
    rc = lib.fluxb_peer_signal(None, 2, 0, 0, None)
    assert rc == -1
    rc = lib.fluxb_peer_alloc(16, ctypes.byref(c_void_p()))
    assert rc == -1


def test_signal_wait_and_bounded_wait(lib):
    from triton_kernels_b200 import _lib

    assert lib.fluxb_peer_header_bytes() == 512
    arenas = []
    for _ in range(2):
        p = c_void_p()
        assert lib.fluxb_peer_alloc(4096, ctypes.byref(p)) == 0
        arenas.append(p.value)
    tbl = (c_void_p * 2)(*arenas)
    stream = _lib.stream_handle()
    try:
        _lib.device_status()  # clear
        # two "ranks" on one GPU, all signals enqueued before any wait: three rounds on barrier
        # 0, one on barrier 1
        for barrier, rounds in ((0, 3), (1, 1)):
            for _ in range(rounds):
                for r in range(2):
                    assert lib.fluxb_peer_signal(tbl, 2, r, barrier, stream) == 0
                for r in range(2):
                    assert lib.fluxb_peer_wait(tbl, 2, r, barrier, stream) == 0
        assert _lib.device_status() == (0, 0)
        # rank 0 waits for a round that rank 1 never signals: the wait gives up by itself
        assert lib.fluxb_peer_signal(tbl, 2, 0, 1, stream) == 0
        assert lib.fluxb_peer_wait(tbl, 2, 0, 1, stream) == 0
        code, where = _lib.device_status()
        assert (code, where) == (_lib.ERR_TIMEOUT, 62)
        # the context is still usable
        x = torch.ones(1024, device="cuda")
        assert float(x.sum()) == 1024.0
        assert _lib.device_status() == (0, 0)
    finally:
        torch.cuda.synchronize()
        for a in arenas:
            lib.fluxb_peer_free(a)
