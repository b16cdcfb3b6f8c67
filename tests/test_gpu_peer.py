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
