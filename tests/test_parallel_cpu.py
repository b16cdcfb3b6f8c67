"""Host-side logic of the multi-GPU shardings on CPU ranks (gloo, world size 2): the Ulysses
all-to-all layouts reproduce full attention, and the batch / token shard helpers partition
their inputs exactly."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import flux_oracle as O


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ulysses_rank(rank: int, world: int, port: int, B: int, q_out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from triton_kernels_b200.parallel import SequenceParallel

        sp = SequenceParallel()
        H, D, L = 4, 16, 24
        g = torch.Generator().manual_seed(77)
        q, k, v = (torch.randn(B, H, L, D, generator=g) for _ in range(3))
        want = O.scaled_dot_product_attention(q, k, v).permute(0, 2, 1, 3).reshape(B, L, H * D)
        L_loc = L // world
        rows = slice(rank * L_loc, (rank + 1) * L_loc)
        # what the q/k/v assembly kernel writes for this rank's tokens
        shape, (Hp, sb, sg, sh, sl) = sp.send_layout(B, L_loc, H, D)
        send = torch.zeros(shape)
        flat = send.view(-1)
        for i, t in enumerate((q, k, v)):
            for b in range(B):
                for h in range(H):
                    for l in range(L_loc):
                        off = i * Hp * D + b * sb + (h // Hp) * sg + (h % Hp) * sh + l * sl
                        flat[off : off + D] = t[b, h, rows][l]
        full = sp.tokens_to_heads(send)  # [B, L, 3, Hp, D]
        assert full.shape == (B, L, 3, Hp, D)
        qh, kh, vh = (full[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        torch.testing.assert_close(qh, q[:, rank * Hp : (rank + 1) * Hp])  # all tokens, local heads, original order
        o = O.scaled_dot_product_attention(qh, kh, vh).permute(0, 2, 1, 3).reshape(B, L, Hp * D).contiguous()
        wide = torch.zeros(B, L_loc, H * D + 8)
        got = sp.heads_to_tokens(o, wide[:, :, : H * D])
        torch.testing.assert_close(got, want[:, rows], atol=1e-6, rtol=1e-6)
        assert float(wide[:, :, H * D :].abs().max()) == 0.0
        q_out.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q_out.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B", [1, 2])
def test_ulysses_exchange_reproduces_full_attention(B):
    world = 2
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ulysses_rank, args=(r, world, port, B, q_out)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q_out.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_shard_helpers_partition_exactly():
    from triton_kernels_b200.parallel import shard_batch, shard_joint_sequence

    for batch, world in [(8, 8), (8, 4), (5, 2), (3, 4)]:
        got = [i for r in range(world) for i in range(batch)[shard_batch(batch, r, world)]]
        assert got == list(range(batch))
    Lt, Li = 8, 24
    txt = torch.arange(Lt).float().view(1, Lt, 1)
    img = 100 + torch.arange(Li).float().view(1, Li, 1)
    pe = torch.arange(Lt + Li).float().view(1, 1, Lt + Li, 1, 1, 1).expand(1, 1, Lt + Li, 2, 2, 2)
    seen_t, seen_i = [], []
    for r in range(4):
        t, i, p = shard_joint_sequence(txt, img, pe, r, 4)
        seen_t += t.flatten().tolist()
        seen_i += i.flatten().tolist()
        # table rows follow the local order: this rank's text rows, then its image rows
        assert p[0, 0, :, 0, 0, 0].tolist() == t.flatten().tolist() + [x - 100 + Lt for x in i.flatten().tolist()]
    assert seen_t == txt.flatten().tolist() and seen_i == img.flatten().tolist()
    with pytest.raises(AssertionError):
        shard_joint_sequence(txt, img, pe, 0, 3)


@pytest.mark.parametrize("B,P", [(1, 2), (2, 4)])
def test_peer_exchange_layout_places_every_element_once(B, P):
    """The address tables of the peer exchange, replayed on CPU: every rank "stores" its q/k/v
    with the scatter kernel's addressing rule into flat per-rank arenas, attention is done per
    head group on what arrived, its output is "stored" with the attention kernel's rule, and
    every rank must end up with full-sequence attention for its own tokens."""
    import torch.nn.functional as F

    from triton_kernels_b200.parallel import peer_exchange_layout

    H, D, L_loc = 4, 8, 6
    L = P * L_loc
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(B, H, L, D, generator=g) for _ in range(3))
    # rank-major token order is the global order here
    want = F.scaled_dot_product_attention(q, k, v).permute(0, 2, 1, 3).reshape(B, L, H * D)
    lays = [peer_exchange_layout(B, L_loc, H, D, P, r, 4) for r in range(P)]
    arenas = [torch.full((lays[0]["nbytes"] // 4,), float("nan")) for _ in range(P)]
    Hp = lays[0]["Hp"]
    for r, lay in enumerate(lays):  # assembly kernel of rank r
        sb, sh, sl = lay["qkv_strides"]
        for h in range(H):
            grp, hh = divmod(h, Hp)
            base = lay["q_offsets"][grp] // 4
            for part, t in ((0, q), (lay["k_off"], k), (lay["v_off"], v)):
                for b in range(B):
                    for l in range(L_loc):
                        o = base + part + b * sb + hh * sh + l * sl
                        arenas[grp][o:o + D] = t[b, h, r * L_loc + l]
    for r, lay in enumerate(lays):  # attention of rank r over its head group, then its stores
        n = B * L * 3 * Hp * D
        recv = arenas[r][:n].view(lay["recv_shape"])
        assert not torch.isnan(recv).any()
        qv, kv, vv = (recv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        o = F.scaled_dot_product_attention(qv, kv, vv)  # [B, Hp, L, D]
        sb, sh, sl = lay["o_strides"]
        for row in range(L):
            owner, lr = divmod(row, L_loc)
            for b in range(B):
                for hh in range(Hp):
                    a = lay["o_offsets"][owner] // 4 + b * sb + hh * sh + lr * sl
                    arenas[owner][a:a + D] = o[b, hh, row]
    for r, lay in enumerate(lays):
        off = lay["out_offset"] // 4
        out = arenas[r][off:off + B * L_loc * H * D].view(lay["out_shape"])
        torch.testing.assert_close(out, want[:, r * L_loc:(r + 1) * L_loc], atol=1e-5, rtol=1e-5)


def test_key_split_estimate_picks_only_part_filled_last_waves():
    """The attention launch is cut along the keys only where that pays: three local heads at
    16896 tokens (eight-way sequence parallelism: 198 CTAs on 148 SMs) yes; 6, 12 or 24 heads, the
    benchmark's single-GPU shape and short sequences no."""
    from triton_kernels_b200.kernels.attention import key_splits_for

    assert key_splits_for(1, 3, 16896, 16896, 128, 148) == 2
    assert [key_splits_for(1, h, 16896, 16896, 128, 148) for h in (6, 12, 24)] == [1, 1, 1]
    assert key_splits_for(1, 24, 4608, 4608, 128, 148) == 1
    assert key_splits_for(2, 4, 512, 512, 128, 148) == 1  # fewer than eight key tiles: never
    assert key_splits_for(1, 2, 20480, 20480, 128, 148) == 2


def test_exchange_pieces_are_whole_gemm_tiles():
    from triton_kernels_b200.parallel.ulysses import exchange_pieces

    for rows in (512, 1024, 2048, 4096, 8192, 9984, 600, 257):
        pieces = exchange_pieces(rows, 2)
        assert pieces[0][0] == 0 and pieces[-1][1] == rows
        assert all(a1 == b0 for (_, a1), (b0, _) in zip(pieces[:-1], pieces[1:]))  # contiguous, in order
        assert all((b - a) % 256 == 0 for a, b in pieces[:-1])  # only the last piece may be ragged
        assert len(pieces) <= 2 and all(b > a for a, b in pieces)
    assert exchange_pieces(2048, 2) == [(0, 1024), (1024, 2048)]
    assert exchange_pieces(9984, 2) == [(0, 5120), (5120, 9984)]
    assert exchange_pieces(256, 2) == [(0, 256)]
    assert exchange_pieces(4096, 4) == [(0, 1024), (1024, 2048), (2048, 3072), (3072, 4096)]
