"""Ulysses sequence parallelism for the joint attention of the Flux blocks.

Every rank holds L/P tokens of each stream and runs LayerNorm, all GEMMs, QK-norm and RoPE on
them for all H heads.  Around attention the sharding is switched from tokens to heads:

  send   [P, B, L_loc, 3, H/P, D]   written directly by the q/k/v assembly kernel: chunk g holds
                                     this rank's tokens for the heads of rank g, q|k|v
                                     interleaved per token
  all-to-all (equal splits, one call for q, k and v together)
  recv   [P, B, L_loc, 3, H/P, D]   chunk s = tokens of rank s; with B = 1 this IS the full
                                     sequence [L, 3, H/P, D], token-major, and the attention
                                     kernel reads q, k, v from it through strides (no copy)
  attention over all L tokens for the local H/P heads -> [B, L, (H/P)*D]
  all-to-all back (chunk s = the rows rank s owns), then one strided copy interleaves the head
  groups into [B, L_loc, H*D].

Softmax attention does not depend on the order of the keys, and each query row is independent,
so the gathered order (rank-major: txt_0 img_0 txt_1 img_1 ...) need not equal the single-GPU
order (all text, then all image) as long as RoPE was applied with each token's own table row
before the exchange — which is how the assembly kernel is called.

The exchange functions are plain torch.distributed calls on whatever device the tensors live
on, so the layout logic is exercised on CPU ranks (gloo) as well as on GPUs (NCCL).

With `exchange="peer"` (GPUs of one NVSwitch box) neither all-to-all is a separate step: the
assembly kernel stores each head group straight into the arena of the rank that will attend
over it, laid out as [B, L, 3, H/P, D], and the attention kernel stores each query row straight
into the arena of the rank that owns the token, laid out as [B, L_loc, H*D]
(triton_kernels_b200/parallel/peer.py).  Two flag barriers per attention order the stores:
one after the assembly (all q/k/v have arrived), one after attention (all outputs have arrived;
it also tells the peers that this rank's receive buffer may be overwritten again).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor


class SequenceParallel:
    """Process-group handle plus the two layout-changing exchanges."""

    def __init__(self, group=None, exchange: str = "nccl", scatter_from_projection: bool = False,
                 pipeline_exchange: bool = True):
        """`pipeline_exchange` (peer exchange only): the double-stream block projects and scatters
        its image tokens in two pieces, the first piece's stores into the peers' arenas running
        beside the second piece's projection on a second stream (1.81 against 1.83 ms per step
        on four B200s with every form timed at the power cap).

        `scatter_from_projection` (peer exchange only): let the q|k|v projection's own epilogue
        store every head group into its owner's arena (fluxb_linear_qkv_grouped_scatter) instead
        of running the assembly kernel after the projection.  Off by default: with half of the
        stores going over NVLink the GEMM's epilogue warps stall on them, and on two B200s the
        block step took 3.57 ms against 3.48 ms with the separate assembly kernel, although the
        same epilogue costs only 4-6 % of the GEMM when all destinations are local."""
        assert exchange in ("nccl", "peer")
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.exchange = exchange
        self.scatter_from_projection = bool(scatter_from_projection) and exchange == "peer"
        self.pipeline_exchange = bool(pipeline_exchange) and exchange == "peer"
        self._peer: dict = {}

    # ---- peer-memory exchange ------------------------------------------------------------
    def peer_buffers(self, B: int, L_loc: int, H: int, D: int, dtype: torch.dtype):
        """Arena and address tables for one problem shape, created (collectively) on first use."""
        key = (B, L_loc, H, D, dtype)
        if key not in self._peer:
            self._peer[key] = _PeerBuffers(self, B, L_loc, H, D, dtype)
        return self._peer[key]

    def close(self) -> None:
        for pb in self._peer.values():
            pb.arena.close()
        self._peer = {}

    def check(self) -> None:
        """Call at a step boundary (it synchronises the device): raises FluxbError if a kernel of
        this rank gave up a bounded wait since the last check.  The flag waits of the peer exchange
        (status sites 61 and 62) stop after two seconds and the stream then carries on with
        whatever the arena holds, so a rank whose peer was held up that long (first-call module
        load, a paused process) has computed attention on stale data; the device status word is
        the only trace.  The word is cleared by the read."""
        from .. import _lib

        code, where = _lib.device_status()
        if code != 0:
            what = "a peer-exchange flag wait" if where in (61, 62) else "a kernel"
            raise _lib.FluxbError(f"{what} on rank {self.rank} reported error {code} at site {where}: "
                                  "the outputs of the steps since the last check are not valid")

    # ---- token-sharded -> head-sharded -------------------------------------------------
    def send_layout(self, B: int, L_loc: int, H: int, D: int) -> tuple[tuple[int, ...], tuple[int, int, int, int, int]]:
        """Shape of the send buffer and the (heads_per_group, batch, group, head, row) strides
        with which q (offset 0), k (offset Hp*D) and v (offset 2*Hp*D) are written into it."""
        P = self.world
        assert H % P == 0, f"{H} heads cannot be split over {P} ranks"
        Hp = H // P
        shape = (P, B, L_loc, 3, Hp, D)
        row = 3 * Hp * D
        return shape, (Hp, L_loc * row, B * L_loc * row, D, row)

    def tokens_to_heads(self, send: Tensor) -> Tensor:
        """send [P, B, L_loc, 3, Hp, D] -> [B, L, 3, Hp, D] with L = P*L_loc (rows ordered by
        source rank).  A view of the receive buffer when B == 1."""
        P, B, L_loc = send.shape[:3]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        if B == 1:
            return recv.view(1, P * L_loc, *send.shape[3:])
        return recv.permute(1, 0, 2, 3, 4, 5).reshape(B, P * L_loc, *send.shape[3:])

    # ---- head-sharded -> token-sharded -------------------------------------------------
    def heads_to_tokens(self, o: Tensor, out: Tensor | None = None) -> Tensor:
        """o [B, L, Hp*D] (rows ordered by owning rank) -> [B, L_loc, H*D] for the local rows.
        `out` may be any [B, L_loc, H*D] view with unit stride on the last dim."""
        P = self.world
        B, L, W = o.shape
        L_loc = L // P
        send = o.view(B, P, L_loc, W).permute(1, 0, 2, 3)
        send = send.contiguous() if B > 1 else send.reshape(P, 1, L_loc, W)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        if out is None:
            out = torch.empty((B, L_loc, P * W), device=o.device, dtype=o.dtype)
        out.unflatten(2, (P, W)).copy_(recv.permute(1, 2, 0, 3))
        return out


def peer_exchange_layout(B: int, L_loc: int, H: int, D: int, P: int, rank: int, elem_size: int) -> dict:
    """Where things live in the arenas of the peer exchange, as seen from `rank` (pure
    arithmetic; offsets in bytes after the arena header, strides in elements).

      recv [B, P*L_loc, 3, Hp, D]  q|k|v of all tokens for the owner's Hp = H/P heads, rows ordered
                                   by source rank
      out  [B, L_loc, H*D]         attention output of all heads for the owner's tokens

    q_offsets[g]: where this rank's rows start in rank g's recv (q of its first token; k and v
    lie k_off / v_off elements further).  o_offsets[r]: where this rank's head columns start in
    rank r's out."""
    assert H % P == 0, f"{H} heads cannot be split over {P} ranks"
    Hp = H // P
    row = 3 * Hp * D
    recv_bytes = (B * P * L_loc * row * elem_size + 255) // 256 * 256
    out_bytes = B * L_loc * H * D * elem_size
    return dict(
        Hp=Hp, row=row,
        recv_shape=(B, P * L_loc, 3, Hp, D), out_shape=(B, L_loc, H * D),
        recv_offset=0, out_offset=recv_bytes, nbytes=recv_bytes + out_bytes,
        q_offsets=[rank * L_loc * row * elem_size] * P, k_off=Hp * D, v_off=2 * Hp * D,
        qkv_strides=(P * L_loc * row, D, row),  # batch, head, token
        o_offsets=[recv_bytes + rank * Hp * D * elem_size] * P,
        o_strides=(L_loc * H * D, D, H * D),  # batch, head, row
    )


class _PeerBuffers:
    """One arena per rank laid out by peer_exchange_layout, plus the address tables the scatter
    kernels take."""

    def __init__(self, sp: SequenceParallel, B: int, L_loc: int, H: int, D: int, dtype: torch.dtype):
        import ctypes

        from .peer import PeerArena

        P = sp.world
        lay = peer_exchange_layout(B, L_loc, H, D, P, sp.rank, torch.empty((), dtype=dtype).element_size())
        self.arena = PeerArena(lay["nbytes"], sp.group)
        self.recv = self.arena.local_view(lay["recv_offset"], lay["recv_shape"], dtype)
        self.out = self.arena.local_view(lay["out_offset"], lay["out_shape"], dtype)
        self.P, self.Hp, self.L_loc = P, lay["Hp"], L_loc
        self.k_off, self.v_off = lay["k_off"], lay["v_off"]
        self._q_addr = [int(self.arena.address(g, off)) for g, off in enumerate(lay["q_offsets"])]
        self._elem_size = torch.empty((), dtype=dtype).element_size()
        self.q_bases = (ctypes.c_void_p * P)(*self._q_addr)
        self._q_bases_from = {0: self.q_bases}
        self.qkv_strides = lay["qkv_strides"]
        self.o_bases = (ctypes.c_void_p * P)(*[self.arena.address(r, off) for r, off in enumerate(lay["o_offsets"])])
        self.o_strides = lay["o_strides"]


    def q_bases_from_row(self, row: int):
        """The q address table for local tokens starting at `row` (a scatter call that handles the
        rows [row, ...) of this rank's tokens numbers them from zero)."""
        if row not in self._q_bases_from:
            import ctypes

            step = row * self.qkv_strides[2] * self._elem_size
            self._q_bases_from[row] = (ctypes.c_void_p * self.P)(*[a + step for a in self._q_addr])
        return self._q_bases_from[row]


def exchange_pieces(rows: int, pieces: int = 2, tile: int = 256) -> list[tuple[int, int]]:
    """Row ranges in which the pipelined peer exchange projects and scatters `rows` image tokens:
    `pieces` ranges of equal size rounded up to whole GEMM row tiles (so that cutting the
    projection does not add a partial tile), the last one taking what is left; empty ranges are
    dropped."""
    per = (rows // pieces + tile - 1) // tile * tile
    cuts = [min(i * per, rows) for i in range(pieces)] + [rows]
    return [(a, b) for a, b in zip(cuts[:-1], cuts[1:]) if b > a]


def shard_joint_sequence(txt: Tensor, img: Tensor, pe: Tensor, rank: int, world: int):
    """This rank's slice of both streams and the matching rows of the RoPE table.

    txt [B, Lt, *], img [B, Li, *], pe [1, 1, Lt + Li, D/2, 2, 2] (text rows first).  Returns
    (txt_loc, img_loc, pe_loc) with pe_loc ordered text-then-image like the local sequence."""
    Lt, Li = txt.shape[1], img.shape[1]
    assert Lt % world == 0 and Li % world == 0, "both stream lengths must be divisible by the number of ranks"
    t0, t1 = rank * (Lt // world), (rank + 1) * (Lt // world)
    i0, i1 = rank * (Li // world), (rank + 1) * (Li // world)
    pe_loc = torch.cat((pe[:, :, t0:t1], pe[:, :, Lt + i0 : Lt + i1]), dim=2).contiguous()
    return txt[:, t0:t1].contiguous(), img[:, i0:i1].contiguous(), pe_loc
