"""Ulysses sequence parallelism on real GPUs (needs at least two): each rank's shard of the
sequence-parallel block output equals the corresponding rows of the single-GPU block output.
Both exchanges are run: the two NCCL all-to-alls, and the peer-memory form in which the
producing kernels store straight into the other GPU's arena (with the assembly kernel and with
the q|k|v projection's own epilogue as the producer).  Ranks are child processes over
NCCL with NVLS switched off; a rank only leaves between steps, after a collective teardown."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, q_out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    import datetime

    torch.cuda.set_device(rank)
    # a short collective timeout: if the peer dies, this rank's next collective ends with an error
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=120))
    try:
        from oracle import flux_oracle as O
        import triton_kernels_b200 as tk
        from triton_kernels_b200 import _lib
        from triton_kernels_b200.parallel import SequenceParallel, shard_joint_sequence

        BF = torch.bfloat16
        C, H, Lt, gh, gw = 3072, 24, 64, 16, 16
        g = torch.Generator().manual_seed(41)  # same draw on every rank
        pd = {k: v.to(BF) for k, v in O.init_params(O.double_block_shapes(C), g, bias_std=0.02, scale_jitter=0.1).items()}
        ps = {k: v.to(BF) for k, v in O.init_params(O.single_block_shapes(C), g, bias_std=0.02, scale_jitter=0.1).items()}
        img = torch.randn(1, gh * gw, C, generator=g).to(BF).cuda()
        txt = torch.randn(1, Lt, C, generator=g).to(BF).cuda()
        vec = torch.randn(1, C, generator=g).to(BF).cuda()
        pe = O.embed_nd(O.flux_position_ids(Lt, gh, gw), [16, 56, 56]).cuda()
        dblk = tk.DoubleStreamBlock(C, H, 4.0).to(BF)
        dblk.load_state_dict(pd)
        dblk = dblk.cuda()
        sblk = tk.SingleStreamBlock(C, H, 4.0).to(BF)
        sblk.load_state_dict(ps)
        sblk = sblk.cuda()

        with torch.no_grad():
            want_img, want_txt = dblk(img, txt, vec, pe)
            want_x = sblk(torch.cat((txt, img), 1), vec, pe)
            txt_l, img_l, pe_l = shard_joint_sequence(txt, img, pe, rank, world)
            Li, Ltl = img.shape[1] // world, Lt // world
            rows_i = slice(rank * Li, (rank + 1) * Li)
            rows_t = slice(rank * Ltl, (rank + 1) * Ltl)

            def rel(a, b):
                return float((a.float() - b.float()).norm() / b.float().norm())

            errs = []
            for exchange, from_projection in (("nccl", False), ("peer", False), ("peer", True)):
                sp = SequenceParallel(exchange=exchange, scatter_from_projection=from_projection)
                dblk.sequence_parallel = sblk.sequence_parallel = sp
                for _ in range(3):  # several rounds: the arenas and their epochs are reused
                    got_img, got_txt = dblk(img_l, txt_l, vec, pe_l)
                    got_x = sblk(torch.cat((txt_l, img_l), 1), vec, pe_l)
                    # same kernels and weights; only the key order inside attention differs
                    errs += [rel(got_img, want_img[:, rows_i]), rel(got_txt, want_txt[:, rows_t]),
                             rel(got_x[:, :Ltl], want_x[:, rows_t]), rel(got_x[:, Ltl:], want_x[:, Lt:][:, rows_i])]
                torch.cuda.synchronize()
                sp.check()  # raises if a flag wait of the peer exchange gave up
                sp.close()
            # A long sequence over few heads: 2 local heads x 80 query blocks = 160 CTAs leave the
            # second wave of the attention launch almost empty, so both exchanges take the
            # key-split form of attention (partial rows merged by their log-sum-exp, the merge
            # pass doing the scatter store under the peer exchange).
            from triton_kernels_b200.kernels.attention import key_splits_for

            C2, H2, Lt2, gh2, gw2 = 512, 4, 512, 156, 128
            assert key_splits_for(1, H2 // world, Lt2 + gh2 * gw2, Lt2 + gh2 * gw2) == 2
            g2 = torch.Generator().manual_seed(42)
            pd2 = {k: v.to(BF) for k, v in O.init_params(O.double_block_shapes(C2), g2, bias_std=0.02, scale_jitter=0.1).items()}
            img2 = torch.randn(1, gh2 * gw2, C2, generator=g2).to(BF).cuda()
            txt2 = torch.randn(1, Lt2, C2, generator=g2).to(BF).cuda()
            vec2 = torch.randn(1, C2, generator=g2).to(BF).cuda()
            pe2 = O.embed_nd(O.flux_position_ids(Lt2, gh2, gw2), [16, 56, 56]).cuda()
            blk2 = tk.DoubleStreamBlock(C2, H2, 4.0).to(BF)
            blk2.load_state_dict(pd2)
            blk2 = blk2.cuda()
            want_i2, want_t2 = blk2(img2, txt2, vec2, pe2)
            txt2_l, img2_l, pe2_l = shard_joint_sequence(txt2, img2, pe2, rank, world)
            ri = slice(rank * (gh2 * gw2 // world), (rank + 1) * (gh2 * gw2 // world))
            rt = slice(rank * (Lt2 // world), (rank + 1) * (Lt2 // world))
            # peer exchange with the image tokens projected and scattered in two halves (the default
            # for 512 local image tokens and more) and in one piece
            for exchange, pipelined in (("peer", True), ("peer", False), ("nccl", False)):
                sp = SequenceParallel(exchange=exchange, pipeline_exchange=pipelined)
                blk2.sequence_parallel = sp
                for _ in range(2):
                    got_i2, got_t2 = blk2(img2_l, txt2_l, vec2, pe2_l)
                    errs += [rel(got_i2, want_i2[:, ri]), rel(got_t2, want_t2[:, rt])]
                torch.cuda.synchronize()
                sp.check()
                sp.close()
        code, where = _lib.device_status()
        assert code == 0, f"device status {code} at {where}"
        dist.barrier()
        q_out.put((rank, max(errs)))
    except Exception as e:  # noqa: BLE001
        # The other rank may be blocked in a collective that this rank will never join: report and
        # leave at once, without the collective teardown; the parent ends the peer.
        q_out.put((rank, repr(e)))
        q_out.close()
        q_out.join_thread()
        os._exit(1)
    dist.destroy_process_group()


def test_sequence_parallel_blocks_match_single_gpu(lib):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q_out)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    try:
        for _ in range(world):
            results.append(q_out.get(timeout=300))
            if not isinstance(results[-1][1], float):
                break  # a rank failed: its peer may never finish
    finally:
        failed = len(results) < world or any(not isinstance(e, float) for _, e in results)
        for p in procs:
            p.join(timeout=5 if failed else 60)
        for p in procs:  # no child may outlive the test holding a GPU
            if p.is_alive():
                p.kill()
                p.join(timeout=30)
    results.sort()
    assert len(results) == world or failed
    for rank, err in results:
        assert isinstance(err, float), f"rank {rank}: {err}"
        assert err < 5e-3, f"rank {rank}: sequence-parallel output differs from single-GPU output by {err}"
