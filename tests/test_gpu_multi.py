"""Two GPUs, one process each, NCCL: the sharded decode paths on real devices.

Skipped on a box with fewer than two GPUs.  Each rank runs as a child process
(``torch.multiprocessing.spawn``), the only exchange on the data path is that of
the per-rank partial ``(out, lse)`` of the sequence split (once as an NCCL
all-gather, once as plain stores into peer-mapped exchange areas); batch shards
need none.  NVLS is switched off for NCCL and the library's own kernel uses plain
peer stores, no multimem.  The failure test makes its failure on the host: a rank
skips a step between two steps.  The result of every rank is compared with the CPU
oracle over the whole sequence, to the tolerance of the single-GPU parity tests."""
import math
import os
import socket

import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, x, ref_seq, ref_batch, bits, group, res):
    import torch.distributed as dist
    import bitladder_b200 as B
    from bitladder_b200 import sharding as S

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        dev = torch.device("cuda", rank)
        scale = 1.0 / math.sqrt(128)
        b, s = x["k"].shape[0], x["k"].shape[1]
        h_k = x["k"].shape[2]

        # ---- sequence split: rank r holds tokens [lo, hi) of every sequence, the last rank the tail
        lo, hi = S.sequence_shard_bounds(s, world, bits)[rank]
        n = hi - lo
        cap = max(n, B.pack_block_tokens(bits))
        bufs = B.alloc_packed_cache(b, cap, h_k, 128, bits, group, device=dev)
        if n > 0:
            B.kvcache_pack_int(x["k"][:, lo:hi].to(dev), bufs[0], bufs[1], x["v"][:, lo:hi].to(dev), bufs[2], bufs[3],
                               None, None, n, "k-channel", group, bits)
        kw = {}
        if rank == world - 1 and res:
            kw = dict(k_res=x["k_res"].to(dev), v_res=x["v_res"].to(dev))
        out, lse = S.decode_sequence_parallel(x["q"].to(dev), *bufs, scale, group, bits, seqlen_k=n,
                                              return_lse=True, **kw)
        err = np.abs(out.float().cpu().numpy()[:, 0] - ref_seq).max()
        assert err <= 2e-3, ("sequence split", rank, err)
        # the same exchange prepared once: over NCCL (one all-gather of a packed buffer, one merge launch) and
        # over peer-mapped exchange areas (one kernel stores, waits and merges), eagerly and as a CUDA graph
        for kind in ("nccl", "peer"):
            sp = S.SequenceParallelStep(x["q"].to(dev), *bufs, scale, group, bits, seqlen_k=n, exchange=kind, **kw)
            for _ in range(3):
                out2 = sp.step()
                err = np.abs(out2.float().cpu().numpy()[:, 0] - ref_seq).max()
                assert err <= 2e-3, ("prepared sequence split", kind, rank, err)
            if kind == "peer":
                sp.check()
                gr = torch.cuda.CUDAGraph()
                side = torch.cuda.Stream(dev)
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    with torch.cuda.graph(gr, stream=side):
                        sp.step()
                        sp.step()
                torch.cuda.current_stream().wait_stream(side)
                for _ in range(3):
                    sp.out.zero_()
                    gr.replay()
                    err = np.abs(sp.out.float().cpu().numpy()[:, 0] - ref_seq).max()
                    assert err <= 2e-3, ("graph replay of the peer exchange", rank, err)
                sp.check()
                dist.barrier()
                # a peer that skips a step (a failure made on the host, between steps): the other rank's
                # bounded wait runs out and its area reports it; nothing faults or hangs
                sp2 = S.SequenceParallelStep(x["q"].to(dev), *bufs, scale, group, bits, seqlen_k=n, exchange="peer",
                                             spin_limit=20000, **kw)
                sp2.step()
                sp2.check()
                dist.barrier()
                if rank == 0:
                    sp2.step()
                    try:
                        sp2.check()
                        raise AssertionError("the missing peer was not noticed")
                    except RuntimeError as exc:
                        assert "wait" in str(exc)
                torch.cuda.synchronize()
                dist.barrier()
                sp2.close()
                sp.close()

        # ---- batch split: rank r holds sequences [lo, hi); no communication at all
        lo, hi = S.shard_range(b, rank, world)
        bufs = B.alloc_packed_cache(hi - lo, s, h_k, 128, bits, group, device=dev)
        B.kvcache_pack_int(x["k"][lo:hi].to(dev), bufs[0], bufs[1], x["v"][lo:hi].to(dev), bufs[2], bufs[3],
                           None, None, s, "k-channel", group, bits)
        out = B.fwd_kvcache_int(x["q"][lo:hi].to(dev), *bufs, None, scale, "k-channel", group, bits)
        err = np.abs(out.float().cpu().numpy()[:, 0] - ref_batch[lo:hi]).max()
        assert err <= 2e-3, ("batch split", rank, err)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("bits,group,res", [(4, 128, 64), (2, 128, 0)])
def test_two_gpus_sequence_and_batch_split(bits, group, res):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    b, s, h, h_k = 4, 4096, 32, 8
    x = H.gen_qkv(b, s, h, h_k, seed=31, res=res)
    pk = H.oracle_pack(x["k"], x["v"], bits, group, "fp16")
    scale = 1.0 / math.sqrt(128)
    ref_seq, _ = H.oracle_decode(x["q"], pk, scale, bits, group, "fp16", k_res=x.get("k_res"), v_res=x.get("v_res"))
    ref_batch, _ = H.oracle_decode(x["q"], pk, scale, bits, group, "fp16")
    mp.spawn(_rank_main, args=(2, _free_port(), x, ref_seq, ref_batch, bits, group, res), nprocs=2, join=True)
