"""CPU, two processes over gloo: the host logic of the multi-GPU paths.

Batch and KV-head sharding need no communication, so they are checked as plain
slicing against the oracle.  The sequence split has one exchange step (all-gather
of the per-rank partial (out, lse)); here each rank's partial comes from the numpy
oracle, travels through ``gather_partials`` over gloo, and the merged result must
equal attention over the whole sequence."""
import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from bitladder_b200 import sharding as S
from oracle import oracle as O
from tests import helpers as H


def test_shard_range_is_a_balanced_partition():
    for n in (0, 1, 7, 8, 33):
        for world in (1, 2, 3, 8):
            spans = [S.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        S.shard_range(4, 2, 2)


def test_sequence_bounds_are_block_aligned():
    for bits, nb in ((4, 128), (2, 256)):
        for s in (0, 100, 1024, 1048576, 33000):
            b = S.sequence_shard_bounds(s, 8, bits)
            assert b[0][0] == 0 and b[-1][1] == s
            assert all(x[1] == y[0] for x, y in zip(b, b[1:]))
            assert all(lo % nb == 0 for lo, _ in b if lo < s)


def test_batch_and_head_shards_reassemble():
    x = H.gen_qkv(4, 256, 8, 4, seed=2)
    pk = H.oracle_pack(x["k"], x["v"], 4, 128, "fp16")
    scale = H.default_scale()
    full, _ = H.oracle_decode(x["q"], pk, scale, 4, 128, "fp16")
    t = {n: torch.from_numpy(pk[n].view(np.int16) if pk[n].dtype == np.uint16 else pk[n]) for n in
         ("k_pack", "k_params", "v_pack", "v_params")}
    back = lambda a: a.numpy().view(np.uint16) if a.dtype == torch.int16 else a.numpy()
    # batch shards
    got = []
    for r in range(2):
        q, kp, kprm, vp, vprm = S.shard_batch([x["q"], t["k_pack"], t["k_params"], t["v_pack"], t["v_params"]], r, 2)
        o, _ = O.decode_from_packed(q.numpy(), back(kp), back(kprm), back(vp), back(vprm), scale, 4, 128)
        got.append(o)
    assert np.allclose(np.concatenate(got, 0), full, atol=1e-6)
    # KV-head shards (query heads follow their KV head)
    got = []
    for r in range(2):
        q, kp, kprm, vp, vprm = S.shard_kv_heads(x["q"], t["k_pack"], t["k_params"], t["v_pack"], t["v_params"], r, 2)
        assert q.shape[2] == 4 and kp.shape[2] == 2 and vprm.shape[2] == 2
        o, _ = O.decode_from_packed(q.numpy(), back(kp), back(kprm), back(vp), back(vprm), scale, 4, 128)
        got.append(o)
    assert np.allclose(np.concatenate(got, 1), full, atol=1e-6)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _seq_split_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x = H.gen_qkv(1, 1024, 8, 2, seed=11, res=24)           # same seeded inputs on every rank
        pk = H.oracle_pack(x["k"], x["v"], 4, 128, "fp16")
        scale = 1.0 / math.sqrt(128)
        lo, hi = S.sequence_shard_bounds(1024, world, 4)[rank]
        kd, vd = O.dequantize(pk["logical"], 128)
        last = rank == world - 1                                  # the tail lives with the end of the sequence
        o, l = O.decode_attention(x["q"][:, 0].float().numpy(), kd[:, lo:hi], vd[:, lo:hi], scale,
                                  k_res=x["k_res"].float().numpy() if last else None,
                                  v_res=x["v_res"].float().numpy() if last else None)
        outs, lses = S.gather_partials(torch.from_numpy(o.astype(np.float32)), torch.from_numpy(l.astype(np.float32)))
        assert len(outs) == world and len(lses) == world
        merged, lse = O.combine_partials([t.numpy() for t in outs], [t.numpy() for t in lses])
        full, full_lse = O.decode_attention(x["q"][:, 0].float().numpy(), kd, vd, scale,
                                            k_res=x["k_res"].float().numpy(), v_res=x["v_res"].float().numpy())
        ret[rank] = (float(np.abs(merged - full).max()), float(np.abs(lse - full_lse).max()))
    finally:
        dist.destroy_process_group()


def test_sequence_split_merge_over_gloo():
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_seq_split_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        assert len(ret) == world
        for rank in range(world):
            derr, lerr = ret[rank]
            assert derr < 1e-6 and lerr < 1e-6, (rank, derr, lerr)
