"""GPU (one device): the cross-GPU exchange-and-merge kernel with the peer emulated on the same GPU.

Two exchange areas live on one device; the "other rank's" partial is published into this rank's area
from the host side (bd_exchange_put: copies and a flag), or by running the same kernel in the other
rank's role afterwards.  Kernels that wait on one another never run at the same time here: whatever a
launch waits for has been published before it starts, or is never published and the bounded wait runs
out (a flag that nothing sets), which is reported in the area's status word."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _areas(lib, world, rows):
    n = lib.bd_exchange_area_bytes(world, rows)
    ptrs = []
    for _ in range(world):
        p = C.c_void_p()
        assert lib.bd_peer_alloc(n, C.byref(p)) == 0
        ptrs.append(p.value)
    return ptrs


def _args(_lib, rank, ptrs, part, lse, out, rows, spin=0):
    arr = (C.c_void_p * len(ptrs))(*ptrs)
    a = _lib.ExchangeArgs(rank=rank, world=len(ptrs), areas=C.cast(arr, C.POINTER(C.c_void_p)), part_out=part.data_ptr(),
                          part_lse=lse.data_ptr(), rows=rows, d=128, out=out.data_ptr(), lse=None,
                          out_dtype=_lib.BD_FP32, spin_limit=spin)
    a._keep = arr
    return a


@pytest.mark.parametrize("world", [3, 8])
def test_exchange_merges_what_the_peers_published_over_three_steps(world):
    from bitladder_b200 import _lib
    lib = _lib.load()
    rows = 40
    ptrs = _areas(lib, world, rows)
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(5)
    try:
        for epoch in (1, 2, 3):
            parts = [torch.randn(rows, 128, generator=g, device="cuda") for _ in range(world)]
            lses = [torch.randn(rows, generator=g, device="cuda") * 3 for _ in range(world)]
            lses[1][7] = float("-inf")                              # a rank with no tokens for one row
            want, _ = O.combine_partials([p.cpu().numpy() for p in parts], [l.cpu().numpy() for l in lses])
            # The ranks run one after the other.  When rank k runs, the ranks before it have already stored
            # their rows into its area (their kernels ran); the ranks after it publish from the host side.
            for k in range(world):
                for r in range(k + 1, world):
                    assert lib.bd_exchange_put(ptrs[k], world, rows, r, epoch, parts[r].data_ptr(), lses[r].data_ptr(), stream) == 0
                out = torch.full((rows, 128), float("nan"), device="cuda")
                assert lib.bd_exchange_combine(C.byref(_args(_lib, k, ptrs, parts[k], lses[k], out, rows)), stream) == 0
                ep = C.c_uint32()
                assert lib.bd_exchange_state(ptrs[k], stream, C.byref(ep)) == 0 and ep.value == epoch
                assert np.abs(out.cpu().numpy() - want).max() <= 1e-5, (epoch, k)
    finally:
        torch.cuda.synchronize()
        for p in ptrs:
            lib.bd_peer_free(p)


@pytest.mark.parametrize("b,s,gq,ragged,world", [(1, 8192, 4, False, 2), (3, 2048, 8, True, 2), (2, 768, 1, False, 2),
                                                 (2, 4096, 4, False, 8), (1, 4096, 2, True, 16), (2, 1536, 4, False, 3)])
def test_decode_fused_with_the_exchange_equals_the_whole_sequence_on_one_gpu(b, s, gq, ragged, world):
    """bd_decode_exchange as rank 0 of `world`: the other ranks' rows (their shards of every sequence,
    decoded on the same GPU beforehand) are published into rank 0's area from the host side; rank 0's step
    decodes the first shard, merges its CTAs' parts, takes the peers' rows and must give the oracle's
    result for the whole sequence.  Two steps in a row (both slots of the area)."""
    import bitladder_b200 as B
    from bitladder_b200 import _lib
    from tests import gpu_util as G, helpers as H
    lib = _lib.load()
    h_k, bits, group = 2, 4, 128
    h = h_k * gq
    x = H.gen_qkv(b, s, h, h_k, seed=31 + b)
    scale = H.default_scale()
    shard = s // world
    assert shard % 128 == 0
    seqlens = None
    if ragged:
        seqlens = np.array([s, s - 700, shard + 1][:b], dtype=np.int32)
    ref = H.oracle_pack(x["k"], x["v"], bits, group, "fp16")
    o_ref, _ = H.oracle_decode(x["q"], ref, scale, bits, group, "fp16", cache_seqlens=seqlens)
    q = x["q"].cuda()
    rows = b * h
    ptrs = _areas(lib, world, rows)
    stream = torch.cuda.current_stream().cuda_stream
    try:
        peers = []
        step = None
        for r in range(world):
            lo, hi = r * shard, (r + 1) * shard
            bufs = G.pack_gpu(B, x["k"][:, lo:hi], x["v"][:, lo:hi], bits, group)
            kw = {}
            if ragged:
                kw = dict(cache_seqlens=torch.from_numpy(np.clip(seqlens - lo, 0, shard).astype(np.int32)).cuda())
            if r == 0:
                step = B.DecodeStep(q, *bufs, None, scale, "k-channel", group, bits, **kw)
            else:
                p, l = B.fwd_kvcache_int(q, *bufs, None, scale, "k-channel", group, bits, out_dtype=torch.float32,
                                         return_lse=True, **kw)
                peers.append((p.reshape(rows, 128).contiguous(), l.reshape(rows).contiguous()))
        arr = (C.c_void_p * world)(*ptrs)
        xa = _lib.ExchangeArgs(rank=0, world=world, areas=C.cast(arr, C.POINTER(C.c_void_p)), part_out=None,
                               part_lse=None, rows=rows, d=128, out=None, lse=None, out_dtype=_lib.BD_FP16, spin_limit=0)
        for epoch in (1, 2):
            for r, (p, l) in enumerate(peers, start=1):
                assert lib.bd_exchange_put(ptrs[0], world, rows, r, epoch, p.data_ptr(), l.data_ptr(), stream) == 0
            step.out.fill_(float("nan"))
            assert lib.bd_decode_exchange(step._ref, C.byref(xa), stream) == 0
            ep = C.c_uint32()
            assert lib.bd_exchange_state(ptrs[0], stream, C.byref(ep)) == 0 and ep.value == epoch
            err = np.abs(step.out[:, 0].float().cpu().numpy() - o_ref).max()
            assert err <= 2e-3, (epoch, err)
        assert step.status() == 0
        # wrong row count: refused before anything is launched
        xa.rows = rows + 1
        assert lib.bd_decode_exchange(step._ref, C.byref(xa), stream) == _lib.BD_ERR_INVALID
    finally:
        torch.cuda.synchronize()
        for p in ptrs:
            lib.bd_peer_free(p)


def test_a_peer_that_never_publishes_is_a_reported_timeout():
    from bitladder_b200 import _lib
    lib = _lib.load()
    world, rows = 2, 16
    ptrs = _areas(lib, world, rows)
    stream = torch.cuda.current_stream().cuda_stream
    try:
        part = torch.randn(rows, 128, device="cuda")
        lse = torch.randn(rows, device="cuda")
        out = torch.full((rows, 128), float("nan"), device="cuda")
        assert lib.bd_exchange_combine(C.byref(_args(_lib, 0, ptrs, part, lse, out, rows, spin=3000)), stream) == 0
        ep = C.c_uint32()
        assert lib.bd_exchange_state(ptrs[0], stream, C.byref(ep)) == _lib.BD_ERR_TIMEOUT
        assert lib.bd_exchange_state(ptrs[0], stream, C.byref(ep)) == 0           # cleared by the read
        assert torch.isnan(out).all()                                             # nothing was written
        assert ep.value == 1                                                      # the step still counts
    finally:
        torch.cuda.synchronize()
        for p in ptrs:
            lib.bd_peer_free(p)


def test_argument_checks():
    from bitladder_b200 import _lib
    lib = _lib.load()
    assert lib.bd_exchange_area_bytes(0, 8) == 0 and lib.bd_exchange_area_bytes(17, 8) == 0
    assert lib.bd_exchange_area_bytes(8, 64) > 2 * 8 * 64 * 129 * 4
    assert lib.bd_exchange_combine(None, None) == -1
