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


def test_exchange_merges_what_the_peers_published_over_three_steps():
    from bitladder_b200 import _lib
    lib = _lib.load()
    world, rows = 3, 40
    ptrs = _areas(lib, world, rows)
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(5)
    try:
        for epoch in (1, 2, 3):
            parts = [torch.randn(rows, 128, generator=g, device="cuda") for _ in range(world)]
            lses = [torch.randn(rows, generator=g, device="cuda") * 3 for _ in range(world)]
            lses[1][7] = float("-inf")                              # a rank with no tokens for one row
            want, _ = O.combine_partials([p.cpu().numpy() for p in parts], [l.cpu().numpy() for l in lses])
            # ranks 1 and 2 publish into rank 0's area from the host side; then rank 0's kernel runs
            for r in (1, 2):
                assert lib.bd_exchange_put(ptrs[0], world, rows, r, epoch, parts[r].data_ptr(), lses[r].data_ptr(), stream) == 0
            outs = [torch.full((rows, 128), float("nan"), device="cuda") for _ in range(world)]
            assert lib.bd_exchange_combine(C.byref(_args(_lib, 0, ptrs, parts[0], lses[0], outs[0], rows)), stream) == 0
            ep = C.c_uint32()
            assert lib.bd_exchange_state(ptrs[0], stream, C.byref(ep)) == 0 and ep.value == epoch
            assert np.abs(outs[0].cpu().numpy() - want).max() <= 1e-5
            # rank 1 in turn: rank 0's kernel has stored its partial into area 1, rank 2's comes from the host
            assert lib.bd_exchange_put(ptrs[1], world, rows, 2, epoch, parts[2].data_ptr(), lses[2].data_ptr(), stream) == 0
            assert lib.bd_exchange_combine(C.byref(_args(_lib, 1, ptrs, parts[1], lses[1], outs[1], rows)), stream) == 0
            assert lib.bd_exchange_state(ptrs[1], stream, C.byref(ep)) == 0 and ep.value == epoch
            assert np.abs(outs[1].cpu().numpy() - want).max() <= 1e-5
            # rank 2: both peers' kernels have published to it
            assert lib.bd_exchange_combine(C.byref(_args(_lib, 2, ptrs, parts[2], lses[2], outs[2], rows)), stream) == 0
            assert lib.bd_exchange_state(ptrs[2], stream, C.byref(ep)) == 0 and ep.value == epoch
            assert np.abs(outs[2].cpu().numpy() - want).max() <= 1e-5
    finally:
        torch.cuda.synchronize()
        for p in ptrs:
            lib.bd_peer_free(p)


@pytest.mark.parametrize("b,s,gq,ragged", [(1, 8192, 4, False), (3, 2048, 8, True), (2, 768, 1, False)])
def test_decode_fused_with_the_exchange_equals_the_whole_sequence_on_one_gpu(b, s, gq, ragged):
    """bd_decode_exchange as rank 0 of two: rank 1's rows (the second half of every sequence, decoded on
    the same GPU beforehand) are published into rank 0's area from the host side; rank 0's step decodes
    the first half, merges its CTAs' parts, takes the peer's rows and must give the oracle's result for
    the whole sequence.  Two steps in a row (both slots of the area)."""
    import bitladder_b200 as B
    from bitladder_b200 import _lib
    from tests import gpu_util as G, helpers as H
    lib = _lib.load()
    h_k, bits, group = 2, 4, 128
    h = h_k * gq
    x = H.gen_qkv(b, s, h, h_k, seed=31 + b)
    scale = H.default_scale()
    half = s // 2
    seqlens = None
    if ragged:
        seqlens = np.array([s, s - 700, half + 1][:b], dtype=np.int32)
    ref = H.oracle_pack(x["k"], x["v"], bits, group, "fp16")
    o_ref, _ = H.oracle_decode(x["q"], ref, scale, bits, group, "fp16", cache_seqlens=seqlens)
    q = x["q"].cuda()
    lo = G.pack_gpu(B, x["k"][:, :half], x["v"][:, :half], bits, group)
    hi = G.pack_gpu(B, x["k"][:, half:], x["v"][:, half:], bits, group)
    kw_lo, kw_hi = {}, {}
    if ragged:
        kw_lo = dict(cache_seqlens=torch.from_numpy(np.minimum(seqlens, half)).cuda())
        kw_hi = dict(cache_seqlens=torch.from_numpy(np.maximum(seqlens - half, 0)).cuda())
    rows = b * h
    ptrs = _areas(lib, 2, rows)
    stream = torch.cuda.current_stream().cuda_stream
    try:
        p1, l1 = B.fwd_kvcache_int(q, *hi, None, scale, "k-channel", group, bits, out_dtype=torch.float32,
                                   return_lse=True, **kw_hi)
        p1 = p1.reshape(rows, 128).contiguous()
        l1 = l1.reshape(rows).contiguous()
        step = B.DecodeStep(q, *lo, None, scale, "k-channel", group, bits, **kw_lo)
        arr = (C.c_void_p * 2)(*ptrs)
        xa = _lib.ExchangeArgs(rank=0, world=2, areas=C.cast(arr, C.POINTER(C.c_void_p)), part_out=None, part_lse=None,
                               rows=rows, d=128, out=None, lse=None, out_dtype=_lib.BD_FP16, spin_limit=0)
        for epoch in (1, 2):
            assert lib.bd_exchange_put(ptrs[0], 2, rows, 1, epoch, p1.data_ptr(), l1.data_ptr(), stream) == 0
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
