"""bd_decode_noalloc: the decode entry point for callers that cannot allocate.

A serving runtime that has given all free device memory to its KV-cache pool, or a
plugin host that forbids allocation after start-up, cannot hand bd_decode a
workspace.  bd_decode_noalloc keeps the scratch in a fixed area inside the library
instead.  These tests call it through the C-ABI (ctypes, raw pointers) and compare
with bd_decode on the same inputs, twice in a row and with a shape change in
between, because the area is shared and keeps the previous call's contents.

The file name sorts last on purpose: a run that stops at the first failure has
then already been through every other test.
"""
import ctypes as C
import math

import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _decode_both(B, x, bufs, bits, group, with_tail, cache_seqlens=None, res_lens=None):
    """Runs bd_decode (caller workspace) and bd_decode_noalloc on the same arguments."""
    from bitladder_b200 import _lib, bit_decode_interface as I

    lib = _lib.load()
    q = x["q"].cuda()
    kw = {}
    if with_tail:
        kw = dict(k_res=x["k_res"].cuda(), v_res=x["v_res"].cuda())
    cs = None if cache_seqlens is None else cache_seqlens.cuda()
    rl = None if res_lens is None else res_lens.cuda()
    outs = []
    for entry in ("bd_decode", "bd_decode_noalloc"):
        out = torch.full_like(q, float("nan"))
        lse = torch.full((q.shape[0], q.shape[2]), float("nan"), dtype=torch.float32, device="cuda")
        a = I._decode_args(q, *bufs, 1.0 / math.sqrt(128), group, bits, kw.get("k_res"), kw.get("v_res"),
                           rl, cs, None, out, lse, 0)
        stream = torch.cuda.current_stream().cuda_stream
        if entry == "bd_decode":
            need = lib.bd_decode_workspace_bytes(C.byref(a))
            ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
            a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
            rc = lib.bd_decode(C.byref(a), stream)
        else:
            a.workspace, a.workspace_bytes = None, 0          # ignored by this entry point
            rc = lib.bd_decode_noalloc(C.byref(a), stream)
        assert rc == 0, _lib.strerror(rc)
        torch.cuda.synchronize()
        if entry == "bd_decode_noalloc":                      # the fixed area's status word: no error
            assert lib.bd_read_status(None, stream) == 0
        outs.append((out.float().cpu().numpy(), lse.cpu().numpy()))
    return outs


def _check(B, b, s, h, h_k, bits, group, res, seed):
    x = H.gen_qkv(b, s, h, h_k, seed=seed, res=res)
    bufs = B.alloc_packed_cache(b, s, h_k, 128, bits, group, device="cuda")
    B.kvcache_pack_int(x["k"].cuda(), bufs[0], bufs[1], x["v"].cuda(), bufs[2], bufs[3], None, None, s,
                       "k-channel", group, bits)
    (o_ws, l_ws), (o_na, l_na) = _decode_both(B, x, bufs, bits, group, res > 0)
    assert np.isfinite(o_na).all() and np.isfinite(l_na).all()
    # same kernels on the same inputs: the tolerance of the parity tests is ample
    assert np.abs(o_na - o_ws).max() <= 2e-3
    assert np.abs(l_na - l_ws).max() <= 2e-3
    # and both sit within the parity bound of the CPU oracle
    ref = H.oracle_pack(x["k"], x["v"], bits, group, "fp16")
    o_ref, _ = H.oracle_decode(x["q"], ref, 1.0 / math.sqrt(128), bits, group, "fp16",
                               k_res=x.get("k_res"), v_res=x.get("v_res"))
    assert np.abs(o_na[:, 0] - o_ref).max() <= 2e-3


def test_noalloc_matches_workspace_entry_point_twice_in_a_row():
    import bitladder_b200 as B
    _check(B, 2, 4096, 32, 8, 4, 128, 64, seed=21)
    _check(B, 2, 4096, 32, 8, 4, 128, 64, seed=22)      # second call: the area holds the first call's partials


def test_noalloc_survives_a_shape_change():
    import bitladder_b200 as B
    _check(B, 4, 2048, 8, 8, 2, 128, 0, seed=23)        # other batch / head count: counters sit elsewhere
    _check(B, 2, 4096, 32, 8, 4, 128, 64, seed=21)


def test_noalloc_rejects_calls_beyond_the_fixed_area():
    import bitladder_b200 as B
    from bitladder_b200 import _lib, bit_decode_interface as I

    lib = _lib.load()
    limit = lib.bd_noalloc_scratch_bytes()
    b, s, h, h_k = 512, 128, 64, 64                      # many (sequence, head) pairs: large partial area
    q = torch.zeros(b, 1, h, 128, dtype=torch.float16, device="cuda")
    bufs = B.alloc_packed_cache(b, s, h_k, 128, 4, 128, device="cuda")
    out = torch.empty_like(q)
    a = I._decode_args(q, *bufs, 1.0, 128, 4, None, None, None, None, None, out, None, 0)
    assert lib.bd_decode_workspace_bytes(C.byref(a)) > limit
    rc = lib.bd_decode_noalloc(C.byref(a), torch.cuda.current_stream().cuda_stream)
    assert rc == -8 and "scratch" in _lib.strerror(rc)


def test_noalloc_with_per_sequence_lengths():
    """Ragged batch: the per-sequence unit table also lives in the fixed area."""
    import bitladder_b200 as B
    b, s, h, h_k, res = 5, 2048, 16, 4, 48
    x = H.gen_qkv(b, s, h, h_k, seed=24, res=res)
    bufs = B.alloc_packed_cache(b, s, h_k, 128, 4, 128, device="cuda")
    B.kvcache_pack_int(x["k"].cuda(), bufs[0], bufs[1], x["v"].cuda(), bufs[2], bufs[3], None, None, s,
                       "k-channel", 128, 4)
    cs = torch.tensor([0, 2048, 1000, 129, 1], dtype=torch.int32)
    rl = torch.tensor([48, 0, 7, 48, 0], dtype=torch.int32)
    for _ in range(2):
        (o_ws, l_ws), (o_na, l_na) = _decode_both(B, x, bufs, 4, 128, True, cs, rl)
        assert np.abs(o_na - o_ws).max() <= 2e-3
        assert np.abs(l_na - l_ws).max() <= 2e-3
    ref = H.oracle_pack(x["k"], x["v"], 4, 128, "fp16")
    o_ref, _ = H.oracle_decode(x["q"], ref, 1.0 / math.sqrt(128), 4, 128, "fp16", cache_seqlens=cs.numpy(),
                               k_res=x["k_res"], v_res=x["v_res"], res_lens=rl.numpy())
    assert np.abs(o_na[:, 0] - o_ref).max() <= 2e-3


def test_noalloc_keeps_an_error_code_until_it_is_read():
    """A step whose bounded wait runs out (test hook, poll limit 2000) leaves BD_ERR_TIMEOUT in the fixed
    area; the next call does not erase it; bd_read_status(NULL, stream) returns and clears it."""
    import bitladder_b200 as B
    from bitladder_b200 import _lib, bit_decode_interface as I
    lib = _lib.load()
    x = H.gen_qkv(2, 2048, 16, 4, seed=25)
    bufs = B.alloc_packed_cache(2, 2048, 4, 128, 4, 128, device="cuda")
    B.kvcache_pack_int(x["k"].cuda(), bufs[0], bufs[1], x["v"].cuda(), bufs[2], bufs[3], None, None, 2048,
                       "k-channel", 128, 4)
    q = x["q"].cuda()
    out = torch.empty_like(q)
    stream = torch.cuda.current_stream().cuda_stream
    a = I._decode_args(q, *bufs, 1.0 / math.sqrt(128), 128, 4, None, None, None, None, None, out, None, 0,
                       spin_limit=2000, test_starve=1)
    assert lib.bd_decode_noalloc(C.byref(a), stream) == 0
    a = I._decode_args(q, *bufs, 1.0 / math.sqrt(128), 128, 4, None, None, None, None, None, out, None, 0)
    assert lib.bd_decode_noalloc(C.byref(a), stream) == 0
    assert lib.bd_read_status(None, stream) == _lib.BD_ERR_TIMEOUT
    assert lib.bd_read_status(None, stream) == 0
    assert lib.bd_decode_noalloc(C.byref(a), stream) == 0
    torch.cuda.synchronize()
    ref = H.oracle_pack(x["k"], x["v"], 4, 128, "fp16")
    o_ref, _ = H.oracle_decode(x["q"], ref, 1.0 / math.sqrt(128), 4, 128, "fp16")
    assert np.abs(out[:, 0].float().cpu().numpy() - o_ref).max() <= 2e-3
