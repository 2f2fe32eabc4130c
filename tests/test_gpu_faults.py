"""GPU: what the decode step does with inputs and conditions that must not turn into a fault.

Nothing here faults, traps or hangs a GPU: the wait that "runs out" is a bounded poll with a limit of
a few thousand iterations, after which the kernel writes a status word and returns normally; the bad
page index and the over-long tail length are clamped before they are used as addresses."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

from tests import gpu_util as G, helpers as H

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_the_workspace_is_reusable():
    """One warp of the first CTA expects 16 bytes more than its first copy delivers (test hook of the
    C-ABI), with a poll limit of 2000: the warp gives up after microseconds, keeps counting in so that
    every sequence still finds its last arrival, and the kernel returns with BD_ERR_TIMEOUT in the
    status word.  The counters are back at zero, and the next, normal call is right."""
    import bitladder_b200 as B
    from bitladder_b200 import _lib
    x = H.gen_qkv(4, 4096, 32, 8, seed=71, res=64)
    ref = H.oracle_pack(x["k"], x["v"], 4, 128, "fp16")
    bufs = G.pack_gpu(B, x["k"], x["v"], 4, 128)
    q = x["q"].cuda()
    kw = dict(k_res=x["k_res"].cuda(), v_res=x["v_res"].cuda())
    need = B.decode_workspace_bytes(q, *bufs, **kw)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    args = (q, *bufs, None, H.default_scale(), "k-channel", 128, 4)
    B.fwd_kvcache_int(*args, workspace=ws, spin_limit=2000, _test_starve=1, **kw)
    stream = torch.cuda.current_stream().cuda_stream
    assert _lib.load().bd_read_status(ws.data_ptr(), stream) == _lib.BD_ERR_TIMEOUT
    assert _lib.load().bd_read_status(ws.data_ptr(), stream) == 0           # reading clears the word
    counters = ws[16:16 + 4 * 4 * 8].view(torch.int32)                       # b * h_k arrival counters
    assert int(counters.abs().sum()) == 0
    with pytest.raises(RuntimeError, match="wait"):
        B.fwd_kvcache_int(*args, workspace=ws, spin_limit=2000, _test_starve=1, check=True, **kw)
    out, lse = B.fwd_kvcache_int(*args, workspace=ws, return_lse=True, check=True, **kw)
    o_ref, l_ref = H.oracle_decode(x["q"], ref, H.default_scale(), 4, 128, "fp16", k_res=x["k_res"], v_res=x["v_res"])
    eo, el = G.errs(out, lse, o_ref, l_ref)
    assert eo <= 2e-3 and el <= 2e-3


def test_decode_step_object_reports_the_status_too():
    import bitladder_b200 as B
    x = H.gen_qkv(2, 2048, 16, 4, seed=72)
    bufs = G.pack_gpu(B, x["k"], x["v"], 4, 128)
    bad = B.DecodeStep(x["q"].cuda(), *bufs, None, H.default_scale(), "k-channel", 128, 4, spin_limit=2000,
                       _test_starve=1)
    with pytest.raises(RuntimeError, match="wait"):
        bad.step(check=True)
    good = B.DecodeStep(x["q"].cuda(), *bufs, None, H.default_scale(), "k-channel", 128, 4)
    good.step(check=True)
    assert good.status() == 0


def test_a_page_index_outside_the_pool_is_masked_and_reported():
    """The last page of one sequence points outside the pool: its tokens are left out (the result
    equals the oracle over the sequence without that page), the status word says BD_ERR_PAGE, no
    address is formed from the bad index."""
    import bitladder_b200 as B
    from bitladder_b200 import _lib
    b, h, h_k, page, pages_per_seq = 2, 16, 4, 256, 4
    s = page * pages_per_seq
    x = H.gen_qkv(b, s, h, h_k, seed=73)
    ref = H.oracle_pack(x["k"], x["v"], 4, 128, "fp16")
    num_pages = b * pages_per_seq
    table = torch.arange(num_pages, dtype=torch.int32).reshape(b, pages_per_seq)
    k_pool = x["k"].reshape(num_pages, page, h_k, 128)
    v_pool = x["v"].reshape(num_pages, page, h_k, 128)
    bufs = B.alloc_packed_cache(num_pages, page, h_k, 128, 4, 128, device="cuda")
    B.kvcache_pack_int(k_pool.cuda(), bufs[0], bufs[1], v_pool.cuda(), bufs[2], bufs[3], table.cuda(), None, page,
                       "k-channel", 128, 4)
    for bad in (num_pages + 5, -3):
        t2 = table.clone()
        t2[1, pages_per_seq - 1] = bad
        q = x["q"].cuda()
        ws = torch.zeros(B.decode_workspace_bytes(q, *bufs, block_table=t2.cuda()), dtype=torch.uint8, device="cuda")
        out, lse = B.fwd_kvcache_int(q, *bufs, t2.cuda(), H.default_scale(), "k-channel", 128, 4, return_lse=True,
                                     workspace=ws)
        rc = _lib.load().bd_read_status(ws.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == _lib.BD_ERR_PAGE
        lens = np.array([s, s - page], dtype=np.int32)
        o_ref, l_ref = H.oracle_decode(x["q"], ref, H.default_scale(), 4, 128, "fp16", cache_seqlens=lens)
        eo, el = G.errs(out, lse, o_ref, l_ref)
        assert eo <= 2e-3 and el <= 2e-3


def test_tail_lengths_beyond_the_buffers_are_clamped():
    """res_lens[ib] larger than the rows the tail buffers hold: the kernel reads the rows there are."""
    import bitladder_b200 as B
    x = H.gen_qkv(3, 512, 8, 2, seed=74, res=40)
    ref = H.oracle_pack(x["k"], x["v"], 4, 128, "fp16")
    bufs = G.pack_gpu(B, x["k"], x["v"], 4, 128)
    rl = torch.tensor([40, 1000, 200], dtype=torch.int32)
    out, lse = B.fwd_kvcache_int(x["q"].cuda(), *bufs, None, H.default_scale(), "k-channel", 128, 4, return_lse=True,
                                 k_res=x["k_res"].cuda(), v_res=x["v_res"].cuda(), res_lens=rl.cuda(), check=True)
    o_ref, l_ref = H.oracle_decode(x["q"], ref, H.default_scale(), 4, 128, "fp16", k_res=x["k_res"], v_res=x["v_res"],
                                   res_lens=np.array([40, 40, 40], dtype=np.int32))
    eo, el = G.errs(out, lse, o_ref, l_ref)
    assert eo <= 2e-3 and el <= 2e-3
