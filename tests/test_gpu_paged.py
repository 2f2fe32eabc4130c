"""Paged KV cache (`opt_block_table`): pages of 256 or 512 tokens scattered over a pool, the
same kernels, against the oracle over the gathered sequences."""
import math

import numpy as np
import pytest
import torch

from tests import gpu_util as G, helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits,group,page,dtype", [(4, 128, 256, "fp16"), (2, 128, 512, "fp16"), (4, 64, 256, "bf16")])
def test_paged_pack_and_decode(bits, group, page, dtype):
    import bitladder_b200 as B

    b, h, h_k, pages_per_seq = 3, 16, 4, 5
    s = page * pages_per_seq
    x = H.gen_qkv(b, s, h, h_k, seed=61, dtype=dtype, res=48)
    num_pages = b * pages_per_seq + 3                     # a few pages of the pool stay unused
    g = torch.Generator().manual_seed(7)
    table = torch.randperm(num_pages, generator=g)[:b * pages_per_seq].reshape(b, pages_per_seq).to(torch.int32)
    tdt = x["k"].dtype
    k_pool = torch.zeros(num_pages, page, h_k, 128, dtype=tdt)
    v_pool = torch.zeros_like(k_pool)
    for ib in range(b):
        for i in range(pages_per_seq):
            k_pool[table[ib, i]] = x["k"][ib, i * page:(i + 1) * page]
            v_pool[table[ib, i]] = x["v"][ib, i * page:(i + 1) * page]
    bufs = B.alloc_packed_cache(num_pages, page, h_k, 128, bits, group, device="cuda")
    tab = table.cuda()
    B.kvcache_pack_int(k_pool.cuda(), bufs[0], bufs[1], v_pool.cuda(), bufs[2], bufs[3], tab, None, page,
                       "k-channel", group, bits)
    # the pool, gathered back into sequences, equals the contiguous pack bit for bit
    ref = H.oracle_pack(x["k"], x["v"], bits, group, dtype)
    pn = 16 // bits
    kp = H.u16(bufs[0]).reshape(num_pages, page // pn, h_k, 128)
    vp = H.u16(bufs[2]).reshape(num_pages, page, h_k, 128 // pn)
    idx = table.numpy().reshape(-1)
    assert np.array_equal(kp[idx].reshape(b, s // pn, h_k, 128), ref["k_pack"])
    assert np.array_equal(vp[idx].reshape(b, s, h_k, 128 // pn), ref["v_pack"])

    lens = torch.tensor([s, page + 37, 3 * page], dtype=torch.int32)
    res_lens = torch.tensor([48, 5, 0], dtype=torch.int32)
    out, lse = B.fwd_kvcache_int(x["q"].cuda(), *bufs, tab, H.default_scale(), "k-channel", group, bits,
                                 cache_seqlens=lens.cuda(), k_res=x["k_res"].cuda(), v_res=x["v_res"].cuda(),
                                 res_lens=res_lens.cuda(), return_lse=True)
    o_ref, l_ref = H.oracle_decode(x["q"], ref, H.default_scale(), bits, group, dtype, cache_seqlens=lens.numpy(),
                                   k_res=x["k_res"], v_res=x["v_res"], res_lens=res_lens.numpy())
    tol = 2e-3 if dtype == "fp16" else 1.6e-2
    assert np.abs(out.float().cpu().numpy()[:, 0] - o_ref).max() <= tol
    assert np.abs(lse.cpu().numpy() - l_ref).max() <= tol


def test_paged_argument_checks():
    import bitladder_b200 as B

    bufs = B.alloc_packed_cache(4, 128, 2, 128, 4, 128, device="cuda")      # 128-token pages: not allowed
    q = torch.zeros(2, 1, 4, 128, dtype=torch.float16, device="cuda")
    table = torch.zeros(2, 2, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError):
        B.fwd_kvcache_int(q, *bufs, table, 1.0, "k-channel", 128, 4)
    bufs = B.alloc_packed_cache(4, 256, 2, 128, 4, 128, device="cuda")
    with pytest.raises(RuntimeError):
        B.fwd_kvcache_int(q, *bufs, table.to(torch.int64), 1.0, "k-channel", 128, 4)
