"""The growing cache (`PackedKVCache`): prefill, token-by-token append with tails that fill up
and get packed, decode after every kind of step, against the CPU oracle over the same history."""
import math

import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _oracle_step(hist_k, hist_v, q, packed_lens, tail_lens, bits, group, dtype):
    b = hist_k.shape[0]
    nb = 32 * (16 // bits)
    cap = max(max(packed_lens), nb)
    pk = H.oracle_pack(hist_k[:, :cap], hist_v[:, :cap], bits, group, dtype)
    tmax = max(max(tail_lens), 1)
    k_res = torch.zeros(b, tmax, *hist_k.shape[2:], dtype=hist_k.dtype)
    v_res = torch.zeros_like(k_res)
    for ib in range(b):
        p, t = packed_lens[ib], tail_lens[ib]
        k_res[ib, :t] = hist_k[ib, p:p + t]
        v_res[ib, :t] = hist_v[ib, p:p + t]
    out, _ = H.oracle_decode(q, pk, 1.0 / math.sqrt(128), bits, group, dtype,
                             cache_seqlens=np.array(packed_lens, np.int32), k_res=k_res, v_res=v_res,
                             res_lens=np.array(tail_lens, np.int32))
    return out


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("bits,group,dtype,prompt", [(4, 128, "fp16", [200, 130]), (2, 128, "bf16", [300, 512]),
                                                      (4, 64, "fp16", [0, 127])])
def test_cache_grows_across_block_boundaries(bits, group, dtype, prompt, fused):
    """fused=False: append (copies) then decode; fused=True: one launch per step that attends over the
    new token and stores it in the tail (`append_and_decode`)."""
    from bitladder_b200.kv_cache import PackedKVCache

    b, h, h_k, steps = 2, 8, 2, 140
    nb = 32 * (16 // bits)
    total = max(prompt) + steps + nb
    x = H.gen_qkv(b, total, h, h_k, seed=41, dtype=dtype)
    tdt = x["k"].dtype
    cache = PackedKVCache(b, total, h_k, 128, bits, group, dtype=tdt, device="cuda")
    s0 = max(prompt)
    cache.prefill(x["k"][:, :s0].cuda(), x["v"][:, :s0].cuda(), seqlens=prompt)
    # each sequence's history: its prompt, then the appended tokens
    hist_k = torch.zeros(b, total + nb, h_k, 128, dtype=tdt)
    hist_v = torch.zeros_like(hist_k)
    lens = list(prompt)
    for ib in range(b):
        hist_k[ib, :lens[ib]] = x["k"][ib, :lens[ib]]
        hist_v[ib, :lens[ib]] = x["v"][ib, :lens[ib]]
    g = torch.Generator().manual_seed(5)
    tol = 2e-3 if dtype == "fp16" else 1.6e-2
    check_at = {0, 1, 2, 55, 56, 57, 58, 125, 126, 127, 128, 129, steps - 1}
    for step in range(steps):
        k_new = torch.randn(b, 1, h_k, 128, generator=g).to(tdt)
        v_new = torch.randn(b, 1, h_k, 128, generator=g).to(tdt)
        q = torch.randn(b, 1, h, 128, generator=g).to(tdt)
        if fused:
            out = cache.append_and_decode(q.cuda(), k_new.cuda(), v_new.cuda(), 1.0 / math.sqrt(128))
        else:
            cache.append(k_new.cuda(), v_new.cuda())
        for ib in range(b):
            hist_k[ib, lens[ib]] = k_new[ib, 0]
            hist_v[ib, lens[ib]] = v_new[ib, 0]
            lens[ib] += 1
        assert cache.seqlens() == lens
        if step in check_at:
            if not fused:
                out = cache.decode(q.cuda(), 1.0 / math.sqrt(128))
            packed = list(cache._packed)          # a full tail is packed lazily, at the next append
            tails = [n - p for n, p in zip(lens, packed)]
            assert all(0 < t <= nb for t in tails)
            ref = _oracle_step(hist_k, hist_v, q, packed, tails, bits, group, dtype)
            err = np.abs(out.float().cpu().numpy()[:, 0] - ref).max()
            assert err <= tol, (step, err)
    # the tails hold exactly the tokens that were appended since the last roll-over
    for ib in range(b):
        p_, t_ = cache._packed[ib], cache._tail[ib]
        assert torch.equal(cache.k_tail[ib, :t_].cpu(), hist_k[ib, p_:p_ + t_])
        assert torch.equal(cache.v_tail[ib, :t_].cpu(), hist_v[ib, p_:p_ + t_])


def test_cache_rejects_bad_calls():
    from bitladder_b200.kv_cache import PackedKVCache

    cache = PackedKVCache(2, 256, 2, 128, 4, 128, device="cuda")
    with pytest.raises(RuntimeError):
        cache.append(torch.zeros(2, 2, 2, 128, dtype=torch.float16, device="cuda"),
                     torch.zeros(2, 2, 2, 128, dtype=torch.float16, device="cuda"))
    with pytest.raises(RuntimeError):
        cache.prefill(torch.zeros(2, 512, 2, 128, dtype=torch.float16, device="cuda"),
                      torch.zeros(2, 512, 2, 128, dtype=torch.float16, device="cuda"))
