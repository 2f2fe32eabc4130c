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
            packed = list(cache._packed)          # append(): a full tail is packed lazily, at the next append;
            tails = [n - p for n, p in zip(lens, packed)]      # append_and_decode(): at once, on the device
            assert all((0 <= t < nb) if fused else (0 < t <= nb) for t in tails)
            if fused:      # the step attended over the tail as it was BEFORE the roll-over, plus the new token
                packed = [p - nb if t == 0 else p for p, t in zip(packed, tails)]
                tails = [nb if t == 0 else t for t in tails]
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


@pytest.mark.parametrize("bits,group,dtype", [(4, 128, "fp16"), (2, 64, "bf16"), (4, 32, "fp16")])
def test_decoder_step_as_a_cuda_graph_rolls_tails_over_on_the_device(bits, group, dtype):
    """The whole decoder step (attend over the new token, file it, pack a tail that filled up, move the
    lengths on) captured ONCE in a CUDA graph and replayed for 300 tokens with fresh q / k_new / v_new in the
    same buffers: no host logic between steps.  Afterwards the lengths on the device are what the history
    says, the packed blocks equal a plain quantize-pack of the same rows bit for bit, and outputs taken
    along the way match the oracle."""
    import bitladder_b200 as B
    from bitladder_b200.kv_cache import PackedKVCache

    b, h, h_k, steps = 3, 8, 2, 300
    nb = 32 * (16 // bits)
    prompt = [5, nb - 2, 2 * nb + 17]
    total = max(prompt) + steps + nb
    x = H.gen_qkv(b, total, h, h_k, seed=43, dtype=dtype)
    tdt = x["k"].dtype
    cache = PackedKVCache(b, total, h_k, 128, bits, group, dtype=tdt, device="cuda")
    s0 = max(prompt)
    cache.prefill(x["k"][:, :s0].cuda(), x["v"][:, :s0].cuda(), seqlens=prompt)
    hist_k = torch.zeros(b, total + nb, h_k, 128, dtype=tdt)
    hist_v = torch.zeros_like(hist_k)
    lens = list(prompt)
    for ib in range(b):
        hist_k[ib, :lens[ib]] = x["k"][ib, :lens[ib]]
        hist_v[ib, :lens[ib]] = x["v"][ib, :lens[ib]]
    q_buf = torch.zeros(b, 1, h, 128, dtype=tdt, device="cuda")
    k_buf = torch.zeros(b, 1, h_k, 128, dtype=tdt, device="cuda")
    v_buf = torch.zeros_like(k_buf)
    step = cache.decoder_step(q_buf, k_buf, v_buf, 1.0 / math.sqrt(128))
    # warm up outside the capture on a clone of the state?  Not needed: the first launch is the capture's replay.
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            step.step()
    torch.cuda.current_stream().wait_stream(side)
    g = torch.Generator().manual_seed(6)
    tol = 2e-3 if dtype == "fp16" else 1.6e-2
    check_at = {0, 1, nb - 3, nb - 2, nb - 1, nb, 2 * nb - 1, 2 * nb, steps - 1}
    for i in range(steps):
        k_new = torch.randn(b, 1, h_k, 128, generator=g).to(tdt)
        v_new = torch.randn(b, 1, h_k, 128, generator=g).to(tdt)
        q = torch.randn(b, 1, h, 128, generator=g).to(tdt)
        q_buf.copy_(q); k_buf.copy_(k_new); v_buf.copy_(v_new)
        before = [(n // nb * nb, n % nb) for n in lens]          # (packed, tail) the step starts from
        graph.replay()
        for ib in range(b):
            hist_k[ib, lens[ib]] = k_new[ib, 0]
            hist_v[ib, lens[ib]] = v_new[ib, 0]
            lens[ib] += 1
        if i in check_at:
            ref = _oracle_step(hist_k, hist_v, q, [p for p, _ in before], [t + 1 for _, t in before], bits, group, dtype)
            err = np.abs(step.out.float().cpu().numpy()[:, 0] - ref).max()
            assert err <= tol, (i, err)
    assert step.status() == 0
    cache.sync_lengths()
    assert cache.seqlens() == lens
    assert cache._packed == [n // nb * nb for n in lens] and cache._tail == [n % nb for n in lens]
    # every packed block, rolled over on the device one at a time, equals a plain pack of the same rows
    for ib in range(b):
        n = lens[ib] // nb * nb
        ref = H.oracle_pack(hist_k[ib:ib + 1, :n], hist_v[ib:ib + 1, :n], bits, group, dtype)
        P = 16 // bits
        assert np.array_equal(H.u16(cache.k_pack[ib:ib + 1, :n // P]), ref["k_pack"])
        assert np.array_equal(H.u16(cache.v_pack[ib:ib + 1, :n]), ref["v_pack"])
        assert np.array_equal(H.f32_as_u16(cache.k_params[ib:ib + 1, :n // group]), ref["k_params"].view(np.uint16))
        assert np.array_equal(H.f32_as_u16(cache.v_params[ib:ib + 1, :, :, :n]), ref["v_params"].view(np.uint16))


def test_a_full_cache_is_reported_not_overrun():
    """advance with no room for the tail's block: the status word says so and nothing is written past the end."""
    import bitladder_b200 as B
    from bitladder_b200 import _lib
    b, h, h_k, nb = 1, 8, 2, 128
    x = H.gen_qkv(b, 2 * nb, h, h_k, seed=44)
    bufs = B.alloc_packed_cache(b, nb, h_k, 128, 4, 128, device="cuda")          # room for ONE block
    B.kvcache_pack_int(x["k"][:, :nb].cuda(), bufs[0], bufs[1], x["v"][:, :nb].cuda(), bufs[2], bufs[3], None, None, nb,
                       "k-channel", 128, 4)
    k_tail = x["k"][:, nb:2 * nb].cuda().clone()
    v_tail = x["v"][:, nb:2 * nb].cuda().clone()
    cs = torch.tensor([nb], dtype=torch.int32, device="cuda")
    rl = torch.tensor([nb - 1], dtype=torch.int32, device="cuda")              # this step's token fills the tail
    q = x["q"].cuda()
    ws = torch.zeros(B.decode_workspace_bytes(q, *bufs, k_res=k_tail, v_res=v_tail, res_lens=rl, cache_seqlens=cs),
                     dtype=torch.uint8, device="cuda")
    before = [t.clone() for t in bufs]
    B.fwd_kvcache_int(q, *bufs, None, H.default_scale(), "k-channel", 128, 4, k_res=k_tail, v_res=v_tail, res_lens=rl,
                      cache_seqlens=cs, k_new=x["k"][:, -1:].cuda(), v_new=x["v"][:, -1:].cuda(), advance=True,
                      workspace=ws)
    assert _lib.load().bd_read_status(ws.data_ptr(), torch.cuda.current_stream().cuda_stream) == _lib.BD_ERR_CAPACITY
    assert int(cs[0]) == nb and int(rl[0]) == nb                                # lengths: the tail stays full
    assert all(torch.equal(a, b_) for a, b_ in zip(before, bufs))
