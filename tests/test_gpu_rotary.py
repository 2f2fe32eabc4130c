"""GPU: rotary embedding of the appended token inside the decode step (the reference's dormant append path,
decode_api.cpp:316, 418; flash.h:149-151; rotary.h): the step must attend with the rotated query over the rotated new key and
file exactly the oracle's rotated key in the tail."""
import math

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import gpu_util as G, helpers as H

pytestmark = pytest.mark.gpu


def _tables(positions, half, tdt, seed):
    g = torch.Generator().manual_seed(seed)
    ang = torch.rand(positions, half, generator=g) * 6.2831853
    return torch.cos(ang).to(tdt), torch.sin(ang).to(tdt)


@pytest.mark.parametrize("dtype,rotary_dim,interleaved,advance", [("fp16", 128, True, False), ("fp16", 64, False, True),
                                                                  ("bf16", 32, True, True), ("bf16", 128, False, False)])
def test_step_with_rotary_equals_the_oracle_on_rotated_inputs(dtype, rotary_dim, interleaved, advance):
    import bitladder_b200 as B
    b, s, h, h_k, bits, group, res_cap = 3, 512, 8, 2, 4, 128, 128
    x = H.gen_qkv(b, s, h, h_k, seed=77, dtype=dtype, res=res_cap)
    tdt = x["q"].dtype
    scale = H.default_scale()
    seqlens = np.array([512, 384, 128], np.int32)
    res_lens = np.array([5, 0, 100], np.int32)
    cos, sin = _tables(1024, rotary_dim // 2, tdt, 3)
    g = torch.Generator().manual_seed(9)
    k_new = torch.randn(b, 1, h_k, 128, generator=g).to(tdt)
    v_new = torch.randn(b, 1, h_k, 128, generator=g).to(tdt)

    # oracle: rotate q and k_new at position cached + tail, append, decode
    pos = seqlens + res_lens
    q_rot = O.apply_rotary(H.to_np(x["q"])[:, 0], H.to_np(cos), H.to_np(sin), pos, interleaved, dtype)
    k_rot = O.apply_rotary(H.to_np(k_new)[:, 0], H.to_np(cos), H.to_np(sin), pos, interleaved, dtype)
    def back(a):
        t = torch.from_numpy(a)
        return t.view(torch.bfloat16) if dtype == "bf16" else t
    k_res = x["k_res"].clone(); v_res = x["v_res"].clone()
    for ib in range(b):
        k_res[ib, res_lens[ib]] = back(k_rot)[ib]
        v_res[ib, res_lens[ib]] = v_new[ib, 0]
    ref = H.oracle_pack(x["k"], x["v"], bits, group, dtype)
    o_ref, _ = H.oracle_decode(back(q_rot)[:, None], ref, scale, bits, group, dtype, cache_seqlens=seqlens,
                               k_res=k_res, v_res=v_res, res_lens=res_lens + 1)

    bufs = G.pack_gpu(B, x["k"], x["v"], bits, group)
    k_tail, v_tail = x["k_res"].cuda(), x["v_res"].cuda()
    cs, rl = torch.from_numpy(seqlens).cuda(), torch.from_numpy(res_lens).cuda()
    out = B.fwd_kvcache_int(x["q"].cuda(), *bufs, None, scale, "k-channel", group, bits, k_res=k_tail, v_res=v_tail,
                            res_lens=rl, cache_seqlens=cs, k_new=k_new.cuda(), v_new=v_new.cuda(), advance=advance,
                            rotary_cos=cos.cuda(), rotary_sin=sin.cuda(), rotary_interleaved=interleaved, check=True)
    tol = G.TOL_O[dtype]
    assert np.abs(out[:, 0].float().cpu().numpy() - o_ref).max() <= tol
    for ib in range(b):          # the filed key is the oracle's rotated key, bit for bit; the value as it came
        assert torch.equal(k_tail[ib, res_lens[ib]].cpu().view(torch.int16), back(k_rot)[ib].view(torch.int16))
        assert torch.equal(v_tail[ib, res_lens[ib]].cpu(), v_new[ib, 0])
    if advance:
        assert rl.cpu().tolist() == (res_lens + 1).tolist()


def test_a_position_beyond_the_tables_is_reported():
    import bitladder_b200 as B
    b, s, h, h_k = 1, 256, 4, 1
    x = H.gen_qkv(b, s, h, h_k, seed=78, res=64)
    bufs = G.pack_gpu(B, x["k"], x["v"], 4, 128)
    cos, sin = _tables(100, 64, torch.float16, 4)            # tables of 100 positions, the token sits at 256 + 3
    rl = torch.tensor([3], dtype=torch.int32, device="cuda")
    kw = dict(k_res=x["k_res"].cuda(), v_res=x["v_res"].cuda(), res_lens=rl, k_new=x["k"][:, :1].cuda(),
              v_new=x["v"][:, :1].cuda(), rotary_cos=cos.cuda(), rotary_sin=sin.cuda())
    with pytest.raises(RuntimeError, match="rotary"):
        B.fwd_kvcache_int(x["q"].cuda(), *bufs, None, 0.1, "k-channel", 128, 4, check=True, **kw)
    # and rotary without an appended token is refused on the host
    kw.pop("k_new"); kw.pop("v_new")
    with pytest.raises(RuntimeError):
        B.fwd_kvcache_int(x["q"].cuda(), *bufs, None, 0.1, "k-channel", 128, 4, **kw)


def test_positions_follow_the_device_side_lengths_in_a_captured_decoder_loop():
    """A decoder step with rotary captured once as a CUDA graph and replayed: the position of every new token
    comes from the lengths the device itself advances, across a roll-over of the tail."""
    from bitladder_b200.kv_cache import PackedKVCache
    b, h, h_k, bits, group, steps = 2, 4, 1, 4, 128, 40
    prompt = [100, 250]
    x = H.gen_qkv(b, 512, h, h_k, seed=81)
    cache = PackedKVCache(b, 1024, h_k, 128, bits, group, dtype=torch.float16, device="cuda")
    cache.prefill(x["k"][:, :256].cuda(), x["v"][:, :256].cuda(), seqlens=prompt)
    cos, sin = _tables(2048, 64, torch.float16, 5)
    q = torch.zeros(b, 1, h, 128, dtype=torch.float16, device="cuda")
    kn = torch.zeros(b, 1, h_k, 128, dtype=torch.float16, device="cuda")
    vn = torch.zeros_like(kn)
    step = cache.decoder_step(q, kn, vn, 0.1, rotary_cos=cos.cuda(), rotary_sin=sin.cuda(), rotary_interleaved=False)
    step.step()                                    # warm-up outside the capture, with zero rows: token 0
    torch.cuda.synchronize()
    gr = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side), torch.cuda.graph(gr, stream=side):
        step.step()
    torch.cuda.current_stream().wait_stream(side)
    g = torch.Generator().manual_seed(6)
    news = []
    for i in range(steps):
        k_i = torch.randn(b, 1, h_k, 128, generator=g).half()
        news.append(k_i)
        kn.copy_(k_i); vn.copy_(k_i); q.copy_(torch.randn(b, 1, h, 128, generator=g).half())
        gr.replay()
    assert step.status() == 0
    cache.note_steps(steps + 1)
    # sequence 0: 100 prompt tokens (tail 100) + warm-up token + 40 tokens: rolled over at 128, tail now 13 rows;
    # the last rows of the tail are the rotated tokens at positions 128 .. 140
    lens = [p + 1 + steps for p in prompt]
    assert cache.seqlens() == lens
    for ib in range(b):
        tail_n = lens[ib] % 128
        for r in range(max(0, tail_n - 5), tail_n):
            pos = lens[ib] - tail_n + r
            i = pos - prompt[ib] - 1                      # index into the replayed tokens
            want = O.apply_rotary(H.to_np(news[i])[ib:ib + 1, 0], H.to_np(cos), H.to_np(sin), [pos], False)
            got = cache.k_tail[ib, r].cpu().numpy()
            assert np.array_equal(got.view(np.uint16), want[0].view(np.uint16)), (ib, r, pos)
