"""CPU: the oracle against known answers, against its independent C restatement and
against the committed golden fixtures."""
import math

import numpy as np
import pytest

from oracle import c_oracle, oracle as O
from tests import helpers as H


def f16(x):
    return np.asarray(x, dtype=np.float16)


# ---------------------------------------------------------------------------
# known-answer cases of the quantizer formula (qpack.h:241-281), worked by hand
# ---------------------------------------------------------------------------
def test_kat_unit_scale_ties_round_away_from_zero():
    # min 0, max 15 -> scale_inv = 15/15 = 1: codes are roundf(x); .5 goes AWAY from zero
    x = np.zeros(128, np.float32)
    x[:8] = [0.0, 0.5, 1.5, 2.5, 14.5, 15.0, 7.49, 7.51]
    codes, scale, zero = O._quantize_lastaxis(x[None], 4)
    assert codes[0, :8].tolist() == [0, 1, 2, 3, 15, 15, 7, 8]     # banker's rounding would give 0, 2, 2, 14
    assert scale[0] == np.float16(1.0) and zero[0] == np.float16(0.0)


def test_kat_constant_group_has_zero_scale():
    x = np.full((1, 128), -3.25, np.float32)
    codes, scale, zero = O._quantize_lastaxis(x, 4)
    assert not codes.any() and scale[0] == 0 and zero[0] == np.float16(-3.25)


def test_kat_asymmetric_range_2bit():
    # min -1, max 2 -> range 3, scale_inv = 3/3 = 1, stored scale 1, zero -1
    x = np.full(128, -1.0, np.float32)
    x[:5] = [-1.0, -0.4, 0.5, 1.49, 2.0]
    codes, scale, zero = O._quantize_lastaxis(x[None], 2)
    assert codes[0, :5].tolist() == [0, 1, 2, 2, 3]                # (x+1) = 0, .6, 1.5, 2.49, 3
    assert scale[0] == np.float16(1.0) and zero[0] == np.float16(-1.0)


def test_kat_scale_is_fp32_reciprocal_rounded_to_fp16():
    # range 1 -> scale_inv = 15, stored scale = fp16(1/15 computed in fp32)
    x = np.zeros(128, np.float32)
    x[1] = 1.0
    _, scale, _ = O._quantize_lastaxis(x[None], 4)
    assert scale[0] == np.float16(np.float32(1.0) / np.float32(15.0))


def test_kat_field_order_low_index_first():
    # K word [p][c]: field j = token p + 32 j; V word [t][p]: field j = dim p + 32 j (4-bit)
    kc = np.zeros((1, 128, 1, 128), np.uint8)
    kc[0, 0, 0, 0], kc[0, 32, 0, 0], kc[0, 64, 0, 0], kc[0, 96, 0, 0] = 1, 2, 3, 4
    assert O.pack_k(kc, 4)[0, 0, 0, 0] == 0x4321
    vc = np.zeros((1, 1, 1, 128), np.uint8)
    vc[0, 0, 0, 0], vc[0, 0, 0, 32], vc[0, 0, 0, 64], vc[0, 0, 0, 96] = 5, 6, 7, 8
    assert O.pack_v(vc, 4)[0, 0, 0, 0] == 0x8765
    kc2 = np.zeros((1, 256, 1, 128), np.uint8)
    for j in range(8):
        kc2[0, 7 + 32 * j, 0, 3] = j % 4
    assert O.pack_k(kc2, 2)[0, 7, 0, 3] == sum((j % 4) << (2 * j) for j in range(8))


def test_kat_dequant_is_one_rounding():
    # code*scale + zero rounded ONCE to fp16 (the reference's __hfma2): 15 * 0.1 - 1.3
    s, z = np.float16(0.1), np.float16(-1.3)
    logical = dict(k_codes=np.full((1, 128, 1, 128), 15, np.uint8), k_scale=np.full((1, 1, 1, 128), s),
                   k_zero=np.full((1, 1, 1, 128), z), v_codes=np.zeros((1, 128, 1, 128), np.uint8),
                   v_scale=np.zeros((1, 128, 1, 1), np.float16), v_zero=np.zeros((1, 128, 1, 1), np.float16))
    k, _ = O.dequantize(logical, 128)
    exact = 15.0 * float(s) + float(z)
    assert k[0, 0, 0, 0] == np.float32(np.float16(exact))
    two_roundings = np.float16(np.float16(15.0 * float(s)) + z)
    assert two_roundings != np.float16(exact)            # the case really distinguishes the two


def test_kat_attention_uniform_scores():
    # q = 0 -> uniform softmax: out = mean of V, lse = log(n)
    q = np.zeros((1, 2, 128), np.float32)
    k = np.random.default_rng(0).standard_normal((1, 64, 1, 128)).astype(np.float32)
    v = np.random.default_rng(1).standard_normal((1, 64, 1, 128)).astype(np.float32)
    out, lse = O.decode_attention(q, k, v, 0.1)
    assert np.allclose(out[0, 0], v[0, :, 0].mean(axis=0)) and np.allclose(lse, math.log(64))


def test_combine_matches_unsplit():
    rng = np.random.default_rng(2)
    q = rng.standard_normal((1, 4, 128)).astype(np.float32)
    k = rng.standard_normal((1, 96, 2, 128)).astype(np.float32)
    v = rng.standard_normal((1, 96, 2, 128)).astype(np.float32)
    full, lse = O.decode_attention(q, k, v, 0.09)
    parts = [O.decode_attention(q, k[:, a:b], v[:, a:b], 0.09) for a, b in ((0, 32), (32, 32), (32, 96))]
    out, l2 = O.combine_partials([p[0] for p in parts], [p[1] for p in parts])
    assert np.allclose(out, full, atol=1e-12) and np.allclose(l2, lse, atol=1e-12)


# ---------------------------------------------------------------------------
# numpy oracle == C oracle, bit for bit on the packed buffers
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("bits,group,dtype", [(4, 128, "fp16"), (2, 128, "fp16"), (4, 64, "fp16"),
                                              (2, 64, "fp16"), (4, 128, "bf16"), (2, 64, "bf16")])
def test_numpy_and_c_oracles_agree(bits, group, dtype):
    x = H.gen_qkv(2, 512, 8, 2, seed=1, dtype=dtype, res=40)
    a = H.oracle_pack(x["k"], x["v"], bits, group, dtype)
    c = c_oracle.quantize_pack(H.to_np(x["k"]), H.to_np(x["v"]), bits, group, dtype)
    for n in ("k_pack", "k_params", "v_pack", "v_params"):
        assert np.array_equal(a[n].view(np.uint16), c[n].view(np.uint16)), n
    assert np.array_equal(O.unpack_k(a["k_pack"], bits), a["logical"]["k_codes"])
    assert np.array_equal(O.unpack_v(a["v_pack"], bits), a["logical"]["v_codes"])
    cs = np.array([512, 130], np.int32)
    rl = np.array([40, 7], np.int32)
    sc = H.default_scale()
    o1, l1 = H.oracle_decode(x["q"], a, sc, bits, group, dtype, cs, x["k_res"], x["v_res"], rl, use_c=False)
    o2, l2 = H.oracle_decode(x["q"], a, sc, bits, group, dtype, cs, x["k_res"], x["v_res"], rl, use_c=True)
    assert np.abs(o1 - o2).max() < 1e-6 and np.abs(l1 - l2).max() < 1e-6


def test_edge_values_zero_group_and_outliers():
    x = H.gen_qkv(1, 256, 4, 1, seed=3)
    k = x["k"].clone()
    k[0, :128, 0, 5] = 0.0                  # an all-zero group
    k[0, :, 0, 9] *= 1000.0                 # a large-magnitude channel
    k[0, 3, 0, 11] = 65504.0                # fp16 max inside a group
    a = H.oracle_pack(k, x["v"], 4, 128, "fp16")
    c = c_oracle.quantize_pack(H.to_np(k), H.to_np(x["v"]), 4, 128, "fp16")
    for n in ("k_pack", "k_params", "v_pack", "v_params"):
        assert np.array_equal(a[n].view(np.uint16), c[n].view(np.uint16)), n
    ks, kz = O.unpack_k_params(a["k_params"])
    assert ks[0, 0, 0, 5] == 0 and kz[0, 0, 0, 5] == 0


# ---------------------------------------------------------------------------
# golden fixtures
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("name", sorted(H.load_golden()))
def test_golden_fixtures_both_oracles(name):
    case = H.load_golden()[name]
    cfg = case["cfg"]
    k, v, q = H.golden_input(case, "k"), H.golden_input(case, "v"), H.golden_input(case, "q")
    for impl in (lambda: O.quantize_pack(k, v, cfg["bits"], cfg["group"], cfg["dtype"]),
                 lambda: c_oracle.quantize_pack(k, v, cfg["bits"], cfg["group"], cfg["dtype"])):
        got = impl()
        for n in ("k_pack", "k_params", "v_pack", "v_params"):
            assert np.array_equal(got[n].view(np.uint16), case[n]), (name, n)
    kw = dict(cache_seqlens=case.get("cache_seqlens"), k_res=H.golden_input(case, "k_res"),
              v_res=H.golden_input(case, "v_res"), res_lens=case.get("res_lens"))
    args = (q, case["k_pack"], case["k_params"].view(np.float32), case["v_pack"], case["v_params"].view(np.float32),
            1.0 / math.sqrt(128), cfg["bits"], cfg["group"], cfg["dtype"])
    for fn in (O.decode_from_packed, c_oracle.decode):
        out, lse = fn(*args, **kw)
        assert np.abs(out - case["out"]).max() < 1e-5 and np.abs(lse - case["lse"]).max() < 1e-5


def test_statistical_anchor_of_the_reference():
    """The reference records mean|out - fp16 attention| = 0.002773 for b1, 32/32 heads, s4096, 4-bit g128
    (benchmark/bench_single_decode.ipynb:92).  Other RNG stream here, so the match is statistical."""
    x = H.gen_qkv(1, 4096, 32, 32, seed=0)
    a = c_oracle.quantize_pack(H.to_np(x["k"]), H.to_np(x["v"]), 4, 128, "fp16")
    sc = H.default_scale()
    out, _ = c_oracle.decode(H.to_np(x["q"]), a["k_pack"], a["k_params"], a["v_pack"], a["v_params"], sc, 4, 128)
    ref, _ = O.decode_attention(x["q"][:, 0].float().numpy(), x["k"].float().numpy(), x["v"].float().numpy(), sc)
    mae = np.abs(out.astype(np.float16).astype(np.float64) - ref.astype(np.float16).astype(np.float64)).mean()
    assert 0.0022 < mae < 0.0034, mae
