"""CPU: the oracle against what the reference's own CUDA kernels wrote (tests/golden/ref_i4.npz).

The fixtures come from the reference's quantize-pack and split-KV decode kernels compiled for sm_100a
(oracle/build_ref.py) and run on a B200 (tests/golden/make_ref_golden.py), 4-bit, group 128 and 32,
once built as the reference ships (``--use_fast_math``, key ``fast``) and once without that flag
(key ``ieee``).  These tests pin the CPU restatement to those bytes."""
import math

import numpy as np
import pytest

from oracle import c_oracle, oracle as O
from tests import helpers as H

KEYS = ("k_pack", "k_params", "v_pack", "v_params")


def _oracle_packs(case, use_c):
    fn = c_oracle.quantize_pack if use_c else O.quantize_pack
    return fn(case["k"].numpy(), case["v"].numpy(), 4, case["cfg"]["group"], "fp16")


@pytest.mark.parametrize("name", H.REF_STORED)
@pytest.mark.parametrize("use_c", [False, True])
def test_packed_bytes_equal_the_reference_built_without_fast_math(name, use_c):
    case = H.load_ref_case(name)
    pk = _oracle_packs(case, use_c)
    for key in KEYS:
        ref = case["blob"][f"{name}/ieee/{key}"]
        mine = pk[key].view(np.uint16).reshape(ref.shape)
        if key.endswith("params"):
            assert H.params_equal(mine, ref), key
        else:
            assert np.array_equal(mine, ref), key


@pytest.mark.parametrize("name", H.REF_HASHED)
def test_packed_bytes_of_the_larger_shapes_by_hash(name):
    """evaluation/test.py's own shape (b1, 32/32 heads, 4096 tokens) and two GQA shapes: every byte of
    the four buffers, compared through SHA-256 (the inputs are regenerated from the seed)."""
    case = H.load_ref_case(name)
    if case["k"] is None:
        pytest.skip("this torch build draws different random numbers than the one that made the fixtures")
    pk = _oracle_packs(case, True)
    for key in KEYS:
        assert np.array_equal(case["sha"](pk[key].view(np.uint16)), case["blob"][f"{name}/ieee/{key}_sha"]), key


@pytest.mark.parametrize("name", H.REF_STORED)
def test_fast_math_build_differs_only_at_exact_rounding_ties(name):
    """The reference as shipped divides with the GPU's approximate reciprocal.  Its scales and zeros
    still equal the IEEE ones; its codes differ from them only where (x - min) * 15 / range is exactly
    k + 0.5, by one step, and only a few times in 10^5."""
    case = H.load_ref_case(name)
    g = case["cfg"]["group"]
    blob = case["blob"]
    for key in ("k_params", "v_params"):
        assert H.params_equal(blob[f"{name}/fast/{key}"], blob[f"{name}/ieee/{key}"])
    k = case["k"].numpy().astype(np.float64)
    v = case["v"].numpy().astype(np.float64)
    b, s, h, d = k.shape
    kg = k.reshape(b, s // g, g, h, d)
    k_true = (kg - kg.min(2, keepdims=True)) * 15.0 / np.maximum(kg.max(2, keepdims=True) - kg.min(2, keepdims=True), 1e-30)
    vg = v.reshape(b, s, h, d // g, g)
    v_true = (vg - vg.min(4, keepdims=True)) * 15.0 / np.maximum(vg.max(4, keepdims=True) - vg.min(4, keepdims=True), 1e-30)
    for pack_key, unpack, true in (("k_pack", O.unpack_k, k_true.reshape(b, s, h, d)),
                                   ("v_pack", O.unpack_v, v_true.reshape(b, s, h, d))):
        fast = unpack(blob[f"{name}/fast/{pack_key}"], 4).astype(np.int32)
        ieee = unpack(blob[f"{name}/ieee/{pack_key}"], 4).astype(np.int32)
        diff = fast != ieee
        assert diff.sum() <= 2e-4 * diff.size + 4
        assert np.all(np.abs(fast - ieee)[diff] == 1)
        frac = true[diff] - np.floor(true[diff])
        assert np.all(frac == 0.5), "a code moved where the exact value is not a tie"


def _group_errors(o, ref, h_k):
    """max |o - ref| per (sequence, KV head)."""
    b, h, d = o.shape
    return np.abs(o - ref).reshape(b, h_k, (h // h_k) * d).max(axis=2)


@pytest.mark.parametrize("name", ("mha_g128",) + H.REF_HASHED)
def test_decode_oracle_against_the_reference_decode_kernel(name):
    """Dequantize-then-attention on the oracle's packed bytes (equal to the reference's) against the
    output of the reference's split-KV kernel, IEEE build.  The reference returns fp16: 1e-4 of |out|
    up to 0.3 is its own rounding.

    llama_g128 (b2, 32q/8kv, 2048 tokens): the reference's result for ONE (sequence, KV head) pair is
    the right attention output times 0.91-0.92 (all four query heads, every dim, residual 4e-5) in the
    IEEE build's run and not in the fast-math build's run of the same inputs: one of its sixteen splits
    is empty there and its split combine weighs something that was never written.  Not reproducible
    arithmetic, so that case asks for all pairs but one."""
    case = H.load_ref_case(name)
    if case["k"] is None:
        pytest.skip("this torch build draws different random numbers than the one that made the fixtures")
    cfg = case["cfg"]
    pk = _oracle_packs(case, True)
    o, _ = c_oracle.decode(case["q"].numpy(), pk["k_pack"], pk["k_params"], pk["v_pack"], pk["v_params"],
                           1.0 / math.sqrt(128), 4, cfg["group"])
    ref = case["blob"][f"{name}/ieee/out"].view(np.float16).astype(np.float64)[:, 0]
    err = _group_errors(o, ref, cfg["h_k"])
    bad = int((err > 3e-4).sum())
    print(name, "max err", err.max(), "pairs over 3e-4:", bad, "of", err.size)
    assert bad <= (1 if name == "llama_g128" else 0)
