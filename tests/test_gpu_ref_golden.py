"""GPU: the CUDA path against what the reference's own kernels wrote on a B200
(tests/golden/ref_i4.npz, see tests/golden/make_ref_golden.py): packed bytes bit for bit, decode
output within the stated 2e-3."""
import math

import numpy as np
import pytest
import torch

from oracle import c_oracle
from tests import gpu_util as G, helpers as H

pytestmark = pytest.mark.gpu
KEYS = ("k_pack", "k_params", "v_pack", "v_params")


def _pack(B, case, fast):
    cfg = case["cfg"]
    bufs = B.alloc_packed_cache(cfg["b"], cfg["s"], cfg["h_k"], 128, 4, cfg["group"], device="cuda")
    B.kvcache_pack_int(case["k"].cuda(), bufs[0], bufs[1], case["v"].cuda(), bufs[2], bufs[3], None, None, cfg["s"],
                       "k-channel", cfg["group"], 4, reference_fast_math=fast)
    torch.cuda.synchronize()
    return bufs


def _bytes(bufs):
    return dict(k_pack=H.u16(bufs[0]), k_params=H.f32_as_u16(bufs[1]), v_pack=H.u16(bufs[2]),
                v_params=H.f32_as_u16(bufs[3]))


@pytest.mark.parametrize("name", H.REF_STORED + H.REF_HASHED)
@pytest.mark.parametrize("variant", ["ieee", "fast"])
def test_pack_writes_the_reference_kernels_bytes(name, variant):
    """Default division against the reference built without --use_fast_math, reference_fast_math=True
    against the reference as shipped: every byte of the four buffers (group 128 and group 32)."""
    import bitladder_b200 as B
    case = H.load_ref_case(name)
    if case["k"] is None:
        pytest.skip("this torch build draws different random numbers than the one that made the fixtures")
    got = _bytes(_pack(B, case, fast=(variant == "fast")))
    blob = case["blob"]
    for key in KEYS:
        if f"{name}/{variant}/{key}" in blob.files:
            ref = blob[f"{name}/{variant}/{key}"]
            mine = got[key].reshape(ref.shape)
            if key.endswith("params"):
                assert H.params_equal(mine, ref), key
            else:
                assert np.array_equal(mine, ref), key
        elif not case["cfg"]["crafted"]:
            assert np.array_equal(case["sha"](got[key]), blob[f"{name}/{variant}/{key}_sha"]), key


def _group_errors(o, ref, h_k):
    b, h, d = o.shape
    return np.abs(o - ref).reshape(b, h_k, (h // h_k) * d).max(axis=2)


@pytest.mark.parametrize("name", ("mha_g128",) + H.REF_HASHED)
@pytest.mark.parametrize("variant", ["ieee", "fast"])
def test_decode_against_the_reference_decode_kernel(name, variant):
    """fwd_kvcache_int over the bytes the reference's pack kernel wrote, against the output of the
    reference's split-KV decode kernel on those bytes (fp16), per (sequence, KV head).

    One pair of the IEEE run of llama_g128 is off in the REFERENCE (its result there is the right
    output times 0.91-0.92: an empty split weighs in its combine; the fast-math run of the same
    inputs does not show it), so that case asks for all pairs but one."""
    import bitladder_b200 as B
    case = H.load_ref_case(name)
    if case["k"] is None:
        pytest.skip("this torch build draws different random numbers than the one that made the fixtures")
    cfg, blob = case["cfg"], case["blob"]
    bufs = _pack(B, case, fast=(variant == "fast"))
    out, lse = B.fwd_kvcache_int(case["q"].cuda(), *bufs, None, 1.0 / math.sqrt(128), "k-channel", cfg["group"], 4,
                                 return_lse=True, check=True)
    o = out[:, 0].float().cpu().numpy().astype(np.float64)
    ref = blob[f"{name}/{variant}/out"].view(np.float16).astype(np.float64)[:, 0]
    err = _group_errors(o, ref, cfg["h_k"])
    bad = int((err > 2e-3).sum())
    print(f"{name}/{variant}: max|dO| vs reference kernel {np.sort(err.ravel())[-2 if name == 'llama_g128' else -1]:.2e}"
          f" (pairs over 2e-3: {bad} of {err.size})")
    assert bad <= (1 if name == "llama_g128" else 0)
    # and the oracle on the same bytes
    pk = _bytes(bufs)
    o_ref, l_ref = c_oracle.decode(case["q"].numpy(), pk["k_pack"], pk["k_params"].view(np.float32),
                                   pk["v_pack"], pk["v_params"].view(np.float32), 1.0 / math.sqrt(128), 4, cfg["group"])
    eo, el = G.errs(out, lse, o_ref, l_ref)
    print(f"   vs oracle: max|dO|={eo:.2e} max|dLSE|={el:.2e}")
    assert eo <= 2e-3 and el <= 2e-3
