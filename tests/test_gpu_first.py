"""First GPU parity checks: quantize-pack bit-exact, decode within 2e-3 of the oracle."""
import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _pack_gpu(B, k, v, bits, group):
    b, s, h_k, d = k.shape
    bufs = B.alloc_packed_cache(b, s, h_k, d, bits, group, device="cuda")
    B.kvcache_pack_int(k.cuda(), bufs[0], bufs[1], v.cuda(), bufs[2], bufs[3], None, None, s,
                       "k-channel", group, bits)
    torch.cuda.synchronize()
    return bufs


@pytest.mark.parametrize("bits,group,dtype", [(4, 128, "fp16"), (2, 128, "fp16"), (4, 64, "fp16"),
                                              (2, 64, "fp16"), (4, 128, "bf16"), (2, 64, "bf16")])
def test_pack_bit_exact(bits, group, dtype):
    import bitladder_b200 as B
    x = H.gen_qkv(2, 1024, 8, 2, seed=11, dtype=dtype)
    ref = H.oracle_pack(x["k"], x["v"], bits, group, dtype)
    kp, kprm, vp, vprm = _pack_gpu(B, x["k"], x["v"], bits, group)
    assert np.array_equal(H.u16(kp), ref["k_pack"])
    assert np.array_equal(H.u16(vp), ref["v_pack"])
    assert np.array_equal(H.f32_as_u16(kprm), ref["k_params"].view(np.uint16))
    assert np.array_equal(H.f32_as_u16(vprm), ref["v_params"].view(np.uint16))


@pytest.mark.parametrize("bits,group,h,h_k,s,splits", [
    (4, 128, 32, 8, 4096, 0), (4, 128, 32, 8, 1024, 1), (4, 128, 8, 8, 512, 2),
    (2, 128, 32, 8, 2048, 0), (4, 64, 32, 8, 1024, 0), (2, 64, 32, 8, 2048, 0),
    (4, 128, 64, 8, 1024, 0), (4, 128, 32, 2, 1024, 0),
])
def test_decode_matches_oracle(bits, group, h, h_k, s, splits):
    import bitladder_b200 as B
    x = H.gen_qkv(2, s, h, h_k, seed=5)
    ref = H.oracle_pack(x["k"], x["v"], bits, group, "fp16")
    bufs = _pack_gpu(B, x["k"], x["v"], bits, group)
    scale = H.default_scale()
    out, lse = B.fwd_kvcache_int(x["q"].cuda(), *bufs, None, scale, "k-channel", group, bits,
                                 return_lse=True, num_splits=splits)
    torch.cuda.synchronize()
    o_ref, l_ref = H.oracle_decode(x["q"], ref, scale, bits, group, "fp16")
    err = np.abs(out[:, 0].float().cpu().numpy().astype(np.float64) - o_ref).max()
    lerr = np.abs(lse.cpu().numpy().astype(np.float64) - l_ref).max()
    print(f"max|dO|={err:.3e} max|dLSE|={lerr:.3e}")
    assert err <= 2e-3, err
    assert lerr <= 2e-3, lerr


@pytest.mark.parametrize("bits,group,dtype,h,h_k,s,res,ragged", [
    (4, 128, "fp16", 32, 8, 1024, 64, False),
    (4, 128, "fp16", 32, 8, 2048, 37, True),
    (4, 128, "bf16", 32, 32, 1024, 127, True),
    (2, 64, "fp16", 32, 8, 2048, 200, True),
    (2, 128, "bf16", 64, 8, 1024, 16, False),
    (4, 64, "fp16", 16, 1, 4096, 256, True),
])
def test_decode_tail_and_ragged(bits, group, dtype, h, h_k, s, res, ragged):
    import bitladder_b200 as B
    b = 5
    x = H.gen_qkv(b, s, h, h_k, seed=9, dtype=dtype, res=res)
    ref = H.oracle_pack(x["k"], x["v"], bits, group, dtype)
    bufs = _pack_gpu(B, x["k"], x["v"], bits, group)
    scale = H.default_scale()
    kw = dict(k_res=x["k_res"].cuda(), v_res=x["v_res"].cuda())
    cs = rl = None
    if ragged:
        g = torch.Generator().manual_seed(3)
        cs = torch.randint(0, s + 1, (b,), generator=g, dtype=torch.int32)
        cs[0] = 0                      # a sequence with only a tail
        cs[1] = s                      # a full one
        rl = torch.randint(0, res + 1, (b,), generator=g, dtype=torch.int32)
        rl[0] = res
        rl[2] = 0
        kw.update(cache_seqlens=cs.cuda(), res_lens=rl.cuda())
    out, lse = B.fwd_kvcache_int(x["q"].cuda(), *bufs, None, scale, "k-channel", group, bits,
                                 return_lse=True, **kw)
    torch.cuda.synchronize()
    o_ref, l_ref = H.oracle_decode(x["q"], ref, scale, bits, group, dtype,
                                   cache_seqlens=None if cs is None else cs.numpy(),
                                   k_res=x["k_res"], v_res=x["v_res"],
                                   res_lens=None if rl is None else rl.numpy())
    err = np.abs(out[:, 0].float().cpu().numpy().astype(np.float64) - o_ref).max()
    lerr = np.abs(lse.cpu().numpy().astype(np.float64) - l_ref).max()
    tol = 2e-3 if dtype == "fp16" else 1.6e-2
    print(f"max|dO|={err:.3e} max|dLSE|={lerr:.3e}")
    assert err <= tol, err
    assert lerr <= (2e-3 if dtype == "fp16" else 1.6e-2), lerr
