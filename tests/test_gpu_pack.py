"""GPU: quantize-pack must be bit-exact against the oracle (codes, scales, zeros)."""
import numpy as np
import pytest
import torch

from tests import gpu_util as G, helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits,group,dtype", [(4, 128, "fp16"), (2, 128, "fp16"), (4, 64, "fp16"),
                                              (2, 64, "fp16"), (4, 128, "bf16"), (2, 128, "bf16"),
                                              (4, 64, "bf16"), (2, 64, "bf16"), (4, 32, "fp16"),
                                              (2, 32, "fp16"), (4, 32, "bf16"), (2, 32, "bf16")])
def test_pack_bit_exact(bits, group, dtype):
    import bitladder_b200 as B
    x = H.gen_qkv(2, 1024, 8, 2, seed=11, dtype=dtype)
    G.assert_pack_equal(G.pack_gpu(B, x["k"], x["v"], bits, group), H.oracle_pack(x["k"], x["v"], bits, group, dtype))


@pytest.mark.parametrize("bits,group", [(4, 128), (2, 64), (4, 32), (2, 32)])
def test_pack_edge_values(bits, group):
    """All-zero and constant groups (scale 0), fp16 max, huge and tiny magnitudes, outlier channels."""
    import bitladder_b200 as B
    x = H.gen_qkv(1, 512, 4, 4, seed=13, outlier_frac=0.05)
    k, v = x["k"].clone(), x["v"].clone()
    k[0, :256, 0, 3] = 0.0
    k[0, :, 1, 7] = 2.5
    k[0, 5, 2, 9] = 65504.0
    k[0, 6, 2, 9] = -65504.0
    k[0, :, 3, :] *= 6e-5                      # near the fp16 subnormal range
    v[0, 17, 0, :] = 0.0
    v[0, 18, 1, :] = -1.0
    v[0, 19, 2, :64] = 100.0
    G.assert_pack_equal(G.pack_gpu(B, k, v, bits, group), H.oracle_pack(k, v, bits, group, "fp16"))


def test_pack_strided_inputs_and_offset():
    """Non-contiguous K/V views (as slices of a larger cache) and packing block by block at an offset."""
    import bitladder_b200 as B
    x = H.gen_qkv(2, 512, 4, 2, seed=17)
    ref = H.oracle_pack(x["k"], x["v"], 4, 128, "fp16")
    big_k = torch.zeros(2, 512, 3, 256, dtype=torch.float16, device="cuda")
    big_v = torch.zeros_like(big_k)
    big_k[:, :, 1:3, 64:192] = x["k"].cuda()
    big_v[:, :, 1:3, 64:192] = x["v"].cuda()
    kview, vview = big_k[:, :, 1:3, 64:192], big_v[:, :, 1:3, 64:192]
    bufs = B.alloc_packed_cache(2, 512, 2, 128, 4, 128, device="cuda")
    for start in (0, 128, 256, 384):           # one pack block at a time, as a growing cache would
        B.kvcache_pack_int(kview[:, start:start + 128], bufs[0], bufs[1], vview[:, start:start + 128], bufs[2],
                           bufs[3], None, None, 128, "k-channel", 128, 4, dst_token_offset=start)
    torch.cuda.synchronize()
    G.assert_pack_equal(bufs, ref)


def test_pack_reference_call_convention():
    """Positional call exactly as the reference's evaluation script makes it (evaluation/test.py:87-96),
    including the cu_seqlens tensor it passes and the uint16 / float32 buffer dtypes."""
    import bitladder_b200 as B
    b, s, h_k, d = 1, 4096, 8, 128
    x = H.gen_qkv(b, s, 32, h_k, seed=0)
    k_pack = torch.zeros((b, s // 4, h_k, d), dtype=torch.uint16, device="cuda")
    k_params = torch.zeros((b, s // 128, h_k, d), dtype=torch.float32, device="cuda")
    v_pack = torch.zeros((b, s, h_k, d // 4), dtype=torch.uint16, device="cuda")
    v_params = torch.zeros((b, d // 128, h_k, s), dtype=torch.float32, device="cuda")
    cu = torch.arange(0, (b + 1) * s, s, dtype=torch.int32, device="cuda")
    B.kvcache_pack_int(x["k"].cuda(), k_pack, k_params, x["v"].cuda(), v_pack, v_params, None, cu, s,
                       "k-channel", 128, 4)
    torch.cuda.synchronize()
    G.assert_pack_equal((k_pack, k_params, v_pack, v_params), H.oracle_pack(x["k"], x["v"], 4, 128, "fp16"))
