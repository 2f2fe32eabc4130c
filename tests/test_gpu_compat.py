"""GPU: the reference's extension-module interface (``bit_decode_cuda``) served by this library, driven
with the call sequence of the reference's evaluation script (``evaluation/test.py:76-108`` through
``bit_decode/bit_decode_interface.py:19-83``): flattened K/V, caller-allocated buffers, fifteen
positional arguments on the decode call."""
import math

import numpy as np
import pytest
import torch

from tests import gpu_util as G, helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("num_bits,group_size,h,h_k", [(4, 128, 32, 32), (4, 32, 32, 8), (2, 128, 32, 8)])
def test_evaluation_script_call_sequence(num_bits, group_size, h, h_k):
    import bitladder_b200.compat as compat
    bit_decode_cuda = compat.install()
    pack = bit_decode_cuda.kvcache_pack_i4 if num_bits == 4 else bit_decode_cuda.kvcache_pack_i2
    fwd = bit_decode_cuda.fwd_kvcache_i4 if num_bits == 4 else bit_decode_cuda.fwd_kvcache_i2
    batch_size, seqlen_kv, d = 1, 4096, 128
    pack_nums = 16 // num_bits
    x = H.gen_qkv(batch_size, seqlen_kv, h, h_k, seed=0)
    q, k_cache, v_cache = x["q"].cuda(), x["k"].cuda(), x["v"].cuda()
    k_pack = torch.zeros((batch_size, seqlen_kv // pack_nums, h_k, d), dtype=torch.uint16, device="cuda")
    k_params = torch.zeros((batch_size, seqlen_kv // group_size, h_k, d), dtype=torch.float32, device="cuda")
    v_pack = torch.zeros((batch_size, seqlen_kv, h_k, d // pack_nums), dtype=torch.uint16, device="cuda")
    v_params = torch.zeros((batch_size, d // group_size, h_k, seqlen_kv), dtype=torch.float32, device="cuda")
    cu_seqlens_k = torch.arange(0, (batch_size + 1) * seqlen_kv, seqlen_kv, dtype=torch.int32, device="cuda")
    pack(k_cache.reshape(batch_size * seqlen_kv, h_k, d), k_pack, k_params,
         v_cache.reshape(batch_size * seqlen_kv, h_k, d), v_pack, v_params, None, cu_seqlens_k, seqlen_kv,
         "k-channel", group_size)
    sm_scale = 1.0 / math.sqrt(d)
    out = fwd(q, k_pack, k_params, v_pack, v_params, None, sm_scale, "k-channel", group_size,
              False, -1, -1, 0.0, True, 0)
    torch.cuda.synchronize()
    assert out.shape == (batch_size, 1, h, d) and out.dtype == torch.float16
    ref = H.oracle_pack(x["k"], x["v"], num_bits, group_size, "fp16")
    G.assert_pack_equal((k_pack, k_params, v_pack, v_params), ref)
    o_ref, _ = H.oracle_decode(x["q"], ref, sm_scale, num_bits, group_size, "fp16")
    assert np.abs(out[:, 0].float().cpu().numpy() - o_ref).max() <= 2e-3


def test_arguments_the_library_cannot_honour_raise():
    import bitladder_b200.compat as compat
    m = compat.install()
    q = torch.zeros(1, 1, 8, 128, dtype=torch.float16, device="cuda")
    import bitladder_b200 as B
    bufs = B.alloc_packed_cache(1, 256, 2, 128, 4, 128, device="cuda")
    with pytest.raises(RuntimeError, match="window"):
        m.fwd_kvcache_i4(q, *bufs, None, 1.0, "k-channel", 128, False, 128, -1, 0.0, True, 0)
    with pytest.raises(RuntimeError, match="softcap"):
        m.fwd_kvcache_i4(q, *bufs, None, 1.0, "k-channel", 128, False, -1, -1, 30.0, True, 0)
    with pytest.raises(RuntimeError, match="quant_mode"):
        m.fwd_kvcache_i4(q, *bufs, None, 1.0, "k-tensor", 128, False, -1, -1, 0.0, True, 0)
