"""`DecodeStep`: the prepared step must do exactly what `fwd_kvcache_int` does, call after call,
while the contents of its tensors change."""
import math

import pytest
import torch

from tests import gpu_util as G, helpers as H

pytestmark = pytest.mark.gpu


def test_prepared_step_equals_the_plain_call_and_follows_content_changes():
    import bitladder_b200 as B
    x = H.gen_qkv(3, 2048, 32, 8, seed=17, res=32)
    bufs = G.pack_gpu(B, x["k"], x["v"], 4, 128)
    q = x["q"].cuda()
    k_res, v_res = x["k_res"].cuda(), x["v_res"].cuda()
    res_lens = torch.tensor([32, 7, 0], dtype=torch.int32, device="cuda")
    lens = torch.tensor([2048, 1000, 128], dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(128)
    run = B.DecodeStep(q, *bufs, None, scale, "k-channel", 128, 4, k_res=k_res, v_res=v_res, res_lens=res_lens,
                       cache_seqlens=lens, return_lse=True)
    for it in range(3):
        o_ref, l_ref = B.fwd_kvcache_int(q, *bufs, None, scale, "k-channel", 128, 4, k_res=k_res, v_res=v_res,
                                         res_lens=res_lens, cache_seqlens=lens, return_lse=True)
        o, l = run.step()
        assert torch.equal(o, o_ref) and torch.equal(l, l_ref)
        # new contents in the same buffers: the prepared step must see them
        q.copy_(torch.randn_like(q))
        res_lens.copy_(torch.tensor([5 + it, 32, 1], dtype=torch.int32))
        lens.copy_(torch.tensor([1024, 2048 - 128 * it, 0], dtype=torch.int32))
