"""GPU: the committed golden fixtures (tests/golden) through the public entry points."""
import math

import numpy as np
import pytest
import torch

from tests import gpu_util as G, helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", sorted(H.load_golden()))
def test_golden_fixture(name):
    import bitladder_b200 as B
    case = H.load_golden()[name]
    cfg = case["cfg"]
    k, v, q = (H.golden_torch(case, n) for n in ("k", "v", "q"))
    bufs = G.pack_gpu(B, k, v, cfg["bits"], cfg["group"])
    ref = dict(k_pack=case["k_pack"], v_pack=case["v_pack"], k_params=case["k_params"], v_params=case["v_params"])
    G.assert_pack_equal(bufs, ref)
    kw = {}
    if "k_res" in case:
        kw.update(k_res=H.golden_torch(case, "k_res", "cuda"), v_res=H.golden_torch(case, "v_res", "cuda"))
    if "cache_seqlens" in case:
        kw["cache_seqlens"] = torch.from_numpy(case["cache_seqlens"]).cuda()
    if "res_lens" in case:
        kw["res_lens"] = torch.from_numpy(case["res_lens"]).cuda()
    out, lse = B.fwd_kvcache_int(q.cuda(), *bufs, None, 1.0 / math.sqrt(128), "k-channel", cfg["group"], cfg["bits"],
                                 return_lse=True, **kw)
    eo, el = G.errs(out, lse, case["out"].astype(np.float64), case["lse"].astype(np.float64))
    tol = G.tol_o(cfg["dtype"], case["out"])
    assert eo <= tol and el <= 2 * tol, (name, eo, el, tol)
