"""Helpers shared by the GPU parity tests (device side goes through the public entry points,
which cross the C-ABI with raw pointers)."""
import numpy as np
import torch

from tests import helpers as H


def pack_gpu(B, k, v, bits, group, device="cuda"):
    b, s, h_k, d = k.shape
    bufs = B.alloc_packed_cache(b, s, h_k, d, bits, group, device=device)
    B.kvcache_pack_int(k.to(device), bufs[0], bufs[1], v.to(device), bufs[2], bufs[3], None, None, s,
                       "k-channel", group, bits)
    torch.cuda.synchronize()
    return bufs


def assert_pack_equal(bufs, ref):
    kp, kprm, vp, vprm = bufs
    assert np.array_equal(H.u16(kp), ref["k_pack"]), "K codes differ"
    assert np.array_equal(H.u16(vp), ref["v_pack"]), "V codes differ"
    assert np.array_equal(H.f32_as_u16(kprm), ref["k_params"].view(np.uint16)), "K scales/zeros differ"
    assert np.array_equal(H.f32_as_u16(vprm), ref["v_params"].view(np.uint16)), "V scales/zeros differ"


def errs(out, lse, o_ref, l_ref):
    o = out[:, 0].float().cpu().numpy().astype(np.float64)
    l = lse.cpu().numpy().astype(np.float64)
    both_inf = np.isinf(l) & np.isinf(l_ref) & (np.sign(l) == np.sign(l_ref))
    ldiff = np.where(both_inf, 0.0, np.abs(l - l_ref))
    return float(np.abs(o - o_ref).max()), float(np.nanmax(ldiff))


TOL_O = {"fp16": 2e-3, "bf16": 1.6e-2}      # fp16: the stated bound of the path; bf16: 8x coarser mantissa
TOL_LSE = {"fp16": 2e-3, "bf16": 1.6e-2}


def tol_o(dtype, o_ref):
    """The stated absolute bound, taken relative to the output magnitude where outputs exceed 1
    (peaked softmax over outlier channels): fp16 cannot hold 2e-3 absolute on values of size 2."""
    return TOL_O[dtype] * max(1.0, float(np.abs(o_ref).max()))
