"""Shared input generators and oracle glue for the tests (CPU side is numpy)."""
from __future__ import annotations

import math

import numpy as np
import torch

from oracle import c_oracle, oracle as O


def gen_qkv(b, s, h, h_k, d=128, seed=0, dtype="fp16", res=0, outlier_frac=0.0):
    """Seeded N(0,1) q/k/v (+ optional tail of `res` tokens) as torch CPU tensors.

    outlier_frac > 0 scales that fraction of K channels (seeded choice per KV
    head) by 10, the way the 2-bit long-context configuration is specified."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    tdt = torch.float16 if dtype == "fp16" else torch.bfloat16
    q = torch.randn(b, 1, h, d, generator=g).to(tdt)
    k = torch.randn(b, s, h_k, d, generator=g)
    v = torch.randn(b, s, h_k, d, generator=g).to(tdt)
    if outlier_frac > 0:
        n_out = round(outlier_frac * d)
        for ih in range(h_k):
            idx = torch.randperm(d, generator=g)[:n_out]
            k[:, :, ih, idx] *= 10.0
    k = k.to(tdt)
    out = dict(q=q, k=k, v=v)
    if res:
        out["k_res"] = torch.randn(b, res, h_k, d, generator=g).to(tdt)
        out["v_res"] = torch.randn(b, res, h_k, d, generator=g).to(tdt)
    return out


def to_np(t: torch.Tensor):
    """torch fp16 -> numpy fp16; torch bf16 -> numpy uint16 bit patterns."""
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.uint16).numpy()
    return t.contiguous().numpy()


def oracle_pack(k, v, bits, group, dtype):
    return O.quantize_pack(to_np(k), to_np(v), bits, group, dtype)


def oracle_decode(q, packed, scale, bits, group, dtype, cache_seqlens=None, k_res=None, v_res=None,
                  res_lens=None, use_c=True):
    fn = c_oracle.decode if use_c else O.decode_from_packed
    return fn(to_np(q), packed["k_pack"], packed["k_params"], packed["v_pack"], packed["v_params"],
              scale, bits, group, dtype, cache_seqlens=cache_seqlens,
              k_res=None if k_res is None else to_np(k_res),
              v_res=None if v_res is None else to_np(v_res), res_lens=res_lens)


def default_scale(d=128):
    return 1.0 / math.sqrt(d)


def u16(t: torch.Tensor) -> np.ndarray:
    """CUDA/CPU uint16 tensor -> numpy uint16."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def f32_as_u16(t: torch.Tensor) -> np.ndarray:
    """float32-typed parameter storage -> numpy uint16 view (fp16 bit patterns)."""
    return t.detach().cpu().contiguous().numpy().view(np.uint16)


# ---------------------------------------------------------------------------
# golden fixtures (tests/golden/pack_decode_small.npz, made by tests/golden/make_golden.py)
# ---------------------------------------------------------------------------
import os as _os

GOLDEN_PATH = _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "golden", "pack_decode_small.npz")


def load_golden():
    """{case name: {array name: ndarray}} with meta decoded into a dict."""
    blob = np.load(GOLDEN_PATH)
    cases = {}
    for key in blob.files:
        name, arr = key.split("/", 1)
        cases.setdefault(name, {})[arr] = blob[key]
    for c in cases.values():
        m = c.pop("meta")
        c["cfg"] = dict(bits=int(m[0]), group=int(m[1]), dtype="bf16" if m[2] else "fp16", b=int(m[3]), s=int(m[4]),
                        h=int(m[5]), h_k=int(m[6]), res=int(m[7]), ragged=bool(m[8]))
    return cases


def golden_input(case, name):
    """Input array of a golden case the way the oracles take it (fp16 array, or bf16 bit patterns)."""
    if name not in case:
        return None
    a = case[name]
    return a.view(np.float16) if case["cfg"]["dtype"] == "fp16" else a


def golden_torch(case, name, device="cpu"):
    if name not in case:
        return None
    tdt = torch.float16 if case["cfg"]["dtype"] == "fp16" else torch.bfloat16
    return torch.from_numpy(case[name].view(np.int16).copy()).view(tdt).to(device)
