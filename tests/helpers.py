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


# ---------------------------------------------------------------------------
# golden vectors written by the reference's own CUDA kernels (tests/golden/ref_i4.npz, made on a
# B200 by tests/golden/make_ref_golden.py from the modules oracle/build_ref.py builds)
# ---------------------------------------------------------------------------
REF_GOLDEN_PATH = _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "golden", "ref_i4.npz")
REF_STORED = ("gqa_g128", "mha_g128", "gqa_g32")            # inputs and packed buffers stored
REF_HASHED = ("eval_g128", "llama_g128", "llama_g32")       # inputs regenerated from the seed, buffers as SHA-256


def _ref_generator():
    import importlib.util
    path = _os.path.join(_os.path.dirname(GOLDEN_PATH), "make_ref_golden.py")
    spec = importlib.util.spec_from_file_location("make_ref_golden", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_ref_case(name):
    """One case of the reference-kernel fixtures: dict(cfg, q, k, v as torch fp16 CPU tensors, blob, sha).
    Inputs of the hashed cases are regenerated with the generator script's own function and checked
    against the recorded hashes (None is returned for q/k/v if this torch build draws other numbers)."""
    gen = _ref_generator()
    blob = np.load(REF_GOLDEN_PATH)
    b, s, h, h_k, group, seed, store, crafted = (int(x) for x in blob[f"{name}/meta"])
    cfg = dict(b=b, s=s, h=h, h_k=h_k, group=group, bits=4, crafted=bool(crafted))
    if store:
        q, k, v = (torch.from_numpy(blob[f"{name}/{n}"].view(np.int16).copy()).view(torch.float16) for n in "qkv")
    else:
        q, k, v = gen.make_inputs(b, s, h, h_k, seed, bool(crafted))
        got = np.concatenate([gen.sha(t.numpy().view(np.uint16)) for t in (q, k, v)])
        if not np.array_equal(got, blob[f"{name}/in_sha"]):
            q = k = v = None
    return dict(cfg=cfg, q=q, k=k, v=v, blob=blob, sha=gen.sha, name=name)


def params_equal(a_u16: np.ndarray, b_u16: np.ndarray) -> bool:
    """fp16 scale/zero bit patterns equal, +0.0 and -0.0 taken as the same value (the sign of a
    zero group minimum depends on the order the reference's reduction meets +0.0 and -0.0)."""
    a, b = a_u16.ravel(), b_u16.ravel()
    return bool(np.all((a == b) | (((a | b) & 0x7FFF) == 0)))
