#!/usr/bin/env python
"""Generates the committed golden fixtures for the pack / decode parity tests.

    python tests/golden/make_golden.py

The reference cannot be run without a GPU and ships no golden vectors for this
path, so the fixtures come from the numpy restatement of its algorithm
(``oracle/oracle.py``): seeded inputs (fp16/bf16 bit patterns) together with the
packed buffers and the attention result they must produce.  They pin the oracle
against regressions, are re-checked against the independent C restatement on
the CPU, and are what the CUDA kernels are compared with on the GPU.  Inputs are
small (one or two pack blocks, two KV heads) so the file stays a few hundred KB.
"""
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle as O  # noqa: E402

CASES = [
    # name, bits, group, dtype, b, s, h, h_k, res, ragged
    ("i4_g128_fp16", 4, 128, "fp16", 1, 256, 8, 2, 0, False),
    ("i4_g128_fp16_tail_ragged", 4, 128, "fp16", 2, 128, 4, 1, 19, True),
    ("i2_g128_fp16", 2, 128, "fp16", 1, 256, 4, 1, 0, False),
    ("i4_g64_fp16", 4, 64, "fp16", 1, 128, 4, 1, 0, False),
    ("i2_g64_fp16_outliers", 2, 64, "fp16", 1, 256, 4, 1, 5, False),
    ("i4_g128_bf16_mha", 4, 128, "bf16", 1, 128, 2, 2, 33, True),
]


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def make_case(name, bits, group, dtype, b, s, h, h_k, res, ragged, seed):
    g = torch.Generator().manual_seed(seed)
    tdt = torch.float16 if dtype == "fp16" else torch.bfloat16
    d = 128
    q = torch.randn(b, 1, h, d, generator=g).to(tdt)
    k = torch.randn(b, s, h_k, d, generator=g)
    if "outliers" in name:
        idx = torch.randperm(d, generator=g)[:6]
        k[:, :, :, idx] *= 10.0
    k = k.to(tdt)
    v = torch.randn(b, s, h_k, d, generator=g).to(tdt)
    case = dict(q=bits16(q), k=bits16(k), v=bits16(v))
    as_np = (lambda t: t.numpy()) if dtype == "fp16" else bits16
    packed = O.quantize_pack(as_np(k), as_np(v), bits, group, dtype)
    for n in ("k_pack", "v_pack"):
        case[n] = packed[n]
    case["k_params"] = packed["k_params"].view(np.uint16)
    case["v_params"] = packed["v_params"].view(np.uint16)
    kr = vr = cs = rl = None
    if res:
        kr = torch.randn(b, res, h_k, d, generator=g).to(tdt)
        vr = torch.randn(b, res, h_k, d, generator=g).to(tdt)
        case["k_res"], case["v_res"] = bits16(kr), bits16(vr)
    if ragged:
        cs = torch.randint(1, s + 1, (b,), generator=g, dtype=torch.int32).numpy()
        rl = torch.randint(0, res + 1, (b,), generator=g, dtype=torch.int32).numpy() if res else None
        case["cache_seqlens"] = cs
        if rl is not None:
            case["res_lens"] = rl
    scale = 1.0 / math.sqrt(d)
    out, lse = O.decode_from_packed(as_np(q), packed["k_pack"], packed["k_params"], packed["v_pack"],
                                    packed["v_params"], scale, bits, group, dtype, cache_seqlens=cs,
                                    k_res=None if kr is None else as_np(kr),
                                    v_res=None if vr is None else as_np(vr), res_lens=rl)
    case["out"] = out.astype(np.float32)
    case["lse"] = lse.astype(np.float32)
    case["meta"] = np.array([bits, group, int(dtype == "bf16"), b, s, h, h_k, res, int(ragged)], dtype=np.int32)
    return case


def main():
    blob = {}
    for i, c in enumerate(CASES):
        case = make_case(*c, seed=4242 + i)
        for key, val in case.items():
            blob[f"{c[0]}/{key}"] = val
    path = os.path.join(HERE, "pack_decode_small.npz")
    np.savez_compressed(path, **blob)
    print(path, os.path.getsize(path), "bytes,", len(CASES), "cases")


if __name__ == "__main__":
    main()
