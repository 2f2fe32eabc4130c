"""ctypes binding of the C restatement of the oracle (``oracle/bd_oracle.c``).

Test infrastructure only.  ``build()`` compiles the shared object with the
Makefile beside this file; ``quantize_pack`` / ``decode`` mirror the numpy
oracle's functions on contiguous numpy arrays.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libbd_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "bd_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "libbd_oracle.so"])
    return _SO


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
        _lib.bdo_num_threads.restype = ctypes.c_int
        _lib.bdo_quantize_pack.restype = ctypes.c_int
        _lib.bdo_decode.restype = ctypes.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _bits16(a):
    """fp16 array or uint16 bit patterns -> contiguous uint16 view."""
    a = np.ascontiguousarray(a)
    return a.view(np.uint16) if a.dtype == np.float16 else a.astype(np.uint16, copy=False)


def num_threads() -> int:
    return int(lib().bdo_num_threads())


def set_num_threads(n: int) -> None:
    """Use ``n`` OpenMP threads from now on (overrides an ``OMP_NUM_THREADS`` inherited from a launcher)."""
    f = lib().bdo_set_num_threads
    f.argtypes, f.restype = [ctypes.c_int], None
    f(int(n))


def quantize_pack(k, v, bits: int, group: int, dtype: str = "fp16"):
    k16, v16 = _bits16(k), _bits16(v)
    b, s, h, d = k16.shape
    P = 16 // bits
    k_pack = np.zeros((b, s // P, h, d), np.uint16)
    k_params = np.zeros((b, s // group, h, 2 * d), np.uint16)
    v_pack = np.zeros((b, s, h, d // P), np.uint16)
    v_params = np.zeros((b, d // group, h, 2 * s), np.uint16)
    rc = lib().bdo_quantize_pack(_p(k16), _p(v16), int(dtype == "bf16"), b, s, h, d, bits, group,
                                 _p(k_pack), _p(k_params), _p(v_pack), _p(v_params))
    if rc != 0:
        raise ValueError("bdo_quantize_pack rejected the sizes")
    return dict(k_pack=k_pack, k_params=k_params.view(np.float32),
                v_pack=v_pack, v_params=v_params.view(np.float32))


def decode(q, k_pack, k_params, v_pack, v_params, softmax_scale, bits, group, dtype="fp16",
           cache_seqlens=None, k_res=None, v_res=None, res_lens=None):
    q16 = _bits16(q)
    if q16.ndim == 4:
        q16 = np.ascontiguousarray(q16[:, 0])
    b, h, d = q16.shape
    s, h_k = v_pack.shape[1], v_pack.shape[2]
    out = np.zeros((b, h, d), np.float64)
    lse = np.zeros((b, h), np.float64)
    cs = None if cache_seqlens is None else np.ascontiguousarray(cache_seqlens, dtype=np.int32)
    rl = None if res_lens is None else np.ascontiguousarray(res_lens, dtype=np.int32)
    kr = None if k_res is None else _bits16(k_res)
    vr = None if v_res is None else _bits16(v_res)
    res_cap = 0 if kr is None else kr.shape[1]
    kprm = np.ascontiguousarray(k_params).view(np.uint16)
    vprm = np.ascontiguousarray(v_params).view(np.uint16)
    rc = lib().bdo_decode(_p(q16), int(dtype == "bf16"),
                          _p(np.ascontiguousarray(k_pack)), _p(kprm),
                          _p(np.ascontiguousarray(v_pack)), _p(vprm),
                          b, h, h_k, d, s, bits, group, ctypes.c_float(softmax_scale),
                          _p(cs), _p(kr), _p(vr), res_cap, _p(rl), res_cap,
                          _p(out), _p(lse))
    if rc != 0:
        raise ValueError("bdo_decode rejected the sizes")
    return out, lse
