"""ctypes binding of ``libbitdecode.so`` (the C-ABI declared in ``include/bitdecode.h``).

There is no fallback: if the shared library is missing or does not export a
symbol, importing the operators fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("BITDECODE_LIB") or os.path.join(_HERE, "libbitdecode.so")

BD_OK = 0
BD_FP16, BD_BF16, BD_FP32 = 0, 1, 2
BD_MAX_PARTS = 16
BD_PACK_APPROX_DIV = 1
BD_ERR_INVALID, BD_ERR_TIMEOUT, BD_ERR_SCRATCH_LIMIT, BD_ERR_PAGE, BD_ERR_CAPACITY, BD_ERR_POSITION = -1, -7, -8, -9, -10, -11

EXPORTS = (
    "bd_pack", "bd_decode", "bd_decode_workspace_bytes", "bd_plan_splits", "bd_decode_plan",
    "bd_combine", "bd_read_status", "bd_strerror", "bd_version",
    "bd_partition_segments", "bd_partition_parts",
    "bd_decode_noalloc", "bd_noalloc_scratch_bytes",
    "bd_exchange_area_bytes", "bd_peer_alloc", "bd_peer_free", "bd_peer_export", "bd_peer_open", "bd_peer_close",
    "bd_exchange_combine", "bd_exchange_put", "bd_exchange_state", "bd_decode_exchange",
)


class PackArgs(C.Structure):
    _fields_ = [
        ("k", C.c_void_p), ("v", C.c_void_p),
        ("k_stride_b", C.c_int64), ("k_stride_s", C.c_int64), ("k_stride_h", C.c_int64),
        ("v_stride_b", C.c_int64), ("v_stride_s", C.c_int64), ("v_stride_h", C.c_int64),
        ("k_pack", C.c_void_p), ("k_params", C.c_void_p), ("v_pack", C.c_void_p), ("v_params", C.c_void_p),
        ("k_pack_stride_b", C.c_int64), ("k_params_stride_b", C.c_int64), ("v_pack_stride_b", C.c_int64),
        ("v_params_stride_b", C.c_int64), ("v_params_stride_g", C.c_int64), ("v_params_stride_h", C.c_int64),
        ("b", C.c_int32), ("s", C.c_int32), ("h_k", C.c_int32), ("d", C.c_int32),
        ("dst_token_offset", C.c_int32),
        ("bits", C.c_int32), ("group", C.c_int32), ("dtype", C.c_int32),
        ("flags", C.c_int32),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("out", C.c_void_p), ("lse", C.c_void_p),
        ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64),
        ("out_stride_b", C.c_int64), ("out_stride_h", C.c_int64),
        ("k_pack", C.c_void_p), ("k_params", C.c_void_p), ("v_pack", C.c_void_p), ("v_params", C.c_void_p),
        ("k_pack_stride_b", C.c_int64), ("k_params_stride_b", C.c_int64), ("v_pack_stride_b", C.c_int64),
        ("v_params_stride_b", C.c_int64), ("v_params_stride_g", C.c_int64), ("v_params_stride_h", C.c_int64),
        ("cache_seqlens", C.c_void_p),
        ("k_res", C.c_void_p), ("v_res", C.c_void_p),
        ("res_stride_b", C.c_int64), ("res_stride_s", C.c_int64), ("res_stride_h", C.c_int64),
        ("res_lens", C.c_void_p),
        ("res_len", C.c_int32),
        ("b", C.c_int32), ("h", C.c_int32), ("h_k", C.c_int32), ("d", C.c_int32),
        ("s", C.c_int32), ("s_cap", C.c_int32),
        ("bits", C.c_int32), ("group", C.c_int32),
        ("dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("softmax_scale", C.c_float),
        ("num_splits", C.c_int32),
        ("k_new", C.c_void_p), ("v_new", C.c_void_p), ("new_stride_b", C.c_int64), ("new_stride_h", C.c_int64),
        ("block_table", C.c_void_p), ("block_table_stride", C.c_int32), ("num_pages", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("advance", C.c_int32), ("spin_limit", C.c_uint32), ("test_starve", C.c_int32),
        ("rotary_cos", C.c_void_p), ("rotary_sin", C.c_void_p),
        ("rotary_dim", C.c_int32), ("rotary_interleaved", C.c_int32), ("rotary_positions", C.c_int32),
        ("reserved0", C.c_int32),
    ]


class CombineArgs(C.Structure):
    _fields_ = [
        ("n_parts", C.c_int32),
        ("part_out", C.POINTER(C.c_void_p)),
        ("part_lse", C.POINTER(C.c_void_p)),
        ("rows", C.c_int64),
        ("d", C.c_int32),
        ("out", C.c_void_p),
        ("lse", C.c_void_p),
        ("out_dtype", C.c_int32),
    ]


class ExchangeArgs(C.Structure):
    _fields_ = [
        ("rank", C.c_int32), ("world", C.c_int32),
        ("areas", C.POINTER(C.c_void_p)),
        ("part_out", C.c_void_p), ("part_lse", C.c_void_p),
        ("rows", C.c_int64),
        ("d", C.c_int32),
        ("out", C.c_void_p), ("lse", C.c_void_p),
        ("out_dtype", C.c_int32), ("spin_limit", C.c_uint32),
    ]


_lib = None


def load():
    """Load the shared library once; raise loudly if it is absent or incomplete."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} not found: the CUDA library is not built. Run "
            "`python -m bitladder_b200.build` (needs nvcc); there is no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    for name in EXPORTS:
        if not hasattr(lib, name):
            raise RuntimeError(f"{LIB_PATH} does not export {name}; rebuild it")
    lib.bd_pack.argtypes = [C.POINTER(PackArgs), C.c_void_p]
    lib.bd_pack.restype = C.c_int
    lib.bd_decode.argtypes = [C.POINTER(DecodeArgs), C.c_void_p]
    lib.bd_decode.restype = C.c_int
    lib.bd_decode_noalloc.argtypes = [C.POINTER(DecodeArgs), C.c_void_p]
    lib.bd_decode_noalloc.restype = C.c_int
    lib.bd_noalloc_scratch_bytes.argtypes = []
    lib.bd_noalloc_scratch_bytes.restype = C.c_size_t
    lib.bd_decode_workspace_bytes.argtypes = [C.POINTER(DecodeArgs)]
    lib.bd_decode_workspace_bytes.restype = C.c_size_t
    lib.bd_plan_splits.argtypes = [C.c_int, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int]
    lib.bd_plan_splits.restype = C.c_int
    lib.bd_decode_plan.argtypes = [C.POINTER(DecodeArgs), C.POINTER(C.c_int32)]
    lib.bd_decode_plan.restype = C.c_int
    lib.bd_combine.argtypes = [C.POINTER(CombineArgs), C.c_void_p]
    lib.bd_combine.restype = C.c_int
    lib.bd_partition_segments.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int]
    lib.bd_partition_segments.restype = C.c_int
    lib.bd_partition_parts.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int]
    lib.bd_partition_parts.restype = C.c_int
    lib.bd_read_status.argtypes = [C.c_void_p, C.c_void_p]
    lib.bd_read_status.restype = C.c_int
    lib.bd_exchange_area_bytes.argtypes = [C.c_int, C.c_int64]
    lib.bd_exchange_area_bytes.restype = C.c_size_t
    lib.bd_peer_alloc.argtypes = [C.c_size_t, C.POINTER(C.c_void_p)]
    lib.bd_peer_free.argtypes = [C.c_void_p]
    lib.bd_peer_export.argtypes = [C.c_void_p, C.c_void_p]
    lib.bd_peer_open.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    lib.bd_peer_close.argtypes = [C.c_void_p]
    lib.bd_exchange_combine.argtypes = [C.POINTER(ExchangeArgs), C.c_void_p]
    lib.bd_decode_exchange.argtypes = [C.POINTER(DecodeArgs), C.POINTER(ExchangeArgs), C.c_void_p]
    lib.bd_exchange_put.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.bd_exchange_state.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint32)]
    for name in ("bd_peer_alloc", "bd_peer_free", "bd_peer_export", "bd_peer_open", "bd_peer_close",
                 "bd_exchange_combine", "bd_exchange_put", "bd_exchange_state", "bd_decode_exchange"):
        getattr(lib, name).restype = C.c_int
    lib.bd_strerror.argtypes = [C.c_int]
    lib.bd_strerror.restype = C.c_char_p
    lib.bd_version.restype = C.c_int
    _lib = lib
    return lib


def strerror(code: int) -> str:
    return load().bd_strerror(code).decode()


def check(code: int, what: str) -> None:
    if code != BD_OK:
        raise RuntimeError(f"{what} failed: {strerror(code)} (code {code})")
