"""Stand-in for the reference's compiled extension module ``bit_decode_cuda``.

The reference's Python layer (``bit_decode/bit_decode_interface.py:8``) imports a pybind11 module of
this name and calls four functions in it (``csrc/bit_decode/decode_api.cpp:605-611``).  This module
exports the same four names with the same positional arguments and hands the work to this library's
C-ABI (``libbitdecode.so``), so the reference's own, unmodified Python file runs on top of it::

    import bitladder_b200.compat as compat
    compat.install()                 # registers ``bit_decode_cuda`` (and ``bit_decode``) in sys.modules
    import bit_decode                # the reference's package, or this library's copy of its two entry points

Arguments the reference's kernels ignore are accepted and ignored here too (``cu_seqlens_k`` is never
read, ``decode_api.cpp:585``; causal / window / softcap / rotary are hard-wired off in its Python layer,
``bit_decode_interface.py:62-67``); values this library cannot honour raise ``RuntimeError``.
"""
from __future__ import annotations

import torch

from .. import bit_decode_interface as _I

__all__ = ["kvcache_pack_i2", "kvcache_pack_i4", "fwd_kvcache_i2", "fwd_kvcache_i4"]


def _pack(num_bits, k, k_pack, k_params, v, v_pack, v_params, opt_block_table, cu_seqlens_k, max_seqlen_k,
          quant_mode, group_size):
    # decode_api.cpp:518-529: k and v come flattened to (b * seqlen_k, h_k, d); the batch is what the
    # pack buffers say (the reference takes it from cu_seqlens_k.numel() - 1, :554)
    if k.dim() != 3 or v.dim() != 3:
        raise RuntimeError("k and v must be (batch * seqlen_k, nheads_k, head_dim) as the reference's wrapper passes them")
    b = k_pack.shape[0]
    s = int(max_seqlen_k)
    if b * s != k.shape[0]:
        raise RuntimeError("max_seqlen_k times the batch of the pack buffers must equal k's first dimension")
    k4, v4 = k.view(b, s, k.shape[1], k.shape[2]), v.view(b, s, v.shape[1], v.shape[2])
    _I.kvcache_pack_int(k4, k_pack, k_params, v4, v_pack, v_params, opt_block_table, cu_seqlens_k, s, quant_mode,
                        int(group_size), num_bits)


def kvcache_pack_i4(k, k_pack, k_params, v, v_pack, v_params, opt_block_table, cu_seqlens_k, max_seqlen_k,
                    quant_mode, group_size):
    """``kvcache_qpack<4>`` (``decode_api.cpp:517-603``)."""
    _pack(4, k, k_pack, k_params, v, v_pack, v_params, opt_block_table, cu_seqlens_k, max_seqlen_k, quant_mode, group_size)


def kvcache_pack_i2(k, k_pack, k_params, v, v_pack, v_params, opt_block_table, cu_seqlens_k, max_seqlen_k,
                    quant_mode, group_size):
    """``kvcache_qpack<2>``."""
    _pack(2, k, k_pack, k_params, v, v_pack, v_params, opt_block_table, cu_seqlens_k, max_seqlen_k, quant_mode, group_size)


def _fwd(num_bits, q, k_pack, k_params, v_pack, v_params, opt_block_table, softmax_scale, quant_mode, group_size,
         is_causal, window_size_left, window_size_right, softcap, is_rotary_interleaved, num_splits):
    # decode_api.cpp:303-318.  One query token: causal is the same as not causal (:357); windows and
    # softcap have no kernel in the reference either (flash_fwd_launch_template.h:125-131)
    if q.dim() != 4 or q.shape[1] != 1:
        raise RuntimeError("only one query token per sequence (seqlen_q = 1) is supported")
    if window_size_left >= 0 or window_size_right >= 0:
        raise RuntimeError("sliding windows are not supported")
    if softcap != 0.0:
        raise RuntimeError("softcap is not supported")
    return _I.fwd_kvcache_int(q, k_pack, k_params, v_pack, v_params, opt_block_table, float(softmax_scale), quant_mode,
                              int(group_size), num_bits, num_splits=int(num_splits))


def fwd_kvcache_i4(q, k_pack, k_params, v_pack, v_params, opt_block_table, softmax_scale, quant_mode, group_size,
                   is_causal, window_size_left, window_size_right, softcap, is_rotary_interleaved, num_splits):
    """``mha_fwd_kvcache<4>`` (``decode_api.cpp:301-441``); returns ``(b, 1, h, d)`` in q's dtype."""
    return _fwd(4, q, k_pack, k_params, v_pack, v_params, opt_block_table, softmax_scale, quant_mode, group_size,
                is_causal, window_size_left, window_size_right, softcap, is_rotary_interleaved, num_splits)


def fwd_kvcache_i2(q, k_pack, k_params, v_pack, v_params, opt_block_table, softmax_scale, quant_mode, group_size,
                   is_causal, window_size_left, window_size_right, softcap, is_rotary_interleaved, num_splits):
    """``mha_fwd_kvcache<2>``."""
    return _fwd(2, q, k_pack, k_params, v_pack, v_params, opt_block_table, softmax_scale, quant_mode, group_size,
                is_causal, window_size_left, window_size_right, softcap, is_rotary_interleaved, num_splits)
