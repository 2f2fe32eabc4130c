"""B200-native low-bit KV-cache decode attention (quantize-pack, split-KV decode, split combine).

The two public functions keep the names and signatures of the reference's
``bit_decode`` package (reference: ``bit_decode/__init__.py:3-6``).
"""
__version__ = "0.1.0"

from .bit_decode_interface import (  # noqa: F401
    kvcache_pack_int,
    fwd_kvcache_int,
    combine_partials,
    decode_workspace_bytes,
    plan_splits,
    pack_block_tokens,
    alloc_packed_cache,
    DecodeStep,
)
from .kv_cache import PackedKVCache  # noqa: F401
