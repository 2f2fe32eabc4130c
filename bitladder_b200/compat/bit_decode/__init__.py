"""``bit_decode``: the reference package's name with its two entry points
(``bit_decode/__init__.py``, ``bit_decode/bit_decode_interface.py:10-86``), served by this library."""
from ...bit_decode_interface import fwd_kvcache_int, kvcache_pack_int

__version__ = "0.0.1+b200"
__all__ = ["kvcache_pack_int", "fwd_kvcache_int"]
