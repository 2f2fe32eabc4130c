"""Import names of the reference project, served by this library.

``install()`` registers two modules in ``sys.modules``:

* ``bit_decode_cuda`` — the four functions the reference's compiled extension exports
  (``csrc/bit_decode/decode_api.cpp:605-611``), so that the reference's own ``bit_decode`` package
  (its unmodified ``bit_decode_interface.py``) can be imported and used on top of this library;
* ``bit_decode`` — only if no package of that name can be imported already: the reference's two entry
  points as this library implements them (same signatures, plus keyword-only extensions).
"""
from __future__ import annotations

import importlib
import importlib.util
import sys

__all__ = ["install"]


def install(alias_package: bool = True):
    """Make ``import bit_decode_cuda`` (and, when absent, ``import bit_decode``) resolve to this library."""
    from . import bit_decode_cuda
    sys.modules.setdefault("bit_decode_cuda", bit_decode_cuda)
    if alias_package and "bit_decode" not in sys.modules and importlib.util.find_spec("bit_decode") is None:
        sys.modules["bit_decode"] = importlib.import_module(__name__ + ".bit_decode")
    return sys.modules["bit_decode_cuda"]
