"""CPU: the reference's import names on top of this library (``bitladder_b200.compat``)."""
import importlib.util
import inspect
import os
import sys

import pytest
import torch

from oracle import build_ref

REF_IFACE = os.path.join(build_ref.DEFAULT_REFERENCE, "bit_decode", "bit_decode_interface.py")


def test_shim_exports_the_four_functions_with_the_reference_arity():
    import bitladder_b200.compat as compat
    mod = compat.install()
    assert sys.modules["bit_decode_cuda"] is mod
    # csrc/bit_decode/decode_api.cpp:518-529 (11 arguments) and :303-318 (15 arguments)
    for name, n in (("kvcache_pack_i2", 11), ("kvcache_pack_i4", 11), ("fwd_kvcache_i2", 15), ("fwd_kvcache_i4", 15)):
        assert len(inspect.signature(getattr(mod, name)).parameters) == n, name
    import bit_decode
    assert callable(bit_decode.kvcache_pack_int) and callable(bit_decode.fwd_kvcache_int)


@pytest.mark.skipif(not os.path.exists(REF_IFACE), reason="the reference sources are not on this machine")
def test_the_reference_python_layer_runs_on_top_of_the_shim():
    """The reference's own, unmodified bit_decode_interface.py imports ``bit_decode_cuda`` and calls it
    positionally; with the shim installed the call reaches this library, which (on this CPU-only machine)
    refuses the CPU tensors with its own error: the binding is complete up to the device."""
    import bitladder_b200.compat as compat
    compat.install()
    spec = importlib.util.spec_from_file_location("ref_bit_decode_interface", REF_IFACE)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    b, s, h, h_k, d = 1, 256, 8, 2, 128
    k = torch.zeros(b, s, h_k, d, dtype=torch.float16)
    k_pack = torch.zeros(b, s // 4, h_k, d, dtype=torch.uint16)
    k_params = torch.zeros(b, s // 128, h_k, d, dtype=torch.float32)
    v_pack = torch.zeros(b, s, h_k, d // 4, dtype=torch.uint16)
    v_params = torch.zeros(b, 1, h_k, s, dtype=torch.float32)
    cu = torch.arange(0, (b + 1) * s, s, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA"):
        ref.kvcache_pack_int(k, k_pack, k_params, k, v_pack, v_params, None, cu, s, "k-channel", 128, 4)
    q = torch.zeros(b, 1, h, d, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA"):
        ref.fwd_kvcache_int(q, k_pack, k_params, v_pack, v_params, None, 0.088, "k-channel", 128, 4)
