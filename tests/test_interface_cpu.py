"""CPU: the Python entry points keep the reference's signatures and fail loudly (no CPU path)."""
import inspect

import pytest
import torch

import bitladder_b200 as B
from bitladder_b200 import bit_decode_interface as I


def test_signatures_match_the_reference():
    # bit_decode/bit_decode_interface.py:10-17 and :43-50 of the reference
    pack = inspect.signature(B.kvcache_pack_int)
    names = [n for n, p in pack.parameters.items() if p.kind is p.POSITIONAL_OR_KEYWORD]
    assert names == ["k_cache", "k_pack", "k_params", "v_cache", "v_pack", "v_params", "opt_block_table",
                     "cu_seqlens_k", "seqlen_k", "quant_mode", "group_size", "num_bits"]
    assert pack.parameters["quant_mode"].default == "k-channel" and pack.parameters["num_bits"].default == 4
    fwd = inspect.signature(B.fwd_kvcache_int)
    names = [n for n, p in fwd.parameters.items() if p.kind is p.POSITIONAL_OR_KEYWORD]
    assert names == ["q", "k_pack", "k_params", "v_pack", "v_params", "opt_block_table", "softmax_scale",
                     "quant_mode", "group_size", "num_bits"]
    assert fwd.parameters["softmax_scale"].default == 1.0 and fwd.parameters["group_size"].default == 128
    extras = [n for n, p in fwd.parameters.items() if p.kind is p.KEYWORD_ONLY]
    assert {"k_res", "v_res", "cache_seqlens", "return_lse", "workspace"} <= set(extras)


def _cpu_buffers(b=1, s=128, h_k=2, bits=4, group=128):
    return B.alloc_packed_cache(b, s, h_k, 128, bits, group, device="cpu")


def test_cpu_tensors_are_rejected():
    k = torch.zeros(1, 128, 2, 128, dtype=torch.float16)
    bufs = _cpu_buffers()
    with pytest.raises(RuntimeError, match="CUDA"):
        B.kvcache_pack_int(k, bufs[0], bufs[1], k, bufs[2], bufs[3])
    q = torch.zeros(1, 1, 8, 128, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA"):
        B.fwd_kvcache_int(q, *bufs)


@pytest.mark.parametrize("kw,msg", [
    (dict(quant_mode="k-tensor"), "quant_mode"),
    (dict(num_bits=8), "num_bits"),
    (dict(group_size=16), "group_size"),
])
def test_unsupported_configs_raise_instead_of_doing_nothing(kw, msg):
    k = torch.zeros(1, 128, 2, 128, dtype=torch.float16)
    bufs = _cpu_buffers()
    with pytest.raises(RuntimeError, match=msg):
        B.kvcache_pack_int(k, bufs[0], bufs[1], k, bufs[2], bufs[3], **kw)
    q = torch.zeros(1, 1, 8, 128, dtype=torch.float16)
    with pytest.raises(RuntimeError, match=msg):
        B.fwd_kvcache_int(q, *bufs, **kw)


def test_paged_cache_checks_its_page_size():
    """The reference's own check: pages are multiples of 256 tokens (decode_api.cpp:351, 566)."""
    k = torch.zeros(1, 128, 2, 128, dtype=torch.float16)
    bufs = _cpu_buffers()
    table = torch.zeros(1, 1, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="divisible by 256"):
        B.kvcache_pack_int(k, bufs[0], bufs[1], k, bufs[2], bufs[3], table)


def test_shape_checks_of_the_packed_buffers():
    kp, kprm, vp, vprm = _cpu_buffers(s=256)
    assert kp.shape == (1, 64, 2, 128) and kprm.shape == (1, 2, 2, 128)
    assert vp.shape == (1, 256, 2, 32) and vprm.shape == (1, 1, 2, 256)
    assert I._check_packed(kp, kprm, vp, vprm, 4, 128) == (1, 256, 2, 128)
    with pytest.raises(RuntimeError, match="k_params shape"):
        I._check_packed(kp, kprm[:, :1], vp, vprm, 4, 128)
    with pytest.raises(RuntimeError, match="uint16"):
        I._check_packed(kp.to(torch.int32), kprm, vp, vprm, 4, 128)
    kp2, kprm2, vp2, vprm2 = B.alloc_packed_cache(1, 300, 2, 128, 2, 64, device="cpu")
    assert vp2.shape == (1, 512, 2, 16) and kp2.shape == (1, 64, 2, 128) and vprm2.shape == (1, 2, 2, 512)
    assert B.pack_block_tokens(4) == 128 and B.pack_block_tokens(2) == 256


def test_missing_library_is_an_error_not_a_fallback(monkeypatch, tmp_path):
    from bitladder_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.load()
