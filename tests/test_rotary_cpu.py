"""CPU: the oracle's rotary embedding (oracle.apply_rotary) against the rotation written as a complex product
in float64, its special cases, and the struct fields that carry it across the C-ABI."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O


@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("rotary_dim", [32, 128])
def test_rotation_equals_a_complex_product(interleaved, rotary_dim):
    rng = np.random.default_rng(7)
    b, heads, half = 3, 5, rotary_dim // 2
    x = rng.standard_normal((b, heads, 128)).astype(np.float16)
    ang = rng.uniform(0, 2 * np.pi, (40, half))
    cos, sin = np.cos(ang).astype(np.float16), np.sin(ang).astype(np.float16)
    pos = [0, 17, 39]
    y = O.apply_rotary(x, cos, sin, pos, interleaved).astype(np.float64)
    xf = x.astype(np.float64)
    for ib, p in enumerate(pos):
        if interleaved:
            x0, x1 = xf[ib, :, 0:rotary_dim:2], xf[ib, :, 1:rotary_dim:2]
            y0, y1 = y[ib, :, 0:rotary_dim:2], y[ib, :, 1:rotary_dim:2]
        else:
            x0, x1 = xf[ib, :, :half], xf[ib, :, half:rotary_dim]
            y0, y1 = y[ib, :, :half], y[ib, :, half:rotary_dim]
        r = (x0 + 1j * x1) * (cos[p].astype(np.float64) + 1j * sin[p].astype(np.float64))
        assert np.abs(r.real - y0).max() <= 4e-3 and np.abs(r.imag - y1).max() <= 4e-3      # fp16 rounding of the result
    assert np.array_equal(y[:, :, rotary_dim:], xf[:, :, rotary_dim:])                       # dims beyond: copied


def test_identity_tables_and_bf16():
    rng = np.random.default_rng(8)
    x = rng.standard_normal((2, 4, 128)).astype(np.float16)
    cos, sin = np.ones((4, 64), np.float16), np.zeros((4, 64), np.float16)
    assert np.array_equal(O.apply_rotary(x, cos, sin, [1, 3], True), x)
    # a quarter turn swaps the pair with a sign
    y = O.apply_rotary(x, sin, cos, [0, 0], False)
    assert np.array_equal(y[:, :, :64], -x[:, :, 64:]) and np.array_equal(y[:, :, 64:], x[:, :, :64])
    xb = O.f32_to_bf16_bits(x.astype(np.float32))
    one, zero = O.f32_to_bf16_bits(np.ones((4, 64), np.float32)), O.f32_to_bf16_bits(np.zeros((4, 64), np.float32))
    assert np.array_equal(O.apply_rotary(xb, one, zero, [2, 2], True, "bf16"), xb)


def test_abi_carries_the_rotary_fields_behind_the_older_ones():
    from bitladder_b200 import _lib
    a = _lib.DecodeArgs
    assert a.rotary_cos.offset == a.test_starve.offset + 8            # int32 + padding, then the two pointers
    assert a.rotary_positions.offset == C.sizeof(a) - 8 and C.sizeof(a) % 8 == 0
    assert _lib.BD_ERR_POSITION == -11
