"""CPU oracle for the low-bit KV-cache decode-attention path (numpy).

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this
module; it exists so the tests, the smoke check and the CPU-baseline leg of the
benchmark can compare the CUDA kernels against an independent restatement of
the reference algorithm.

Parity status: *pinned for 4-bit, group 128 and 32*.  The reference has no CPU
implementation and ships no golden vectors, but its CUDA kernels compile for
sm_100a (``oracle/build_ref.py``); what they write on seeded inputs on a B200 is
committed as ``tests/golden/ref_i4.npz`` (``tests/golden/make_ref_golden.py``).
``tests/test_ref_golden.py`` checks this restatement against those bytes: packed
codes, scales and zeros equal the reference built without ``--use_fast_math`` byte
for byte (a group minimum of -0.0 may come out as +0.0); against the reference as
shipped (``--use_fast_math``: the GPU's approximate reciprocal gives a
``scale_inv`` that is one ulp off in about a quarter of the groups) codes differ
only where ``(x - min) * 15 / range`` is exactly ``k + 0.5``, by one step.  The
attention output agrees with the reference decode kernel's to 1e-4 on those
inputs.  2-bit, group 64 and bf16 have no runnable reference kernel (the 2-bit V
packer indexes past its fragment): those are defined by this build and anchored
on (a) hand-computed known-answer cases, (b) the independent C restatement
(``oracle/bd_oracle.c``) that must agree bit for bit, and (c) the one aggregate
the reference records (mean-abs error 0.002773 against fp16 attention,
``benchmark/bench_single_decode.ipynb:92``), reproduced statistically.

Reference files restated here (paths relative to the reference project):

* quantizer math          ``csrc/bit_decode/src/include/qpack.h:219-300`` (4-bit)
                          and ``:110-217`` (2-bit)
* group geometry          ``csrc/bit_decode/src/flash_fwd_kernel.h:919-957``
* packed layouts          ``qpack.h:283-294`` (fields, low index first) and the
                          parameter stores at ``flash_fwd_kernel.h:939-957``
* affine dequantisation   ``csrc/bit_decode/src/include/dequantize.h:253-384``
                          (one fused multiply-add in fp16, single rounding)
* softmax / LSE           ``csrc/bit_decode/src/include/softmax.h:188-309``
* GQA head mapping        ``csrc/bit_decode/decode_api.cpp:360-368``
* split combine           ``csrc/bit_decode/src/flash_fwd_kernel.h:1217-1298``

Layouts (``P = 16 // bits`` codes per 16-bit word, ``NB = 32 * P`` tokens per
pack block, ``G`` = group size, ``d`` = head dim):

* ``k_pack[b, 32*blk + p, h, c]``: field ``j`` (bits ``bits*j ...``) is the code
  of token ``NB*blk + p + 32*j``, channel ``c``.
* ``k_params[b, g, h, :]`` viewed as ``2*d`` fp16: ``[0:d]`` scales and
  ``[d:2d]`` zeros of token group ``g`` (``G`` consecutive tokens), per channel.
* ``v_pack[b, t, h, p]``: field ``j`` is the code of dim ``p + (d/P)*j``.
* ``v_params[b, gd, h, :]`` viewed as ``2*s`` fp16: for each run of 128 tokens
  ``tb``, ``[256*tb : 256*tb+128]`` are the scales and ``[256*tb+128 :
  256*tb+256]`` the zeros of tokens ``128*tb ... 128*tb+127`` for dim group
  ``gd`` (``G`` consecutive dims).

For 4-bit with G=128 and G=32 these are byte-identical to what the reference
kernels write.  With 4-bit / G=32 the reference stores the parameters in the order
its MMA fragments hold them (``flash_fwd_kernel.h:939-957`` with ``num_params = 4``):
the scale of (group ``g`` of the pack block / 128-token run, element ``c``) sits in
parameter row ``2*(g%2) + (c//8)%2`` at fp16 column ``16*(c//16) + 8*(g//2) + c%8``
(see ``param_slots``).  The 2-bit and G=64 layouts are defined by this build (the
reference's 2-bit V packer is not usable and it has no G=64 instantiation) and use
the natural order.
"""
from __future__ import annotations

import numpy as np

__all__ = [
    "pack_block_tokens", "bf16_bits_to_f32", "f32_to_bf16_bits", "to_f32",
    "quantize_kv", "pack_k", "pack_v", "pack_k_params", "pack_v_params",
    "unpack_k", "unpack_v", "unpack_k_params", "unpack_v_params", "param_slots",
    "quantize_pack", "dequantize", "decode_attention", "combine_partials",
    "decode_from_packed",
]


# ----------------------------------------------------------------------------
# dtype helpers
# ----------------------------------------------------------------------------

def pack_block_tokens(bits: int) -> int:
    """Tokens covered by one K pack block (32 rows of 16-bit words)."""
    return 32 * (16 // bits)


def bf16_bits_to_f32(bits_u16: np.ndarray) -> np.ndarray:
    return (bits_u16.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + (np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1)))
    return (rounded >> 16).astype(np.uint16)


def to_f32(x: np.ndarray, dtype: str) -> np.ndarray:
    """Input tensor (fp16 array, or uint16 bit patterns for bf16) -> fp32."""
    if dtype == "fp16":
        return np.asarray(x, dtype=np.float16).astype(np.float32)
    if dtype == "bf16":
        return bf16_bits_to_f32(np.asarray(x, dtype=np.uint16))
    raise ValueError(dtype)


def _round_half_away_nonneg(x: np.ndarray) -> np.ndarray:
    """roundf() for x >= 0 (ties away from zero), exact in fp32.

    ``x - trunc(x)`` is exact, so the comparison with 0.5 sees the true
    fraction; ``floor(x + 0.5)`` would be wrong for 0.49999997.
    """
    r = np.trunc(x)
    return r + ((x - r) >= np.float32(0.5)).astype(np.float32)


# ----------------------------------------------------------------------------
# quantizer (qpack.h:219-300, :110-217)
# ----------------------------------------------------------------------------

def _quantize_lastaxis(x: np.ndarray, bits: int):
    """Asymmetric min-max quantisation of groups laid along the last axis.

    x: fp32 (..., G).  Returns codes uint8 (..., G), scale fp16 (...), zero fp16 (...).
    Follows qpack.h:241-252 (range, scale_inv, stored scale and zero) and
    :266-281 (subtract, multiply, roundf, clamp), all in IEEE fp32.
    """
    maxv = np.float32((1 << bits) - 1)
    mx = x.max(axis=-1)
    mn = x.min(axis=-1)
    rng = (mx - mn).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        scale_inv = np.where(rng > 0, maxv / rng, np.float32(0)).astype(np.float32)
        scale = np.where(scale_inv == 0, np.float32(0), np.float32(1) / scale_inv).astype(np.float32)
    val = (x - mn[..., None]).astype(np.float32) * scale_inv[..., None]
    val = val.astype(np.float32)
    val = np.minimum(np.maximum(_round_half_away_nonneg(val), np.float32(0)), maxv)
    return val.astype(np.uint8), scale.astype(np.float16), mn.astype(np.float16)


def quantize_kv(k_f32: np.ndarray, v_f32: np.ndarray, bits: int, group: int):
    """Logical quantisation of K (per channel) and V (per token).

    k_f32, v_f32: (b, s, h, d) fp32 holding fp16/bf16 values.
    Returns dict with
      k_codes (b,s,h,d) u8, k_scale/k_zero (b, s/G, h, d) fp16,
      v_codes (b,s,h,d) u8, v_scale/v_zero (b, s, h, d/G) fp16.
    K groups: G consecutive tokens of one channel.  V groups: G consecutive
    dims of one token (flash_fwd_kernel.h:919-937).
    """
    b, s, h, d = k_f32.shape
    if s % group or d % group:
        raise ValueError("s and d must be multiples of group")
    kg = k_f32.reshape(b, s // group, group, h, d).transpose(0, 1, 3, 4, 2)
    kc, ks, kz = _quantize_lastaxis(np.ascontiguousarray(kg), bits)
    k_codes = kc.transpose(0, 1, 4, 2, 3).reshape(b, s, h, d)
    vg = v_f32.reshape(b, s, h, d // group, group)
    vc, vs, vz = _quantize_lastaxis(vg, bits)
    return dict(k_codes=np.ascontiguousarray(k_codes), k_scale=ks, k_zero=kz,
                v_codes=vc.reshape(b, s, h, d), v_scale=vs, v_zero=vz)


# ----------------------------------------------------------------------------
# physical layouts
# ----------------------------------------------------------------------------

def pack_k(k_codes: np.ndarray, bits: int) -> np.ndarray:
    P = 16 // bits
    NB = 32 * P
    b, s, h, d = k_codes.shape
    if s % NB:
        raise ValueError("s must be a multiple of the pack block")
    c = k_codes.reshape(b, s // NB, P, 32, h, d).astype(np.uint16)   # token = NB*blk + 32*j + p
    out = np.zeros((b, s // NB, 32, h, d), dtype=np.uint16)
    for j in range(P):
        out |= c[:, :, j] << np.uint16(bits * j)
    return out.reshape(b, s // P, h, d)


def unpack_k(k_pack: np.ndarray, bits: int) -> np.ndarray:
    P = 16 // bits
    NB = 32 * P
    b, rows, h, d = k_pack.shape
    w = k_pack.reshape(b, rows // 32, 32, h, d)
    mask = np.uint16((1 << bits) - 1)
    out = np.empty((b, rows // 32, P, 32, h, d), dtype=np.uint8)
    for j in range(P):
        out[:, :, j] = ((w >> np.uint16(bits * j)) & mask).astype(np.uint8)
    return out.reshape(b, rows * P, h, d)


def pack_v(v_codes: np.ndarray, bits: int) -> np.ndarray:
    P = 16 // bits
    b, s, h, d = v_codes.shape
    c = v_codes.reshape(b, s, h, P, d // P).astype(np.uint16)        # dim = (d/P)*j + p
    out = np.zeros((b, s, h, d // P), dtype=np.uint16)
    for j in range(P):
        out |= c[:, :, :, j] << np.uint16(bits * j)
    return out


def unpack_v(v_pack: np.ndarray, bits: int) -> np.ndarray:
    P = 16 // bits
    b, s, h, dp = v_pack.shape
    mask = np.uint16((1 << bits) - 1)
    out = np.empty((b, s, h, P, dp), dtype=np.uint8)
    for j in range(P):
        out[:, :, :, j] = ((v_pack >> np.uint16(bits * j)) & mask).astype(np.uint8)
    return out.reshape(b, s, h, P * dp)


def param_slots(bits: int, group: int):
    """Index arrays ``(row, col)`` of shape (4, 128) for the 4-bit / group-32 parameter order of
    the reference (``flash_fwd_kernel.h:939-957``), or ``None`` where the order is the natural one:
    the scale of (group ``g`` of a block or run, element ``c``) is stored in row ``row[g, c]`` at
    fp16 column ``col[g, c]``."""
    if not (bits == 4 and group == 32):
        return None
    g = np.arange(4)[:, None]
    c = np.arange(128)[None, :]
    return 2 * (g % 2) + (c // 8) % 2 + 0 * c, 16 * (c // 16) + 8 * (g // 2) + c % 8


def pack_k_params(k_scale: np.ndarray, k_zero: np.ndarray, bits: int = 4, group: int = 128) -> np.ndarray:
    """(b, s/G, h, d) fp16 x2 -> (b, s/G, h, d) float32-typed storage."""
    slots = param_slots(bits, group)
    if slots is not None:
        row, col = slots
        b, ng, h, d = k_scale.shape
        out = []
        for t in (k_scale, k_zero):
            src = t.reshape(b, ng // 4, 4, h, d)
            dst = np.empty_like(src)
            for g in range(4):
                dst[:, :, row[g], :, col[g]] = np.moveaxis(src[:, :, g], -1, 0)
            out.append(dst.reshape(b, ng, h, d))
        k_scale, k_zero = out
    both = np.concatenate([k_scale, k_zero], axis=-1).astype(np.float16)   # (b, ng, h, 2d)
    return np.ascontiguousarray(both).view(np.float32)


def unpack_k_params(k_params: np.ndarray, bits: int = 4, group: int = 128):
    halves = np.ascontiguousarray(k_params).view(np.float16)
    d = k_params.shape[-1]
    sc, ze = halves[..., :d].copy(), halves[..., d:].copy()
    slots = param_slots(bits, group)
    if slots is not None:
        row, col = slots
        b, ng, h, _ = sc.shape
        out = []
        for t in (sc, ze):
            src = t.reshape(b, ng // 4, 4, h, d)
            dst = np.empty_like(src)
            for g in range(4):
                dst[:, :, g] = np.moveaxis(src[:, :, row[g], :, col[g]], 0, -1)
            out.append(dst.reshape(b, ng, h, d))
        sc, ze = out
    return sc, ze


def pack_v_params(v_scale: np.ndarray, v_zero: np.ndarray, bits: int = 4, group: int = 128) -> np.ndarray:
    """(b, s, h, d/G) fp16 x2 -> (b, d/G, h, s) float32-typed storage."""
    b, s, h, ng = v_scale.shape
    if s % 128:
        raise ValueError("s must be a multiple of 128")
    sc = v_scale.transpose(0, 3, 2, 1).reshape(b, ng, h, s // 128, 1, 128)
    ze = v_zero.transpose(0, 3, 2, 1).reshape(b, ng, h, s // 128, 1, 128)
    both = np.concatenate([sc, ze], axis=4).astype(np.float16)              # (b, ng, h, s/128, 2, 128)
    slots = param_slots(bits, group)
    if slots is not None:
        row, col = slots
        dst = np.empty_like(both)
        for g in range(4):
            dst[:, row[g], :, :, :, col[g]] = np.moveaxis(both[:, g], -1, 0)
        both = dst
    return np.ascontiguousarray(both.reshape(b, ng, h, 2 * s)).view(np.float32)


def unpack_v_params(v_params: np.ndarray, bits: int = 4, group: int = 128):
    b, ng, h, s = v_params.shape
    halves = np.ascontiguousarray(v_params).view(np.float16).reshape(b, ng, h, s // 128, 2, 128)
    slots = param_slots(bits, group)
    if slots is not None:
        row, col = slots
        dst = np.empty_like(halves)
        for g in range(4):
            dst[:, g] = np.moveaxis(halves[:, row[g], :, :, :, col[g]], 0, -1)
        halves = dst
    sc = halves[:, :, :, :, 0].reshape(b, ng, h, s).transpose(0, 3, 2, 1)
    ze = halves[:, :, :, :, 1].reshape(b, ng, h, s).transpose(0, 3, 2, 1)
    return np.ascontiguousarray(sc), np.ascontiguousarray(ze)


def quantize_pack(k, v, bits: int, group: int, dtype: str = "fp16"):
    """Full restatement of the quantize-pack entry point; returns the four
    caller-visible buffers plus the logical result."""
    q = quantize_kv(to_f32(k, dtype), to_f32(v, dtype), bits, group)
    return dict(
        k_pack=pack_k(q["k_codes"], bits),
        k_params=pack_k_params(q["k_scale"], q["k_zero"], bits, group),
        v_pack=pack_v(q["v_codes"], bits),
        v_params=pack_v_params(q["v_scale"], q["v_zero"], bits, group),
        logical=q,
    )


# ----------------------------------------------------------------------------
# dequantise + attention
# ----------------------------------------------------------------------------

def dequantize(logical: dict, group: int, out_dtype: str = "fp16"):
    """code * scale + zero with a single rounding (the reference's __hfma2,
    dequantize.h:291,372-375).  Returns fp32 arrays (b, s, h, d) holding
    fp16 values, or bf16 values when out_dtype == 'bf16' (the fp16 result
    rounded once more to bf16, the definition this build uses for bf16 caches).
    """
    kc = logical["k_codes"].astype(np.float64)
    b, s, h, d = kc.shape
    ks = np.repeat(logical["k_scale"].astype(np.float64), group, axis=1)
    kz = np.repeat(logical["k_zero"].astype(np.float64), group, axis=1)
    k = (kc * ks + kz).astype(np.float16).astype(np.float32)
    vc = logical["v_codes"].astype(np.float64)
    vs = np.repeat(logical["v_scale"].astype(np.float64), group, axis=3)
    vz = np.repeat(logical["v_zero"].astype(np.float64), group, axis=3)
    v = (vc * vs + vz).astype(np.float16).astype(np.float32)
    if out_dtype == "bf16":
        k = bf16_bits_to_f32(f32_to_bf16_bits(k))
        v = bf16_bits_to_f32(f32_to_bf16_bits(v))
    return k, v


def decode_attention(q_f32, k_f32, v_f32, softmax_scale, cache_seqlens=None,
                     k_res=None, v_res=None, res_lens=None):
    """One decode step: softmax(scale * q k^T) v over the first
    ``cache_seqlens[b]`` cached tokens followed by the first ``res_lens[b]``
    residual tokens, one joint softmax (softmax.h:188-309 semantics).

    q_f32 (b, h, d); k_f32/v_f32 (b, s, h_k, d); k_res/v_res (b, r, h_k, d).
    Query head ``hq`` reads KV head ``hq // (h / h_k)`` (decode_api.cpp:365).
    Returns out float64 (b, h, d) and lse float64 (b, h) = natural-log
    log-sum-exp of the scaled scores.  A row with no valid token gives
    out = 0, lse = -inf.
    """
    b, h, d = q_f32.shape
    s, h_k = k_f32.shape[1], k_f32.shape[2]
    gq = h // h_k
    out = np.zeros((b, h, d), dtype=np.float64)
    lse = np.full((b, h), -np.inf, dtype=np.float64)
    for ib in range(b):
        n = s if cache_seqlens is None else int(cache_seqlens[ib])
        ks = [k_f32[ib, :n]]
        vs = [v_f32[ib, :n]]
        if k_res is not None:
            r = k_res.shape[1] if res_lens is None else int(res_lens[ib])
            ks.append(k_res[ib, :r])
            vs.append(v_res[ib, :r])
        kk = np.concatenate(ks, axis=0).astype(np.float64)      # (n_tot, h_k, d)
        vv = np.concatenate(vs, axis=0).astype(np.float64)
        if kk.shape[0] == 0:
            continue
        qq = q_f32[ib].astype(np.float64).reshape(h_k, gq, d)
        sc = np.einsum("hgd,thd->hgt", qq, kk) * float(softmax_scale)
        m = sc.max(axis=-1, keepdims=True)
        p = np.exp(sc - m)
        l = p.sum(axis=-1, keepdims=True)
        o = np.einsum("hgt,thd->hgd", p, vv) / l
        out[ib] = o.reshape(h, d)
        lse[ib] = (m + np.log(l)).reshape(h)
    return out, lse


def combine_partials(outs, lses):
    """Merge partial (O, LSE) pairs (flash_fwd_kernel.h:1217-1231,1280-1298).

    outs: (n, ..., d) each normalised within its part; lses: (n, ...).
    Parts with lse = -inf contribute nothing; if all are -inf the result is
    out = 0, lse = -inf.
    """
    outs = np.asarray(outs, dtype=np.float64)
    lses = np.asarray(lses, dtype=np.float64)
    m = lses.max(axis=0)
    safe_m = np.where(np.isfinite(m), m, 0.0)
    w = np.exp(lses - safe_m)
    tot = w.sum(axis=0)
    with np.errstate(divide="ignore", invalid="ignore"):
        lse = np.where(tot > 0, safe_m + np.log(tot), -np.inf)
        wn = np.where(tot > 0, w / np.where(tot > 0, tot, 1.0), 0.0)
    out = (wn[..., None] * outs).sum(axis=0)
    return out, lse


def decode_from_packed(q, k_pack, k_params, v_pack, v_params, softmax_scale, bits, group,
                       dtype="fp16", cache_seqlens=None, k_res=None, v_res=None, res_lens=None):
    """Dequantize-then-attention from the four packed buffers (the path the
    decode entry point must match).  q is (b, 1, h, d) or (b, h, d)."""
    kc = unpack_k(k_pack, bits)
    vc = unpack_v(v_pack, bits)
    ks, kz = unpack_k_params(k_params, bits, group)
    vs, vz = unpack_v_params(v_params, bits, group)
    logical = dict(k_codes=kc, k_scale=ks, k_zero=kz, v_codes=vc, v_scale=vs, v_zero=vz)
    kd, vd = dequantize(logical, group, out_dtype=dtype)
    qf = to_f32(q, dtype)
    if qf.ndim == 4:
        qf = qf[:, 0]
    kr = None if k_res is None else to_f32(k_res, dtype)
    vr = None if v_res is None else to_f32(v_res, dtype)
    return decode_attention(qf, kd, vd, softmax_scale, cache_seqlens, kr, vr, res_lens)


def apply_rotary(x, cos, sin, positions, interleaved: bool, dtype: str = "fp16"):
    """Rotary embedding of one token per sequence, the arithmetic of the reference's dormant append path
    (csrc/bit_decode/src/include/rotary.h:56-63 interleaved pairs, :116-131 pairs half a rotary_dim apart).

    x: (b, heads, d) in `dtype` (fp16 array, or uint16 bf16 bit patterns); cos / sin: (positions, rotary_dim/2)
    likewise; positions: (b,) row of the tables per sequence.  For a pair (x0, x1):
        x0' = x0 cos - x1 sin,   x1' = x0 sin + x1 cos
    in fp32, every product and the sum rounded separately, then rounded once to `dtype`.  Dims from rotary_dim
    on are copied.  Returns an array like x."""
    xf = to_f32(x, dtype).copy()
    cf, sf = to_f32(cos, dtype), to_f32(sin, dtype)
    half = cf.shape[1]
    out = xf.copy()
    for ib in range(xf.shape[0]):
        c = cf[int(positions[ib])][None, :]
        s = sf[int(positions[ib])][None, :]
        if interleaved:
            x0, x1 = xf[ib, :, 0:2 * half:2], xf[ib, :, 1:2 * half:2]
        else:
            x0, x1 = xf[ib, :, :half], xf[ib, :, half:2 * half]
        y0 = (x0 * c).astype(np.float32) - (x1 * s).astype(np.float32)
        y1 = (x0 * s).astype(np.float32) + (x1 * c).astype(np.float32)
        if interleaved:
            out[ib, :, 0:2 * half:2], out[ib, :, 1:2 * half:2] = y0, y1
        else:
            out[ib, :, :half], out[ib, :, half:2 * half] = y0, y1
    if dtype == "bf16":
        return f32_to_bf16_bits(out)
    return out.astype(np.float16)
