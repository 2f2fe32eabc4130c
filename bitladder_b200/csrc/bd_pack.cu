// Quantize-pack kernel: K per channel (groups of G consecutive tokens), V per
// token (groups of G consecutive dims), asymmetric min-max to 4 or 2 bits.
//
// Arithmetic follows the reference quantizer step by step in IEEE fp32
// (reference: csrc/bit_decode/src/include/qpack.h:241-252 for range, scale_inv,
// stored scale and zero; :266-281 for subtract, multiply, roundf, clamp; :283-294
// for the field order inside a word).  Explicit round-to-nearest intrinsics keep
// the result independent of compiler flags, so codes, scales and zeros are
// bit-identical to a CPU evaluation of the same formulas, and to what the reference's kernel
// writes when it is built without --use_fast_math (4-bit, group 128 and 32).  PackParams::approx_div
// selects the division of the reference as shipped instead (see scale_from_minmax).
//
// One CTA handles one pack block (NB = 32 * 16/bits tokens) of one KV head.
// The work is pure streaming (read 2*NB*d*2 bytes, write a quarter or an eighth
// of that): every thread keeps 64 packed pairs in flight for K, rows are read
// and written in 128-byte warp segments, and nothing is re-read.
#include <type_traits>
#include "bd_common.cuh"
#include "bd_kernels.h"

namespace bd {

template <bool BF16>
__device__ __forceinline__ float2 pair_to_float2(uint32_t w) {
    if constexpr (BF16) {
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    } else {
        return __half22float2(*reinterpret_cast<__half2 *>(&w));
    }
}

// Running min / max of packed pairs in their own format (exact: no rounding is involved, and a
// NaN operand yields the other operand, like fminf / fmaxf).  +inf / -inf as the neutral starts.
template <bool BF16>
__device__ __forceinline__ uint32_t pair_min(uint32_t a, uint32_t b) {
    if constexpr (BF16) {
        __nv_bfloat162 r = __hmin2(*reinterpret_cast<__nv_bfloat162 *>(&a), *reinterpret_cast<__nv_bfloat162 *>(&b));
        return *reinterpret_cast<uint32_t *>(&r);
    } else {
        __half2 r = __hmin2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b));
        return *reinterpret_cast<uint32_t *>(&r);
    }
}
template <bool BF16>
__device__ __forceinline__ uint32_t pair_max(uint32_t a, uint32_t b) {
    if constexpr (BF16) {
        __nv_bfloat162 r = __hmax2(*reinterpret_cast<__nv_bfloat162 *>(&a), *reinterpret_cast<__nv_bfloat162 *>(&b));
        return *reinterpret_cast<uint32_t *>(&r);
    } else {
        __half2 r = __hmax2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b));
        return *reinterpret_cast<uint32_t *>(&r);
    }
}
template <bool BF16> constexpr uint32_t kPairPosInf = BF16 ? 0x7f807f80u : 0x7c007c00u;
template <bool BF16> constexpr uint32_t kPairNegInf = BF16 ? 0xff80ff80u : 0xfc00fc00u;

// Code of x as a bit field, in four instructions (subtract, multiply, add, logic op).
//   v = (x - mn) * scale_inv lies in [0, maxv + 1e-6] (x >= mn, and (mx - mn) * fl(maxv / (mx - mn))
//   exceeds maxv by a few ulps at most), or is NaN (NaN or infinite inputs), which the reference's
//   fminf(fmaxf(roundf(v), 0), maxv) turns into 0; its clamp from above never acts.
//   * The multiply is by scale_inv / 2^BITS (a power of two: the product is v / 2^BITS, rounded exactly
//     as v is) with saturation to [0, 1], which also turns NaN into 0: t = v / 2^BITS in [0, 1).
//   * t + (2^m + 2^-(BITS+1)), rounded toward zero, leaves floor(v + 0.5) = roundf(v) (v >= 0, ties
//     away from zero) in the mantissa at bit 23 - m - BITS and up: the ulp of the sum is 2^(m-23), the
//     half is representable beside 2^m for m <= 22 - BITS, and cutting first to that ulp and then to
//     the integer is one floor.  m is chosen per field so that the code lands where the field sits in
//     the 16-bit word (field 0 one bit higher, shifted down afterwards).
template <int BITS, int J>
__device__ __forceinline__ uint32_t put_field(uint32_t acc, float x, float mn, float scale_inv_div) {
    constexpr int kPos = (J == 0) ? 1 : BITS * J;                  // bit where the code lands
    constexpr int m = 23 - BITS - kPos;
    static_assert(m >= 0 && m <= 22 - BITS, "magic constant out of range");
    constexpr float kMagic = float(1u << m) + 1.0f / float(1u << (BITS + 1));
    float t;
    asm("mul.rn.sat.f32 %0, %1, %2;" : "=f"(t) : "f"(__fsub_rn(x, mn)), "f"(scale_inv_div));
    const uint32_t bits = __float_as_uint(__fadd_rz(t, kMagic));
    constexpr uint32_t kMask = ((1u << BITS) - 1u) << (BITS * J);
    if constexpr (J == 0) return acc | ((bits >> 1) & kMask);
    else return acc | (bits & kMask);
}

// approx_div: divide the way the reference does as it is shipped (built with --use_fast_math,
// setup.py:149): maxv / range becomes maxv times the GPU's approximate reciprocal, which is one ulp
// off the IEEE quotient in about a quarter of the groups and so moves a code by one step where
// (x - mn) * maxv / range is exactly k + 0.5.  Same bytes as that build on the same GPU; not
// reproducible on a CPU.  Default (0): IEEE division, the bytes the reference writes when built
// without that flag, and what a CPU evaluation of the formulas gives.
__device__ __forceinline__ void scale_from_minmax(float mn, float mx, float maxv, bool approx_div, float &scale_inv,
                                                  float &scale) {
    const float range = __fsub_rn(mx, mn);
    if (approx_div) {
        scale_inv = (range > 0.0f) ? __fdividef(maxv, range) : 0.0f;
        scale = (scale_inv == 0.0f) ? 0.0f : __fdividef(1.0f, scale_inv);
    } else {
        scale_inv = (range > 0.0f) ? __fdiv_rn(maxv, range) : 0.0f;
        scale = (scale_inv == 0.0f) ? 0.0f : __fdiv_rn(1.0f, scale_inv);
    }
}

// Where the parameters of (group g of the block / 128-token run, element c of 0..127) are stored:
// natural order, except 4-bit with group 32, where the reference keeps the order of its MMA
// fragments (csrc/bit_decode/src/flash_fwd_kernel.h:939-957 with num_params = 4): row
// 2*(g%2) + (c/8)%2, fp16 column 16*(c/16) + 8*(g/2) + c%8.  Pairs (c even, c + 1) stay adjacent.
template <int BITS, int GROUP>
__device__ __forceinline__ void param_slot(int g, int c, int &row, int &col) {
    if constexpr (BITS == 4 && GROUP == 32) {
        row = 2 * (g & 1) + ((c >> 3) & 1);
        col = 16 * (c >> 4) + 8 * (g >> 1) + (c & 7);
    } else {
        row = g;
        col = c;
    }
}

// Four token subsets of 64 threads per CTA; resident threads per SM (and with them the
// registers a thread may hold) chosen by measurement: 768 at 4 bits, 512 at 2 bits, where a
// thread keeps twice as many fields.
constexpr int kPackSubsets = 4;
constexpr int kPackThreads = 64 * kPackSubsets;
template <int BITS, int GROUP, bool BF16>
__global__ void __launch_bounds__(kPackThreads, (BITS == 4 ? 768 : 512) / kPackThreads)
bd_pack_kernel(const PackParams p) {
    constexpr int P = 16 / BITS;            // codes per 16-bit word
    constexpr int NB = 32 * P;              // tokens per pack block
    constexpr int NT = kPackSubsets;        // token subsets (threads = 64 * NT)
    constexpr int NTHREADS = 64 * NT;
    constexpr int PPT = 32 / NT;            // pack rows per thread (K)
    constexpr int NGK = NB / GROUP;         // K token groups per block
    constexpr int FPG = GROUP / 32;         // K fields per group
    constexpr int D = kHeadDim;
    constexpr int DP = D / P;               // words per V row
    constexpr int NGD = D / GROUP;          // V dim groups
    constexpr int FPGV = P / NGD;           // V fields per dim group
    const float maxv = static_cast<float>((1 << BITS) - 1);
    const bool approx_div = p.approx_div != 0;

    __shared__ float red[NT][NGK][2][D];
    __shared__ __half vprm[NGD][2][NB];

    const int tid = threadIdx.x;
    // heads vary fastest: CTAs that run together read neighbouring 256-byte pieces of the same token rows
    const int ih = blockIdx.x, blk = blockIdx.y, ib = blockIdx.z;
    int dst_off = p.dst_token_offset;
    if (p.roll_res_lens != nullptr) {          // roll-over: only sequences whose tail this step's token filled
        // The roll-over is staged early behind the decode kernel that files the token, and the kernel that moves
        // the lengths on is staged behind this one: every CTA waits for the decode kernel before it reads a tail
        // row or leaves (a CTA that left without waiting would let the lengths move under that kernel).
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (p.roll_res_lens[ib] + 1 != NB) return;
        dst_off = p.roll_cache_seqlens[ib];
        if (dst_off < 0 || dst_off % NB != 0 || dst_off + NB > p.roll_s_cap) return;   // no room: reported by the advance kernel
    }
    const int dst_blk = blk + dst_off / NB;
    const uint16_t *kin = static_cast<const uint16_t *>(p.k);
    const uint16_t *vin = static_cast<const uint16_t *>(p.v);

    // ------------------------------------------------------------------ K
    {
        const int cp = tid & 63, T = tid >> 6;
        const uint16_t *kbase = kin + ib * p.k_stride_b + static_cast<int64_t>(blk) * NB * p.k_stride_s +
                                ih * p.k_stride_h + 2 * cp;
        uint32_t raw[PPT][P];
#pragma unroll
        for (int pi = 0; pi < PPT; ++pi)
#pragma unroll
            for (int j = 0; j < P; ++j) {
                const int t = T * PPT + pi + 32 * j;
                raw[pi][j] = __ldg(reinterpret_cast<const unsigned int *>(kbase + t * p.k_stride_s));
            }
        float mn[NGK][2], mx[NGK][2];
        {
            uint32_t pmn[NGK], pmx[NGK];        // both channels at once, in the input format
#pragma unroll
            for (int gk = 0; gk < NGK; ++gk) { pmn[gk] = kPairPosInf<BF16>; pmx[gk] = kPairNegInf<BF16>; }
#pragma unroll
            for (int pi = 0; pi < PPT; ++pi)
#pragma unroll
                for (int j = 0; j < P; ++j) {
                    const int gk = j / FPG;
                    pmn[gk] = pair_min<BF16>(pmn[gk], raw[pi][j]);
                    pmx[gk] = pair_max<BF16>(pmx[gk], raw[pi][j]);
                }
#pragma unroll
            for (int gk = 0; gk < NGK; ++gk) {
                const float2 a = pair_to_float2<BF16>(pmn[gk]), b2 = pair_to_float2<BF16>(pmx[gk]);
                mn[gk][0] = a.x; mn[gk][1] = a.y; mx[gk][0] = b2.x; mx[gk][1] = b2.y;
            }
        }
#pragma unroll
        for (int gk = 0; gk < NGK; ++gk) {
            red[T][gk][0][2 * cp] = mn[gk][0]; red[T][gk][0][2 * cp + 1] = mn[gk][1];
            red[T][gk][1][2 * cp] = mx[gk][0]; red[T][gk][1][2 * cp + 1] = mx[gk][1];
        }
        __syncthreads();
        float sinv[NGK][2];
#pragma unroll
        for (int gk = 0; gk < NGK; ++gk)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float a = red[0][gk][0][2 * cp + e], b = red[0][gk][1][2 * cp + e];
#pragma unroll
                for (int t2 = 1; t2 < NT; ++t2) {
                    a = fminf(a, red[t2][gk][0][2 * cp + e]);
                    b = fmaxf(b, red[t2][gk][1][2 * cp + e]);
                }
                mn[gk][e] = a;
                float sc;
                scale_from_minmax(a, b, maxv, approx_div, sinv[gk][e], sc);
                sinv[gk][e] *= 1.0f / float(1 << BITS);      // exact; see put_field
                mx[gk][e] = sc;   // reuse as the stored scale
            }
        if (T == 0) {
#pragma unroll
            for (int gk = 0; gk < NGK; ++gk) {
                int prow, pcol;
                param_slot<BITS, GROUP>(gk, 2 * cp, prow, pcol);
                const int64_t grow = static_cast<int64_t>(dst_blk) * NGK + prow;
                __half *prm = reinterpret_cast<__half *>(p.k_params) +
                              2 * (ib * p.k_params_stride_b + (grow * p.h_k + ih) * D);
                *reinterpret_cast<__half2 *>(prm + pcol) = __floats2half2_rn(mx[gk][0], mx[gk][1]);
                *reinterpret_cast<__half2 *>(prm + D + pcol) = __floats2half2_rn(mn[gk][0], mn[gk][1]);
            }
        }
        uint16_t *kp = static_cast<uint16_t *>(p.k_pack) + ib * p.k_pack_stride_b +
                       ((static_cast<int64_t>(dst_blk) * 32 + T * PPT) * p.h_k + ih) * D + 2 * cp;
#pragma unroll
        for (int pi = 0; pi < PPT; ++pi) {
            uint32_t lo = 0, hi = 0;
            auto put = [&](auto jc) {
                constexpr int J = decltype(jc)::value;
                const float2 x = pair_to_float2<BF16>(raw[pi][J]);
                constexpr int gk = J / FPG;
                lo = put_field<BITS, J>(lo, x.x, mn[gk][0], sinv[gk][0]);
                hi = put_field<BITS, J>(hi, x.y, mn[gk][1], sinv[gk][1]);
            };
            put(std::integral_constant<int, 0>{}); put(std::integral_constant<int, 1>{});
            put(std::integral_constant<int, 2>{}); put(std::integral_constant<int, 3>{});
            if constexpr (P == 8) {
                put(std::integral_constant<int, 4>{}); put(std::integral_constant<int, 5>{});
                put(std::integral_constant<int, 6>{}); put(std::integral_constant<int, 7>{});
            }
            *reinterpret_cast<uint32_t *>(kp + static_cast<int64_t>(pi) * p.h_k * D) = lo | (hi << 16);
        }
    }

    // ------------------------------------------------------------------ V
    {
        // A thread owns 8 consecutive output words of one token (one 16-byte store) and so needs,
        // for every field j, the 8 dims  p0 + DP*j .. +7: P loads of 16 bytes.  DP/8 threads per token
        // (4 at 4 bits, 2 at 2 bits): the min/max over a token's group takes one or two shuffles.
        constexpr int TPT = DP / 8;              // threads per token
        constexpr int TPI = NTHREADS / TPT;      // tokens per iteration
        constexpr int VITER = NB / TPI;
        static_assert(VITER * TPI == NB, "token tiling");
        const int q8 = tid % TPT, tsub = tid / TPT;
        const uint16_t *vbase = vin + ib * p.v_stride_b + static_cast<int64_t>(blk) * NB * p.v_stride_s +
                                ih * p.v_stride_h + 8 * q8;
        uint16_t *vp = static_cast<uint16_t *>(p.v_pack) + ib * p.v_pack_stride_b +
                       (static_cast<int64_t>(dst_blk) * NB * p.h_k + ih) * DP + 8 * q8;
        uint4 raw[VITER][P];
#pragma unroll
        for (int u = 0; u < VITER; ++u) {
            const int t = u * TPI + tsub;
#pragma unroll
            for (int j = 0; j < P; ++j)
                raw[u][j] = __ldg(reinterpret_cast<const uint4 *>(vbase + t * p.v_stride_s + DP * j));
        }
#pragma unroll
        for (int u = 0; u < VITER; ++u) {
            const int t = u * TPI + tsub;
            float mn[NGD], mx[NGD];
            {
                uint32_t pmn[NGD], pmx[NGD];
#pragma unroll
                for (int gd = 0; gd < NGD; ++gd) { pmn[gd] = kPairPosInf<BF16>; pmx[gd] = kPairNegInf<BF16>; }
#pragma unroll
                for (int j = 0; j < P; ++j) {
                    const int gd = j / FPGV;
                    const uint32_t w4[4] = {raw[u][j].x, raw[u][j].y, raw[u][j].z, raw[u][j].w};
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        pmn[gd] = pair_min<BF16>(pmn[gd], w4[r]);
                        pmx[gd] = pair_max<BF16>(pmx[gd], w4[r]);
                    }
                }
#pragma unroll
                for (int gd = 0; gd < NGD; ++gd) {
                    const float2 a = pair_to_float2<BF16>(pmn[gd]), b2 = pair_to_float2<BF16>(pmx[gd]);
                    mn[gd] = fminf(a.x, a.y);
                    mx[gd] = fmaxf(b2.x, b2.y);
                }
            }
            float sinv[NGD];
#pragma unroll
            for (int gd = 0; gd < NGD; ++gd) {
#pragma unroll
                for (int off = 1; off < TPT; off <<= 1) {
                    mn[gd] = fminf(mn[gd], __shfl_xor_sync(0xffffffffu, mn[gd], off));
                    mx[gd] = fmaxf(mx[gd], __shfl_xor_sync(0xffffffffu, mx[gd], off));
                }
                float sc;
                scale_from_minmax(mn[gd], mx[gd], maxv, approx_div, sinv[gd], sc);
                sinv[gd] *= 1.0f / float(1 << BITS);         // exact; see put_field
                if (q8 == 0) {
                    vprm[gd][0][t] = __float2half_rn(sc);
                    vprm[gd][1][t] = __float2half_rn(mn[gd]);
                }
            }
            uint32_t outw[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                uint32_t lo = 0, hi = 0;
                auto put = [&](auto jc) {
                    constexpr int J = decltype(jc)::value;
                    const uint32_t w = r == 0 ? raw[u][J].x : (r == 1 ? raw[u][J].y : (r == 2 ? raw[u][J].z : raw[u][J].w));
                    const float2 x = pair_to_float2<BF16>(w);
                    constexpr int gd = J / FPGV;
                    lo = put_field<BITS, J>(lo, x.x, mn[gd], sinv[gd]);
                    hi = put_field<BITS, J>(hi, x.y, mn[gd], sinv[gd]);
                };
                put(std::integral_constant<int, 0>{}); put(std::integral_constant<int, 1>{});
                put(std::integral_constant<int, 2>{}); put(std::integral_constant<int, 3>{});
                if constexpr (P == 8) {
                    put(std::integral_constant<int, 4>{}); put(std::integral_constant<int, 5>{});
                    put(std::integral_constant<int, 6>{}); put(std::integral_constant<int, 7>{});
                }
                outw[r] = lo | (hi << 16);
            }
            *reinterpret_cast<uint4 *>(vp + static_cast<int64_t>(t) * p.h_k * DP) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
        }
        __syncthreads();
        // scales / zeros of this block's tokens: per dim group, per run of 128 tokens,
        // 128 scales then 128 zeros.
        constexpr int RUNS = NB / 128;
        const int64_t run0 = static_cast<int64_t>(dst_blk) * RUNS;
        for (int i = tid; i < NGD * RUNS * 2 * 64; i += NTHREADS) {
            const int w = i & 63;                  // pair index inside 128 values
            const int z = (i >> 6) & 1;            // 0 scales, 1 zeros
            const int run = (i >> 7) % RUNS;
            const int gd = (i >> 7) / RUNS;
            int plane, pcol;
            param_slot<BITS, GROUP>(gd, 2 * w, plane, pcol);
            __half *dst = reinterpret_cast<__half *>(p.v_params) +
                          2 * (ib * p.v_params_stride_b + plane * p.v_params_stride_g + ih * p.v_params_stride_h) +
                          256 * (run0 + run) + 128 * z + pcol;
            *reinterpret_cast<__half2 *>(dst) = *reinterpret_cast<const __half2 *>(&vprm[gd][z][128 * run + 2 * w]);
        }
    }
}

template <int BITS, int GROUP, bool BF16>
static cudaError_t launch_pack_t(const PackParams &p, cudaStream_t stream) {
    constexpr int NB = 32 * (16 / BITS);
    constexpr int NTHREADS = kPackThreads;
    dim3 grid(p.h_k, p.s / NB, p.b);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(NTHREADS);
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = p.roll_res_lens != nullptr ? 1 : 0;           // the roll-over of a decoder step only
    return cudaLaunchKernelEx(&cfg, bd_pack_kernel<BITS, GROUP, BF16>, p);
}

cudaError_t launch_pack(const PackParams &p, int bits, int group, int dtype, cudaStream_t stream) {
    const bool bf = dtype == BD_BF16;
    if (bits == 4 && group == 128) return bf ? launch_pack_t<4, 128, true>(p, stream) : launch_pack_t<4, 128, false>(p, stream);
    if (bits == 4 && group == 64)  return bf ? launch_pack_t<4, 64, true>(p, stream)  : launch_pack_t<4, 64, false>(p, stream);
    if (bits == 2 && group == 128) return bf ? launch_pack_t<2, 128, true>(p, stream) : launch_pack_t<2, 128, false>(p, stream);
    if (bits == 2 && group == 64)  return bf ? launch_pack_t<2, 64, true>(p, stream)  : launch_pack_t<2, 64, false>(p, stream);
    if (bits == 4 && group == 32)  return bf ? launch_pack_t<4, 32, true>(p, stream)  : launch_pack_t<4, 32, false>(p, stream);
    if (bits == 2 && group == 32)  return bf ? launch_pack_t<2, 32, true>(p, stream)  : launch_pack_t<2, 32, false>(p, stream);
    return cudaErrorInvalidValue;
}

}  // namespace bd
