// Split-KV decode attention over the packed low-bit KV cache (one query token
// per sequence), written for sm_100a.
//
// What it computes matches the reference's split-KV kernel (reference:
// csrc/bit_decode/src/flash_fwd_kernel.h:66-728 with the dequantisation of
// csrc/bit_decode/src/include/dequantize.h:253-384 and the online softmax of
// csrc/bit_decode/src/include/softmax.h:188-309); how it computes it does not:
//
//  * One CTA = (KV head, sequence split, batch).  Warp 4 is a TMA producer; warps
//    0-3 are consumers.  Each consumer owns whole pack blocks (NB tokens) and a
//    private ring of RD shared-memory slots, so K and V tiles of later blocks
//    stream in while a block is being processed, and no consumer ever waits for
//    another: each keeps its own running (max, sum, O) and the four are merged
//    once at the end with the log-sum-exp rule.
//  * Packed codes go global -> shared with tiled TMA copies (128-byte swizzle
//    for K, 64/32-byte swizzle for V, which makes the transposing ldmatrix on V
//    bank-conflict free), completion on mbarriers.
//  * The GQA query group is the N dimension of mma.m16n8k16 and tokens (for
//    QK^T) / head dims (for PV) are the M dimension, so a packed 32-bit word
//    turns into A-fragment registers with one AND per field: the masked field
//    is read as an fp16 subnormal (code * 2^-24 * 16^k), which the tensor core
//    multiplies exactly; the power-of-two factor is folded into the softmax
//    scale (K) or the epilogue (V).
//  * The affine part of the dequantisation is folded out of the inner loop:
//    per-channel K scales multiply q once per token group, K zeros contribute
//    q.zero per group (one extra row of MMAs), per-token V scales multiply the
//    probabilities, V zeros contribute sum_t p_t zero_t (one extra MMA per 16
//    tokens).  Products are exact in fp32; only q*scale and p*scale are rounded
//    to fp16.
//
// tcgen05 is not used: its MMA needs M >= 64 rows of real work per instruction
// and operands staged through shared memory or TMEM, while this kernel has at
// most 16 query rows and is bound by HBM bandwidth, not tensor throughput.
#include "bd_common.cuh"
#include "bd_kernels.h"

#ifndef BD_SUBNORMAL_CODES
#define BD_SUBNORMAL_CODES 1
#endif

namespace bd {

constexpr int kConsumerWarps = 4;
constexpr int kDecodeThreads = (kConsumerWarps + 1) * 32;
constexpr int kTailMax = 256;          // longest unquantized tail the kernel accepts
constexpr int kPartStride = 132;       // floats per (row) in the epilogue partials (bank spread)

template <int BITS, int GROUP, int NQT>
struct Cfg {
    static constexpr int P = 16 / BITS;
    static constexpr int NB = 32 * P;
    static constexpr int NGK = NB / GROUP;              // K token groups per block
    static constexpr int FPG = GROUP / 32;              // K fields per token group
    static constexpr int NGD = kHeadDim / GROUP;        // V dim groups
    static constexpr int FPGV = P / NGD;                // V fields per dim group
    static constexpr int DP = kHeadDim / P;             // 16-bit words per V row
    static constexpr int RUNS = NB / 128;               // 128-token runs per block (V params)
    static constexpr int PRM_BYTES = 512 * NGK;         // == NGD * RUNS * 512
    static constexpr int CODE_BYTES = 8192;
    static constexpr int RD = (PRM_BYTES <= 1024) ? 3 : 2;   // ring depth per consumer warp
    static constexpr int NSLOT = RD * kConsumerWarps;
    static constexpr int QROWS = NQT * 8;
    static constexpr size_t OFF_PRM = size_t(NSLOT) * CODE_BYTES;
    static constexpr size_t OFF_BAR = OFF_PRM + size_t(NSLOT) * PRM_BYTES;
    static constexpr size_t SMEM = OFF_BAR + 2 * NSLOT * 8 + 16 + 1024;   // + alignment slack
    // epilogue / tail scratch live in the (then idle) ring memory
    static constexpr size_t OFF_PART = 0;                                  // [5][QROWS][kPartStride] f32
    static constexpr size_t OFF_ML = OFF_PART + size_t(5) * QROWS * kPartStride * 4;   // [5][QROWS][2] f32
    static constexpr size_t OFF_TAIL = OFF_ML + size_t(5) * QROWS * 2 * 4;             // [QROWS][kTailMax] f32
    static_assert(OFF_TAIL + size_t(QROWS) * kTailMax * 4 <= OFF_PRM, "epilogue scratch must fit in the ring");
};

// Field j of a packed word as two fp16 lanes.  `wsh` is the word shifted right
// by 8 (4-bit) or 10 (2-bit) so that every field lands inside the fp16 mantissa.
template <int BITS, int J>
__device__ __forceinline__ uint32_t field(uint32_t w, uint32_t wsh) {
    uint32_t x;
    if constexpr (BITS == 4) {
        constexpr uint32_t m = (J & 1) ? 0x00f000f0u : 0x000f000fu;
        x = ((J & 2) ? wsh : w) & m;
    } else {
        constexpr uint32_t m = 0x00030003u << (2 * (J < 5 ? J : J - 5));
        x = ((J < 5) ? w : wsh) & m;
    }
#if !BD_SUBNORMAL_CODES
    x |= 0x64006400u;   // 1024 + code * 16^k, then remove the 1024 exactly
    __half2 h = __hsub2(*reinterpret_cast<__half2 *>(&x), __half2half2(__ushort_as_half(0x6400)));
    x = *reinterpret_cast<uint32_t *>(&h);
#endif
    return x;
}
// Value of the fp16 lane produced by field<J> divided by the code.
template <int BITS>
__host__ __device__ constexpr float field_weight(int j) {
    float f = 1.0f;
    if (BITS == 4) {
        f = (j & 1) ? 16.0f : 1.0f;
    } else {
        int e = j < 5 ? j : j - 5;
        for (int i = 0; i < e; ++i) f *= 4.0f;
    }
#if BD_SUBNORMAL_CODES
    return f * (1.0f / 16777216.0f);
#else
    return f;
#endif
}

__device__ __forceinline__ void consumer_bar() {
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
}

template <bool BF16>
__device__ __forceinline__ void load4(const void *ptr, float (&x)[4]) {
    const uint2 w = *reinterpret_cast<const uint2 *>(ptr);
    if constexpr (BF16) {
        x[0] = __uint_as_float(w.x << 16); x[1] = __uint_as_float(w.x & 0xffff0000u);
        x[2] = __uint_as_float(w.y << 16); x[3] = __uint_as_float(w.y & 0xffff0000u);
    } else {
        float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&w.x));
        float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&w.y));
        x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
    }
}
__device__ __forceinline__ float load1(const void *base, int64_t idx, bool bf16) {
    const uint16_t v = static_cast<const uint16_t *>(base)[idx];
    return bf16 ? __uint_as_float(static_cast<uint32_t>(v) << 16) : __half2float(__ushort_as_half(v));
}

// Unquantized tail: softmax partial over res_n fp16/bf16 tokens, computed by the
// four consumer warps with plain FMAs (the tail is at most kTailMax tokens).
// Leaves O (unnormalised), row max (log2 units) and row sum in partial slot 4.
template <int NQT>
__device__ void tail_partial(const DecodeParams &p, uint8_t *smem, int ib, int ih, int res_n, int tid) {
    constexpr int QROWS = NQT * 8;
    using C = Cfg<4, 128, NQT>;   // only the scratch offsets, identical for every config
    float *part = reinterpret_cast<float *>(smem + C::OFF_PART) + 4 * QROWS * kPartStride;
    float *ml = reinterpret_cast<float *>(smem + C::OFF_ML) + 4 * QROWS * 2;
    float *sc = reinterpret_cast<float *>(smem + C::OFF_TAIL);
    const int warp = tid >> 5, lane = tid & 31;
    const bool bf = p.dtype == BD_BF16;
    const int64_t esz = 2;
    const uint8_t *kres = static_cast<const uint8_t *>(p.k_res) +
                          (ib * p.res_stride_b + ih * p.res_stride_h) * esz;
    const uint8_t *vres = static_cast<const uint8_t *>(p.v_res) +
                          (ib * p.res_stride_b + ih * p.res_stride_h) * esz;
    // 1. scores
    float qv[QROWS][4];
#pragma unroll
    for (int r = 0; r < QROWS; ++r) {
        if (r < p.gq) {
            const uint8_t *qp = static_cast<const uint8_t *>(p.q) +
                                (ib * p.q_stride_b + (int64_t(ih) * p.gq + r) * p.q_stride_h + 4 * lane) * esz;
            if (bf) load4<true>(qp, qv[r]); else load4<false>(qp, qv[r]);
        } else {
            qv[r][0] = qv[r][1] = qv[r][2] = qv[r][3] = 0.f;
        }
    }
    for (int t = warp; t < res_n; t += kConsumerWarps) {
        float kv[4];
        const uint8_t *kp = kres + (int64_t(t) * p.res_stride_s + 4 * lane) * esz;
        if (bf) load4<true>(kp, kv); else load4<false>(kp, kv);
#pragma unroll
        for (int r = 0; r < QROWS; ++r) {
            float d = qv[r][0] * kv[0] + qv[r][1] * kv[1] + qv[r][2] * kv[2] + qv[r][3] * kv[3];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
            if (lane == 0) sc[r * kTailMax + t] = d * p.scale_log2;
        }
    }
    consumer_bar();
    // 2. softmax per query row
    for (int r = warp; r < QROWS; r += kConsumerWarps) {
        float mx = -INFINITY;
        for (int t = lane; t < res_n; t += 32) mx = fmaxf(mx, sc[r * kTailMax + t]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        float sum = 0.f;
        for (int t = lane; t < res_n; t += 32) {
            const float e = ex2f(sc[r * kTailMax + t] - mx);
            sc[r * kTailMax + t] = e;
            sum += e;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        if (lane == 0) { ml[2 * r] = mx; ml[2 * r + 1] = sum; }
    }
    consumer_bar();
    // 3. weighted sum of V rows; thread = head dim
    float acc[QROWS];
#pragma unroll
    for (int r = 0; r < QROWS; ++r) acc[r] = 0.f;
    for (int t = 0; t < res_n; ++t) {
        const float v = load1(vres, int64_t(t) * p.res_stride_s + tid, bf);
#pragma unroll
        for (int r = 0; r < QROWS; ++r) acc[r] = fmaf(sc[r * kTailMax + t], v, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < QROWS; ++r) part[r * kPartStride + tid] = acc[r];
}

template <int BITS, int GROUP, int NQT>
__global__ void __launch_bounds__(kDecodeThreads, 2)
bd_decode_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap kmap,
                 const __grid_constant__ CUtensorMap vmap) {
    using C = Cfg<BITS, GROUP, NQT>;
    constexpr int P = C::P, NB = C::NB, NGK = C::NGK, FPG = C::FPG, NGD = C::NGD, FPGV = C::FPGV;
    constexpr int DP = C::DP, RUNS = C::RUNS, PRM = C::PRM_BYTES, RD = C::RD, NSLOT = C::NSLOT;
    constexpr int QROWS = C::QROWS;

    extern __shared__ uint8_t smem_unaligned[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_base + uint32_t(C::OFF_BAR);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (NSLOT + s); };
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + C::OFF_BAR + 2 * NSLOT * 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ih = blockIdx.x, split = blockIdx.y, ib = blockIdx.z;

    int seqlen = p.s;
    if (p.cache_seqlens) seqlen = min(max(p.cache_seqlens[ib], 0), p.s);
    const int nblk = (seqlen + NB - 1) / NB;
    const int nsplit_b = max(1, (nblk + p.chunk_blocks - 1) / p.chunk_blocks);
    if (split >= nsplit_b) return;                       // whole CTA: nothing to do for this sequence
    const int blk_begin = split * p.chunk_blocks;
    const int nloc = max(0, min(nblk, blk_begin + p.chunk_blocks) - blk_begin);
    int res_n = 0;
    if (p.k_res != nullptr && split == nsplit_b - 1) {
        res_n = p.res_lens ? p.res_lens[ib] : p.res_len;
        res_n = min(max(res_n, 0), kTailMax);
    }

    if (tid == 0) {
        for (int s = 0; s < NSLOT; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        *abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();

    // ======================================================================
    // producer warp
    // ======================================================================
    if (warp == kConsumerWarps) {
        if (lane == 0) {
            tma_prefetch_desc(&kmap);
            tma_prefetch_desc(&vmap);
            const uint16_t *kprm_g = p.k_params + ib * p.k_params_stride_b;
            const uint16_t *vprm_g = p.v_params + ib * p.v_params_stride_b + ih * p.v_params_stride_h;
            for (int i = 0; i < nloc; ++i) {
                const int blk = blk_begin + i;
                const int cw = i % kConsumerWarps;
                const int lseq = 2 * (i / kConsumerWarps);
                // ---- K slot
                {
                    const int slot = cw * RD + lseq % RD;
                    const uint32_t par = (lseq / RD) & 1;
                    if (!mbar_wait_bounded(empty_bar(slot), par ^ 1)) { *abort_flag = 1; break; }
                    const uint32_t dst = smem_base + slot * C::CODE_BYTES;
                    const uint32_t prm = smem_base + uint32_t(C::OFF_PRM) + slot * PRM;
                    mbar_arrive_expect_tx(full_bar(slot), C::CODE_BYTES + PRM);
                    const int row0 = ib * p.k_batch_rows + blk * 32;
                    tma_load_2d(dst, &kmap, full_bar(slot), ih * kHeadDim, row0);
                    tma_load_2d(dst + 4096, &kmap, full_bar(slot), ih * kHeadDim + 64, row0);
#pragma unroll
                    for (int gk = 0; gk < NGK; ++gk)
                        bulk_load_1d(prm + gk * 512,
                                     kprm_g + ((int64_t(blk) * NGK + gk) * p.h_k + ih) * (2 * kHeadDim), 512,
                                     full_bar(slot));
                }
                // ---- V slot
                {
                    const int slot = cw * RD + (lseq + 1) % RD;
                    const uint32_t par = ((lseq + 1) / RD) & 1;
                    if (!mbar_wait_bounded(empty_bar(slot), par ^ 1)) { *abort_flag = 1; break; }
                    const uint32_t dst = smem_base + slot * C::CODE_BYTES;
                    const uint32_t prm = smem_base + uint32_t(C::OFF_PRM) + slot * PRM;
                    mbar_arrive_expect_tx(full_bar(slot), C::CODE_BYTES + PRM);
                    tma_load_2d(dst, &vmap, full_bar(slot), ih * DP, ib * p.v_batch_rows + blk * NB);
#pragma unroll
                    for (int gd = 0; gd < NGD; ++gd)
                        bulk_load_1d(prm + gd * (RUNS * 512),
                                     vprm_g + gd * p.v_params_stride_g + int64_t(blk) * RUNS * 256, RUNS * 512,
                                     full_bar(slot));
                }
            }
        }
        return;
    }

    // ======================================================================
    // consumer warps
    // ======================================================================
    const int g = lane >> 2, l = lane & 3;
    const bool bf16 = p.dtype == BD_BF16;

    // Query rows as B fragments: thread (g, l) holds q[row g][32a + 8l .. +7], a = 0..3.
    uint32_t qr[NQT][4][4];
#pragma unroll
    for (int nq = 0; nq < NQT; ++nq) {
        const int row = nq * 8 + g;
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < p.gq) {
                const uint16_t *qp = static_cast<const uint16_t *>(p.q) + ib * p.q_stride_b +
                                     (int64_t(ih) * p.gq + row) * p.q_stride_h + 32 * a + 8 * l;
                v = *reinterpret_cast<const uint4 *>(qp);
                if (bf16) {
                    v.x = bf16x2_to_f16x2(v.x); v.y = bf16x2_to_f16x2(v.y);
                    v.z = bf16x2_to_f16x2(v.z); v.w = bf16x2_to_f16x2(v.w);
                }
            }
            qr[nq][a][0] = v.x; qr[nq][a][1] = v.y; qr[nq][a][2] = v.z; qr[nq][a][3] = v.w;
        }
    }

    // thread-constant shared-memory offsets
    // K tile: two halves of 64 channels, each [32 pack rows][128 B] with the 128-byte
    // TMA swizzle (16-byte chunk index XOR row % 8); this thread reads rows g and g + 8.
    const uint32_t k_row_off = g * 128;
    const uint32_t k_chunk_off[2] = {uint32_t((l ^ g) << 4), uint32_t(((4 + l) ^ g) << 4)};
    const int v_slot = (lane & 7) + 8 * ((lane >> 4) & 1);                 // token slot this lane addresses
    const int v_cpar = (lane >> 3) & 1;
    uint32_t v_off[2];
    if constexpr (BITS == 4) {
        v_off[0] = v_slot * 64 + (((0 + v_cpar) ^ ((v_slot >> 1) & 3)) << 4);
        v_off[1] = v_slot * 64 + (((2 + v_cpar) ^ ((v_slot >> 1) & 3)) << 4);
    } else {
        v_off[0] = v_slot * 32 + ((v_cpar ^ ((v_slot >> 2) & 1)) << 4);
        v_off[1] = 0;
    }

    float O[8][NQT][4];
    float ZS[NQT][4];
    float m_run[NQT][2], l_run[NQT][2];
#pragma unroll
    for (int nq = 0; nq < NQT; ++nq) {
#pragma unroll
        for (int mt = 0; mt < 8; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) O[mt][nq][e] = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) ZS[nq][e] = 0.f;
        m_run[nq][0] = m_run[nq][1] = -INFINITY;
        l_run[nq][0] = l_run[nq][1] = 0.f;
    }

    bool aborted = false;
    for (int i = warp; i < nloc; i += kConsumerWarps) {
        const int blk = blk_begin + i;
        const int lseq = 2 * (i / kConsumerWarps);
        const int kslot = warp * RD + lseq % RD;
        const int vslot = warp * RD + (lseq + 1) % RD;
        const uint32_t kpar = (lseq / RD) & 1, vpar = ((lseq + 1) / RD) & 1;
        const uint32_t kcode = smem_base + kslot * C::CODE_BYTES;
        const uint32_t kprm = smem_base + uint32_t(C::OFF_PRM) + kslot * PRM;
        const uint32_t vcode = smem_base + vslot * C::CODE_BYTES;
        const uint32_t vprm = smem_base + uint32_t(C::OFF_PRM) + vslot * PRM;
        const bool need_mask = (blk + 1) * NB > seqlen;

        // ------------------------------------------------------------ K phase
        if (!mbar_wait_bounded(full_bar(kslot), kpar)) { aborted = true; break; }

        // q . zero per token group (rows of the A operand all equal the zero vector)
        float Zc[NGK][NQT][2];
        {
            float Z[NGK][NQT][4];
#pragma unroll
            for (int gk = 0; gk < NGK; ++gk)
#pragma unroll
                for (int nq = 0; nq < NQT; ++nq)
#pragma unroll
                    for (int e = 0; e < 4; ++e) Z[gk][nq][e] = 0.f;
#pragma unroll
            for (int gk = 0; gk < NGK; ++gk)
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    uint32_t z0, z1, z2, z3;
                    lds128(kprm + gk * 512 + 256 + (32 * a + 8 * l) * 2, z0, z1, z2, z3);
#pragma unroll
                    for (int nq = 0; nq < NQT; ++nq) {
                        mma_f16(Z[gk][nq], z0, z0, z1, z1, qr[nq][a][0], qr[nq][a][1]);
                        mma_f16(Z[gk][nq], z2, z2, z3, z3, qr[nq][a][2], qr[nq][a][3]);
                    }
                }
#pragma unroll
            for (int gk = 0; gk < NGK; ++gk)
#pragma unroll
                for (int nq = 0; nq < NQT; ++nq) {
                    Zc[gk][nq][0] = Z[gk][nq][0] * p.scale_log2;
                    Zc[gk][nq][1] = Z[gk][nq][1] * p.scale_log2;
                }
        }

        // With one token group per block, q * scale is computed once per block.
        uint32_t qs1[NQT][4][4];
        if constexpr (NGK == 1) {
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                uint32_t s0, s1, s2, s3;
                lds128(kprm + (32 * a + 8 * l) * 2, s0, s1, s2, s3);
#pragma unroll
                for (int nq = 0; nq < NQT; ++nq) {
                    qs1[nq][a][0] = hmul2_u32(qr[nq][a][0], s0);
                    qs1[nq][a][1] = hmul2_u32(qr[nq][a][1], s1);
                    qs1[nq][a][2] = hmul2_u32(qr[nq][a][2], s2);
                    qs1[nq][a][3] = hmul2_u32(qr[nq][a][3], s3);
                }
            }
        }
        uint32_t Pb[2][P][NQT][2];      // probabilities as B fragments (fp16), per unit and field
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            float S[P][NQT][4];
#pragma unroll
            for (int j = 0; j < P; ++j)
#pragma unroll
                for (int nq = 0; nq < NQT; ++nq)
#pragma unroll
                    for (int e = 0; e < 4; ++e) S[j][nq][e] = 0.f;
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                // q * scale for the token groups of this block, channels 32a + 8l .. +7
                uint32_t qs[NGK][NQT][4];
                if constexpr (NGK == 1) {
#pragma unroll
                    for (int nq = 0; nq < NQT; ++nq)
#pragma unroll
                        for (int x = 0; x < 4; ++x) qs[0][nq][x] = qs1[nq][a][x];
                } else {
#pragma unroll
                    for (int gk = 0; gk < NGK; ++gk) {
                        uint32_t s0, s1, s2, s3;
                        lds128(kprm + gk * 512 + (32 * a + 8 * l) * 2, s0, s1, s2, s3);
#pragma unroll
                        for (int nq = 0; nq < NQT; ++nq) {
                            qs[gk][nq][0] = hmul2_u32(qr[nq][a][0], s0);
                            qs[gk][nq][1] = hmul2_u32(qr[nq][a][1], s1);
                            qs[gk][nq][2] = hmul2_u32(qr[nq][a][2], s2);
                            qs[gk][nq][3] = hmul2_u32(qr[nq][a][3], s3);
                        }
                    }
                }
                uint32_t wl[4], wh[4];
                const uint32_t base = kcode + (a >> 1) * 4096 + u * 2048 + k_row_off + k_chunk_off[a & 1];
                lds128(base, wl[0], wl[1], wl[2], wl[3]);
                lds128(base + 1024, wh[0], wh[1], wh[2], wh[3]);
                uint32_t wls[4], whs[4];
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    wls[x] = wl[x] >> (BITS == 4 ? 8 : 10);
                    whs[x] = wh[x] >> (BITS == 4 ? 8 : 10);
                }
                // fields (compile-time index) -> one MMA per (field, k-slice)
                auto do_field = [&](auto jc) {
                    constexpr int J = decltype(jc)::value;
                    constexpr int gk = J / FPG;
#pragma unroll
                    for (int nq = 0; nq < NQT; ++nq) {
                        mma_f16(S[J][nq], field<BITS, J>(wl[0], wls[0]), field<BITS, J>(wh[0], whs[0]),
                                field<BITS, J>(wl[1], wls[1]), field<BITS, J>(wh[1], whs[1]),
                                qs[gk][nq][0], qs[gk][nq][1]);
                        mma_f16(S[J][nq], field<BITS, J>(wl[2], wls[2]), field<BITS, J>(wh[2], whs[2]),
                                field<BITS, J>(wl[3], wls[3]), field<BITS, J>(wh[3], whs[3]),
                                qs[gk][nq][2], qs[gk][nq][3]);
                    }
                };
                do_field(std::integral_constant<int, 0>{});
                do_field(std::integral_constant<int, 1>{});
                do_field(std::integral_constant<int, 2>{});
                do_field(std::integral_constant<int, 3>{});
                if constexpr (P == 8) {
                    do_field(std::integral_constant<int, 4>{});
                    do_field(std::integral_constant<int, 5>{});
                    do_field(std::integral_constant<int, 6>{});
                    do_field(std::integral_constant<int, 7>{});
                }
            }

            // ---------------------------------------------- online softmax (this unit)
#pragma unroll
            for (int nq = 0; nq < NQT; ++nq) {
                float t[P][4];
                float cmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < P; ++j) {
                    const float mj = p.scale_log2 * (1.0f / field_weight<BITS>(j));
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float x = fmaf(S[j][nq][e], mj, Zc[j / FPG][nq][e & 1]);
                        if (need_mask) {
                            const int tok = blk * NB + 16 * u + 32 * j + g + 8 * (e >> 1);
                            if (tok >= seqlen) x = -INFINITY;
                        }
                        t[j][e] = x;
                        cmax[e & 1] = fmaxf(cmax[e & 1], x);
                    }
                }
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    cmax[c] = fmaxf(cmax[c], __shfl_xor_sync(0xffffffffu, cmax[c], 4));
                    cmax[c] = fmaxf(cmax[c], __shfl_xor_sync(0xffffffffu, cmax[c], 8));
                    cmax[c] = fmaxf(cmax[c], __shfl_xor_sync(0xffffffffu, cmax[c], 16));
                }
                float mnew[2], msafe[2];
                bool changed = false;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    mnew[c] = fmaxf(m_run[nq][c], cmax[c]);
                    msafe[c] = (mnew[c] == -INFINITY) ? 0.f : mnew[c];
                    changed |= (mnew[c] != m_run[nq][c]);
                }
                if (__any_sync(0xffffffffu, changed)) {
                    float f[2];
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        f[c] = ex2f(m_run[nq][c] - msafe[c]);
                        l_run[nq][c] *= f[c];
                        m_run[nq][c] = mnew[c];
                    }
#pragma unroll
                    for (int mt = 0; mt < 8; ++mt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) O[mt][nq][e] *= f[e & 1];
#pragma unroll
                    for (int e = 0; e < 4; ++e) ZS[nq][e] *= f[e & 1];
                    if (u == 1) {
                        // The first unit's probabilities are still waiting (as B fragments,
                        // column = g) for the V phase: bring them to the new maximum too.
                        const float f0 = __shfl_sync(0xffffffffu, f[0], g >> 1);
                        const float f1 = __shfl_sync(0xffffffffu, f[1], g >> 1);
                        const float fq = (g & 1) ? f1 : f0;
                        const uint32_t fh = pack_f16x2(fq, fq);
#pragma unroll
                        for (int j = 0; j < P; ++j) {
                            Pb[0][j][nq][0] = hmul2_u32(Pb[0][j][nq][0], fh);
                            Pb[0][j][nq][1] = hmul2_u32(Pb[0][j][nq][1], fh);
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < P; ++j) {
                    float pe[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        pe[e] = ex2f(t[j][e] - msafe[e & 1]);
                        l_run[nq][e & 1] += pe[e];
                    }
                    Pb[u][j][nq][0] = movmatrix_trans(pack_f16x2(pe[0], pe[1]));
                    Pb[u][j][nq][1] = movmatrix_trans(pack_f16x2(pe[2], pe[3]));
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(kslot));

        // ------------------------------------------------------------ V phase
        if (!mbar_wait_bounded(full_bar(vslot), vpar)) { aborted = true; break; }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
#pragma unroll
            for (int j = 0; j < P; ++j) {
                const int T0 = 16 * u + 32 * j;                       // first token of this k-slice
                const int r0 = T0 + 2 * l;                            // tokens of fragment register 0
                const uint32_t pofs = (r0 >> 7) * 512 + (r0 & 127) * 2;   // run, position (r0+8 stays in the run)
                uint32_t sc0[NGD], sc1[NGD], ze0[NGD], ze1[NGD];
#pragma unroll
                for (int gd = 0; gd < NGD; ++gd) {
                    const uint32_t b0 = vprm + gd * (RUNS * 512) + pofs;
                    sc0[gd] = lds32(b0);
                    sc1[gd] = lds32(b0 + 16);
                    ze0[gd] = lds32(b0 + 256);
                    ze1[gd] = lds32(b0 + 256 + 16);
                    if (need_mask) {      // params of tokens past the end may be uninitialised
                        const int tok = blk * NB + r0;
                        const uint32_t k0 = (tok < seqlen ? 0x0000ffffu : 0u) | (tok + 1 < seqlen ? 0xffff0000u : 0u);
                        const uint32_t k1 = (tok + 8 < seqlen ? 0x0000ffffu : 0u) | (tok + 9 < seqlen ? 0xffff0000u : 0u);
                        sc0[gd] &= k0; ze0[gd] &= k0; sc1[gd] &= k1; ze1[gd] &= k1;
                    }
                }
                uint32_t pv[NGD][NQT][2];
#pragma unroll
                for (int nq = 0; nq < NQT; ++nq) {
                    // sum_t p_t * zero_t  (rows 0-7: dim group 0, rows 8-15: dim group 1)
                    mma_f16(ZS[nq], ze0[0], ze0[NGD - 1], ze1[0], ze1[NGD - 1], Pb[u][j][nq][0], Pb[u][j][nq][1]);
#pragma unroll
                    for (int gd = 0; gd < NGD; ++gd) {
                        pv[gd][nq][0] = hmul2_u32(Pb[u][j][nq][0], sc0[gd]);
                        pv[gd][nq][1] = hmul2_u32(Pb[u][j][nq][1], sc1[gd]);
                    }
                }
                constexpr int NCB = (BITS == 4) ? 2 : 1;              // ldmatrix.x4 per k-slice
#pragma unroll
                for (int cb = 0; cb < NCB; ++cb) {
                    uint32_t r0w, r1w, r2w, r3w;
                    ldsm_x4_trans(vcode + T0 * (DP * 2) + v_off[cb], r0w, r1w, r2w, r3w);
                    const uint32_t s0w = r0w >> (BITS == 4 ? 8 : 10), s1w = r1w >> (BITS == 4 ? 8 : 10);
                    const uint32_t s2w = r2w >> (BITS == 4 ? 8 : 10), s3w = r3w >> (BITS == 4 ? 8 : 10);
                    auto do_vfield = [&](auto jc) {
                        constexpr int JV = decltype(jc)::value;
                        constexpr int gd = JV / FPGV;
                        const int mt = (BITS == 4) ? (cb * 4 + JV) : JV;
#pragma unroll
                        for (int nq = 0; nq < NQT; ++nq)
                            mma_f16(O[mt][nq], field<BITS, JV>(r0w, s0w), field<BITS, JV>(r1w, s1w),
                                    field<BITS, JV>(r2w, s2w), field<BITS, JV>(r3w, s3w),
                                    pv[gd][nq][0], pv[gd][nq][1]);
                    };
                    do_vfield(std::integral_constant<int, 0>{});
                    do_vfield(std::integral_constant<int, 1>{});
                    do_vfield(std::integral_constant<int, 2>{});
                    do_vfield(std::integral_constant<int, 3>{});
                    if constexpr (P == 8) {
                        do_vfield(std::integral_constant<int, 4>{});
                        do_vfield(std::integral_constant<int, 5>{});
                        do_vfield(std::integral_constant<int, 6>{});
                        do_vfield(std::integral_constant<int, 7>{});
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(vslot));
    }
    if (aborted) *abort_flag = 1;

    // ======================================================================
    // epilogue: merge the four warp partials (+ the tail) and write the result
    // ======================================================================
    // Drain: a consumer that gave up must still see every copy that was issued for
    // it complete before the block's shared memory may be reused or released.
    consumer_bar();
    const bool any_abort = *abort_flag != 0;
    if (any_abort) {
        if (tid == 0) atomicExch(p.status, BD_ERR_TIMEOUT);
        // give copies that are still in flight time to land before the block's
        // shared memory is released
        for (int it = 0; it < 2000; ++it) __nanosleep(1000);
        consumer_bar();
        return;
    }

    float *part = reinterpret_cast<float *>(smem + C::OFF_PART);
    float *ml = reinterpret_cast<float *>(smem + C::OFF_ML);
    {
        float *mypart = part + warp * QROWS * kPartStride;
#pragma unroll
        for (int nq = 0; nq < NQT; ++nq) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float s = l_run[nq][c];
                s += __shfl_xor_sync(0xffffffffu, s, 4);
                s += __shfl_xor_sync(0xffffffffu, s, 8);
                s += __shfl_xor_sync(0xffffffffu, s, 16);
                if (g == 0) {
                    ml[(warp * QROWS + nq * 8 + 2 * l + c) * 2] = m_run[nq][c];
                    ml[(warp * QROWS + nq * 8 + 2 * l + c) * 2 + 1] = s;
                }
            }
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                const int jv = (BITS == 4) ? (mt & 3) : mt;
                const int pbase = (BITS == 4) ? 16 * (mt >> 2) : 0;
                const float wgt = 1.0f / field_weight<BITS>(jv);
                const int gd = jv / FPGV;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int dim = pbase + g + 8 * (e >> 1) + DP * jv;
                    const int row = nq * 8 + 2 * l + (e & 1);
                    const float zs = ZS[nq][(gd == 0 ? 0 : 2) + (e & 1)];
                    mypart[row * kPartStride + dim] = fmaf(O[mt][nq][e], wgt, zs);
                }
            }
        }
    }
    if (res_n > 0) {
        consumer_bar();
        tail_partial<NQT>(p, smem, ib, ih, res_n, tid);
    } else if (tid < QROWS) {
        ml[(4 * QROWS + tid) * 2] = -INFINITY;
        ml[(4 * QROWS + tid) * 2 + 1] = 0.f;
    }
    consumer_bar();

    // thread = head dim; loop over the query rows of this KV head
    for (int r = 0; r < p.gq; ++r) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 5; ++w) M = fmaxf(M, ml[(w * QROWS + r) * 2]);
        float L = 0.f, acc = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 5; ++w) {
                const float mw = ml[(w * QROWS + r) * 2];
                if (mw != -INFINITY) {
                    const float f = ex2f(mw - M);
                    L = fmaf(ml[(w * QROWS + r) * 2 + 1], f, L);
                    acc = fmaf(part[(w * QROWS + r) * kPartStride + tid], f, acc);
                }
            }
        }
        const float o = (L > 0.f) ? acc / L : 0.f;
        const float lse = (L > 0.f) ? fmaf(M, 0.6931471805599453f, logf(L)) : -INFINITY;
        const int hq = ih * p.gq + r;
        if (p.num_splits > 1) {
            const int64_t prow = (int64_t(ib) * p.h + hq) * p.num_splits + split;
            p.part_out[prow * kHeadDim + tid] = o;
            if (tid == 0) p.part_lse[prow] = lse;
        } else {
            const int64_t oidx = ib * p.out_stride_b + int64_t(hq) * p.out_stride_h + tid;
            if (p.out_dtype == BD_FP16) static_cast<__half *>(p.out)[oidx] = __float2half_rn(o);
            else if (p.out_dtype == BD_BF16) static_cast<__nv_bfloat16 *>(p.out)[oidx] = __float2bfloat16_rn(o);
            else static_cast<float *>(p.out)[oidx] = o;
            if (tid == 0 && p.lse) p.lse[int64_t(ib) * p.h + hq] = lse;
        }
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
template <int BITS, int GROUP, int NQT>
static cudaError_t launch_t(const DecodeParams &p, const CUtensorMap &kmap, const CUtensorMap &vmap,
                            cudaStream_t stream) {
    using C = Cfg<BITS, GROUP, NQT>;
    auto kern = bd_decode_kernel<BITS, GROUP, NQT>;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 64 && !configured[dev]) {
        err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(C::SMEM));
        if (err != cudaSuccess) return err;
        configured[dev] = true;
    }
    dim3 grid(p.h_k, p.num_splits, p.b);
    kern<<<grid, kDecodeThreads, C::SMEM, stream>>>(p, kmap, vmap);
    return cudaGetLastError();
}

template <int BITS, int GROUP>
static cudaError_t launch_bg(const DecodeParams &p, const CUtensorMap &kmap, const CUtensorMap &vmap,
                             cudaStream_t stream) {
    if (p.gq <= 8) return launch_t<BITS, GROUP, 1>(p, kmap, vmap, stream);
    return launch_t<BITS, GROUP, 2>(p, kmap, vmap, stream);
}

cudaError_t launch_decode(const DecodeParams &p, const CUtensorMap &kmap, const CUtensorMap &vmap,
                          int bits, int group, cudaStream_t stream) {
    if (bits == 4 && group == 128) return launch_bg<4, 128>(p, kmap, vmap, stream);
    if (bits == 4 && group == 64) return launch_bg<4, 64>(p, kmap, vmap, stream);
    if (bits == 2 && group == 128) return launch_bg<2, 128>(p, kmap, vmap, stream);
    if (bits == 2 && group == 64) return launch_bg<2, 64>(p, kmap, vmap, stream);
    return cudaErrorInvalidValue;
}

size_t decode_smem_bytes(int bits, int group, int gq) {
    const int nqt = gq <= 8 ? 1 : 2;
    if (bits == 4 && group == 128) return nqt == 1 ? Cfg<4, 128, 1>::SMEM : Cfg<4, 128, 2>::SMEM;
    if (bits == 4 && group == 64) return nqt == 1 ? Cfg<4, 64, 1>::SMEM : Cfg<4, 64, 2>::SMEM;
    if (bits == 2 && group == 128) return nqt == 1 ? Cfg<2, 128, 1>::SMEM : Cfg<2, 128, 2>::SMEM;
    if (bits == 2 && group == 64) return nqt == 1 ? Cfg<2, 64, 1>::SMEM : Cfg<2, 64, 2>::SMEM;
    return 0;
}

int decode_ctas_per_sm_default() { return 2; }

}  // namespace bd
