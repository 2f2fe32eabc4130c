// Split-KV decode attention over the packed low-bit KV cache (one query token
// per sequence), written for sm_100a.
//
// What it computes matches the reference's split-KV kernel (reference:
// csrc/bit_decode/src/flash_fwd_kernel.h:66-728 with the dequantisation of
// csrc/bit_decode/src/include/dequantize.h:253-384 and the online softmax of
// csrc/bit_decode/src/include/softmax.h:188-309); how it computes it does not:
//
//  * Work is cut into equal ranges of units (pack blocks, then chunks of the unquantized
//    tail) per KV head (see Partition in bd_kernels.h), one CTA per (range, head), one CTA
//    per SM, every CTA resident at once; inside the CTA the same cut gives every warp one
//    contiguous range.
//  * A CTA is up to twelve independent warps.  Each warp owns whole pack blocks (NB
//    tokens), two shared-memory slots (one K tile, one V tile) and their
//    mbarriers, and refills a slot itself, with TMA, as soon as it has consumed
//    it: the next block's K streams in during the V phase and vice versa.  No
//    warp ever waits for another, anywhere in the kernel; each keeps its own running
//    (max, sum, O).  At the end of a sequence's share the warps that hold a part of it
//    deposit their partials and count in; the last to count in merges them in a fixed
//    order, and the CTA that finishes a sequence last merges the CTAs' parts the same
//    way.  The unquantized fp16/bf16 tail goes through the same tensor-core path and
//    the same running state.
//  * Packed codes go global -> shared with tiled TMA copies (128-byte swizzle
//    for K, 64/32-byte swizzle for V, which makes the transposing ldmatrix on V
//    bank-conflict free), completion on mbarriers.
//  * The GQA query group is the N dimension of mma.m16n8k16 and tokens (for
//    QK^T) / head dims (for PV) are the M dimension, so a packed 32-bit word
//    turns into A-fragment registers with one AND per field: the masked field
//    is read as an fp16 subnormal (code * 2^-24 * 16^k), which the tensor core
//    multiplies exactly; the power-of-two factor is folded into the softmax
//    scale (K) or the epilogue (V).  4-bit words come apart in byte pairs (see field()).
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
#include <type_traits>

#include "bd_common.cuh"
#include "bd_kernels.h"

#ifndef BD_SUBNORMAL_CODES
#define BD_SUBNORMAL_CODES 1
#endif

namespace bd {

#ifdef BD_TRACE
// Timing trace for development builds only (-DBD_TRACE): per CTA its SM, start, the time every warp
// left the streaming loop, and the CTA's end, in nanoseconds of the global timer.
__device__ unsigned long long g_trace[4096 * 32];
__device__ unsigned long long g_trace2[4096 * 64];      // per warp: loop entry, after 1, 2, 4 blocks (slots 16 w + k)
#define BD_TRACE_WARP(k) do { if (lane == 0 && blockIdx.x < 4096 && warp < 16) g_trace2[blockIdx.x * 64 + 4 * warp + (k)] = trace_now(); } while (0)
__device__ __forceinline__ unsigned long long trace_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define BD_TRACE_MARK(slot) do { if (lane == 0 && blockIdx.x < 4096) g_trace[blockIdx.x * 32 + (slot)] = trace_now(); } while (0)
__device__ __forceinline__ unsigned trace_smid() {
    unsigned r;
    asm volatile("mov.u32 %0, %smid;" : "=r"(r));
    return r;
}
#endif

#ifndef BD_TRACE
#define BD_TRACE_WARP(k) do { } while (0)
#define BD_TRACE_MARK(slot) do { } while (0)
#endif

#ifndef BD_MAX_WARPS
#define BD_MAX_WARPS 12
#endif
// Streaming warps per CTA: as many as fit one CTA per SM, at most this (three per
// scheduler; 384 threads keep 168 registers each).  All warps of an SM then belong to
// one CTA and have the same age: with several CTAs per SM the scheduler favoured the
// warps of the CTA that was launched first and the others finished up to 40 % later.
constexpr int kMaxWarps = BD_MAX_WARPS;
constexpr int kSmemLimit = 232448;     // 227 KB of shared memory per CTA
constexpr float kRescaleSlack = 8.0f;  // keep a stale row max until it is exceeded by 2^8

// TWO = 1: half as many warps per CTA and two CTAs per SM.  One CTA of twelve same-age warps per SM is
// the faster arrangement wherever rows * KV heads fills the machine; with many KV heads (rows are tied
// to whole KV heads: 32 heads leave 20 of 148 SMs without a CTA) twice as many smaller CTAs fill it better.
template <int BITS, int GROUP, int NQT, int TWO = 0>
struct Cfg {
    static constexpr int P = 16 / BITS;
    static constexpr int NB = 32 * P;
    static constexpr int NGK = NB / GROUP;              // K token groups per block
    static constexpr int FPG = GROUP / 32;              // K fields per token group
    static constexpr int NGD = kHeadDim / GROUP;        // V dim groups
    static constexpr int NZ = (NGD + 1) / 2;            // accumulators of sum_t p_t * zero_t (two dim groups each)
    static constexpr int FPGV = P / NGD;                // V fields per dim group
    static constexpr int DP = kHeadDim / P;             // 16-bit words per V row
    static constexpr int RUNS = NB / 128;               // 128-token runs per block (V params)
    static constexpr int PRM_BYTES = 512 * NGK;         // == NGD * RUNS * 512
    static constexpr int CODE_BYTES = 8192;             // one K tile (32 pack rows) or one V tile (NB tokens)
    static constexpr int QROWS = NQT * 8;
    static constexpr int NACC = 8 * NQT * 4 + 4 * NQT;  // floats per thread handed over in a merge
    // per warp: one K tile and one V tile, then their scales/zeros
    static constexpr int WARP_BYTES = 2 * CODE_BYTES + 2 * PRM_BYTES + 16;
    static constexpr int FIT = (kSmemLimit - 32) / (WARP_BYTES + 32);
    // Twelve warps leave a thread 168 registers (three warps per scheduler; so do 9 to 11).  One query tile
    // fits them at 4 bits and, taking a block unit by unit, at 2 bits (C3 48.4 -> 44.6 us, C5a 2-bit 349 ->
    // 340 us against eight warps with 255 registers); two query tiles and group 32 (four parameter sets per
    // block) need more and run eight warps.
    static constexpr int CAP = (NQT == 1 && GROUP >= 64) ? kMaxWarps : (kMaxWarps < 8 ? kMaxWarps : 8);
    static constexpr int WARPS = (FIT < CAP ? FIT : CAP) / (TWO ? 2 : 1);
    static constexpr int THREADS = WARPS * 32;
    static constexpr size_t OFF_PRM = size_t(WARPS) * 2 * CODE_BYTES;
    static constexpr size_t OFF_BAR = OFF_PRM + size_t(WARPS) * 2 * PRM_BYTES;
    static constexpr size_t OFF_FLAGS = OFF_BAR + 2 * WARPS * 8;            // abort flag, arrivals[WARPS], segment notes[WARPS][4]
    static constexpr size_t OFF_NOTES = OFF_FLAGS + 16 + ((WARPS * 4 + 15) / 16) * 16;
    static constexpr size_t SMEM = OFF_NOTES + WARPS * 16;
    static constexpr int DEPOSIT_FLOATS = NACC * 32;                        // one warp's share of a segment
    static_assert(DEPOSIT_FLOATS * 4 <= 2 * CODE_BYTES, "a deposit fits the warp's own tile slots");
    static constexpr int CTAS_PER_SM = (SMEM + 1024) * 3 <= 233472 ? 3 : ((SMEM + 1024) * 2 <= 233472 ? 2 : 1);
    static_assert(WARPS >= 1 && WARPS < 16, "one mask bit per warp; the segment notes use lanes 0..WARPS and 16, 17");
    static_assert(SMEM <= size_t(kSmemLimit), "shared memory");
};

// A packed 32-bit register (two 16-bit words) and the helper word the field extraction
// needs: 4-bit: the high bytes of both words moved to the low bytes (one byte permute);
// 2-bit: the register shifted right by 10.
template <int BITS>
__device__ __forceinline__ uint32_t aux_word(uint32_t w) {
    if constexpr (BITS == 4) return __byte_perm(w, 0u, 0x4341u);
    else return w >> 10;
}
// Field j of a packed word as two fp16 lanes, every field inside the fp16 mantissa.
//
// 4-bit words are taken apart in PAIRS: an even field comes out together with the odd
// field above it (f_j + 16 f_{j+1}, a whole byte: still an exact fp16 subnormal), the odd
// field alone (16 f_{j+1}).  The products are linear, so the even field's sum is the
// difference of the two accumulators, taken once after the last MMA; that saves the
// shift and one of the masks on the high byte.  kFieldPairs tells the callers (with one field
// per quantization group, group 32, the two fields of a byte have different scales and every
// field is masked out alone).
template <int BITS, int J, bool PAIRS>
__device__ __forceinline__ uint32_t field(uint32_t w, uint32_t aux) {
    uint32_t x;
    if constexpr (BITS == 4) {
        if constexpr (J == 0) x = w & (PAIRS ? 0x00ff00ffu : 0x000f000fu);
        else if constexpr (J == 1) x = w & 0x00f000f0u;
        else if constexpr (J == 2) x = PAIRS ? aux : (aux & 0x000f000fu);
        else x = aux & 0x00f000f0u;
    } else {
        constexpr uint32_t m = 0x00030003u << (2 * (J < 5 ? J : J - 5));
        x = ((J < 5) ? w : aux) & m;
    }
#if !BD_SUBNORMAL_CODES
    x |= 0x64006400u;   // 1024 + value, then remove the 1024 exactly
    __half2 h = __hsub2(*reinterpret_cast<__half2 *>(&x), __half2half2(__ushort_as_half(0x6400)));
    x = *reinterpret_cast<uint32_t *>(&h);
#endif
    return x;
}
// Pairs need both fields of a byte to meet the same scale: two or more fields per group.
template <int BITS, int GROUP> constexpr bool kFieldPairs = (BITS == 4 && GROUP >= 64);
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

// Byte offset, inside a warp's K parameter tile, of the 8 scales of token group gk for channels
// 32a + 8l .. +7 (the zeros sit 256 bytes on), and inside its V parameter tile of the scales of
// tokens r0, r0 + 1 (hi = 0) or r0 + 8, r0 + 9 (hi = 1) of dim group gd, r0 even with r0 % 16 < 8.
// Natural order, except 4-bit with group 32: the reference's fragment order (element c of group g in
// row 2*(g%2) + (c/8)%2, column 16*(c/16) + 8*(g/2) + c%8; flash_fwd_kernel.h:939-957).
template <int BITS, int GROUP>
__device__ __forceinline__ uint32_t kprm_off(int gk, int a, int l) {
    if constexpr (BITS == 4 && GROUP == 32) return (2 * (gk & 1) + (l & 1)) * 512 + (16 * (2 * a + (l >> 1)) + 8 * (gk >> 1)) * 2;
    else return gk * 512 + (32 * a + 8 * l) * 2;
}
template <int BITS, int GROUP>
__device__ __forceinline__ uint32_t vprm_off(int gd, int r0, int hi) {
    constexpr int RUNS = (32 * (16 / BITS)) / 128;
    if constexpr (BITS == 4 && GROUP == 32) return (2 * (gd & 1) + hi) * 512 + (16 * (r0 >> 4) + 8 * (gd >> 1) + (r0 & 7)) * 2;
    else return gd * (RUNS * 512) + (r0 >> 7) * 512 + (r0 & 127) * 2 + 16 * hi;
}

// One online-softmax step for NT score tiles (m16n8 accumulators, columns = query
// rows).  On entry t holds the scores in log2 units MINUS the running maximum of
// their column (minus 0 while the column has no maximum yet); on exit it holds
// the probabilities.  The running max moves lazily: only when it is exceeded by
// more than 2^kRescaleSlack, so probabilities stay below 2^8 and the accumulators
// are rescaled a handful of times per sequence.  With ACC_L the probabilities are
// also added to l_run (otherwise the caller gets the row sums elsewhere).
// Returns true when a rescale happened (f holds the factor per column parity).
template <int NT, bool ACC_L, int NZ>
__device__ __forceinline__ bool softmax_step(float (&t)[NT][4], float (&m_run)[2], float (&l_run)[2],
                                             float (&O)[8][4], float (&ZS)[NZ][4], float (&f)[2]) {
    float cmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) cmax[e & 1] = fmaxf(cmax[e & 1], t[j][e]);
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        cmax[c] = fmaxf(cmax[c], __shfl_xor_sync(0xffffffffu, cmax[c], 4));
        cmax[c] = fmaxf(cmax[c], __shfl_xor_sync(0xffffffffu, cmax[c], 8));
        cmax[c] = fmaxf(cmax[c], __shfl_xor_sync(0xffffffffu, cmax[c], 16));
    }
    bool changed = false;
#pragma unroll
    for (int c = 0; c < 2; ++c)
        changed |= cmax[c] > kRescaleSlack || (m_run[c] == -INFINITY && cmax[c] != -INFINITY);
    const bool any = __any_sync(0xffffffffu, changed);
    if (any) {
        float shift[2];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const bool first = m_run[c] == -INFINITY;
            const bool move = cmax[c] > kRescaleSlack || (first && cmax[c] != -INFINITY);
            shift[c] = move ? cmax[c] : 0.f;
            f[c] = move ? (first ? 0.f : ex2f(-cmax[c])) : 1.f;
            if (move) m_run[c] = (first ? 0.f : m_run[c]) + cmax[c];
            l_run[c] *= f[c];
        }
#pragma unroll
        for (int mt = 0; mt < 8; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) O[mt][e] *= f[e & 1];
#pragma unroll
        for (int z = 0; z < NZ; ++z)
#pragma unroll
            for (int e = 0; e < 4; ++e) ZS[z][e] *= f[e & 1];
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) t[j][e] -= shift[e & 1];
    }
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            t[j][e] = ex2f(t[j][e]);
            if (ACC_L) l_run[e & 1] += t[j][e];
        }
    return any;
}

// This warp's position in its stream of pack blocks: walks the segments of the warp's
// row and, inside a segment, its pack blocks in order (tail chunks, the units behind a
// sequence's blocks, are not copied by TMA and are skipped here).
struct BlockCursor {
    SegWalk walk;
    Segment sg;
    const int32_t *cache_seqlens;
    int32_t s, block_tokens;
    int32_t u, uend;
    bool valid;

    __device__ __forceinline__ bool seek() {
        while (walk.next(sg)) {
            const int32_t nblk = seq_blocks(cache_seqlens ? cache_seqlens[sg.ib] : s, s, block_tokens);
            u = sg.u0;
            uend = sg.u1 < nblk ? sg.u1 : nblk;
            if (u < uend) return true;
        }
        return false;
    }
    // starts from a walk that stands at the beginning of the warp's row
    __device__ __forceinline__ void init(const SegWalk &start, const int32_t *cs, int32_t s_, int32_t nb) {
        walk = start;
        cache_seqlens = cs; s = s_; block_tokens = nb;
        valid = seek();
    }
    __device__ __forceinline__ void advance() {
        if (++u < uend) return;
        valid = seek();
    }
};

template <int BITS, int GROUP, int NQT, int TWO>
__global__ void __launch_bounds__(Cfg<BITS, GROUP, NQT, TWO>::THREADS, Cfg<BITS, GROUP, NQT, TWO>::CTAS_PER_SM)
bd_decode_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap kmap,
                 const __grid_constant__ CUtensorMap vmap) {
    using C = Cfg<BITS, GROUP, NQT, TWO>;
    constexpr int P = C::P, NB = C::NB, NGK = C::NGK, FPG = C::FPG, NGD = C::NGD, FPGV = C::FPGV;
    constexpr int DP = C::DP, RUNS = C::RUNS, PRM = C::PRM_BYTES, NACC = C::NACC, NZ = C::NZ;
    constexpr int kWarps = C::WARPS;

    // The swizzled TMA tiles need a 1024-byte aligned base; dynamic shared memory
    // starts at the beginning of the CTA's window, which is, and the kernel checks it.
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t smem_base = smem_u32(smem);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + C::OFF_FLAGS);
    int *arrivals = reinterpret_cast<int *>(smem + C::OFF_FLAGS + 16);     // per first sharing warp of a segment

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ih = blockIdx.x % p.h_k, row = blockIdx.x / p.h_k;
    const int g = lane >> 2, l = lane & 3;
    int4 *note = reinterpret_cast<int4 *>(smem + C::OFF_NOTES) + warp;       // this warp's notes on its current segment
#ifdef BD_TRACE
    if (tid == 0 && blockIdx.x < 4096) {
        g_trace[blockIdx.x * 32 + 0] = trace_smid();
        g_trace[blockIdx.x * 32 + 1] = trace_now();
    }
#endif
    if ((smem_base & 1023u) != 0) {                      // never seen; refuse rather than read garbage
        if (tid == 0) atomicExch(p.status, BD_ERR_ALIGNMENT);
        return;
    }

    // this warp's slots and barriers
    const uint32_t kcode = smem_base + (warp * 2) * C::CODE_BYTES;
    const uint32_t vcode = kcode + C::CODE_BYTES;
    const uint32_t kprm = smem_base + uint32_t(C::OFF_PRM) + (warp * 2) * PRM;
    const uint32_t vprm = kprm + PRM;
    const uint32_t kbar = smem_base + uint32_t(C::OFF_BAR) + warp * 16;
    const uint32_t vbar = kbar + 8;

    if (lane == 0) {
        mbar_init(kbar, 1);
        mbar_init(vbar, 1);
        if (warp == 0) *abort_flag = 0;
        arrivals[warp] = 0;
        fence_mbar_init();
        tma_prefetch_desc(&kmap);
        tma_prefetch_desc(&vmap);
    }
    BD_TRACE_MARK(25);
    // The warps are the rows of the partition with kWarps times the CTA rows.
    Partition wpart = p.part;
    wpart.R = p.part.R * kWarps;
    const int wrow = row * kWarps + warp;

    // ---- TMA issue (one lane) ------------------------------------------------
    // Paged cache: block `blk` of sequence `ib` sits in page block_table[ib][blk / blocks_per_page]
    // at block blk % blocks_per_page; the page takes the place of the batch index in every address
    // below (pages are laid out exactly like the sequences of a contiguous cache).
    // A page index outside the pool is never used as an address: the copy then reads page 0
    // (in bounds), the block is masked where it is consumed and the status word reports it.
    auto resolve = [&](int &ib, int &blk) -> bool {
        if (p.block_table == nullptr) return true;
        const int pg = blk / p.blocks_per_page;
        blk -= pg * p.blocks_per_page;
        const int page = p.block_table[int64_t(ib) * p.block_table_stride + pg];
        const bool ok = page >= 0 && page < p.num_pages;
        ib = ok ? page : 0;
        return ok;
    };
    bool starve = p.test_starve != 0 && blockIdx.x == 0;     // test hook: the first K copy of every warp of CTA 0
    auto issue_k = [&](int ib, int blk) {
        resolve(ib, blk);
        mbar_arrive_expect_tx(kbar, C::CODE_BYTES + PRM + (starve ? 16 : 0));
        starve = false;
        const int row0 = ib * p.k_batch_rows + blk * 32;
        tma_load_2d(kcode, &kmap, kbar, ih * kHeadDim, row0);
        tma_load_2d(kcode + 4096, &kmap, kbar, ih * kHeadDim + 64, row0);
        const uint16_t *src = p.k_params + ib * p.k_params_stride_b;
#pragma unroll
        for (int gk = 0; gk < NGK; ++gk)
            bulk_load_1d(kprm + gk * 512, src + ((int64_t(blk) * NGK + gk) * p.h_k + ih) * (2 * kHeadDim), 512, kbar);
    };
    auto issue_v = [&](int ib, int blk) {
        resolve(ib, blk);
        mbar_arrive_expect_tx(vbar, C::CODE_BYTES + PRM);
        tma_load_2d(vcode, &vmap, vbar, ih * DP, ib * p.v_batch_rows + blk * NB);
        const uint16_t *src = p.v_params + ib * p.v_params_stride_b + ih * p.v_params_stride_h;
#pragma unroll
        for (int gd = 0; gd < NGD; ++gd)
            bulk_load_1d(vprm + gd * (RUNS * 512), src + gd * p.v_params_stride_g + int64_t(blk) * RUNS * 256,
                         RUNS * 512, vbar);
    };

    // ---- prologue: first block of this warp ------------------------------------
    SegWalk walk;                   // this warp's segments, in order
    if (wpart.table != nullptr) {
        // ragged batch: the sequence that holds the first unit of this warp's range, looked for by all lanes
        // at once (smallest ib with first(ib) + count(ib) > f0 or first(ib) >= f0; one round per 32 sequences)
        const int64_t Tw = wpart.total();
        const int64_t f0 = wpart.row_begin(wrow, Tw);
        int start = wpart.b;
        for (int base = 0; base < wpart.b; base += 32) {
            const int i = base + lane;
            bool ok = false;
            if (i < wpart.b) {
                const int2 e = *reinterpret_cast<const int2 *>(wpart.table + 2 * i);
                ok = int64_t(e.x) + e.y > f0 || int64_t(e.x) >= f0;
            }
            const uint32_t m = __ballot_sync(0xffffffffu, ok);
            if (m != 0) { start = base + __ffs(m) - 1; break; }
        }
        walk.init_at(wpart, wrow, Tw, start);
    } else {
        walk.init(wpart, wrow);
    }
    BD_TRACE_MARK(26);
    BlockCursor ld;                 // next block to copy into this warp's tiles
    ld.init(walk, p.cache_seqlens, p.s, NB);
    BD_TRACE_MARK(27);
    if (ld.valid && lane == 0) {
        issue_k(ld.sg.ib, ld.u);
        issue_v(ld.sg.ib, ld.u);
    }
    if (ld.valid) { BD_TRACE_MARK(20); }
    if (ld.valid) ld.advance();
    __syncthreads();          // every warp's flags and barriers are set up (its own first copies are already on their way)

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
    float mjs[P];          // softmax scale times the inverse field weight
#pragma unroll
    for (int j = 0; j < P; ++j) mjs[j] = p.scale_log2 * (1.0f / field_weight<BITS>(j));

    const bool bf16 = p.dtype == BD_BF16;
    uint32_t phase = 0;    // parity of both barriers: one completion each per consumed block
    bool aborted = false;

    Segment sg;
    while (walk.next(sg)) {
        const int ib = sg.ib;
        if (sg.u1 <= sg.u0) {
            // A sequence without any token, answered for by this warp: the defined result is
            // out = 0, lse = -inf.
            if (sg.owns_empty) {
                for (int qrow = 0; qrow < p.gq; ++qrow) {
                    const int64_t hq = int64_t(ih) * p.gq + qrow;
                    const int64_t oi = ib * p.out_stride_b + hq * p.out_stride_h + 4 * lane;
                    if (p.out_dtype == BD_FP32) {
                        *reinterpret_cast<float4 *>(static_cast<float *>(p.out) + oi) = make_float4(0.f, 0.f, 0.f, 0.f);
                    } else {                       // fp16 and bf16 zeros are the same bits
                        *reinterpret_cast<uint2 *>(static_cast<uint16_t *>(p.out) + oi) = make_uint2(0u, 0u);
                    }
                    if (lane == 0 && p.lse) p.lse[int64_t(ib) * p.h + hq] = -INFINITY;
                }
            }
            continue;
        }
        int seqlen = p.s;
        if (p.cache_seqlens) seqlen = min(max(p.cache_seqlens[ib], 0), p.s);
        int res_n = 0;                                // tail tokens of this sequence
        if (p.k_res != nullptr) res_n = min(max(p.res_lens ? p.res_lens[ib] : p.res_len, 0), min(kTailMax, p.res_cap));
        // Fused append: the token of this step is tail row res_old.  It is read from k_new / v_new
        // (nobody reads that row of the tail buffers during this launch) and the warp that streams
        // it also stores it there, for the steps to come.
        const int res_old = res_n;
        const bool has_new = p.k_new != nullptr && res_n < min(kTailMax, p.res_cap);
        if (has_new) res_n += 1;
        // this warp's units of the sequence: pack blocks [blk0, blk1), tail tokens [tail0, tail1)
        const int nblk = (seqlen + NB - 1) / NB;
        const int blk0 = sg.u0, blk1 = min(sg.u1, nblk);
        const int tail0 = max(sg.u0 - nblk, 0) * kTailChunk, tail1 = min(max(sg.u1 - nblk, 0) * kTailChunk, res_n);
        if (has_new && res_old >= tail0 && res_old < tail1 && res_old < p.res_cap) {
            // this warp streams the chunk that holds the new row: it also files the row in the tail
            // buffers (8 bytes of K and of V per lane), as it came
            const int64_t src = ib * p.new_stride_b + ih * p.new_stride_h + 4 * lane;
            const int64_t dst = ib * p.res_stride_b + ih * p.res_stride_h + int64_t(res_old) * p.res_stride_s + 4 * lane;
            const uint2 kw = __ldg(reinterpret_cast<const uint2 *>(static_cast<const uint16_t *>(p.k_new) + src));
            const uint2 vw = __ldg(reinterpret_cast<const uint2 *>(static_cast<const uint16_t *>(p.v_new) + src));
            *reinterpret_cast<uint2 *>(static_cast<uint16_t *>(p.k_res_out) + dst) = kw;
            *reinterpret_cast<uint2 *>(static_cast<uint16_t *>(p.v_res_out) + dst) = vw;
        }

        // Query rows as B fragments: thread (g, l) holds q[row g][32a + 8l .. +7], a = 0..3.
        uint32_t qr[NQT][4][4];
#pragma unroll
        for (int nq = 0; nq < NQT; ++nq) {
            const int qrow = nq * 8 + g;
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                uint4 v = make_uint4(0, 0, 0, 0);
                if (qrow < p.gq) {
                    const uint16_t *qp = static_cast<const uint16_t *>(p.q) + ib * p.q_stride_b +
                                         (int64_t(ih) * p.gq + qrow) * p.q_stride_h + 32 * a + 8 * l;
                    v = *reinterpret_cast<const uint4 *>(qp);
                    if (bf16) {
                        v.x = bf16x2_to_f16x2(v.x); v.y = bf16x2_to_f16x2(v.y);
                        v.z = bf16x2_to_f16x2(v.z); v.w = bf16x2_to_f16x2(v.w);
                    }
                }
                qr[nq][a][0] = v.x; qr[nq][a][1] = v.y; qr[nq][a][2] = v.z; qr[nq][a][3] = v.w;
            }
        }

        // Which warps of this CTA share the sequence, which of them goes on with another sequence
        // afterwards, and how many CTA rows hold a part of it: worked out now, while the first copies
        // and the query loads are in flight, and kept in shared memory (not in registers across the
        // streaming loop).  One division per lane: lanes 0..kWarps the first unit of each warp's range,
        // lanes 16 and 17 the first and the last CTA row that holds a part of the sequence.
        {
            const int64_t Tw = wpart.total();
            const int64_t seq_first = wpart.first(ib), seq_n = wpart.count(ib), seq_end = seq_first + seq_n;
            int64_t num = (int64_t(row) * kWarps + lane) * Tw, den = wpart.R;
            if (lane >= 16) {
                num = (seq_first + (lane == 16 ? 1 : seq_n)) * p.part.R - 1;
                den = Tw;
            }
            const int64_t quo = div_nn(num, den > 0 ? den : 1);
            const int64_t lo = quo, hi = __shfl_down_sync(0xffffffffu, quo, 1);
            const bool shares = lane < kWarps && max(lo, seq_first) < min(hi, seq_end);
            const uint32_t share_mask = __ballot_sync(0xffffffffu, shares);
            const uint32_t on_mask = __ballot_sync(0xffffffffu, shares && hi > seq_end);
            const int goes_on = on_mask ? 31 - __clz(on_mask) : -1;
            PartRange pr{0, -1, true};
            if (seq_n > 0 && Tw > 0) {
                pr.c0 = int(__shfl_sync(0xffffffffu, quo, 16));
                pr.c1 = int(__shfl_sync(0xffffffffu, quo, 17));
                pr.dense = Tw >= p.part.R;
            }
            int nparts = pr.c1 - pr.c0 + 1;
            if (!pr.dense) {
                nparts = 0;
                for (int c = pr.c0; c <= pr.c1; ++c) nparts += row_has_part(p.part, ib, c) ? 1 : 0;
            }
            if (lane == 0)
                *note = make_int4(int(share_mask), (goes_on + 1) | ((pr.c1 - pr.c0 + 1) << 8), pr.c0, (nparts << 1) | (pr.dense ? 1 : 0));
            __syncwarp();
        }

        float O[NQT][8][4];
        float ZS[NQT][NZ][4];
        float m_run[NQT][2], l_run[NQT][2];
#pragma unroll
        for (int nq = 0; nq < NQT; ++nq) {
#pragma unroll
            for (int mt = 0; mt < 8; ++mt)
#pragma unroll
                for (int e = 0; e < 4; ++e) O[nq][mt][e] = 0.f;
#pragma unroll
            for (int z = 0; z < NZ; ++z)
#pragma unroll
                for (int e = 0; e < 4; ++e) ZS[nq][z][e] = 0.f;
            m_run[nq][0] = m_run[nq][1] = -INFINITY;
            l_run[nq][0] = l_run[nq][1] = 0.f;
        }

        // ------------------------------------------------------------------
        // Unquantized tail (fp16 / bf16 rows), 16 tokens per step, spread over the
        // warps: K rows are A fragments as they are (128-bit loads), V rows are
        // transposed in registers (movmatrix); same running state as the packed
        // blocks, done first so that its loads overlap the TMA copies in flight.
        // ------------------------------------------------------------------
        for (int tok0 = tail0; tok0 < tail1; tok0 += 16) {
            const int tA = tok0 + g, tB = tA + 8;
            const bool okA = tA < res_n, okB = tB < res_n;
            // rows past the end are read from the last valid row (in bounds) and zeroed afterwards,
            // so that every load below is unconditional and all of them are in flight together
            const int rA = min(tA, res_n - 1), rB = min(tB, res_n - 1);
            const uint16_t *kres = static_cast<const uint16_t *>(p.k_res) + ib * p.res_stride_b + ih * p.res_stride_h;
            const uint16_t *vres = static_cast<const uint16_t *>(p.v_res) + ib * p.res_stride_b + ih * p.res_stride_h;
            const uint16_t *kA = kres + int64_t(rA) * p.res_stride_s + 8 * l, *kB = kres + int64_t(rB) * p.res_stride_s + 8 * l;
            const uint16_t *vA = vres + int64_t(rA) * p.res_stride_s + 2 * l, *vB = vres + int64_t(rB) * p.res_stride_s + 2 * l;
            if (has_new) {
                const uint16_t *knew = static_cast<const uint16_t *>(p.k_new) + ib * p.new_stride_b + ih * p.new_stride_h;
                const uint16_t *vnew = static_cast<const uint16_t *>(p.v_new) + ib * p.new_stride_b + ih * p.new_stride_h;
                if (rA == res_old) { kA = knew + 8 * l; vA = vnew + 2 * l; }
                if (rB == res_old) { kB = knew + 8 * l; vB = vnew + 2 * l; }
            }
            uint4 ka[4], kb[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                ka[a] = __ldg(reinterpret_cast<const uint4 *>(kA + 32 * a));
                kb[a] = __ldg(reinterpret_cast<const uint4 *>(kB + 32 * a));
            }
            uint32_t va[16], vb[16];     // word i: dims 8 i + 2 l, + 1 of the two token rows
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                va[i] = __ldg(reinterpret_cast<const unsigned int *>(vA + 8 * i));
                vb[i] = __ldg(reinterpret_cast<const unsigned int *>(vB + 8 * i));
            }
            if (bf16) {
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    ka[a].x = bf16x2_to_f16x2(ka[a].x); ka[a].y = bf16x2_to_f16x2(ka[a].y);
                    ka[a].z = bf16x2_to_f16x2(ka[a].z); ka[a].w = bf16x2_to_f16x2(ka[a].w);
                    kb[a].x = bf16x2_to_f16x2(kb[a].x); kb[a].y = bf16x2_to_f16x2(kb[a].y);
                    kb[a].z = bf16x2_to_f16x2(kb[a].z); kb[a].w = bf16x2_to_f16x2(kb[a].w);
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) { va[i] = bf16x2_to_f16x2(va[i]); vb[i] = bf16x2_to_f16x2(vb[i]); }
            }
            float S1[NQT][1][4];
#pragma unroll
            for (int nq = 0; nq < NQT; ++nq)
#pragma unroll
                for (int e = 0; e < 4; ++e) S1[nq][0][e] = 0.f;
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int nq = 0; nq < NQT; ++nq) {
                    mma_f16(S1[nq][0], ka[a].x, kb[a].x, ka[a].y, kb[a].y, qr[nq][a][0], qr[nq][a][1]);
                    mma_f16(S1[nq][0], ka[a].z, kb[a].z, ka[a].w, kb[a].w, qr[nq][a][2], qr[nq][a][3]);
                }
            uint32_t pb[NQT][2];
#pragma unroll
            for (int nq = 0; nq < NQT; ++nq) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const bool ok = (e < 2) ? okA : okB;
                    const float mu = m_run[nq][e & 1] == -INFINITY ? 0.f : m_run[nq][e & 1];
                    S1[nq][0][e] = ok ? fmaf(S1[nq][0][e], p.scale_log2, -mu) : -INFINITY;
                }
                float f[2];
                softmax_step<1, true, NZ>(S1[nq], m_run[nq], l_run[nq], O[nq], ZS[nq], f);
                pb[nq][0] = movmatrix_trans(pack_f16x2(S1[nq][0][0], S1[nq][0][1]));
                pb[nq][1] = movmatrix_trans(pack_f16x2(S1[nq][0][2], S1[nq][0][3]));
            }
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                const int jv = (BITS == 4) ? (mt & 3) : mt;
                // rows 0-7 of this m-tile are dims d0 .. d0+7, rows 8-15 are d0+8 .. d0+15
                const int i0 = (((BITS == 4) ? 16 * (mt >> 2) : 0) + DP * jv) / 8;
                const uint32_t a0 = movmatrix_trans(okA ? va[i0] : 0u);
                const uint32_t a1 = movmatrix_trans(okA ? va[i0 + 1] : 0u);
                const uint32_t a2 = movmatrix_trans(okB ? vb[i0] : 0u);
                const uint32_t a3 = movmatrix_trans(okB ? vb[i0 + 1] : 0u);
                const float fw = field_weight<BITS>(jv);   // O is kept in the units of its packed field
#pragma unroll
                for (int nq = 0; nq < NQT; ++nq) {
                    float ot[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_f16(ot, a0, a1, a2, a3, pb[nq][0], pb[nq][1]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        O[nq][mt][e] = fmaf(ot[e], fw, O[nq][mt][e]);
                        if constexpr (kFieldPairs<BITS, GROUP>) {          // the accumulator below holds the pair sum
                            if (mt & 1) O[nq][mt - 1][e] = fmaf(ot[e], fw, O[nq][mt - 1][e]);
                        }
                    }
                }
            }
        }

        for (int blk = blk0; blk < blk1 && !aborted; ++blk) {
            if (phase == 0 && blk == blk0) { BD_TRACE_MARK(21); }
            if (blk == blk0) { BD_TRACE_WARP(0); }
            if (blk == blk0 + 1) { BD_TRACE_WARP(1); }
            if (blk == blk0 + 2) { BD_TRACE_WARP(2); }
            if (blk == blk0 + 5) { BD_TRACE_WARP(3); }
            int seqlen_blk = seqlen;              // tokens of the sequence this block may use
            if (p.block_table != nullptr) {
                int pib = ib, pblk = blk;
                if (!resolve(pib, pblk)) {        // page index outside the pool: the whole block is masked
                    seqlen_blk = blk * NB;
                    if (lane == 0) atomicExch(p.status, BD_ERR_PAGE);
                }
            }
            const bool need_mask = (blk + 1) * NB > seqlen_blk;

            // ------------------------------------------------------------ K phase
            if (!mbar_wait_bounded(kbar, phase, p.spin_limit)) { aborted = true; break; }
            if (phase == 0 && blk == blk0) { BD_TRACE_MARK(22); }

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
                        lds128(kprm + kprm_off<BITS, GROUP>(gk, a, l) + 256, z0, z1, z2, z3);
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

            // V phase of one unit (16 token slices of the V tile): O += P V for the unit's probabilities.
            auto v_unit = [&](const int u, const uint32_t (&pbu)[P][NQT][2]) {
#pragma unroll
                for (int j = 0; j < P; ++j) {
                    const int T0 = 16 * u + 32 * j;                       // first token of this k-slice
                    const int r0 = T0 + 2 * l;                            // tokens of fragment register 0
                    uint32_t sc0[NGD], sc1[NGD], ze0[NGD], ze1[NGD];    // tokens r0, r0+1 and r0+8, r0+9 (same run)
#pragma unroll
                    for (int gd = 0; gd < NGD; ++gd) {
                        const uint32_t b0 = vprm + vprm_off<BITS, GROUP>(gd, r0, 0), b1 = vprm + vprm_off<BITS, GROUP>(gd, r0, 1);
                        sc0[gd] = lds32(b0);
                        sc1[gd] = lds32(b1);
                        ze0[gd] = lds32(b0 + 256);
                        ze1[gd] = lds32(b1 + 256);
                    }
                    if (need_mask) {          // params of tokens past the end may be uninitialised
                        const int tok = blk * NB + r0;
                        const uint32_t k0 = (tok < seqlen_blk ? 0x0000ffffu : 0u) | (tok + 1 < seqlen_blk ? 0xffff0000u : 0u);
                        const uint32_t k1 = (tok + 8 < seqlen_blk ? 0x0000ffffu : 0u) | (tok + 9 < seqlen_blk ? 0xffff0000u : 0u);
#pragma unroll
                        for (int gd = 0; gd < NGD; ++gd) { sc0[gd] &= k0; ze0[gd] &= k0; sc1[gd] &= k1; ze1[gd] &= k1; }
                    }
                    uint32_t pv[NGD][NQT][2];
#pragma unroll
                    for (int nq = 0; nq < NQT; ++nq) {
                        // rows 0-7: sum_t p_t * zero_t of dim group 0; rows 8-15: the same for dim
                        // group 1 or, with a single dim group, sum_t p_t (the softmax denominator,
                        // from the same rounded probabilities the numerator uses)
                        constexpr uint32_t kOnes = 0x3c003c00u;
#pragma unroll
                        for (int z = 0; z < NZ; ++z)
                            mma_f16(ZS[nq][z], ze0[2 * z], NGD > 1 ? ze0[NGD > 1 ? 2 * z + 1 : 0] : kOnes, ze1[2 * z],
                                    NGD > 1 ? ze1[NGD > 1 ? 2 * z + 1 : 0] : kOnes, pbu[j][nq][0], pbu[j][nq][1]);
#pragma unroll
                        for (int gd = 0; gd < NGD; ++gd) {
                            pv[gd][nq][0] = hmul2_u32(pbu[j][nq][0], sc0[gd]);
                            pv[gd][nq][1] = hmul2_u32(pbu[j][nq][1], sc1[gd]);
                        }
                    }
                    constexpr int NCB = (BITS == 4) ? 2 : 1;              // ldmatrix.x4 per k-slice
#pragma unroll
                    for (int cb = 0; cb < NCB; ++cb) {
                        uint32_t r0w, r1w, r2w, r3w;
                        ldsm_x4_trans(vcode + T0 * (DP * 2) + v_off[cb], r0w, r1w, r2w, r3w);
                        const uint32_t s0w = aux_word<BITS>(r0w), s1w = aux_word<BITS>(r1w), s2w = aux_word<BITS>(r2w), s3w = aux_word<BITS>(r3w);
                        auto do_vfield = [&](auto jc) {
                            constexpr int JV = decltype(jc)::value;
                            constexpr int gd = JV / FPGV;
                            const int mt = (BITS == 4) ? (cb * 4 + JV) : JV;
#pragma unroll
                            for (int nq = 0; nq < NQT; ++nq)
                                mma_f16(O[nq][mt], field<BITS, JV, kFieldPairs<BITS, GROUP>>(r0w, s0w),
                                        field<BITS, JV, kFieldPairs<BITS, GROUP>>(r1w, s1w),
                                        field<BITS, JV, kFieldPairs<BITS, GROUP>>(r2w, s2w),
                                        field<BITS, JV, kFieldPairs<BITS, GROUP>>(r3w, s3w),
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
            };

            // Units (16 pack rows) that share one softmax step: both of a 4-bit block (one
            // step per block), one of a 2-bit block (its 8 fields fill the registers).
            constexpr int UG = (P == 4) ? 2 : 1;
            // With one unit per softmax step (2 bits) a unit goes all the way, K phase, softmax step, V
            // phase, before the next one starts: one unit's probabilities are alive at a time and the
            // whole block body is one rolled loop over the two units (half the instruction bytes).
            constexpr bool kUnitByUnit = (UG == 1);
            uint32_t Pb[kUnitByUnit ? 1 : 2][P][NQT][2];      // probabilities as B fragments (fp16), per unit and field
            // One group at 4 bits; at 2 bits the two units run through the same (rolled) code.
            constexpr int kGroupUnroll = kUnitByUnit ? 1 : 2;
#pragma unroll kGroupUnroll
            for (int ug = 0; ug < 2 / UG; ++ug) {
                float S[UG][P][NQT][4];
#pragma unroll
                for (int uu = 0; uu < UG; ++uu)
#pragma unroll
                    for (int j = 0; j < P; ++j)
#pragma unroll
                        for (int nq = 0; nq < NQT; ++nq)
#pragma unroll
                            for (int e = 0; e < 4; ++e) S[uu][j][nq][e] = 0.f;
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    // q * scale for the token groups of this block, channels 32a + 8l .. +7
                    uint32_t qs[NGK][NQT][4];
#pragma unroll
                    for (int gk = 0; gk < NGK; ++gk) {
                        uint32_t s0, s1, s2, s3;
                        lds128(kprm + kprm_off<BITS, GROUP>(gk, a, l), s0, s1, s2, s3);
#pragma unroll
                        for (int nq = 0; nq < NQT; ++nq) {
                            qs[gk][nq][0] = hmul2_u32(qr[nq][a][0], s0);
                            qs[gk][nq][1] = hmul2_u32(qr[nq][a][1], s1);
                            qs[gk][nq][2] = hmul2_u32(qr[nq][a][2], s2);
                            qs[gk][nq][3] = hmul2_u32(qr[nq][a][3], s3);
                        }
                    }
#pragma unroll
                    for (int uu = 0; uu < UG; ++uu) {
                        const int u = ug * UG + uu;
                        uint32_t wl[4], wh[4];
                        const uint32_t base = kcode + (a >> 1) * 4096 + u * 2048 + k_row_off + k_chunk_off[a & 1];
                        lds128(base, wl[0], wl[1], wl[2], wl[3]);
                        lds128(base + 1024, wh[0], wh[1], wh[2], wh[3]);
                        uint32_t wls[4], whs[4];
#pragma unroll
                        for (int x = 0; x < 4; ++x) { wls[x] = aux_word<BITS>(wl[x]); whs[x] = aux_word<BITS>(wh[x]); }
                        // all fields first, then the MMAs of the first k-slice, then of the second:
                        // consecutive MMAs never share an accumulator
                        uint32_t F[P][8];
                        auto extract = [&](auto jc) {
                            constexpr int J = decltype(jc)::value;
#pragma unroll
                            for (int x = 0; x < 4; ++x) {
                                F[J][2 * x] = field<BITS, J, kFieldPairs<BITS, GROUP>>(wl[x], wls[x]);
                                F[J][2 * x + 1] = field<BITS, J, kFieldPairs<BITS, GROUP>>(wh[x], whs[x]);
                            }
                        };
                        extract(std::integral_constant<int, 0>{});
                        extract(std::integral_constant<int, 1>{});
                        extract(std::integral_constant<int, 2>{});
                        extract(std::integral_constant<int, 3>{});
                        if constexpr (P == 8) {
                            extract(std::integral_constant<int, 4>{});
                            extract(std::integral_constant<int, 5>{});
                            extract(std::integral_constant<int, 6>{});
                            extract(std::integral_constant<int, 7>{});
                        }
#pragma unroll
                        for (int half = 0; half < 2; ++half)
#pragma unroll
                            for (int j = 0; j < P; ++j)
#pragma unroll
                                for (int nq = 0; nq < NQT; ++nq)
                                    mma_f16(S[uu][j][nq], F[j][4 * half], F[j][4 * half + 1], F[j][4 * half + 2],
                                            F[j][4 * half + 3], qs[j / FPG][nq][2 * half], qs[j / FPG][nq][2 * half + 1]);
                    }
                }

                // ---------------------------------------------- online softmax (these units)
#pragma unroll
                for (int nq = 0; nq < NQT; ++nq) {
                    float t[UG * P][4];
                    float zm[NGK][2];       // q.zero term minus the running max of the column
#pragma unroll
                    for (int gk = 0; gk < NGK; ++gk)
#pragma unroll
                        for (int c = 0; c < 2; ++c)
                            zm[gk][c] = Zc[gk][nq][c] - (m_run[nq][c] == -INFINITY ? 0.f : m_run[nq][c]);
#pragma unroll
                    for (int uu = 0; uu < UG; ++uu)
#pragma unroll
                        for (int j = 0; j < P; ++j)
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                float sv = S[uu][j][nq][e];
                                if constexpr (kFieldPairs<BITS, GROUP>) {
                                    if ((j & 1) == 0) sv -= S[uu][j + 1][nq][e];   // pair sum minus the odd field
                                }
                                t[uu * P + j][e] = fmaf(sv, mjs[j], zm[j / FPG][e & 1]);
                            }
                    if (need_mask) {
#pragma unroll
                        for (int uu = 0; uu < UG; ++uu)
#pragma unroll
                            for (int j = 0; j < P; ++j)
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const int tok = blk * NB + 16 * (ug * UG + uu) + 32 * j + g + 8 * (e >> 1);
                                    if (tok >= seqlen_blk) t[uu * P + j][e] = -INFINITY;
                                }
                    }
                    float f[2];
                    softmax_step<UG * P, (NGD > 1), NZ>(t, m_run[nq], l_run[nq], O[nq], ZS[nq], f);
#pragma unroll
                    for (int uu = 0; uu < UG; ++uu)
#pragma unroll
                        for (int j = 0; j < P; ++j) {
                            Pb[uu][j][nq][0] = movmatrix_trans(pack_f16x2(t[uu * P + j][0], t[uu * P + j][1]));
                            Pb[uu][j][nq][1] = movmatrix_trans(pack_f16x2(t[uu * P + j][2], t[uu * P + j][3]));
                        }
                }
                if constexpr (kUnitByUnit) {
                    if (ug == 1) {
                        // K tile consumed: refill it with the next block's K
                        __syncwarp();
                        if (lane == 0 && ld.valid) {
                            fence_proxy_async();
                            issue_k(ld.sg.ib, ld.u);
                        }
                    } else if (!mbar_wait_bounded(vbar, phase, p.spin_limit)) {
                        aborted = true;
                        break;
                    }
                    v_unit(ug, Pb[0]);
                }
            }
            if constexpr (kUnitByUnit) {
                if (aborted) break;
            } else {
            // K tile consumed: refill it with the next block's K while V is processed
            __syncwarp();
            if (lane == 0 && ld.valid) {
                fence_proxy_async();
                issue_k(ld.sg.ib, ld.u);
            }

            // ------------------------------------------------------------ V phase
            if (phase == 0 && blk == blk0) { BD_TRACE_MARK(23); }
            if (!mbar_wait_bounded(vbar, phase, p.spin_limit)) { aborted = true; break; }
            if (phase == 0 && blk == blk0) { BD_TRACE_MARK(24); }
            // The two units run through the same code (a rolled loop: half the instruction bytes of
            // the largest part of the block's code); their probabilities are picked with selects.
#pragma unroll 1
            for (int u = 0; u < 2; ++u) {
                uint32_t pbu[P][NQT][2];
#pragma unroll
                for (int j = 0; j < P; ++j)
#pragma unroll
                    for (int nq = 0; nq < NQT; ++nq) {
                        pbu[j][nq][0] = u ? Pb[1][j][nq][0] : Pb[0][j][nq][0];
                        pbu[j][nq][1] = u ? Pb[1][j][nq][1] : Pb[0][j][nq][1];
                    }
                v_unit(u, pbu);
            }
            }
            // V tile consumed: refill it, then move the load cursor on
            __syncwarp();
            if (ld.valid) {
                if (lane == 0) {
                    fence_proxy_async();
                    issue_v(ld.sg.ib, ld.u);
                }
                ld.advance();
            }
            phase ^= 1;
        }
        if (aborted) *abort_flag = 1;
#ifdef BD_TRACE
        if (lane == 0 && blockIdx.x < 4096 && warp < 13) g_trace[blockIdx.x * 32 + 2 + warp] = trace_now();
#endif

        // ------------------------------------------------------------------
        // End of this warp's share of the sequence: its partial (O, m, l in the fragment layout, the
        // same in every warp) in final units.
        // ------------------------------------------------------------------
        float acc[NACC];       // O in final units (field weights and zero sums applied), then m, l
#pragma unroll
        for (int nq = 0; nq < NQT; ++nq) {
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                const int jv = (BITS == 4) ? (mt & 3) : mt;
                const float wgt = 1.0f / field_weight<BITS>(jv);
                const int gd = jv / FPGV;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float ov = O[nq][mt][e];
                    if constexpr (kFieldPairs<BITS, GROUP>) {
                        if ((mt & 1) == 0) ov -= O[nq][mt + 1][e];      // pair sum minus the odd field
                    }
                    acc[(nq * 8 + mt) * 4 + e] = fmaf(ov, wgt, ZS[nq][gd >> 1][2 * (gd & 1) + (e & 1)]);
                }
            }
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float sum = l_run[nq][c];           // tail probabilities (and all of them with two dim groups)
                sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                sum += __shfl_xor_sync(0xffffffffu, sum, 8);
                sum += __shfl_xor_sync(0xffffffffu, sum, 16);
                if (NGD == 1) sum += ZS[nq][0][2 + c];  // every row of the ones block holds the column sum
                acc[32 * NQT + nq * 4 + c] = m_run[nq][c];
                acc[32 * NQT + nq * 4 + 2 + c] = sum;
            }
        }
        // The warps that share the sequence each deposit their partial and count in; the one that counts
        // in last folds the deposits in warp order (so the result does not depend on who was last).  A
        // warp whose range ends inside the sequence deposits into its own tile slots; the one warp in
        // whose range the sequence ends goes on streaming and deposits through global memory.
        const int4 nt = *note;
        const uint32_t share_mask = uint32_t(nt.x);
        const int goes_on = (nt.y & 0xff) - 1;
        const int nshare = __popc(share_mask);
        bool finisher = true;
        if (nshare > 1) {
            float *gdep = p.warp_acc + (int64_t(ib) * p.h_k + ih) * C::DEPOSIT_FLOATS;
            if (goes_on == warp) {
#pragma unroll
                for (int i = 0; i < NACC; ++i) __stcg(gdep + i * 32 + lane, acc[i]);
                __threadfence();
            } else {
                float *mine = reinterpret_cast<float *>(smem + size_t(warp) * 2 * C::CODE_BYTES);
#pragma unroll
                for (int i = 0; i < NACC; ++i) mine[i * 32 + lane] = acc[i];
                __threadfence_block();
            }
            __syncwarp();
            int old = 0;
            if (lane == 0) old = atomicAdd(arrivals + (__ffs(share_mask) - 1), 1);
            old = __shfl_sync(0xffffffffu, old, 0);
            finisher = old == nshare - 1;
            if (finisher) {
                BD_TRACE_MARK(16);
                if (goes_on >= 0) __threadfence(); else __threadfence_block();
                // generic loads serve shared and (written past L1, never read before) global deposits
                auto deposit_of = [&](int w) {
                    return (w == goes_on) ? static_cast<const float *>(gdep)
                                          : reinterpret_cast<const float *>(smem + size_t(w) * 2 * C::CODE_BYTES);
                };
                uint32_t rest = share_mask;
                int w = __ffs(rest) - 1;
                rest &= rest - 1;
                {
                    const float *dep = deposit_of(w);
#pragma unroll
                    for (int i = 0; i < NACC; ++i) acc[i] = dep[i * 32 + lane];
                }
#pragma unroll 1
                while (rest) {
                    w = __ffs(rest) - 1;
                    rest &= rest - 1;
                    const float *dep = deposit_of(w);
                    float v[NACC];
#pragma unroll
                    for (int i = 0; i < NACC; ++i) v[i] = dep[i * 32 + lane];
#pragma unroll
                    for (int nq = 0; nq < NQT; ++nq) {
                        float fa[2], fv[2];
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            const float ma = acc[32 * NQT + nq * 4 + c], mv = v[32 * NQT + nq * 4 + c];
                            const float mx = fmaxf(ma, mv);
                            fa[c] = (ma == -INFINITY) ? 0.f : ex2f(ma - mx);
                            fv[c] = (mv == -INFINITY) ? 0.f : ex2f(mv - mx);
                            acc[32 * NQT + nq * 4 + c] = mx;
                            acc[32 * NQT + nq * 4 + 2 + c] =
                                fmaf(fv[c], v[32 * NQT + nq * 4 + 2 + c], fa[c] * acc[32 * NQT + nq * 4 + 2 + c]);
                        }
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc[nq * 32 + i] = fmaf(fv[i & 1], v[nq * 32 + i], fa[i & 1] * acc[nq * 32 + i]);
                    }
                }
            }
        }
        if (finisher) {
            BD_TRACE_MARK(17);
            // How many rows hold a part of this sequence?  One: this is the final result.
            // More: leave a normalised partial; the row that arrives last merges them all.
            const int nparts = nt.w >> 1;
            PartRange pr;
            pr.c0 = nt.z; pr.dense = (nt.w & 1) != 0;
            pr.c1 = pr.c0 + (nt.y >> 8) - 1;
            const bool final_here = nparts <= 1 && !p.leave_parts;     // (a sequence split over GPUs always leaves parts)
            const int64_t slot = (int64_t(row) + ib) * p.h_k + ih;
            // normalise in place, then one straight run of stores per destination kind
            bool row_ok[NQT][2];
#pragma unroll
            for (int nq = 0; nq < NQT; ++nq) {
                float inv[2];
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const float M = acc[32 * NQT + nq * 4 + c], L = acc[32 * NQT + nq * 4 + 2 + c];
                    inv[c] = (L > 0.f) ? 1.0f / L : 0.f;
                    const float lse = (L > 0.f) ? fmaf(M, 0.6931471805599453f, logf(L)) : -INFINITY;
                    const int qrow = nq * 8 + 2 * l + c;
                    row_ok[nq][c] = qrow < p.gq;
                    if (g == 0 && row_ok[nq][c]) {
                        if (!final_here) p.part_lse[slot * p.gq + qrow] = lse;
                        else if (p.lse) p.lse[int64_t(ib) * p.h + int64_t(ih) * p.gq + qrow] = lse;
                    }
                }
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[nq * 32 + i] *= inv[i & 1];
            }
            // element (nq, mt, e) of this thread: query row nq*8 + 2l + (e&1), head dim dim_of(mt, e) + g
            auto dim_of = [](int mt, int e) {
                const int jv = (BITS == 4) ? (mt & 3) : mt;
                const int pbase = (BITS == 4) ? 16 * (mt >> 2) : 0;
                return pbase + 8 * (e >> 1) + DP * jv;
            };
            auto store_rows = [&](auto *base, int64_t row_stride, auto cvt) {
#pragma unroll
                for (int nq = 0; nq < NQT; ++nq)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        if (!row_ok[nq][c]) continue;
                        auto *rp = base + (nq * 8 + c) * row_stride;
#pragma unroll
                        for (int mt = 0; mt < 8; ++mt)
#pragma unroll
                            for (int eh = 0; eh < 2; ++eh)
                                rp[dim_of(mt, 2 * eh + c)] = cvt(acc[(nq * 8 + mt) * 4 + 2 * eh + c]);
                    }
            };
            if (!final_here) {
                store_rows(p.part_out + (slot * p.gq + 2 * l) * kHeadDim + g, int64_t(kHeadDim), [](float x) { return x; });
            } else {
                const int64_t o0 = ib * p.out_stride_b + (int64_t(ih) * p.gq + 2 * l) * p.out_stride_h + g;
                if (p.out_dtype == BD_FP16)
                    store_rows(static_cast<__half *>(p.out) + o0, p.out_stride_h, [](float x) { return __float2half_rn(x); });
                else if (p.out_dtype == BD_BF16)
                    store_rows(static_cast<__nv_bfloat16 *>(p.out) + o0, p.out_stride_h,
                               [](float x) { return __float2bfloat16_rn(x); });
                else
                    store_rows(static_cast<float *>(p.out) + o0, p.out_stride_h, [](float x) { return x; });
            }
            // With many parts per sequence (few long sequences) the merge is left to a second,
            // fully parallel kernel: one warp doing it here would be the tail of the whole step.
            if (!final_here && !p.defer_merge) {
                // publish the partial, count arrivals; the last one merges (same arithmetic as
                // the reference's combine kernel, flash_fwd_kernel.h:1217-1231, 1280-1298)
                __threadfence();
                __syncwarp();
                int old = 0;
                if (lane == 0) old = atomicAdd(p.counters + int64_t(ib) * p.h_k + ih, 1);
                old = __shfl_sync(0xffffffffu, old, 0);
                BD_TRACE_MARK(18);
                if (old == nparts - 1) {
                    __threadfence();
                    // Parts sit in consecutive rows, so consecutive slots h_k apart (rows that
                    // hold no part, possible only with more rows than units, weigh zero).
                    // Each lane owns 4 head dims; query rows go four at a time, every load of a
                    // round independent of the others.
                    const int nrows = pr.c1 - pr.c0 + 1;
                    const int64_t slot0 = (int64_t(pr.c0) + ib) * p.h_k + ih;
                    // final row `qrow` of this KV head: o holds the weighted sum of this lane's 4 dims
                    auto write_row = [&](int qrow, float (&o)[4], float mxv, float sumv) {
                        float lse_f = -INFINITY;
                        if (mxv != -INFINITY) {
                            const float inv = 1.0f / sumv;
                            o[0] *= inv; o[1] *= inv; o[2] *= inv; o[3] *= inv;
                            lse_f = mxv + logf(sumv);
                        }
                        const int64_t hq = int64_t(ih) * p.gq + qrow;
                        const int64_t oi = ib * p.out_stride_b + hq * p.out_stride_h + 4 * lane;
                        if (p.out_dtype == BD_FP16) {
                            __half2 a = __floats2half2_rn(o[0], o[1]), b2 = __floats2half2_rn(o[2], o[3]);
                            *reinterpret_cast<uint2 *>(static_cast<__half *>(p.out) + oi) =
                                make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b2));
                        } else if (p.out_dtype == BD_BF16) {
                            __nv_bfloat162 a = __floats2bfloat162_rn(o[0], o[1]), b2 = __floats2bfloat162_rn(o[2], o[3]);
                            *reinterpret_cast<uint2 *>(static_cast<__nv_bfloat16 *>(p.out) + oi) =
                                make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b2));
                        } else {
                            *reinterpret_cast<float4 *>(static_cast<float *>(p.out) + oi) = make_float4(o[0], o[1], o[2], o[3]);
                        }
                        if (lane == 0 && p.lse) p.lse[int64_t(ib) * p.h + hq] = lse_f;
                    };
                    if (pr.dense && nrows <= 4) {
                        // The usual case, a sequence cut into a few parts: every load of a round
                        // (4 query rows x 4 parts: the LSEs and this lane's 16 bytes of each part) is
                        // issued before any is used, one trip to L2 for all of them.
#pragma unroll 1
                        for (int q0 = 0; q0 < p.gq; q0 += 4) {
                            float ls[4][4];
                            float4 v[4][4];
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj) {
                                const int64_t sl = slot0 + int64_t(jj) * p.h_k;
#pragma unroll
                                for (int qq = 0; qq < 4; ++qq) {
                                    const bool live = jj < nrows && q0 + qq < p.gq;
                                    ls[jj][qq] = -INFINITY;
                                    v[jj][qq] = make_float4(0.f, 0.f, 0.f, 0.f);
                                    if (live) {
                                        ls[jj][qq] = __ldcg(p.part_lse + sl * p.gq + q0 + qq);
                                        v[jj][qq] = __ldcg(reinterpret_cast<const float4 *>(
                                            p.part_out + (sl * p.gq + q0 + qq) * kHeadDim + 4 * lane));
                                    }
                                }
                            }
#pragma unroll
                            for (int qq = 0; qq < 4; ++qq) {
                                if (q0 + qq >= p.gq) continue;
                                const float mxv = fmaxf(fmaxf(ls[0][qq], ls[1][qq]), fmaxf(ls[2][qq], ls[3][qq]));
                                float sumv = 0.f;
                                float o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                                for (int jj = 0; jj < 4; ++jj) {
                                    const float wv = (ls[jj][qq] == -INFINITY) ? 0.f : __expf(ls[jj][qq] - mxv);
                                    sumv += wv;
                                    if (wv != 0.f) {
                                        o[0] = fmaf(wv, v[jj][qq].x, o[0]); o[1] = fmaf(wv, v[jj][qq].y, o[1]);
                                        o[2] = fmaf(wv, v[jj][qq].z, o[2]); o[3] = fmaf(wv, v[jj][qq].w, o[3]);
                                    }
                                }
                                write_row(q0 + qq, o, mxv, sumv);
                            }
                        }
                    } else {
                    for (int q0 = 0; q0 < p.gq; q0 += 4) {
                        // pass 1: lane i reads the LSEs of row c0 + i (32 rows per round); one
                        // round trip to L2 for all of them, then warp reductions
                        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                        for (int base = 0; base < nrows; base += 32) {
                            const int i = base + lane;
                            const bool live = i < nrows && (pr.dense || row_has_part(p.part, ib, pr.c0 + i));
                            const float *lp = p.part_lse + (slot0 + int64_t(i) * p.h_k) * p.gq + q0;
#pragma unroll
                            for (int qq = 0; qq < 4; ++qq) {
                                float v = (live && q0 + qq < p.gq) ? __ldcg(lp + qq) : -INFINITY;
#pragma unroll
                                for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
                                mx[qq] = fmaxf(mx[qq], v);
                            }
                        }
                        // pass 2: weights per lane, then the weighted sum; four rows' worth of
                        // loads (16 x 16 bytes per lane) are in flight together
                        float sum[4] = {0.f, 0.f, 0.f, 0.f};
                        float o[4][4];
#pragma unroll
                        for (int qq = 0; qq < 4; ++qq) o[qq][0] = o[qq][1] = o[qq][2] = o[qq][3] = 0.f;
                        for (int base = 0; base < nrows; base += 32) {
                            const int i = base + lane;
                            const bool live = i < nrows && (pr.dense || row_has_part(p.part, ib, pr.c0 + i));
                            const float *lp = p.part_lse + (slot0 + int64_t(i) * p.h_k) * p.gq + q0;
                            float w[4];
#pragma unroll
                            for (int qq = 0; qq < 4; ++qq)
                                w[qq] = (live && q0 + qq < p.gq && mx[qq] != -INFINITY) ? __expf(__ldcg(lp + qq) - mx[qq]) : 0.f;
                            const int cnt = min(32, nrows - base);
                            for (int j0 = 0; j0 < cnt; j0 += 4) {
                                float4 v[4][4];
                                float wj[4][4];
#pragma unroll
                                for (int jj = 0; jj < 4; ++jj) {
                                    const int64_t sl = slot0 + int64_t(base + j0 + jj) * p.h_k;
#pragma unroll
                                    for (int qq = 0; qq < 4; ++qq) {
                                        wj[jj][qq] = __shfl_sync(0xffffffffu, w[qq], (j0 + jj) & 31);
                                        if (j0 + jj >= cnt) wj[jj][qq] = 0.f;
                                        v[jj][qq] = make_float4(0.f, 0.f, 0.f, 0.f);
                                        if (wj[jj][qq] != 0.f)
                                            v[jj][qq] = __ldcg(reinterpret_cast<const float4 *>(
                                                p.part_out + (sl * p.gq + q0 + qq) * kHeadDim + 4 * lane));
                                    }
                                }
#pragma unroll
                                for (int jj = 0; jj < 4; ++jj)
#pragma unroll
                                    for (int qq = 0; qq < 4; ++qq) {
                                        sum[qq] += wj[jj][qq];
                                        o[qq][0] = fmaf(wj[jj][qq], v[jj][qq].x, o[qq][0]);
                                        o[qq][1] = fmaf(wj[jj][qq], v[jj][qq].y, o[qq][1]);
                                        o[qq][2] = fmaf(wj[jj][qq], v[jj][qq].z, o[qq][2]);
                                        o[qq][3] = fmaf(wj[jj][qq], v[jj][qq].w, o[qq][3]);
                                    }
                            }
                        }
#pragma unroll
                        for (int qq = 0; qq < 4; ++qq)
                            if (q0 + qq < p.gq) write_row(q0 + qq, o[qq], mx[qq], sum[qq]);
                    }
                    }
                    if (lane == 0) p.counters[int64_t(ib) * p.h_k + ih] = 0;   // ready for the next step
                    BD_TRACE_MARK(19);
                }
            }
        }
        // a warp that gave up keeps walking its segments (without streaming) and keeps
        // counting in, so that every segment still finds its last arrival
    }

    // ======================================================================
    // after the stream: error exit
    // ======================================================================
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // a merge kernel staged behind this one may be placed
    __syncthreads();
#ifdef BD_TRACE
    if (tid == 0 && blockIdx.x < 4096) g_trace[blockIdx.x * 32 + 15] = trace_now();
#endif
    if (*abort_flag != 0) {
        if (tid == 0) atomicExch(p.status, BD_ERR_TIMEOUT);
        // give copies that are still in flight time to land before the block's
        // shared memory is released
        for (int it = 0; it < 2000; ++it) __nanosleep(1000);
        __syncthreads();
        return;
    }
}

// ---------------------------------------------------------------------------
// Merge of the CTAs' parts as a kernel of its own, for steps with many parts per sequence
// (DecodeParams::defer_merge): one warp per (sequence, query head), lane i weighs part i, each
// lane owns 4 head dims.  Same arithmetic as the in-kernel merge and as the reference's combine
// (flash_fwd_kernel.h:1217-1231, 1280-1298).  Sequences with at most one part were finished by
// the decode kernel itself.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128, 1) bd_merge_parts_kernel(const DecodeParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t rowid = int64_t(blockIdx.x) * 4 + warp;
    // (a warp that has nothing to merge still waits for the decode kernel before it leaves: kernels staged behind
    // this one rely on this kernel not finishing before that one)
    if (rowid >= int64_t(p.b) * p.h) { asm volatile("griddepcontrol.wait;" ::: "memory"); return; }
    const int ib = int(rowid / p.h), hq = int(rowid % p.h);
    const int ih = hq / p.gq, qrow = hq % p.gq;
    const PartRange pr = part_range(p.part, ib);
    const int nrows = pr.c1 - pr.c0 + 1;
    if (nrows <= 1) { asm volatile("griddepcontrol.wait;" ::: "memory"); return; }
    if (!pr.dense) {
        int nparts = 0;
        for (int c = pr.c0; c <= pr.c1; ++c) nparts += row_has_part(p.part, ib, c) ? 1 : 0;
        if (nparts <= 1) { asm volatile("griddepcontrol.wait;" ::: "memory"); return; }
    }
    const int64_t slot0 = (int64_t(pr.c0) + ib) * p.h_k + ih;
    auto lse_of = [&](int i) {
        const bool live = i < nrows && (pr.dense || row_has_part(p.part, ib, pr.c0 + i));
        return live ? __ldcg(p.part_lse + (slot0 + int64_t(i) * p.h_k) * p.gq + qrow) : -INFINITY;
    };
    // Launched early (see launch_merge_parts), the integer work above ran beside the decode kernel's end (the
    // partition and a ragged batch's table were final before that kernel started); everything it wrote is
    // visible after this.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // Up to 32 parts a round: lane i weighs part i, and every lane asks for its 16 bytes of all the parts of
    // the round together with the round's log-sum-exps before any answer is used (the rows do not depend on
    // the weights): one trip to L2 per round.  Rows of parts that weigh nothing are never used (select, not
    // multiply).  A later round brings what was summed so far to the new maximum.
    float mx = -INFINITY, sum = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
    for (int base = 0; base < nrows; base += 32) {
        const int cnt = min(32, nrows - base);
        float4 v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (j < cnt)
                v[j] = __ldcg(reinterpret_cast<const float4 *>(
                    p.part_out + ((slot0 + int64_t(base + j) * p.h_k) * p.gq + qrow) * kHeadDim + 4 * lane));
        }
        const float ls = lse_of(base + lane);
        float m2 = ls;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m2 = fmaxf(m2, __shfl_xor_sync(0xffffffffu, m2, off));
        m2 = fmaxf(m2, mx);
        const float fold = (mx == -INFINITY) ? 0.f : __expf(mx - m2);
        sum *= fold; o[0] *= fold; o[1] *= fold; o[2] *= fold; o[3] *= fold;
        mx = m2;
        const float w = (ls == -INFINITY || mx == -INFINITY) ? 0.f : __expf(ls - mx);
        float t = w;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
        sum += t;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float wj = __shfl_sync(0xffffffffu, w, j);
            if (j < cnt && wj != 0.f) {
                o[0] = fmaf(wj, v[j].x, o[0]); o[1] = fmaf(wj, v[j].y, o[1]);
                o[2] = fmaf(wj, v[j].z, o[2]); o[3] = fmaf(wj, v[j].w, o[3]);
            }
        }
    }
    float lse_f = -INFINITY;
    if (mx != -INFINITY && sum > 0.f) {
        const float inv = 1.0f / sum;
        o[0] *= inv; o[1] *= inv; o[2] *= inv; o[3] *= inv;
        lse_f = mx + logf(sum);
    }
    const int64_t oi = ib * p.out_stride_b + int64_t(hq) * p.out_stride_h + 4 * lane;
    if (p.out_dtype == BD_FP16) {
        __half2 a = __floats2half2_rn(o[0], o[1]), b2 = __floats2half2_rn(o[2], o[3]);
        *reinterpret_cast<uint2 *>(static_cast<__half *>(p.out) + oi) =
            make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b2));
    } else if (p.out_dtype == BD_BF16) {
        __nv_bfloat162 a = __floats2bfloat162_rn(o[0], o[1]), b2 = __floats2bfloat162_rn(o[2], o[3]);
        *reinterpret_cast<uint2 *>(static_cast<__nv_bfloat16 *>(p.out) + oi) =
            make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b2));
    } else {
        *reinterpret_cast<float4 *>(static_cast<float *>(p.out) + oi) = make_float4(o[0], o[1], o[2], o[3]);
    }
    if (lane == 0 && p.lse) p.lse[int64_t(ib) * p.h + hq] = lse_f;
}

#ifdef BD_TRACE
extern "C" int bd_trace_read(void *dst, size_t bytes) {
    return int(cudaMemcpyFromSymbol(dst, g_trace, bytes < sizeof(g_trace) ? bytes : sizeof(g_trace)));
}
extern "C" int bd_trace2_read(void *dst, size_t bytes) {
    return int(cudaMemcpyFromSymbol(dst, g_trace2, bytes < sizeof(g_trace2) ? bytes : sizeof(g_trace2)));
}
#endif

// `early`: launched as a programmatic dependent of the decode kernel before it: the launch is staged and the
// kernel's integer set-up runs while that kernel drains; the merge itself still waits for all of it.
// Measured: 0.3 to 1.4 us less per step (4 sequences per GPU of C2 38.2 -> 36.8 us, C3 40.3 -> 39.7 us).
cudaError_t launch_merge_parts(const DecodeParams &p, bool early, cudaStream_t stream) {
    const int64_t rows = int64_t(p.b) * p.h;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned((rows + 3) / 4));
    cfg.blockDim = dim3(128);
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = early ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, bd_merge_parts_kernel, p);
}

// ---------------------------------------------------------------------------
// Per-sequence unit table for ragged batches: (first unit, unit count) for each
// sequence and (T, 0) at the end.  One block; b is at most a few thousand.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) bd_prefix_kernel(const PrefixParams p) {
    __shared__ int32_t partial[256];
    const int tid = threadIdx.x;
    const int per = (p.b + 255) / 256;
    const int lo = min(tid * per, p.b), hi = min(lo + per, p.b);
    int32_t sum = 0;
    auto units = [&](int i) {
        return seq_blocks(p.cache_seqlens ? p.cache_seqlens[i] : p.s, p.s, p.block_tokens) +
               tail_chunks(min(max(p.res_lens ? p.res_lens[i] : p.res_len, 0), p.res_len) + p.res_extra);
    };
    for (int i = lo; i < hi; ++i) sum += units(i);
    partial[tid] = sum;
    __syncthreads();
    if (tid == 0) {
        int32_t run = 0;
        for (int i = 0; i < 256; ++i) { const int32_t v = partial[i]; partial[i] = run; run += v; }
        p.table[2 * p.b] = run;
        p.table[2 * p.b + 1] = 0;
    }
    __syncthreads();
    int32_t run = partial[tid];
    for (int i = lo; i < hi; ++i) {
        const int32_t n = units(i);
        p.table[2 * i] = run;
        p.table[2 * i + 1] = n;
        run += n;
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
template <int BITS, int GROUP, int NQT, int TWO>
static cudaError_t launch_t(const DecodeParams &p, const CUtensorMap &kmap, const CUtensorMap &vmap,
                            cudaStream_t stream) {
    using C = Cfg<BITS, GROUP, NQT, TWO>;
    auto kern = bd_decode_kernel<BITS, GROUP, NQT, TWO>;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 64 && !configured[dev]) {
        err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(C::SMEM));
        if (err != cudaSuccess) return err;
        configured[dev] = true;
    }
    const unsigned grid = unsigned(p.part.R) * unsigned(p.h_k);
    kern<<<grid, C::THREADS, C::SMEM, stream>>>(p, kmap, vmap);
    return cudaGetLastError();
}

template <int BITS, int GROUP>
static cudaError_t launch_bg(const DecodeParams &p, const CUtensorMap &kmap, const CUtensorMap &vmap,
                             cudaStream_t stream) {
    if (p.gq <= 8) {
        if constexpr (BITS == 4 && GROUP >= 64) {
            if (p.two_ctas) return launch_t<BITS, GROUP, 1, 1>(p, kmap, vmap, stream);
        }
        return launch_t<BITS, GROUP, 1, 0>(p, kmap, vmap, stream);
    }
    return launch_t<BITS, GROUP, 2, 0>(p, kmap, vmap, stream);
}

cudaError_t launch_decode(const DecodeParams &p, const CUtensorMap &kmap, const CUtensorMap &vmap,
                          int bits, int group, cudaStream_t stream) {
    if (bits == 4 && group == 128) return launch_bg<4, 128>(p, kmap, vmap, stream);
    if (bits == 4 && group == 64) return launch_bg<4, 64>(p, kmap, vmap, stream);
    if (bits == 2 && group == 128) return launch_bg<2, 128>(p, kmap, vmap, stream);
    if (bits == 2 && group == 64) return launch_bg<2, 64>(p, kmap, vmap, stream);
    if (bits == 4 && group == 32) return launch_bg<4, 32>(p, kmap, vmap, stream);
    if (bits == 2 && group == 32) return launch_bg<2, 32>(p, kmap, vmap, stream);
    return cudaErrorInvalidValue;
}

// ---------------------------------------------------------------------------
// After a step that appended a token to every tail: the lengths the next step will read.  Mirrors
// what the decode kernel did (a tail that was already full took no token) and what the roll-over
// pack did (a tail that reached one pack block was packed, room permitting).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) bd_advance_kernel(const AdvanceParams p) {
    // staged early behind the roll-over pack kernel (which itself waits for the decode kernel): the lengths
    // may only move when both are done
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= p.b) return;
    const int cap = min(kTailMax, p.res_cap);
    int r = min(max(p.res_lens[i], 0), cap);
    if (r < cap) r += 1;                                  // the decode kernel filed this step's token
    if (r == p.block_tokens) {
        const int cs = p.cache_seqlens[i];
        if (cs >= 0 && cs % p.block_tokens == 0 && cs + p.block_tokens <= p.s_cap) {
            p.cache_seqlens[i] = cs + p.block_tokens;
            r = 0;
        } else {
            atomicExch(p.status, BD_ERR_CAPACITY);
        }
    }
    p.res_lens[i] = r;
}

cudaError_t launch_advance(const AdvanceParams &p, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned((p.b + 255) / 256));
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;     // staged behind the kernel before it
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, bd_advance_kernel, p);
}

cudaError_t launch_prefix(const PrefixParams &p, cudaStream_t stream) {
    bd_prefix_kernel<<<1, 256, 0, stream>>>(p);
    return cudaGetLastError();
}

#define BD_CFG_PICK(FIELD)                                                                              \
    const int nqt = gq <= 8 ? 1 : 2;                                                                   \
    if (two && decode_two_ctas_built(bits, group, gq))                                                 \
        return group == 128 ? Cfg<4, 128, 1, 1>::FIELD : Cfg<4, 64, 1, 1>::FIELD;                       \
    if (bits == 4 && group == 128) return nqt == 1 ? Cfg<4, 128, 1>::FIELD : Cfg<4, 128, 2>::FIELD;     \
    if (bits == 4 && group == 64) return nqt == 1 ? Cfg<4, 64, 1>::FIELD : Cfg<4, 64, 2>::FIELD;        \
    if (bits == 2 && group == 128) return nqt == 1 ? Cfg<2, 128, 1>::FIELD : Cfg<2, 128, 2>::FIELD;     \
    if (bits == 2 && group == 64) return nqt == 1 ? Cfg<2, 64, 1>::FIELD : Cfg<2, 64, 2>::FIELD;        \
    if (bits == 4 && group == 32) return nqt == 1 ? Cfg<4, 32, 1>::FIELD : Cfg<4, 32, 2>::FIELD;        \
    if (bits == 2 && group == 32) return nqt == 1 ? Cfg<2, 32, 1>::FIELD : Cfg<2, 32, 2>::FIELD;

// Whether the two-CTAs-per-SM variant exists for this configuration (4-bit, group 64 / 128, up to 8
// query heads per KV head: the variants that otherwise run twelve warps per CTA).
bool decode_two_ctas_built(int bits, int group, int gq) { return bits == 4 && group >= 64 && gq <= 8; }
// Streaming warps per CTA of the kernel that serves this configuration.
int decode_warps(int bits, int group, int gq, int two) {
    BD_CFG_PICK(WARPS)
    return 1;
}
// Floats of one warp's deposit (its partial of a segment).
int decode_deposit_floats(int bits, int group, int gq, int two) {
    BD_CFG_PICK(DEPOSIT_FLOATS)
    return 0;
}
int decode_ctas_per_sm(int bits, int group, int gq, int two) {
    BD_CFG_PICK(CTAS_PER_SM)
    return 1;
}

}  // namespace bd
