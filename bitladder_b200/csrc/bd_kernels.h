// Internal parameter blocks, the work partition shared by the decode and the
// combine kernels, and launch prototypes.  Plain structs passed by value to the
// kernels (the reference passes one large Flash_fwd_params for everything,
// reference: csrc/bit_decode/src/include/flash.h:24-198).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#ifndef BD_HD
#define BD_HD __host__ __device__ __forceinline__
#endif

struct bd_exchange_args;

namespace bd {

struct PackParams {
    const void *k, *v;
    int64_t k_stride_b, k_stride_s, k_stride_h;
    int64_t v_stride_b, v_stride_s, v_stride_h;
    void *k_pack, *k_params, *v_pack, *v_params;
    int64_t k_pack_stride_b;      // u16 elements
    int64_t k_params_stride_b;    // 4-byte slots
    int64_t v_pack_stride_b;      // u16 elements
    int64_t v_params_stride_b, v_params_stride_g, v_params_stride_h;   // 4-byte slots
    int32_t b, s, h_k;
    int32_t dst_token_offset;
    int32_t approx_div;           // divide like the reference built with --use_fast_math (see bd_pack.cu)
    // Roll-over of full tails (null: plain pack).  The source rows are a sequence's tail buffer; a
    // sequence is packed only if roll_res_lens[ib] + 1 equals one pack block (this step's token filled
    // the tail), into the block that starts at token roll_cache_seqlens[ib] (room permitting).
    const int32_t *roll_res_lens;
    const int32_t *roll_cache_seqlens;
    int32_t roll_s_cap;
};

struct AdvanceParams {
    int32_t *cache_seqlens, *res_lens;
    int32_t b, block_tokens, s_cap, res_cap;
    int32_t *status;
};

// ---------------------------------------------------------------------------
// Work partition of one decode step.
//
// A UNIT is one pack block of the quantized cache or one chunk of kTailChunk tokens
// of the unquantized tail.  Per KV head, the units of all sequences form one flat
// list of T units (sequence 0's blocks, then its tail chunks, then sequence 1's,
// ...).  The list is cut into R equal ranges ("rows"); CTA (row c, head ih) streams
// range c of head ih, so all CTAs carry the same number of units (+-1) whatever the
// batch size and however ragged the lengths are, and the CTAs of one row touch the
// same tokens of neighbouring heads at the same time.  Inside the CTA the same cut
// is applied once more: the warps are the rows of the partition with R * W rows
// (row c * W + w is warp w of CTA row c; floor(cW * T / (RW)) = floor(c * T / R), so
// the two levels agree), every warp streams one contiguous range.
// A range that crosses a sequence boundary yields one partial result per sequence
// it touches ("segment"); the segment of (CTA row c, sequence ib) owns partial slot
// c + ib, which is unique because rows and sequences both advance monotonically
// along the list.  A sequence without any unit is owned by the row whose range
// holds its position (the last row when it sits behind the last unit); the owner
// writes the defined result for it.  The merge walks the same arithmetic to find
// the parts.
// ---------------------------------------------------------------------------
constexpr int kTailChunk = 32;    // tokens of the unquantized tail per unit (two 16-token steps: about the time of a pack block)
constexpr int kTailMax = 256;     // longest unquantized tail the kernel accepts

// Units of one sequence: pack blocks of `len` cached tokens (clamped to the capacity s),
// then chunks of `res_n` tail tokens.
BD_HD int32_t seq_blocks(int32_t len, int32_t s, int32_t block_tokens) {
    len = len < 0 ? 0 : (len > s ? s : len);
    return (len + block_tokens - 1) / block_tokens;
}
BD_HD int32_t tail_chunks(int32_t res_n) {
    res_n = res_n < 0 ? 0 : (res_n > kTailMax ? kTailMax : res_n);
    return (res_n + kTailChunk - 1) / kTailChunk;
}

// Non-negative 64-bit quotient; takes the cheap 32-bit divide when both fit (they
// almost always do: unit counts and row counts), the emulated one otherwise.
BD_HD int64_t div_nn(int64_t a, int64_t b) {
    return ((a | b) >> 32) == 0 ? int64_t(uint32_t(a) / uint32_t(b)) : a / b;
}

struct Partition {
    const int32_t *table;     // ragged: (first unit, unit count) per sequence, then (T, 0); null when uniform
    int32_t b;
    int32_t n_uniform;        // units per sequence when table is null
    int32_t R;                // rows

    BD_HD int64_t total() const { return table ? int64_t(table[2 * b]) : int64_t(b) * n_uniform; }
    BD_HD int64_t first(int ib) const { return table ? int64_t(table[2 * ib]) : int64_t(ib) * n_uniform; }
    BD_HD int32_t count(int ib) const { return table ? table[2 * ib + 1] : n_uniform; }
    // first unit of row c (c == R gives T)
    BD_HD int64_t row_begin(int64_t c, int64_t T) const { return div_nn(c * T, R); }
    // row that holds unit f (0 <= f < T)
    BD_HD int32_t row_of(int64_t f, int64_t T) const { return int32_t(div_nn((f + 1) * R - 1, T)); }
};

// One segment of a row: units [u0, u1) of sequence ib, or (u1 <= u0, owns_empty) a
// sequence without units that this row answers for.
struct Segment {
    int32_t ib, u0, u1;
    bool owns_empty;
};

// Walks the segments of row c in order.  Pure integer arithmetic on the
// partition, shared by the decode kernel and by host-side tests.
struct SegWalk {
    const Partition *ptp;
    int64_t T, f0, f1;
    int32_t c, ib;

    BD_HD void init(const Partition &p, int row) {
        ptp = &p;
        c = row;
        T = p.total();
        f0 = p.row_begin(row, T);
        f1 = p.row_begin(int64_t(row) + 1, T);
        ib = find_start();
    }
    // the same with the first sequence found by the caller (the decode kernel searches a ragged table with
    // all lanes of the warp at once instead of a binary search of dependent loads)
    BD_HD void init_at(const Partition &p, int row, int64_t T_, int32_t ib_start) {
        ptp = &p;
        c = row;
        T = T_;
        f0 = p.row_begin(row, T);
        f1 = p.row_begin(int64_t(row) + 1, T);
        ib = ib_start;
    }
    // smallest ib with first(ib) >= f0 or first(ib) + count(ib) > f0
    BD_HD int32_t find_start() const {
        const Partition &pt = *ptp;
        if (!pt.table) return pt.n_uniform > 0 ? int32_t(div_nn(f0, pt.n_uniform)) : 0;
        int32_t lo = 0, hi = pt.b;
        while (lo < hi) {
            const int32_t mid = (lo + hi) >> 1;
            const bool ok = pt.first(mid) + pt.count(mid) > f0 || pt.first(mid) >= f0;
            if (ok) hi = mid; else lo = mid + 1;
        }
        return lo;
    }
    BD_HD bool next(Segment &sg) {
        const Partition &pt = *ptp;
        while (ib < pt.b) {
            const int64_t fb = pt.first(ib);
            const bool trailing = (c == pt.R - 1) && fb >= T;      // empty sequences after the last unit
            if (fb >= f1 && !trailing) break;
            const int64_t n = pt.count(ib);
            const int64_t lo = fb > f0 ? fb : f0;
            const int64_t hi = fb + n < f1 ? fb + n : f1;
            sg.ib = ib;
            sg.u0 = int32_t(lo - fb);
            sg.u1 = int32_t(hi - fb);
            sg.owns_empty = n <= 0 && (trailing || (fb >= f0 && fb < f1));
            ++ib;
            if (sg.u1 > sg.u0 || sg.owns_empty) return true;
        }
        return false;
    }
};

// Rows that hold a part of sequence ib (the merge side of the same arithmetic); none
// for a sequence without units.  When every row has units (T >= R, the normal case)
// the parts are the consecutive rows c0 .. c1; with more rows than units some rows in
// between are empty.
struct PartRange {
    int32_t c0, c1;           // inclusive; c1 < c0: no part
    bool dense;               // every row of the range holds a part
};
BD_HD PartRange part_range(const Partition &pt, int ib) {
    const int64_t T = pt.total();
    const int64_t first = pt.first(ib), n = pt.count(ib);
    PartRange r{0, -1, true};
    if (n > 0 && T > 0) {
        r.c0 = pt.row_of(first, T);
        r.c1 = pt.row_of(first + n - 1, T);
        r.dense = T >= pt.R;
    }
    return r;
}
BD_HD bool row_has_part(const Partition &pt, int ib, int64_t c) {
    const int64_t T = pt.total();
    const int64_t first = pt.first(ib), n = pt.count(ib);
    if (n <= 0) return false;
    const int64_t b0 = pt.row_begin(c, T), b1 = pt.row_begin(c + 1, T);
    const int64_t lo = b0 > first ? b0 : first, hi = b1 < first + n ? b1 : first + n;
    return hi > lo;
}
template <class F>
BD_HD void for_each_part(const Partition &pt, int ib, F &&f) {
    const PartRange r = part_range(pt, ib);
    for (int c = r.c0; c <= r.c1; ++c)
        if (r.dense || row_has_part(pt, ib, c)) f(c);
}

struct DecodeParams {
    const void *q;
    int64_t q_stride_b, q_stride_h;
    const uint16_t *k_params;     // viewed as fp16
    const uint16_t *v_params;
    int64_t k_params_stride_b;    // in fp16 elements
    int64_t v_params_stride_b, v_params_stride_g, v_params_stride_h;   // in fp16 elements
    const int32_t *cache_seqlens;
    const int32_t *block_table;   // paged cache: [b][block_table_stride] page indices; null: contiguous
    int32_t block_table_stride, blocks_per_page;
    int32_t num_pages;            // pages the packed buffers hold (page indices outside [0, num_pages) are refused)
    const void *k_res, *v_res;
    void *k_res_out, *v_res_out;  // the same buffers, written by the fused append
    const void *k_new, *v_new;    // (b, 1, h_k, d): this step's token, appended to the tail; null: no append
    int64_t new_stride_b, new_stride_h;
    int64_t res_stride_b, res_stride_s, res_stride_h;
    const int32_t *res_lens;
    int32_t res_len;
    int32_t res_cap;              // token rows the tail buffers hold
    int32_t b, h, h_k, gq;
    int32_t s;
    int32_t k_batch_rows;         // K batch stride in pack rows
    int32_t v_batch_rows;         // V batch stride in token rows
    int32_t dtype;
    float scale_log2;             // softmax_scale * log2(e)
    Partition part;
    float *part_out;              // [(R + b) * h_k segment slots][gq][128] fp32, normalised
    float *part_lse;              // [(R + b) * h_k][gq]
    int32_t *counters;            // [b * h_k] parts arrived per (sequence, KV head); zero between steps
    float *warp_acc;              // [b * h_k][deposit floats]: the share of the warp in whose range a sequence ends
    void *out;                    // (b, h, d) final result
    float *lse;                   // optional (b, h)
    int64_t out_stride_b, out_stride_h;
    int32_t out_dtype;
    int32_t defer_merge;          // the parts of a sequence are merged by a kernel launched next
    int32_t leave_parts;          // every segment leaves a part, also where a sequence has a single one (the exchange merges)
    int32_t two_ctas;             // launch the variant with two smaller CTAs per SM
    uint32_t spin_limit;          // polls a wait on a copy may take before the warp gives up
    int32_t test_starve;          // test hook: the warps of CTA 0 expect 16 bytes more than their first copy brings
    int32_t *status;
};

struct PrefixParams {
    const int32_t *cache_seqlens;     // null: every sequence has s tokens
    const int32_t *res_lens;          // null: every sequence has res_len tail tokens
    int32_t *table;
    int32_t b, s, block_tokens, res_len;   // res_len: rows the tail buffers hold (per-sequence lengths are clamped to it)
    int32_t res_extra;                // 1 when the step appends a token to every tail
};

struct CombinePartsParams {
    const float *part_out[16];
    const float *part_lse[16];
    void *out;
    float *lse;
    int64_t rows;
    int32_t n_parts;
    int32_t out_dtype;
};

// Rotary embedding of the step's token (bd_rope.cu): q and k_new rotated at the token's position into
// scratch copies (b, h, 128) and (b, h_k, 128) that the decode kernel then reads instead (v_new is copied
// beside them as it is: the decode kernel takes one pair of strides for both new rows).
struct RopeParams {
    const void *q, *k_new, *v_new;
    int64_t q_stride_b, q_stride_h, new_stride_b, new_stride_h;
    void *q_out, *k_out, *v_out;      // contiguous
    const void *cos_tab, *sin_tab;    // (positions, rotary_dim / 2), q's dtype
    const int32_t *cache_seqlens, *res_lens;
    int32_t s, res_len;               // lengths of every sequence when the arrays are null
    int32_t b, h, h_k;
    int32_t rotary_dim, interleaved, positions, dtype;
    int32_t *status;
};
cudaError_t launch_rope(const RopeParams &p, cudaStream_t stream);

// Exchange of a sequence split's partials between GPUs (bd_exchange.cu).
struct ExchangeParams {
    uint8_t *area[16];               // area of every rank as mapped into this process; area[rank] is local
    const float *part_out;           // this rank's normalised partial (rows, 128), or the decode kernel's parts
    const float *part_lse;
    void *out;
    float *lse;
    int64_t rows;                    // b * h
    int64_t out_stride_b, out_stride_h;
    int32_t h;                       // rows per sequence
    int32_t rank, world, out_dtype;
    uint32_t spin_limit;
    // fused with the decode step: where the decode kernel's CTAs left their parts
    Partition part;
    int32_t h_k, gq;
};
cudaError_t launch_exchange_parts(const ExchangeParams &p, cudaStream_t stream);
// checks the exchange half of a call and fills areas, rank, world, rows and the poll limit from it
int fill_exchange_params(const ::bd_exchange_args *a, ExchangeParams &p);

cudaError_t launch_pack(const PackParams &p, int bits, int group, int dtype, cudaStream_t stream);
cudaError_t launch_prefix(const PrefixParams &p, cudaStream_t stream);
cudaError_t launch_advance(const AdvanceParams &p, cudaStream_t stream);
cudaError_t launch_merge_parts(const DecodeParams &p, bool early, cudaStream_t stream);
cudaError_t launch_decode(const DecodeParams &p, const CUtensorMap &kmap, const CUtensorMap &vmap,
                          int bits, int group, cudaStream_t stream);
// `two`: the variant with half as many warps per CTA and two CTAs per SM (see Cfg in bd_decode.cu)
bool decode_two_ctas_built(int bits, int group, int gq);
int decode_ctas_per_sm(int bits, int group, int gq, int two);
int decode_warps(int bits, int group, int gq, int two);
int decode_deposit_floats(int bits, int group, int gq, int two);
cudaError_t launch_combine_parts(const CombinePartsParams &p, cudaStream_t stream);

}  // namespace bd
