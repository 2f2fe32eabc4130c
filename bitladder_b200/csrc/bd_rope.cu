// Rotary position embedding of the token a decoder step appends: the query rows and the new key rows of
// every sequence are rotated at the token's position before the decode kernel attends with them and files
// the key in the tail.  The reference carries this for its append path (rotary_cos / rotary_sin, rotary_dim,
// is_rotary_interleaved: csrc/bit_decode/src/include/flash.h:121, 149-151, 189 and decode_api.cpp:316; the arithmetic of
// csrc/bit_decode/src/include/rotary.h:56-63 for interleaved pairs and :116-131 for pairs half a rotary_dim
// apart), switched off in its snapshot (rotary_dim = 0, decode_api.cpp:418).
//
// For a pair (x0, x1) of a head and the table row of the token's position:
//     x0' = x0 cos - x1 sin,   x1' = x0 sin + x1 cos
// in fp32 with separately rounded products (no fused multiply-add, so a CPU evaluation gives the same bits),
// rounded once to the input type.  Dims from rotary_dim on are copied.  One thread per pair, one CTA of 64
// threads per (sequence, head): every load of the step is in flight at once.
#include "bd_common.cuh"
#include "bd_kernels.h"

namespace bd {

__device__ __forceinline__ float rope_load(const void *p, int64_t i, bool bf16) {
    if (bf16) return __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
    return __half2float(static_cast<const __half *>(p)[i]);
}
__device__ __forceinline__ void rope_store(void *p, int64_t i, float v, bool bf16) {
    if (bf16) static_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
    else static_cast<__half *>(p)[i] = __float2half_rn(v);
}

// grid (q heads + 2 x KV heads, b), 64 threads: thread t is pair t of one head's row: a q head, then a k head
// (both rotated), then a v head (copied beside them)
__global__ void __launch_bounds__(64) bd_rope_kernel(const RopeParams p) {
    const int ib = blockIdx.y;
    const bool bf16 = p.dtype == BD_BF16;
    const int cached = p.cache_seqlens ? max(p.cache_seqlens[ib], 0) : p.s;
    const int tail = p.res_lens ? max(p.res_lens[ib], 0) : p.res_len;
    int pos = cached + tail;
    if (pos >= p.positions) {
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicExch(p.status, BD_ERR_POSITION);
        pos = p.positions - 1;
    }
    const int half = p.rotary_dim / 2;
    constexpr int kPairs = kHeadDim / 2;
    {
        const int head = blockIdx.x;
        int pr = threadIdx.x;
        const bool is_q = head < p.h, is_v = head >= p.h + p.h_k;
        const void *src = is_q ? p.q : (is_v ? p.v_new : p.k_new);
        void *dst = is_q ? p.q_out : (is_v ? p.v_out : p.k_out);
        const int hh = is_q ? head : (is_v ? head - p.h - p.h_k : head - p.h);
        const int64_t s0 = is_q ? ib * p.q_stride_b + hh * p.q_stride_h : ib * p.new_stride_b + hh * p.new_stride_h;
        const int64_t d0 = (int64_t(ib) * (is_q ? p.h : p.h_k) + hh) * kHeadDim;
        if (is_v) pr += kPairs;                   // never a rotated pair
        // pair pr of the head: dims (i0, i1) and the table column they share
        int i0, i1, col;
        if (pr < half) {
            if (p.interleaved) { i0 = 2 * pr; i1 = 2 * pr + 1; }
            else { i0 = pr; i1 = pr + half; }
            col = pr;
        } else {                                  // beyond the rotated dims, and V: two dims copied as they are
            const int pc = is_v ? pr - kPairs : pr;
            i0 = is_v ? 2 * pc : p.rotary_dim + 2 * (pc - half);
            i1 = i0 + 1;
            col = -1;
        }
        const float x0 = rope_load(src, s0 + i0, bf16), x1 = rope_load(src, s0 + i1, bf16);
        float y0 = x0, y1 = x1;
        if (col >= 0) {
            const float c = rope_load(p.cos_tab, int64_t(pos) * half + col, bf16);
            const float sn = rope_load(p.sin_tab, int64_t(pos) * half + col, bf16);
            y0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn));
            y1 = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c));
        }
        rope_store(dst, d0 + i0, y0, bf16);
        rope_store(dst, d0 + i1, y1, bf16);
    }
}

cudaError_t launch_rope(const RopeParams &p, cudaStream_t stream) {
    static_assert(kHeadDim / 2 == 64, "one thread per pair of a 128-dim head");
    bd_rope_kernel<<<dim3(unsigned(p.h + 2 * p.h_k), unsigned(p.b)), 64, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace bd
