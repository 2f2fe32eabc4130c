// Log-sum-exp merge of partial attention results.
//
//   LSE = log sum_i exp(lse_i),   out = sum_i exp(lse_i - LSE) * out_i
//
// Same arithmetic as the reference's split combine (reference:
// csrc/bit_decode/src/flash_fwd_kernel.h:1217-1231 for the LSE, :1280-1298 for
// the weighted sum).  One warp per (batch, query head) row, each lane owns four
// consecutive head dims (one 16-byte load per partial).
//
// Inside one decode step the merge of the per-range partials is done by the
// decode kernel itself (the range that finishes last merges); this file holds
// the stand-alone variant that takes one pointer per part, for partial results
// that come from other GPUs: the pointers may point into a peer's memory (plain
// loads over NVLink, no multicast, no TMA).
#include "bd_common.cuh"
#include "bd_kernels.h"

namespace bd {

constexpr int kCombineWarps = 4;

__device__ __forceinline__ void store_out4(void *out, int64_t idx, const float (&o)[4], int out_dtype) {
    if (out_dtype == BD_FP16) {
        __half2 a = __floats2half2_rn(o[0], o[1]), b = __floats2half2_rn(o[2], o[3]);
        uint2 w = make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b));
        *reinterpret_cast<uint2 *>(static_cast<__half *>(out) + idx) = w;
    } else if (out_dtype == BD_BF16) {
        __nv_bfloat162 a = __floats2bfloat162_rn(o[0], o[1]), b = __floats2bfloat162_rn(o[2], o[3]);
        uint2 w = make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b));
        *reinterpret_cast<uint2 *>(static_cast<__nv_bfloat16 *>(out) + idx) = w;
    } else {
        *reinterpret_cast<float4 *>(static_cast<float *>(out) + idx) = make_float4(o[0], o[1], o[2], o[3]);
    }
}

__global__ void __launch_bounds__(kCombineWarps * 32)
bd_combine_parts_kernel(const CombinePartsParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = int64_t(blockIdx.x) * kCombineWarps + warp;
    if (row >= p.rows) return;
    float l[16];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        l[i] = (i < p.n_parts) ? p.part_lse[i][row] : -INFINITY;
        mx = fmaxf(mx, l[i]);
    }
    float sum = 0.f;
    if (mx != -INFINITY) {
#pragma unroll
        for (int i = 0; i < 16; ++i) sum += (i < p.n_parts) ? __expf(l[i] - mx) : 0.f;
    }
    const float lse = (sum > 0.f) ? mx + logf(sum) : -INFINITY;
    float o[4] = {0.f, 0.f, 0.f, 0.f};
    if (sum > 0.f) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (i < p.n_parts) {
                const float w = __expf(l[i] - lse);
                const float4 v = *reinterpret_cast<const float4 *>(p.part_out[i] + row * kHeadDim + 4 * lane);
                o[0] = fmaf(w, v.x, o[0]); o[1] = fmaf(w, v.y, o[1]);
                o[2] = fmaf(w, v.z, o[2]); o[3] = fmaf(w, v.w, o[3]);
            }
        }
    }
    store_out4(p.out, row * kHeadDim + 4 * lane, o, p.out_dtype);
    if (lane == 0 && p.lse) p.lse[row] = lse;
}

cudaError_t launch_combine_parts(const CombinePartsParams &p, cudaStream_t stream) {
    const unsigned grid = unsigned((p.rows + kCombineWarps - 1) / kCombineWarps);
    bd_combine_parts_kernel<<<grid, kCombineWarps * 32, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace bd
