// Internal parameter blocks and launch prototypes shared by the kernel
// translation units and the C-ABI layer.  Plain structs passed by value to
// the kernels (the reference passes one large Flash_fwd_params for everything,
// reference: csrc/bit_decode/src/include/flash.h:24-198).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

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
};

struct DecodeParams {
    const void *q;
    void *out;
    float *lse;
    int64_t q_stride_b, q_stride_h, out_stride_b, out_stride_h;
    const uint16_t *k_params;     // viewed as fp16
    const uint16_t *v_params;
    int64_t k_params_stride_b;    // in fp16 elements
    int64_t v_params_stride_b, v_params_stride_g, v_params_stride_h;   // in fp16 elements
    const int32_t *cache_seqlens;
    const void *k_res, *v_res;
    int64_t res_stride_b, res_stride_s, res_stride_h;
    const int32_t *res_lens;
    int32_t res_len;
    int32_t b, h, h_k, gq;
    int32_t s;
    int32_t chunk_blocks;         // pack blocks per split
    int32_t num_splits;
    int32_t k_batch_rows;         // K batch stride in pack rows
    int32_t v_batch_rows;         // V batch stride in token rows
    int32_t dtype, out_dtype;
    float scale_log2;             // softmax_scale * log2(e)
    float *part_out;              // (b*h, num_splits, d) fp32
    float *part_lse;              // (b*h, num_splits) fp32
    int32_t *status;
};

struct CombineSplitParams {
    const float *part_out, *part_lse;
    void *out;
    float *lse;
    int64_t out_stride_b, out_stride_h;
    const int32_t *cache_seqlens;
    int32_t b, h, s, num_splits, chunk_tokens;
    int32_t out_dtype;
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

cudaError_t launch_pack(const PackParams &p, int bits, int group, int dtype, cudaStream_t stream);
cudaError_t launch_decode(const DecodeParams &p, const CUtensorMap &kmap, const CUtensorMap &vmap,
                          int bits, int group, cudaStream_t stream);
size_t decode_smem_bytes(int bits, int group, int gq);
int decode_ctas_per_sm_default();
cudaError_t launch_combine_splits(const CombineSplitParams &p, cudaStream_t stream);
cudaError_t launch_combine_parts(const CombinePartsParams &p, cudaStream_t stream);

}  // namespace bd
