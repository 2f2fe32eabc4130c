// C-ABI layer: argument checks, split planning, tensor-map construction and
// kernel dispatch.  Takes the place of the reference's host API (reference:
// csrc/bit_decode/decode_api.cpp:22-180 parameter marshalling, :234-299 split
// heuristic and workspace, :301-441 decode entry, :517-603 pack entry), minus
// everything that needs ATen: no tensors, no allocation, no device sync.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/bitdecode.h"
#include "bd_kernels.h"

namespace {

using bd::DecodeParams;
using bd::PackParams;

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct DeviceInfo {
    bool ok = false;
    int sm_count = 0;
    int cc_major = 0;
};

int current_device_info(DeviceInfo &info) {
    static DeviceInfo cache[64];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return BD_ERR_CUDA;
    if (dev < 0 || dev >= 64) return BD_ERR_CUDA;
    std::lock_guard<std::mutex> lock(mu);
    if (!cache[dev].ok) {
        int sm = 0, major = 0;
        if (cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return BD_ERR_CUDA;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return BD_ERR_CUDA;
        cache[dev].sm_count = sm;
        cache[dev].cc_major = major;
        cache[dev].ok = true;
    }
    info = cache[dev];
    return BD_OK;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time
// dependency on libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

// 2-D map over 16-bit words: dim0 = contiguous words of one row (all heads),
// dim1 = rows.  Box = (box_w words, box_rows rows).
int make_map_2d(CUtensorMap *map, const void *base, uint64_t row_words, uint64_t rows, uint32_t box_w,
                uint32_t box_rows, CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return BD_ERR_CUDA;
    cuuint64_t dims[2] = {row_words, rows};
    cuuint64_t strides[1] = {row_words * 2};
    cuuint32_t box[2] = {box_w, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? BD_OK : BD_ERR_CUDA;
}

int pack_block_tokens(int bits) { return 32 * (16 / bits); }

bool config_supported(int bits, int group, int d) {
    return (bits == 2 || bits == 4) && (group == 32 || group == 64 || group == 128) && d == 128;
}

struct DecodePlan {
    int rows;                 // R: ranges the block list of one KV head is cut into
    int two_ctas;             // two smaller CTAs per SM instead of one (fills the machine better with many KV heads)
    bool ragged;
    int32_t n_uniform;        // units per sequence when the batch is not ragged
    size_t off_counters, off_table, off_part_out, off_part_lse, off_warp_acc, off_rope_q, off_rope_k, off_rope_v, total_bytes;
};

inline size_t align16(size_t x) { return (x + 15) & ~size_t(15); }

// Every CTA of the decode grid should be resident at once (one wave) and carry
// the same number of pack blocks: then all of them stream at the same rate and
// finish together.  rows * h_k CTAs fill the resident slots.
int plan_rows(int b, int h_k, int64_t max_s, int bits, int sm_count, int ctas_per_sm) {
    if (b <= 0 || h_k <= 0 || max_s <= 0) return 1;
    const int nb = pack_block_tokens(bits);
    const int64_t nblk = (max_s + nb - 1) / nb;
    if (ctas_per_sm <= 0) ctas_per_sm = bd::decode_ctas_per_sm(bits, 128, 4, 0);
    const int64_t slots = int64_t(sm_count) * ctas_per_sm;
    int64_t rows = std::max<int64_t>(1, slots / h_k);
    // a row holds at least two blocks (one block per warp is as fine as the work gets; more rows than that only
    // add parts to merge); small problems cut into more than four parts per sequence take the parts-merge
    // kernel, which measured faster than fewer rows merged inside the decode kernel (b1, 4096 tokens: 12.7 us
    // with 4 rows, 10.5 us with 16)
    rows = std::min<int64_t>(rows, std::max<int64_t>(1, (int64_t(b) * nblk + 1) / 2));
    return int(std::min<int64_t>(rows, 1 << 20));
}

int make_plan(const bd_decode_args *a, int sm_count, DecodePlan &plan) {
    const int nb = pack_block_tokens(a->bits);
    const int64_t nblk = (int64_t(a->s) + nb - 1) / nb;
    const int gq = a->h / a->h_k;
    int64_t rows;
    plan.two_ctas = 0;
    if (a->num_splits > 0) {
        rows = std::min<int64_t>(int64_t(a->num_splits) * a->b, std::max<int64_t>(1, int64_t(a->b) * (nblk + 4)));
    } else {
        // One CTA per SM unless whole rows of KV heads leave more than a tenth of the SMs without a CTA and
        // two smaller CTAs per SM fill that gap (measured: 32 KV heads, 128 -> 288 CTAs, 4.5 % faster; with
        // 8 KV heads, 144 -> 296 CTAs, 12 % slower).
        const int c1 = bd::decode_ctas_per_sm(a->bits, a->group, gq, 0);
        if (bd::decode_two_ctas_built(a->bits, a->group, gq) && a->h_k <= sm_count) {
            const int c2 = bd::decode_ctas_per_sm(a->bits, a->group, gq, 1);
            const double u1 = double((int64_t(sm_count) * c1 / a->h_k) * a->h_k) / (double(sm_count) * c1);
            const double u2 = double((int64_t(sm_count) * c2 / a->h_k) * a->h_k) / (double(sm_count) * c2);
            const int64_t units = int64_t(a->b) * nblk;
            if (u2 > 1.1 * u1 && units >= 8 * int64_t(sm_count) * c2) plan.two_ctas = 1;
        }
        rows = plan_rows(a->b, a->h_k, a->s, a->bits, sm_count, bd::decode_ctas_per_sm(a->bits, a->group, gq, plan.two_ctas));
    }
    plan.rows = int(std::max<int64_t>(1, std::min<int64_t>(rows, 1 << 20)));
    const bool has_tail = a->k_res != nullptr;
    plan.ragged = a->cache_seqlens != nullptr || (has_tail && a->res_lens != nullptr);
    plan.n_uniform = bd::seq_blocks(a->s, a->s, nb) + (has_tail ? bd::tail_chunks(a->res_len + (a->k_new ? 1 : 0)) : 0);
    const size_t slots = (size_t(plan.rows) + a->b) * a->h_k;
    size_t off = 16;                                  // status word
    plan.off_counters = off;
    off = align16(off + size_t(a->b) * a->h_k * sizeof(int32_t));
    plan.off_table = off;
    if (plan.ragged) off = align16(off + (size_t(a->b) + 1) * 2 * sizeof(int32_t));
    plan.off_part_out = off; off += slots * gq * 128 * sizeof(float);
    plan.off_part_lse = off; off = align16(off + slots * gq * sizeof(float));
    plan.off_warp_acc = off;
    off = align16(off + size_t(a->b) * a->h_k * bd::decode_deposit_floats(a->bits, a->group, gq, plan.two_ctas) * sizeof(float));
    plan.off_rope_q = plan.off_rope_k = plan.off_rope_v = off;
    if (a->rotary_dim > 0) {          // rotated copies of q and k_new, and v_new beside them (fp16 / bf16)
        off = align16(off + size_t(a->b) * a->h * 128 * 2);
        plan.off_rope_k = off;
        off = align16(off + size_t(a->b) * a->h_k * 128 * 2);
        plan.off_rope_v = off;
        off = align16(off + size_t(a->b) * a->h_k * 128 * 2);
    }
    plan.total_bytes = off;
    return BD_OK;
}

int check_decode_args(const bd_decode_args *a) {
    if (!a || !a->q || !a->out || !a->k_pack || !a->k_params || !a->v_pack || !a->v_params) return BD_ERR_INVALID;
    if (a->b <= 0 || a->h <= 0 || a->h_k <= 0 || a->s < 0 || a->s_cap <= 0) return BD_ERR_INVALID;
    if (!config_supported(a->bits, a->group, a->d)) return BD_ERR_UNSUPPORTED;
    if (a->dtype != BD_FP16 && a->dtype != BD_BF16) return BD_ERR_UNSUPPORTED;
    if (a->out_dtype != BD_FP16 && a->out_dtype != BD_BF16 && a->out_dtype != BD_FP32) return BD_ERR_UNSUPPORTED;
    if (a->h % a->h_k) return BD_ERR_INVALID;
    if (a->h / a->h_k > 16) return BD_ERR_UNSUPPORTED;
    const int nb = pack_block_tokens(a->bits);
    if (a->block_table == nullptr) {
        if (a->s_cap % nb || a->s > a->s_cap) return BD_ERR_INVALID;
    } else {
        // paged: s_cap is the page size (reference: a multiple of 256, decode_api.cpp:351)
        if (a->s_cap % 256 || a->num_pages <= 0 || a->block_table_stride <= 0) return BD_ERR_INVALID;
        if (int64_t(a->s) > int64_t(a->block_table_stride) * a->s_cap) return BD_ERR_INVALID;
    }
    if ((a->k_res == nullptr) != (a->v_res == nullptr)) return BD_ERR_INVALID;
    if ((a->k_new == nullptr) != (a->v_new == nullptr)) return BD_ERR_INVALID;
    if (a->k_new && (!a->k_res || !a->res_lens)) return BD_ERR_INVALID;       // appends go to a tail with per-sequence lengths
    if (a->k_new && (!aligned16(a->k_new) || !aligned16(a->v_new) || a->new_stride_b % 8 || a->new_stride_h % 8))
        return BD_ERR_ALIGNMENT;
    if (a->k_res && (a->res_len < 0 || a->res_len > 256)) return BD_ERR_UNSUPPORTED;
    if (a->rotary_dim != 0) {      // rotary embedding of the appended token
        if (a->rotary_dim < 0 || a->rotary_dim > 128 || a->rotary_dim % 16) return BD_ERR_UNSUPPORTED;
        if (!a->k_new || !a->rotary_cos || !a->rotary_sin || a->rotary_positions <= 0 || a->b > 65535) return BD_ERR_INVALID;
    }
    if (a->advance) {      // device-side bookkeeping: appends, ragged lengths, a tail that holds a pack block, no pages
        if (!a->k_new || !a->cache_seqlens || !a->res_lens || a->block_table) return BD_ERR_INVALID;
        if (a->res_len < pack_block_tokens(a->bits) || a->b > 65535) return BD_ERR_INVALID;
    }
    if (!aligned16(a->q) || !aligned16(a->out) || !aligned16(a->k_pack) || !aligned16(a->k_params) ||
        !aligned16(a->v_pack) || !aligned16(a->v_params))
        return BD_ERR_ALIGNMENT;
    if (a->k_res && (!aligned16(a->k_res) || !aligned16(a->v_res))) return BD_ERR_ALIGNMENT;
    if (a->q_stride_b % 8 || a->q_stride_h % 8 || a->out_stride_b % 4 || a->out_stride_h % 4) return BD_ERR_ALIGNMENT;
    if (a->k_res && (a->res_stride_b % 8 || a->res_stride_s % 8 || a->res_stride_h % 8)) return BD_ERR_ALIGNMENT;
    // pack buffers: whole rows per batch step so that TMA coordinates stay integral
    const int64_t k_row = int64_t(a->h_k) * 128, v_row = int64_t(a->h_k) * (128 / (16 / a->bits));
    if (a->k_pack_stride_b % k_row || a->v_pack_stride_b % v_row) return BD_ERR_ALIGNMENT;
    if (a->k_params_stride_b % 4 || a->v_params_stride_b % 4 || a->v_params_stride_g % 4 || a->v_params_stride_h % 4)
        return BD_ERR_ALIGNMENT;
    return BD_OK;
}

// Small cache of encoded tensor maps: a decode loop calls with the same buffers
// every step, and encoding costs a few microseconds of host time per map.
struct MapKey {
    const void *base;
    uint64_t row_words, rows;
    uint32_t box_w, box_rows;
    int swz;
    int dev;
    bool operator==(const MapKey &o) const {
        return base == o.base && row_words == o.row_words && rows == o.rows && box_w == o.box_w &&
               box_rows == o.box_rows && swz == o.swz && dev == o.dev;
    }
};
struct MapCache {
    static constexpr int N = 32;
    MapKey keys[N];
    CUtensorMap maps[N];
    bool used[N] = {};
    int next = 0;
    std::mutex mu;
};

int get_map(CUtensorMap *out, const void *base, uint64_t row_words, uint64_t rows, uint32_t box_w,
            uint32_t box_rows, CUtensorMapSwizzle swz) {
    static MapCache cache;
    int dev = 0;
    cudaGetDevice(&dev);
    MapKey key{base, row_words, rows, box_w, box_rows, int(swz), dev};
    std::lock_guard<std::mutex> lock(cache.mu);
    for (int i = 0; i < MapCache::N; ++i)
        if (cache.used[i] && cache.keys[i] == key) {
            *out = cache.maps[i];
            return BD_OK;
        }
    CUtensorMap m;
    int rc = make_map_2d(&m, base, row_words, rows, box_w, box_rows, swz);
    if (rc != BD_OK) return rc;
    const int slot = cache.next;
    cache.next = (cache.next + 1) % MapCache::N;
    cache.keys[slot] = key;
    cache.maps[slot] = m;
    cache.used[slot] = true;
    *out = m;
    return BD_OK;
}

}  // namespace

extern "C" {

int bd_version(void) { return BD_VERSION; }

int bd_partition_segments(const int32_t *table, int b, int n_uniform, int rows, int row, int32_t *out, int max_segments) {
    if (b <= 0 || rows <= 0 || row < 0 || row >= rows || !out || max_segments < 0) return BD_ERR_INVALID;
    bd::Partition pt{table, b, n_uniform, rows};
    bd::SegWalk walk;
    walk.init(pt, row);
    bd::Segment sg;
    int n = 0;
    while (walk.next(sg)) {
        if (n < max_segments) {
            out[4 * n] = sg.ib; out[4 * n + 1] = sg.u0; out[4 * n + 2] = sg.u1; out[4 * n + 3] = sg.owns_empty ? 1 : 0;
        }
        ++n;
    }
    return n;
}

int bd_partition_parts(const int32_t *table, int b, int n_uniform, int rows, int ib, int32_t *out, int max_parts) {
    if (b <= 0 || rows <= 0 || ib < 0 || ib >= b || !out || max_parts < 0) return BD_ERR_INVALID;
    bd::Partition pt{table, b, n_uniform, rows};
    int n = 0;
    bd::for_each_part(pt, ib, [&](int c) {
        if (n < max_parts) out[n] = c;
        ++n;
    });
    return n;
}

const char *bd_strerror(int code) {
    switch (code) {
        case BD_OK: return "ok";
        case BD_ERR_INVALID: return "invalid argument (null pointer, bad size or stride)";
        case BD_ERR_UNSUPPORTED: return "unsupported configuration (bits must be 2 or 4, group 32, 64 or 128, head_dim 128, "
                                        "fp16/bf16, at most 16 query heads per KV head, tail of at most 256 tokens)";
        case BD_ERR_ALIGNMENT: return "pointer or stride not aligned (16-byte pointers, strides in whole rows / multiples of 8)";
        case BD_ERR_WORKSPACE: return "workspace missing or too small (see bd_decode_workspace_bytes)";
        case BD_ERR_CUDA: return "a CUDA runtime or driver call failed";
        case BD_ERR_DEVICE: return "device is not compute capability 10.x";
        case BD_ERR_TIMEOUT: return "a bounded wait inside a kernel ran out";
        case BD_ERR_CAPACITY: return "a tail filled up but the packed buffers have no room for another block";
        case BD_ERR_POSITION: return "a token position lies beyond the rotary tables";
        case BD_ERR_PAGE: return "a block_table entry lies outside [0, num_pages); its tokens were left out";
        case BD_ERR_SCRATCH_LIMIT: return "this call needs more scratch than the library's fixed area holds "
                                          "(bd_noalloc_scratch_bytes); use bd_decode with a workspace";
        default: return "unknown error";
    }
}

int bd_decode_plan(const bd_decode_args *a, int32_t out[4]) {
    if (!out) return BD_ERR_INVALID;
    int rc = check_decode_args(a);
    if (rc != BD_OK) return rc;
    DeviceInfo info;
    rc = current_device_info(info);
    if (rc != BD_OK) return rc;
    DecodePlan plan;
    make_plan(a, info.sm_count, plan);
    const int gq = a->h / a->h_k;
    out[0] = plan.rows;
    out[1] = bd::decode_ctas_per_sm(a->bits, a->group, gq, plan.two_ctas);
    out[2] = bd::decode_warps(a->bits, a->group, gq, plan.two_ctas);
    out[3] = (plan.ragged ? 1 : 0) + (a->rotary_dim > 0 ? 1 : 0) + 1 + (plan.rows > 4 * a->b ? 1 : 0) + (a->advance ? 2 : 0);
    return BD_OK;
}

int bd_plan_splits(int b, int h_k, int64_t max_s, int bits, int sm_count, int ctas_per_sm) {
    if (bits != 2 && bits != 4) return 1;
    return plan_rows(b, h_k, max_s, bits, sm_count, ctas_per_sm);
}

int bd_pack(const bd_pack_args *a, bd_stream_t stream) {
    if (!a || !a->k || !a->v || !a->k_pack || !a->k_params || !a->v_pack || !a->v_params) return BD_ERR_INVALID;
    if (a->b <= 0 || a->h_k <= 0 || a->s < 0 || a->dst_token_offset < 0) return BD_ERR_INVALID;
    if (!config_supported(a->bits, a->group, a->d)) return BD_ERR_UNSUPPORTED;
    if (a->dtype != BD_FP16 && a->dtype != BD_BF16) return BD_ERR_UNSUPPORTED;
    const int nb = pack_block_tokens(a->bits);
    if (a->s % nb || a->dst_token_offset % nb) return BD_ERR_INVALID;
    if (a->s / nb > 65535 || a->b > 65535) return BD_ERR_INVALID;      // grid.y, grid.z
    // 16-byte vector loads of the inputs and 16-byte stores of the V codes
    if ((reinterpret_cast<uintptr_t>(a->k) | reinterpret_cast<uintptr_t>(a->v) |
         reinterpret_cast<uintptr_t>(a->k_pack) | reinterpret_cast<uintptr_t>(a->v_pack) |
         reinterpret_cast<uintptr_t>(a->k_params) | reinterpret_cast<uintptr_t>(a->v_params)) & 15u)
        return BD_ERR_ALIGNMENT;
    if ((a->k_stride_b | a->k_stride_s | a->k_stride_h | a->v_stride_b | a->v_stride_s | a->v_stride_h |
         a->k_pack_stride_b | a->v_pack_stride_b) & 7)
        return BD_ERR_ALIGNMENT;
    if (a->s == 0) return BD_OK;
    DeviceInfo info;
    int rc = current_device_info(info);
    if (rc != BD_OK) return rc;
    if (info.cc_major != 10) return BD_ERR_DEVICE;
    PackParams p;
    std::memset(&p, 0, sizeof(p));
    p.k = a->k; p.v = a->v;
    p.k_stride_b = a->k_stride_b; p.k_stride_s = a->k_stride_s; p.k_stride_h = a->k_stride_h;
    p.v_stride_b = a->v_stride_b; p.v_stride_s = a->v_stride_s; p.v_stride_h = a->v_stride_h;
    p.k_pack = a->k_pack; p.k_params = a->k_params; p.v_pack = a->v_pack; p.v_params = a->v_params;
    p.k_pack_stride_b = a->k_pack_stride_b; p.k_params_stride_b = a->k_params_stride_b;
    p.v_pack_stride_b = a->v_pack_stride_b;
    p.v_params_stride_b = a->v_params_stride_b; p.v_params_stride_g = a->v_params_stride_g;
    p.v_params_stride_h = a->v_params_stride_h;
    p.b = a->b; p.s = a->s; p.h_k = a->h_k; p.dst_token_offset = a->dst_token_offset;
    p.approx_div = (a->flags & BD_PACK_APPROX_DIV) ? 1 : 0;
    cudaError_t err = bd::launch_pack(p, a->bits, a->group, a->dtype, static_cast<cudaStream_t>(stream));
    return err == cudaSuccess ? BD_OK : BD_ERR_CUDA;
}

size_t bd_decode_workspace_bytes(const bd_decode_args *a) {
    if (!a || a->b <= 0 || a->h <= 0 || a->h_k <= 0 || (a->bits != 2 && a->bits != 4)) return 0;
    DeviceInfo info;
    int sm = 148;
    if (a->num_splits <= 0) {
        if (current_device_info(info) != BD_OK) return 0;
        sm = info.sm_count;
    }
    DecodePlan plan;
    make_plan(a, sm, plan);
    return plan.total_bytes;
}

// The decode step; with `x` the step of one rank of a sequence split: every segment leaves its part in
// the workspace and the exchange kernel merges them, sends the rows to the peers and merges theirs.
static int decode_step(const bd_decode_args *a, const bd_exchange_args *x, bd_stream_t stream_) {
    int rc = check_decode_args(a);
    if (rc != BD_OK) return rc;
    bd::ExchangeParams xp;
    if (x) {
        rc = bd::fill_exchange_params(x, xp);
        if (rc != BD_OK) return rc;
        if (x->rows != int64_t(a->b) * a->h) return BD_ERR_INVALID;
    }
    DeviceInfo info;
    rc = current_device_info(info);
    if (rc != BD_OK) return rc;
    if (info.cc_major != 10) return BD_ERR_DEVICE;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);

    DecodePlan plan;
    make_plan(a, info.sm_count, plan);
    if (!a->workspace || a->workspace_bytes < plan.total_bytes) return BD_ERR_WORKSPACE;
    if (!aligned16(a->workspace)) return BD_ERR_ALIGNMENT;

    const int P = 16 / a->bits, nb = 32 * P, dp = 128 / P;
    const int64_t k_row = int64_t(a->h_k) * 128, v_row = int64_t(a->h_k) * dp;
    const int64_t k_batch_rows = a->k_pack_stride_b / k_row, v_batch_rows = a->v_pack_stride_b / v_row;
    const int64_t units = a->block_table ? a->num_pages : a->b;      // sequences, or pages of a paged cache
    const uint64_t k_rows_total = uint64_t(units - 1) * k_batch_rows + uint64_t(a->s_cap / P);
    const uint64_t v_rows_total = uint64_t(units - 1) * v_batch_rows + uint64_t(a->s_cap);
    if (k_rows_total > 0x7fffffffull || v_rows_total > 0x7fffffffull) return BD_ERR_INVALID;
    if (int64_t(plan.rows) * a->h_k > 0x7fffffffll) return BD_ERR_INVALID;

    CUtensorMap kmap, vmap;
    rc = get_map(&kmap, a->k_pack, uint64_t(k_row), k_rows_total, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != BD_OK) return rc;
    rc = get_map(&vmap, a->v_pack, uint64_t(v_row), v_rows_total, uint32_t(dp), uint32_t(nb),
                 a->bits == 4 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    if (rc != BD_OK) return rc;

    uint8_t *ws = static_cast<uint8_t *>(a->workspace);
    bd::Partition part;
    part.table = plan.ragged ? reinterpret_cast<const int32_t *>(ws + plan.off_table) : nullptr;
    part.b = a->b;
    part.n_uniform = plan.n_uniform;
    part.R = plan.rows;

    cudaError_t err;
    if (plan.ragged) {
        bd::PrefixParams pp;
        pp.cache_seqlens = a->cache_seqlens;
        pp.res_lens = a->k_res ? a->res_lens : nullptr;
        pp.res_len = a->k_res ? a->res_len : 0;
        pp.res_extra = a->k_new ? 1 : 0;
        pp.table = reinterpret_cast<int32_t *>(ws + plan.off_table);
        pp.b = a->b; pp.s = a->s; pp.block_tokens = nb;
        err = bd::launch_prefix(pp, stream);
        if (err != cudaSuccess) return BD_ERR_CUDA;
    }

    DecodeParams p;
    std::memset(&p, 0, sizeof(p));
    p.q = a->q;
    p.q_stride_b = a->q_stride_b; p.q_stride_h = a->q_stride_h;
    p.k_params = static_cast<const uint16_t *>(a->k_params);
    p.v_params = static_cast<const uint16_t *>(a->v_params);
    p.k_params_stride_b = 2 * a->k_params_stride_b;
    p.v_params_stride_b = 2 * a->v_params_stride_b;
    p.v_params_stride_g = 2 * a->v_params_stride_g;
    p.v_params_stride_h = 2 * a->v_params_stride_h;
    p.cache_seqlens = a->cache_seqlens;
    p.block_table = a->block_table;
    p.block_table_stride = a->block_table_stride;
    p.blocks_per_page = a->block_table ? a->s_cap / nb : 0;
    p.num_pages = a->num_pages;
    p.spin_limit = a->spin_limit ? a->spin_limit : (1u << 22);
    p.test_starve = a->test_starve;
    p.k_res = a->k_res; p.v_res = a->v_res;
    p.res_stride_b = a->res_stride_b; p.res_stride_s = a->res_stride_s; p.res_stride_h = a->res_stride_h;
    p.res_lens = a->res_lens; p.res_len = a->k_res ? a->res_len : 0;
    p.res_cap = p.res_len;
    p.k_res_out = const_cast<void *>(a->k_res); p.v_res_out = const_cast<void *>(a->v_res);
    p.k_new = a->k_new; p.v_new = a->v_new;
    p.new_stride_b = a->new_stride_b; p.new_stride_h = a->new_stride_h;
    p.b = a->b; p.h = a->h; p.h_k = a->h_k; p.gq = a->h / a->h_k;
    p.s = a->s;
    p.k_batch_rows = int32_t(k_batch_rows);
    p.v_batch_rows = int32_t(v_batch_rows);
    p.dtype = a->dtype;
    p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
    p.part = part;
    // workspace: [status word, 16 B][arrival counters][sequence table][segment partials]
    p.counters = reinterpret_cast<int32_t *>(ws + plan.off_counters);
    p.warp_acc = reinterpret_cast<float *>(ws + plan.off_warp_acc);
    p.out = a->out; p.lse = a->lse;
    p.out_stride_b = a->out_stride_b; p.out_stride_h = a->out_stride_h;
    p.out_dtype = a->out_dtype;
    p.status = reinterpret_cast<int32_t *>(ws);
    p.part_out = reinterpret_cast<float *>(ws + plan.off_part_out);
    p.part_lse = reinterpret_cast<float *>(ws + plan.off_part_lse);

    // More than four parts per sequence on average (few long sequences cut over all SMs): one warp
    // merging them at the end of the decode kernel would be the tail of the step; a second kernel
    // with a warp per (sequence, query head) does it in parallel.
    if (a->rotary_dim > 0) {
        // q and the new key rotated at the token's position into scratch copies; the decode kernel reads those
        bd::RopeParams rp;
        std::memset(&rp, 0, sizeof(rp));
        rp.q = a->q; rp.k_new = a->k_new; rp.v_new = a->v_new;
        rp.q_stride_b = a->q_stride_b; rp.q_stride_h = a->q_stride_h;
        rp.new_stride_b = a->new_stride_b; rp.new_stride_h = a->new_stride_h;
        rp.q_out = ws + plan.off_rope_q; rp.k_out = ws + plan.off_rope_k; rp.v_out = ws + plan.off_rope_v;
        rp.cos_tab = a->rotary_cos; rp.sin_tab = a->rotary_sin;
        rp.cache_seqlens = a->cache_seqlens; rp.res_lens = a->res_lens;
        rp.s = a->s; rp.res_len = a->res_len;
        rp.b = a->b; rp.h = a->h; rp.h_k = a->h_k;
        rp.rotary_dim = a->rotary_dim; rp.interleaved = a->rotary_interleaved ? 1 : 0;
        rp.positions = a->rotary_positions; rp.dtype = a->dtype;
        rp.status = reinterpret_cast<int32_t *>(ws);
        err = bd::launch_rope(rp, stream);
        if (err != cudaSuccess) return BD_ERR_CUDA;
        p.q = rp.q_out; p.q_stride_b = int64_t(a->h) * 128; p.q_stride_h = 128;
        p.k_new = rp.k_out; p.v_new = rp.v_out; p.new_stride_b = int64_t(a->h_k) * 128; p.new_stride_h = 128;
    }
    p.defer_merge = (x || plan.rows > 4 * a->b) ? 1 : 0;
    p.leave_parts = x ? 1 : 0;
    p.two_ctas = plan.two_ctas;
    err = bd::launch_decode(p, kmap, vmap, a->bits, a->group, stream);
    if (err != cudaSuccess) return BD_ERR_CUDA;
    if (x) {
        xp.part_out = p.part_out; xp.part_lse = p.part_lse;
        xp.out = p.out; xp.lse = p.lse;
        xp.out_stride_b = p.out_stride_b; xp.out_stride_h = p.out_stride_h;
        xp.h = p.h; xp.out_dtype = p.out_dtype;
        xp.part = p.part; xp.h_k = p.h_k; xp.gq = p.gq;
        err = bd::launch_exchange_parts(xp, stream);
        if (err != cudaSuccess) return BD_ERR_CUDA;
    } else if (p.defer_merge) {
        err = bd::launch_merge_parts(p, true, stream);
        if (err != cudaSuccess) return BD_ERR_CUDA;
    }

    if (a->advance) {
        // roll-over: tails that this step's token filled become the next pack block of their sequence ...
        PackParams pk;
        std::memset(&pk, 0, sizeof(pk));
        pk.k = a->k_res; pk.v = a->v_res;
        pk.k_stride_b = pk.v_stride_b = a->res_stride_b;
        pk.k_stride_s = pk.v_stride_s = a->res_stride_s;
        pk.k_stride_h = pk.v_stride_h = a->res_stride_h;
        pk.k_pack = const_cast<void *>(a->k_pack); pk.k_params = const_cast<void *>(a->k_params);
        pk.v_pack = const_cast<void *>(a->v_pack); pk.v_params = const_cast<void *>(a->v_params);
        pk.k_pack_stride_b = a->k_pack_stride_b; pk.k_params_stride_b = a->k_params_stride_b;
        pk.v_pack_stride_b = a->v_pack_stride_b;
        pk.v_params_stride_b = a->v_params_stride_b; pk.v_params_stride_g = a->v_params_stride_g;
        pk.v_params_stride_h = a->v_params_stride_h;
        pk.b = a->b; pk.s = nb; pk.h_k = a->h_k;
        pk.roll_res_lens = a->res_lens; pk.roll_cache_seqlens = a->cache_seqlens; pk.roll_s_cap = a->s_cap;
        err = bd::launch_pack(pk, a->bits, a->group, a->dtype, stream);
        if (err != cudaSuccess) return BD_ERR_CUDA;
        // ... and every sequence's lengths move on
        bd::AdvanceParams ad;
        ad.cache_seqlens = const_cast<int32_t *>(a->cache_seqlens);
        ad.res_lens = const_cast<int32_t *>(a->res_lens);
        ad.b = a->b; ad.block_tokens = nb; ad.s_cap = a->s_cap; ad.res_cap = a->res_len;
        ad.status = reinterpret_cast<int32_t *>(ws);
        err = bd::launch_advance(ad, stream);
        if (err != cudaSuccess) return BD_ERR_CUDA;
    }

    return BD_OK;
}

int bd_decode(const bd_decode_args *a, bd_stream_t stream) { return decode_step(a, nullptr, stream); }

int bd_decode_exchange(const bd_decode_args *a, const bd_exchange_args *x, bd_stream_t stream) {
    if (!x) return BD_ERR_INVALID;
    return decode_step(a, x, stream);
}

// ---------------------------------------------------------------------------
// bd_decode_noalloc: decode with the library's own fixed scratch area.
//
// Some callers cannot give bd_decode a workspace because they cannot allocate
// device memory where they call it: a serving runtime that has handed every free
// byte to its KV-cache pool, code on a latency path that must not touch the
// allocator, a plugin whose host forbids cudaMalloc after start-up.  For them the
// scratch lives in a file-scope device array, part of the loaded library image,
// so every GPU that loads the library holds these bytes until the process ends.
//
// The array's name is only a host-side handle, not a device address; the address
// kernels can use comes from cudaGetSymbolAddress, asked once per device (with
// that device current) the first time this entry point runs there.
// ---------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_noalloc_scratch[BD_NOALLOC_SCRATCH_BYTES];

namespace {
void *noalloc_scratch_address(int *rc_out) {
    static void *ptr[64] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { *rc_out = BD_ERR_CUDA; return nullptr; }
    std::lock_guard<std::mutex> lock(mu);
    if (!ptr[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) {
            *rc_out = BD_ERR_CUDA;
            return nullptr;
        }
        ptr[dev] = p;
    }
    *rc_out = BD_OK;
    return ptr[dev];
}
}  // namespace

size_t bd_noalloc_scratch_bytes(void) { return BD_NOALLOC_SCRATCH_BYTES; }

int bd_decode_noalloc(const bd_decode_args *a, bd_stream_t stream_) {
    int rc = check_decode_args(a);
    if (rc != BD_OK) return rc;
    DeviceInfo info;
    rc = current_device_info(info);
    if (rc != BD_OK) return rc;
    if (info.cc_major != 10) return BD_ERR_DEVICE;
    DecodePlan plan;
    make_plan(a, info.sm_count, plan);
    if (plan.total_bytes > BD_NOALLOC_SCRATCH_BYTES) return BD_ERR_SCRATCH_LIMIT;
    void *scratch = noalloc_scratch_address(&rc);
    if (rc != BD_OK) return rc;
    // The area keeps whatever the previous call left (partials of another shape may sit
    // where this call's counters go): clear the arrival counters, the only bytes that must
    // start at zero.  The status word in front of them is left as it is, so an error a step
    // reported stays readable (bd_read_status(NULL, stream) returns and clears it); a freshly
    // loaded library has it at zero.  No allocation: a memset node on the stream.
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (cudaMemsetAsync(static_cast<unsigned char *>(scratch) + plan.off_counters, 0,
                        plan.off_table - plan.off_counters, stream) != cudaSuccess)
        return BD_ERR_CUDA;
    bd_decode_args args = *a;
    args.workspace = scratch;
    args.workspace_bytes = BD_NOALLOC_SCRATCH_BYTES;
    return bd_decode(&args, stream_);
}

int bd_combine(const bd_combine_args *a, bd_stream_t stream) {
    if (!a || !a->part_out || !a->part_lse || !a->out) return BD_ERR_INVALID;
    if (a->n_parts < 1 || a->n_parts > BD_MAX_PARTS || a->rows <= 0) return BD_ERR_INVALID;
    if (a->d != 128) return BD_ERR_UNSUPPORTED;
    if (a->out_dtype != BD_FP16 && a->out_dtype != BD_BF16 && a->out_dtype != BD_FP32) return BD_ERR_UNSUPPORTED;
    if (!aligned16(a->out)) return BD_ERR_ALIGNMENT;
    bd::CombinePartsParams p;
    std::memset(&p, 0, sizeof(p));
    for (int i = 0; i < a->n_parts; ++i) {
        if (!a->part_out[i] || !a->part_lse[i]) return BD_ERR_INVALID;
        if (!aligned16(a->part_out[i])) return BD_ERR_ALIGNMENT;
        p.part_out[i] = a->part_out[i];
        p.part_lse[i] = a->part_lse[i];
    }
    p.out = a->out; p.lse = a->lse; p.rows = a->rows; p.n_parts = a->n_parts; p.out_dtype = a->out_dtype;
    cudaError_t err = bd::launch_combine_parts(p, static_cast<cudaStream_t>(stream));
    return err == cudaSuccess ? BD_OK : BD_ERR_CUDA;
}

int bd_read_status(const void *workspace, bd_stream_t stream) {
    if (!workspace) {            // the fixed area of bd_decode_noalloc on the current device
        int rc = BD_OK;
        workspace = noalloc_scratch_address(&rc);
        if (rc != BD_OK) return rc;
    }
    if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess) return BD_ERR_CUDA;
    int32_t v = 0;   // the status word is the first word of the workspace
    if (cudaMemcpy(&v, workspace, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return BD_ERR_CUDA;
    if (v != 0 && cudaMemset(const_cast<void *>(workspace), 0, sizeof(v)) != cudaSuccess) return BD_ERR_CUDA;
    return v;
}

}  // extern "C"
