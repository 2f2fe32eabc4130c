// Cross-GPU exchange and merge of partial attention results for a sequence that is split over GPUs:
// the one step of the decode path that needs other GPUs (the reference has no multi-GPU code; the
// arithmetic is its split combine, csrc/bit_decode/src/flash_fwd_kernel.h:1217-1231, 1280-1298,
// applied one level up).
//
// Every rank owns an exchange AREA in its own memory that its peers have mapped (CUDA IPC):
//
//   [header: epoch, finished-CTA counter, status]  [flags: one per rank]  [slots: 2 x world partials]
//
// One kernel per step and rank does the whole exchange:
//   1. CTA c of rank r stores r's normalised partial (out rows fp32, then the LSEs) into slot
//      [epoch parity][r] of rank c's area with plain 16-byte stores over NVLink, fences, and sets
//      flag[r] of rank c's area to the epoch (release).
//   2. Every CTA waits until all flags of its OWN area show the epoch (acquire loads of local memory,
//      bounded: after `spin_limit` polls the kernel writes BD_ERR_TIMEOUT to the area's status word and
//      returns without touching `out`).
//   3. The CTAs merge the world partials row by row (one warp per row, loads that bypass L1: the slots
//      are rewritten by peers every second step) and write the result.
//   4. The CTA that finishes last advances the area's epoch for the next step.
// Nothing here uses TMA, bulk copies or multicast on peer memory: plain stores and flag writes only.
// Two slots per rank (epoch parity) make it safe for a fast rank to publish step n + 1 while a slow rank
// still merges step n: step n + 2 can only be published after the slow rank's flag for n + 1 was seen,
// and it sets that flag after its merge of step n is done (same stream).
// Ranks are separate processes, one per GPU; kernels of different ranks never share a GPU.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>

#include "bd_common.cuh"
#include "bd_kernels.h"

namespace bd {

constexpr int kXHeaderBytes = 128;
constexpr int kXFlagStride = 32;              // bytes between flags (one sector each)
constexpr int kXThreads = 256;

struct XLayout {
    size_t flags_off, slots_off, slot_floats, total;
};
__host__ __device__ inline XLayout xchg_layout(int world, int64_t rows) {
    XLayout l;
    l.flags_off = kXHeaderBytes;
    l.slots_off = (l.flags_off + size_t(world) * kXFlagStride + 255) & ~size_t(255);
    l.slot_floats = (size_t(rows) * (kHeadDim + 1) + 63) & ~size_t(63);   // out rows, then LSEs; 256-byte multiple
    l.total = l.slots_off + 2 * size_t(world) * l.slot_floats * sizeof(float);
    return l;
}

struct ExchangeParams {
    uint8_t *area[BD_MAX_PARTS];     // area of every rank as mapped into this process; area[rank] is local
    const float *part_out;           // (rows, 128) this rank's normalised partial
    const float *part_lse;           // (rows)
    void *out;
    float *lse;
    int64_t rows;
    int32_t rank, world, out_dtype;
    uint32_t spin_limit;
};

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kXThreads) bd_exchange_kernel(const ExchangeParams p) {
    __shared__ int timed_out;
    const XLayout L = xchg_layout(p.world, p.rows);
    uint8_t *mine = p.area[p.rank];
    uint32_t *hdr = reinterpret_cast<uint32_t *>(mine);              // [0] epoch, [1] finished CTAs, [2] status
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(hdr) + 1;
    const uint32_t par = epoch & 1u;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) timed_out = 0;

    // ---- 1. publish to the peer this CTA serves (CTAs beyond `world` only help with the merge)
    const int peer = blockIdx.x;
    if (peer < p.world && peer != p.rank) {
        float *dst = reinterpret_cast<float *>(p.area[peer] + L.slots_off) + (size_t(par) * p.world + p.rank) * L.slot_floats;
        const int64_t n4 = p.rows * (kHeadDim / 4);
        const float4 *src = reinterpret_cast<const float4 *>(p.part_out);
        for (int64_t i = tid; i < n4; i += kXThreads) reinterpret_cast<float4 *>(dst)[i] = src[i];
        float *dl = dst + p.rows * kHeadDim;
        for (int64_t i = tid; i < p.rows; i += kXThreads) dl[i] = p.part_lse[i];
        __threadfence_system();
        __syncthreads();
        if (tid == 0)
            st_release_sys(reinterpret_cast<uint32_t *>(p.area[peer] + L.flags_off + size_t(p.rank) * kXFlagStride), epoch);
    }

    // ---- 2. wait for every peer's partial of this epoch in the local area (bounded)
    __syncthreads();
    if (tid < p.world && tid != p.rank) {
        const uint32_t *flag = reinterpret_cast<const uint32_t *>(mine + L.flags_off + size_t(tid) * kXFlagStride);
        bool ok = false;
        for (uint32_t it = 0; it < p.spin_limit; ++it) {
            if (int32_t(ld_acquire_sys(flag) - epoch) >= 0) { ok = true; break; }
            if (it > 32) __nanosleep(it > 4096 ? 1000 : 100);
        }
        if (!ok) timed_out = 1;
    }
    __syncthreads();
    if (timed_out) {
        if (tid == 0) atomicExch(reinterpret_cast<int *>(hdr + 2), BD_ERR_TIMEOUT);
    } else {
        // ---- 3. merge: one warp per row, lane owns 4 head dims; own partial straight from part_out
        const float *slots = reinterpret_cast<const float *>(mine + L.slots_off) + size_t(par) * p.world * L.slot_floats;
        for (int64_t row = int64_t(blockIdx.x) * (kXThreads / 32) + warp; row < p.rows;
             row += int64_t(gridDim.x) * (kXThreads / 32)) {
            float l[BD_MAX_PARTS];
            float mx = -INFINITY;
#pragma unroll
            for (int r = 0; r < BD_MAX_PARTS; ++r) {
                l[r] = -INFINITY;
                if (r < p.world)
                    l[r] = (r == p.rank) ? p.part_lse[row] : __ldcg(slots + size_t(r) * L.slot_floats + p.rows * kHeadDim + row);
                mx = fmaxf(mx, l[r]);
            }
            float sum = 0.f;
            if (mx != -INFINITY) {
#pragma unroll
                for (int r = 0; r < BD_MAX_PARTS; ++r) sum += (r < p.world) ? __expf(l[r] - mx) : 0.f;
            }
            const float lse = (sum > 0.f) ? mx + logf(sum) : -INFINITY;
            float o[4] = {0.f, 0.f, 0.f, 0.f};
            if (sum > 0.f) {
#pragma unroll
                for (int r = 0; r < BD_MAX_PARTS; ++r) {
                    if (r < p.world) {
                        const float4 *src = (r == p.rank) ? reinterpret_cast<const float4 *>(p.part_out)
                                                          : reinterpret_cast<const float4 *>(slots + size_t(r) * L.slot_floats);
                        const float4 v = __ldcg(src + row * (kHeadDim / 4) + lane);
                        const float wgt = __expf(l[r] - lse);
                        o[0] = fmaf(wgt, v.x, o[0]); o[1] = fmaf(wgt, v.y, o[1]);
                        o[2] = fmaf(wgt, v.z, o[2]); o[3] = fmaf(wgt, v.w, o[3]);
                    }
                }
            }
            const int64_t idx = row * kHeadDim + 4 * lane;
            if (p.out_dtype == BD_FP16) {
                __half2 a = __floats2half2_rn(o[0], o[1]), b = __floats2half2_rn(o[2], o[3]);
                *reinterpret_cast<uint2 *>(static_cast<__half *>(p.out) + idx) =
                    make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b));
            } else if (p.out_dtype == BD_BF16) {
                __nv_bfloat162 a = __floats2bfloat162_rn(o[0], o[1]), b = __floats2bfloat162_rn(o[2], o[3]);
                *reinterpret_cast<uint2 *>(static_cast<__nv_bfloat16 *>(p.out) + idx) =
                    make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b));
            } else {
                *reinterpret_cast<float4 *>(static_cast<float *>(p.out) + idx) = make_float4(o[0], o[1], o[2], o[3]);
            }
            if (lane == 0 && p.lse) p.lse[row] = lse;
        }
    }

    // ---- 4. the CTA that finishes last moves the epoch on (every CTA has read it by then)
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(hdr + 1, 1u) == gridDim.x - 1) {
            hdr[1] = 0;
            *reinterpret_cast<volatile uint32_t *>(hdr) = epoch;
        }
    }
}

}  // namespace bd

extern "C" {

size_t bd_exchange_area_bytes(int world, int64_t rows) {
    if (world < 1 || world > BD_MAX_PARTS || rows <= 0) return 0;
    return bd::xchg_layout(world, rows).total;
}

int bd_peer_alloc(size_t bytes, void **ptr) {
    if (!ptr || bytes == 0) return BD_ERR_INVALID;
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return BD_ERR_CUDA;
    if (cudaMemset(p, 0, bytes) != cudaSuccess) { cudaFree(p); return BD_ERR_CUDA; }
    *ptr = p;
    return BD_OK;
}

int bd_peer_free(void *ptr) { return (!ptr || cudaFree(ptr) == cudaSuccess) ? BD_OK : BD_ERR_CUDA; }

int bd_peer_export(const void *ptr, void *handle64) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    if (!ptr || !handle64) return BD_ERR_INVALID;
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, const_cast<void *>(ptr)) != cudaSuccess) return BD_ERR_CUDA;
    std::memcpy(handle64, &h, sizeof(h));
    return BD_OK;
}

int bd_peer_open(const void *handle64, void **ptr) {
    if (!handle64 || !ptr) return BD_ERR_INVALID;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, sizeof(h));
    void *p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return BD_ERR_CUDA;
    *ptr = p;
    return BD_OK;
}

int bd_peer_close(void *ptr) { return (!ptr || cudaIpcCloseMemHandle(ptr) == cudaSuccess) ? BD_OK : BD_ERR_CUDA; }

int bd_exchange_combine(const bd_exchange_args *a, bd_stream_t stream) {
    if (!a || !a->areas || !a->part_out || !a->part_lse || !a->out) return BD_ERR_INVALID;
    if (a->world < 1 || a->world > BD_MAX_PARTS || a->rank < 0 || a->rank >= a->world || a->rows <= 0) return BD_ERR_INVALID;
    if (a->d != 128) return BD_ERR_UNSUPPORTED;
    if (a->out_dtype != BD_FP16 && a->out_dtype != BD_BF16 && a->out_dtype != BD_FP32) return BD_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a->part_out) | reinterpret_cast<uintptr_t>(a->out)) & 15u) return BD_ERR_ALIGNMENT;
    bd::ExchangeParams p;
    std::memset(&p, 0, sizeof(p));
    for (int r = 0; r < a->world; ++r) {
        if (!a->areas[r] || (reinterpret_cast<uintptr_t>(a->areas[r]) & 255u)) return BD_ERR_ALIGNMENT;
        p.area[r] = static_cast<uint8_t *>(a->areas[r]);
    }
    p.part_out = a->part_out; p.part_lse = a->part_lse; p.out = a->out; p.lse = a->lse;
    p.rows = a->rows; p.rank = a->rank; p.world = a->world; p.out_dtype = a->out_dtype;
    p.spin_limit = a->spin_limit ? a->spin_limit : (1u << 22);
    // one CTA per peer to publish; a few more help with the merge when there are many rows
    const int64_t want = (a->rows + (bd::kXThreads / 32) - 1) / (bd::kXThreads / 32);
    const unsigned grid = unsigned(std::max<int64_t>(a->world, std::min<int64_t>(want, 32)));
    bd::bd_exchange_kernel<<<grid, bd::kXThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return cudaGetLastError() == cudaSuccess ? BD_OK : BD_ERR_CUDA;
}

int bd_exchange_put(void *area, int world, int64_t rows, int from_rank, uint32_t epoch, const float *part_out,
                    const float *part_lse, bd_stream_t stream_) {
    if (!area || !part_out || !part_lse || world < 1 || world > BD_MAX_PARTS || from_rank < 0 || from_rank >= world || rows <= 0)
        return BD_ERR_INVALID;
    const bd::XLayout L = bd::xchg_layout(world, rows);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    uint8_t *base = static_cast<uint8_t *>(area);
    float *dst = reinterpret_cast<float *>(base + L.slots_off) + (size_t(epoch & 1u) * world + from_rank) * L.slot_floats;
    if (cudaMemcpyAsync(dst, part_out, size_t(rows) * 128 * sizeof(float), cudaMemcpyDefault, stream) != cudaSuccess) return BD_ERR_CUDA;
    if (cudaMemcpyAsync(dst + rows * 128, part_lse, size_t(rows) * sizeof(float), cudaMemcpyDefault, stream) != cudaSuccess)
        return BD_ERR_CUDA;
    if (cudaMemcpyAsync(base + L.flags_off + size_t(from_rank) * bd::kXFlagStride, &epoch, sizeof(epoch), cudaMemcpyHostToDevice,
                        stream) != cudaSuccess)
        return BD_ERR_CUDA;
    return cudaStreamSynchronize(stream) == cudaSuccess ? BD_OK : BD_ERR_CUDA;   // `epoch` lives on this stack frame
}

int bd_exchange_state(const void *area, bd_stream_t stream, uint32_t *epoch_out) {
    if (!area) return BD_ERR_INVALID;
    if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess) return BD_ERR_CUDA;
    uint32_t hdr[4] = {0, 0, 0, 0};
    if (cudaMemcpy(hdr, area, sizeof(hdr), cudaMemcpyDeviceToHost) != cudaSuccess) return BD_ERR_CUDA;
    if (epoch_out) *epoch_out = hdr[0];
    const int status = int(hdr[2]);
    if (status != 0) {
        const uint32_t zero = 0;
        if (cudaMemcpy(static_cast<uint8_t *>(const_cast<void *>(area)) + 8, &zero, 4, cudaMemcpyHostToDevice) != cudaSuccess)
            return BD_ERR_CUDA;
    }
    return status;
}

}  // extern "C"
