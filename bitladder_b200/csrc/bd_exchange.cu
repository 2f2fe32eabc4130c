// Cross-GPU exchange and merge of partial attention results for a sequence that is split over GPUs:
// the one step of the decode path that needs other GPUs (the reference has no multi-GPU code; the
// arithmetic is its split combine, csrc/bit_decode/src/flash_fwd_kernel.h:1217-1231, 1280-1298,
// applied one level up).
//
// Every rank owns an exchange AREA in its own memory that its peers have mapped (CUDA IPC):
//
//   [header: epoch, finished-CTA counter, status]  [slots: 2 x world x rows records]
//
// A record is one row (one sequence and query head) of a rank's partial: 128 fp32 values and the row's
// log-sum-exp, written as 16-byte units {value, epoch, value, epoch}: every 8-byte half carries the
// step's epoch beside its value, and 8-byte stores arrive whole, so a reader that sees the epoch in a
// half has that half's value: no fence and no separate flag between the data and its "ready" mark,
// one NVLink crossing from the sender's registers to the reader's poll.
//
// One kernel per step and rank does the whole exchange, one warp per row:
//   1. the warp gets the row of this rank's partial: from (part_out, part_lse), or, fused with the
//      decode step (bd_decode_exchange), by merging the parts the decode kernel's CTAs left in its
//      workspace (the work of the local parts-merge kernel, which is then not launched);
//   2. it stores the row into slot [epoch parity][this rank][row] of every peer's area (plain 16-byte
//      stores over NVLink, each lane its 4 values);
//   3. it polls slot [epoch parity][r][row] of its OWN area for every peer r until all halves show the
//      epoch (volatile loads of local memory, bounded: after `spin_limit` polls it puts BD_ERR_TIMEOUT
//      into the area's status word and leaves the row of `out` untouched);
//   4. it merges the world partials of the row and writes the result.
// The CTA that finishes last advances the area's epoch for the next step.
// Nothing here uses TMA, bulk copies or multicast on peer memory: plain stores and loads only.
// Two slots per rank (epoch parity) make it safe for a fast rank to publish step n + 1 while a slow rank
// still merges step n: step n + 2 can only be published after the slow rank's row of n + 1 was seen,
// and it sends that after its merge of step n is done (same stream).  Areas start zero-filled and the
// first epoch is 1; after the first two steps no slot holds a zero epoch any more, so the counter may
// wrap.
// Ranks are separate processes, one per GPU; kernels of different ranks never share a GPU.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <vector>

#include "bd_common.cuh"
#include "bd_kernels.h"

namespace bd {

constexpr int kXHeaderBytes = 256;
constexpr int kXRecordBytes = (kHeadDim / 2 + 1) * 16;     // 64 units of two values, one unit for the log-sum-exp
constexpr int kXWarps = 4;

struct XLayout {
    size_t slots_off, total;
};
__host__ __device__ inline XLayout xchg_layout(int world, int64_t rows) {
    XLayout l;
    l.slots_off = kXHeaderBytes;
    l.total = (l.slots_off + 2 * size_t(world) * size_t(rows) * kXRecordBytes + 255) & ~size_t(255);
    return l;
}
__host__ __device__ inline size_t xchg_record_off(int world, int64_t rows, uint32_t par, int from, int64_t row) {
    return size_t(kXHeaderBytes) + ((size_t(par) * world + from) * size_t(rows) + size_t(row)) * kXRecordBytes;
}

__device__ __forceinline__ void st_unit(uint8_t *p, float a, float b, uint32_t epoch) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(__float_as_uint(a)), "r"(epoch),
                 "r"(__float_as_uint(b)), "r"(epoch)
                 : "memory");
}
__device__ __forceinline__ bool ld_unit(const uint8_t *p, float &a, float &b, uint32_t epoch) {
    uint32_t x, fx, y, fy;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(x), "=r"(fx), "=r"(y), "=r"(fy) : "l"(p) : "memory");
    a = __uint_as_float(x);
    b = __uint_as_float(y);
    return fx == epoch && fy == epoch;
}

#ifdef BD_TRACE
// Timing trace for development builds only: per CTA the time of each stage, global timer nanoseconds.
__device__ unsigned long long g_xtrace[64 * 16];
#define BD_XMARK(slot) do { if (threadIdx.x == 0 && blockIdx.x < 64) { unsigned long long t_; \
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_)); g_xtrace[blockIdx.x * 16 + (slot)] = t_; } } while (0)
#else
#define BD_XMARK(slot) do { } while (0)
#endif

// MAXW: the smallest of 2, 4, 8, 16 that holds the world size (the loops over ranks are unrolled that far:
// the kernel runs once per step from a cold instruction cache, so its code is kept short).
template <bool FROM_PARTS, int MAXW>
__global__ void __launch_bounds__(kXWarps * 32) bd_exchange_kernel(const ExchangeParams p) {
    uint8_t *mine = p.area[p.rank];
    uint32_t *hdr = reinterpret_cast<uint32_t *>(mine);              // [0] epoch, [1] finished CTAs, [2] status
    uint32_t epoch = 0, par = 0;         // read behind the wait: the call before this one may just be moving it on
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    BD_XMARK(0);

    // The kernel is launched early behind the one that produces this rank's partial (programmatic dependent
    // launch): its set-up runs beside that kernel's end, and what that kernel wrote is read after the wait.
    bool waited = false;
    for (int64_t row = int64_t(blockIdx.x) * kXWarps + warp; row < p.rows; row += int64_t(gridDim.x) * kXWarps) {
        const int ib = int(row / p.h), hq = int(row % p.h);
        // ---- 1. this rank's partial of the row: lane owns head dims 4 lane .. 4 lane + 3
        float o[4] = {0.f, 0.f, 0.f, 0.f};
        float lse_mine = -INFINITY;
        if constexpr (!FROM_PARTS) {
            if (!waited) {
                asm volatile("griddepcontrol.wait;" ::: "memory");
                epoch = *reinterpret_cast<volatile uint32_t *>(hdr) + 1;
                par = epoch & 1u;
                waited = true;
            }
            const float4 v = *reinterpret_cast<const float4 *>(p.part_out + row * kHeadDim + 4 * lane);
            o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
            lse_mine = p.part_lse[row];
        } else {
            // the parts of (sequence, head) sit in consecutive CTA rows, slots h_k apart; lane i weighs
            // part i, every lane asks for its 16 bytes of all the parts of a round before any is used
            const int ih = hq / p.gq, qrow = hq % p.gq;
            const PartRange pr = part_range(p.part, ib);
            const int nrows = pr.c1 - pr.c0 + 1;
            const int64_t slot0 = (int64_t(pr.c0) + ib) * p.h_k + ih;
            auto lse_of = [&](int i) {
                const bool live = i < nrows && (pr.dense || row_has_part(p.part, ib, pr.c0 + i));
                return live ? __ldcg(p.part_lse + (slot0 + int64_t(i) * p.h_k) * p.gq + qrow) : -INFINITY;
            };
            if (!waited) {
                asm volatile("griddepcontrol.wait;" ::: "memory");
                epoch = *reinterpret_cast<volatile uint32_t *>(hdr) + 1;
                par = epoch & 1u;
                waited = true;
            }
            // Up to 32 parts a round: lane i weighs part i, and every lane asks for its 16 bytes of all the
            // parts of the round together with the log-sum-exps, before any answer is used: one trip to L2.
            float mx = -INFINITY, sum = 0.f;
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
                // bring what earlier rounds summed to the new maximum
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
            if (mx != -INFINITY && sum > 0.f) {
                const float inv = 1.0f / sum;
                o[0] *= inv; o[1] *= inv; o[2] *= inv; o[3] *= inv;
                lse_mine = mx + logf(sum);
            }
        }
        BD_XMARK(1);

        // ---- 2. the row goes to every peer
#pragma unroll
        for (int r = 0; r < MAXW; ++r) {
            if (r >= p.world || r == p.rank) continue;
            uint8_t *dst = p.area[r] + xchg_record_off(p.world, p.rows, par, p.rank, row);
            st_unit(dst + lane * 32, o[0], o[1], epoch);
            st_unit(dst + lane * 32 + 16, o[2], o[3], epoch);
            if (lane == 0) st_unit(dst + kHeadDim * 8, lse_mine, 0.f, epoch);
        }
        BD_XMARK(2);

        // ---- 3. the peers' rows, as they arrive in this rank's own area (bounded)
        float l[MAXW];
        float pv[MAXW][4];
        bool ok = true;
        for (uint32_t polls = 0;; ++polls) {
            // every peer's record is asked for in each round (all loads in flight together)
            bool got = true;
#pragma unroll
            for (int r = 0; r < MAXW; ++r) {
                l[r] = -INFINITY;
                pv[r][0] = pv[r][1] = pv[r][2] = pv[r][3] = 0.f;
                if (r < p.world && r != p.rank) {
                    const uint8_t *src = mine + xchg_record_off(p.world, p.rows, par, r, row);
                    float unused;
                    got = ld_unit(src + lane * 32, pv[r][0], pv[r][1], epoch) && got;
                    got = ld_unit(src + lane * 32 + 16, pv[r][2], pv[r][3], epoch) && got;
                    got = ld_unit(src + kHeadDim * 8, l[r], unused, epoch) && got;
                }
            }
            if (__all_sync(0xffffffffu, got)) break;
            if (polls + 1 >= p.spin_limit) { ok = false; break; }
            if (polls > 64) __nanosleep(polls > 4096 ? 1000 : 100);
        }
        BD_XMARK(3);
        if (!ok) {
            if (lane == 0) atomicExch(reinterpret_cast<int *>(hdr + 2), BD_ERR_TIMEOUT);
            continue;
        }

        // ---- 4. merge the world partials of the row
        float mx = -INFINITY;
#pragma unroll
        for (int r = 0; r < MAXW; ++r) {
            if (r == p.rank) l[r] = lse_mine;
            if (r < p.world) mx = fmaxf(mx, l[r]);
        }
        float sum = 0.f;
        float w[MAXW];
#pragma unroll
        for (int r = 0; r < MAXW; ++r) {
            w[r] = (r < p.world && mx != -INFINITY && l[r] != -INFINITY) ? __expf(l[r] - mx) : 0.f;
            sum += w[r];
        }
        const float inv = sum > 0.f ? 1.0f / sum : 0.f;
        const float lse = sum > 0.f ? mx + logf(sum) : -INFINITY;
        float res[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < MAXW; ++r) {
            if (r < p.world && w[r] != 0.f) {
                const float wr = w[r] * inv;
                const bool own = r == p.rank;
                res[0] = fmaf(wr, own ? o[0] : pv[r][0], res[0]); res[1] = fmaf(wr, own ? o[1] : pv[r][1], res[1]);
                res[2] = fmaf(wr, own ? o[2] : pv[r][2], res[2]); res[3] = fmaf(wr, own ? o[3] : pv[r][3], res[3]);
            }
        }
        const int64_t idx = ib * p.out_stride_b + int64_t(hq) * p.out_stride_h + 4 * lane;
        if (p.out_dtype == BD_FP16) {
            __half2 a = __floats2half2_rn(res[0], res[1]), b = __floats2half2_rn(res[2], res[3]);
            *reinterpret_cast<uint2 *>(static_cast<__half *>(p.out) + idx) =
                make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b));
        } else if (p.out_dtype == BD_BF16) {
            __nv_bfloat162 a = __floats2bfloat162_rn(res[0], res[1]), b = __floats2bfloat162_rn(res[2], res[3]);
            *reinterpret_cast<uint2 *>(static_cast<__nv_bfloat16 *>(p.out) + idx) =
                make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b));
        } else {
            *reinterpret_cast<float4 *>(static_cast<float *>(p.out) + idx) = make_float4(res[0], res[1], res[2], res[3]);
        }
        if (lane == 0 && p.lse) p.lse[row] = lse;
    }
    BD_XMARK(4);

    // ---- the CTA that finishes last moves the epoch on (every CTA has read it by then)
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(hdr + 1, 1u) == gridDim.x - 1) {
            hdr[1] = 0;
            *reinterpret_cast<volatile uint32_t *>(hdr) = epoch;
        }
    }
}

static unsigned xchg_grid(int64_t rows) {
    const int64_t want = (rows + kXWarps - 1) / kXWarps;
    return unsigned(std::max<int64_t>(1, std::min<int64_t>(want, 148 * 4)));
}

template <bool FROM_PARTS>
static cudaError_t launch_exchange(const ExchangeParams &p, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(xchg_grid(p.rows));
    cfg.blockDim = dim3(kXWarps * 32);
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;     // staged behind the kernel before it
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (p.world <= 2) return cudaLaunchKernelEx(&cfg, bd_exchange_kernel<FROM_PARTS, 2>, p);
    if (p.world <= 4) return cudaLaunchKernelEx(&cfg, bd_exchange_kernel<FROM_PARTS, 4>, p);
    if (p.world <= 8) return cudaLaunchKernelEx(&cfg, bd_exchange_kernel<FROM_PARTS, 8>, p);
    return cudaLaunchKernelEx(&cfg, bd_exchange_kernel<FROM_PARTS, 16>, p);
}
cudaError_t launch_exchange_parts(const ExchangeParams &p, cudaStream_t stream) { return launch_exchange<true>(p, stream); }
static_assert(BD_MAX_PARTS == 16, "the exchange kernel is built for up to 16 ranks");

}  // namespace bd

namespace bd {
// Checks the exchange half of a call and fills the kernel's parameters from it (not the partial's
// source, the output or its strides: the caller's part).
int fill_exchange_params(const bd_exchange_args *a, ExchangeParams &p) {
    if (!a || !a->areas) return BD_ERR_INVALID;
    if (a->world < 1 || a->world > BD_MAX_PARTS || a->rank < 0 || a->rank >= a->world || a->rows <= 0) return BD_ERR_INVALID;
    if (a->d != 128) return BD_ERR_UNSUPPORTED;
    std::memset(&p, 0, sizeof(p));
    for (int r = 0; r < a->world; ++r) {
        if (!a->areas[r] || (reinterpret_cast<uintptr_t>(a->areas[r]) & 255u)) return BD_ERR_ALIGNMENT;
        p.area[r] = static_cast<uint8_t *>(a->areas[r]);
    }
    p.rows = a->rows; p.rank = a->rank; p.world = a->world;
    p.spin_limit = a->spin_limit ? a->spin_limit : (1u << 22);
    return BD_OK;
}
}  // namespace bd

#ifdef BD_TRACE
extern "C" int bd_xtrace_read(void *dst, size_t bytes) {
    return int(cudaMemcpyFromSymbol(dst, bd::g_xtrace, bytes < sizeof(bd::g_xtrace) ? bytes : sizeof(bd::g_xtrace)));
}
#endif

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
    if (!a || !a->part_out || !a->part_lse || !a->out) return BD_ERR_INVALID;
    if (a->out_dtype != BD_FP16 && a->out_dtype != BD_BF16 && a->out_dtype != BD_FP32) return BD_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a->part_out) | reinterpret_cast<uintptr_t>(a->out)) & 15u) return BD_ERR_ALIGNMENT;
    bd::ExchangeParams p;
    const int rc = bd::fill_exchange_params(a, p);
    if (rc != BD_OK) return rc;
    p.part_out = a->part_out; p.part_lse = a->part_lse; p.out = a->out; p.lse = a->lse;
    p.out_dtype = a->out_dtype;
    p.h = int32_t(std::min<int64_t>(a->rows, 0x7fffffff));       // one "sequence" of `rows` rows, contiguous
    p.out_stride_b = 0; p.out_stride_h = bd::kHeadDim;
    if (a->rows > 0x7fffffff) return BD_ERR_INVALID;
    return bd::launch_exchange<false>(p, static_cast<cudaStream_t>(stream)) == cudaSuccess ? BD_OK : BD_ERR_CUDA;
}

int bd_exchange_put(void *area, int world, int64_t rows, int from_rank, uint32_t epoch, const float *part_out,
                    const float *part_lse, bd_stream_t stream_) {
    if (!area || !part_out || !part_lse || world < 1 || world > BD_MAX_PARTS || from_rank < 0 || from_rank >= world || rows <= 0)
        return BD_ERR_INVALID;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    // the records are built on the host: every value beside the epoch, as the kernel's stores write them
    std::vector<float> po(size_t(rows) * bd::kHeadDim), pl(static_cast<size_t>(rows));
    if (cudaMemcpyAsync(po.data(), part_out, po.size() * sizeof(float), cudaMemcpyDefault, stream) != cudaSuccess) return BD_ERR_CUDA;
    if (cudaMemcpyAsync(pl.data(), part_lse, pl.size() * sizeof(float), cudaMemcpyDefault, stream) != cudaSuccess) return BD_ERR_CUDA;
    if (cudaStreamSynchronize(stream) != cudaSuccess) return BD_ERR_CUDA;
    std::vector<uint32_t> rec(size_t(rows) * (bd::kXRecordBytes / 4));
    for (int64_t row = 0; row < rows; ++row) {
        uint32_t *r = rec.data() + size_t(row) * (bd::kXRecordBytes / 4);
        for (int i = 0; i < bd::kHeadDim; ++i) {
            std::memcpy(r + 2 * i, &po[size_t(row) * bd::kHeadDim + i], 4);
            r[2 * i + 1] = epoch;
        }
        std::memcpy(r + 2 * bd::kHeadDim, &pl[size_t(row)], 4);
        r[2 * bd::kHeadDim + 1] = epoch;
        r[2 * bd::kHeadDim + 2] = 0;
        r[2 * bd::kHeadDim + 3] = epoch;
    }
    uint8_t *dst = static_cast<uint8_t *>(area) + bd::xchg_record_off(world, rows, epoch & 1u, from_rank, 0);
    if (cudaMemcpyAsync(dst, rec.data(), rec.size() * 4, cudaMemcpyHostToDevice, stream) != cudaSuccess) return BD_ERR_CUDA;
    return cudaStreamSynchronize(stream) == cudaSuccess ? BD_OK : BD_ERR_CUDA;   // the staging buffers live on this frame
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
