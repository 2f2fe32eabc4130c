/*
 * bitdecode.h — C ABI of the B200-native low-bit KV-cache decode-attention library.
 *
 * One shared library (libbitdecode.so), plain pointers and sizes, no C++ or
 * PyTorch types.  Every entry point returns 0 (BD_OK) or a negative BD_ERR_*
 * code, never throws, never allocates device memory, never synchronises the
 * device and launches its kernels on the stream it is given.  All pointers in
 * the argument structs are device pointers unless stated otherwise.
 *
 * The entry points replace the four functions the reference exports from its
 * pybind11 module `bit_decode_cuda` (reference: csrc/bit_decode/decode_api.cpp:605-611):
 *
 *   kvcache_pack_i2 / kvcache_pack_i4   ->  bd_pack    (bits = 2 / 4)
 *   fwd_kvcache_i2  / fwd_kvcache_i4    ->  bd_decode  (bits = 2 / 4)
 *
 * Packed layouts (P = 16/bits codes per 16-bit word, NB = 32*P tokens per pack
 * block, G = group size, d = head dim = 128):
 *
 *   k_pack   (b, s/P, h_k, d)   u16   word [32*blk + p][c], field j = token NB*blk + p + 32*j
 *   k_params (b, s/G, h_k, d)   f32-sized slots holding 2*d fp16: [0:d] scale, [d:2d] zero
 *   v_pack   (b, s, h_k, d/P)   u16   word [t][p], field j = dim p + (d/P)*j
 *   v_params (b, d/G, h_k, s)   f32-sized slots holding 2*s fp16: per run of 128 tokens,
 *                                     128 scales then 128 zeros
 *
 * For bits = 4 with G = 128 and G = 32 these are the reference's own layouts (reference:
 * csrc/bit_decode/src/include/qpack.h:283-294 and csrc/bit_decode/src/flash_fwd_kernel.h:939-957),
 * checked byte for byte against what its kernels write on a B200 (tests/golden/ref_i4.npz).  With
 * bits = 4, G = 32 the reference keeps the parameters in the order of its MMA fragments: the scale of
 * (group g of a pack block / 128-token run, element c) sits in parameter row 2*(g%2) + (c/8)%2 at
 * fp16 column 16*(c/16) + 8*(g/2) + c%8.  The 2-bit layouts and G = 64 are defined by this library
 * (natural order): the reference's 2-bit V packer is not usable and it has no G = 64 kernels.
 */
#ifndef BITDECODE_H_
#define BITDECODE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BD_VERSION 201

/* status codes */
#define BD_OK                0
#define BD_ERR_INVALID      -1   /* null pointer, non-positive size, bad stride */
#define BD_ERR_UNSUPPORTED  -2   /* (bits, group, dtype, head_dim, GQA ratio) not built */
#define BD_ERR_ALIGNMENT    -3   /* pointer or stride breaks a 16-byte / block rule */
#define BD_ERR_WORKSPACE    -4   /* workspace missing or too small */
#define BD_ERR_CUDA         -5   /* a CUDA runtime / driver call failed */
#define BD_ERR_DEVICE       -6   /* not an sm_100 device */
#define BD_ERR_TIMEOUT      -7   /* a bounded device-side wait ran out (see bd_read_status) */
#define BD_ERR_CAPACITY    -10   /* status word: a tail filled up but the packed buffers have no room for its block */
#define BD_ERR_POSITION    -11   /* status word: a token position beyond the rotary tables (their last row was used) */
#define BD_ERR_PAGE         -9   /* status word: a block_table entry outside [0, num_pages) was met; its
                                    tokens were left out */
#define BD_ERR_SCRATCH_LIMIT -8  /* bd_decode_noalloc: the call needs more than the fixed scratch area */

/* element types */
#define BD_FP16 0
#define BD_BF16 1
#define BD_FP32 2   /* output only */

typedef void *bd_stream_t;   /* a cudaStream_t */

/*
 * Quantize-pack.  Replaces kvcache_pack_i2 / kvcache_pack_i4
 * (reference: csrc/bit_decode/decode_api.cpp:517-603, launch at
 * csrc/bit_decode/src/flash_fwd_launch_template.h:224-250, kernel body
 * csrc/bit_decode/src/flash_fwd_kernel.h:732-1091, quantizer
 * csrc/bit_decode/src/include/qpack.h:110-300).
 *
 * Reads `s` tokens of K and V (s a multiple of NB) and writes their codes,
 * scales and zeros into the pack buffers starting at token `dst_token_offset`
 * (a multiple of NB).  Strides are in elements of the tensor they belong to;
 * the innermost dimension of every tensor is contiguous.
 */
typedef struct bd_pack_args {
    const void *k;            /* (b, s, h_k, d) fp16 or bf16 */
    const void *v;
    int64_t k_stride_b, k_stride_s, k_stride_h;
    int64_t v_stride_b, v_stride_s, v_stride_h;
    void *k_pack;             /* (b, s_cap/P, h_k, d) u16, rows contiguous */
    void *k_params;           /* (b, s_cap/G, h_k, d) 4-byte slots */
    void *v_pack;             /* (b, s_cap, h_k, d/P) u16 */
    void *v_params;           /* (b, d/G, h_k, s_cap) 4-byte slots */
    int64_t k_pack_stride_b, k_params_stride_b, v_pack_stride_b;
    int64_t v_params_stride_b, v_params_stride_g, v_params_stride_h;
    int32_t b, s, h_k, d;
    int32_t dst_token_offset;
    int32_t bits;             /* 2 or 4 */
    int32_t group;            /* 32, 64 or 128 */
    int32_t dtype;            /* BD_FP16 or BD_BF16 */
    int32_t flags;            /* 0, or BD_PACK_APPROX_DIV */
} bd_pack_args;

/*
 * How max_code / range is divided.  Default: IEEE division; the packed bytes equal what the
 * reference's kernel writes when built without --use_fast_math and what a CPU evaluation of
 * its formulas gives.  BD_PACK_APPROX_DIV: the GPU's approximate reciprocal, as in the reference
 * the way it is shipped (--use_fast_math, setup.py:149); byte-identical to that build on the
 * same GPU.  The two differ by one code step where (x - min) * max_code / range is exactly
 * k + 0.5, a few codes in 10^5.
 */
#define BD_PACK_APPROX_DIV 1

int bd_pack(const bd_pack_args *args, bd_stream_t stream);

/*
 * One decode-attention step over the packed cache.  Replaces fwd_kvcache_i2 /
 * fwd_kvcache_i4 (reference: csrc/bit_decode/decode_api.cpp:301-441; split-KV
 * launch csrc/bit_decode/src/flash_fwd_launch_template.h:103-146, kernel body
 * csrc/bit_decode/src/flash_fwd_kernel.h:66-728; combine kernel
 * flash_fwd_launch_template.h:147-171, flash_fwd_kernel.h:1144-1327).
 *
 * out = softmax(scale * q K^T) V with one query token per sequence, over the
 * first cache_seqlens[b] (or `s`) quantized tokens followed by the first
 * res_lens[b] (or `res_len`) tokens of an unquantized tail, one joint softmax.
 * Query head hq reads KV head hq / (h / h_k).  The reference has neither the
 * tail, nor per-sequence lengths, nor a returned LSE; they are extensions.
 *
 * The workspace (bd_decode_workspace_bytes) holds one status word, the arrival
 * counters of the in-kernel merge, the per-sequence block table (ragged
 * batches) and the partial results of every range.  The caller zeroes it once
 * after allocating it, and again before using it with a different (b, h_k) or
 * switching cache_seqlens on or off (the layout moves): every call leaves the
 * counters at zero again and only
 * ever writes a non-zero error code (BD_ERR_TIMEOUT) to the status word, so the
 * hot path has no memset.  After BD_ERR_TIMEOUT zero it again.  The same
 * workspace must not be used by two decode calls that can overlap on the device.
 */
typedef struct bd_decode_args {
    const void *q;            /* (b, h, d) fp16 / bf16 */
    void *out;                /* (b, h, d) in out_dtype */
    float *lse;               /* optional (b, h): natural-log LSE of the scaled scores */
    int64_t q_stride_b, q_stride_h;
    int64_t out_stride_b, out_stride_h;
    const void *k_pack, *k_params, *v_pack, *v_params;
    int64_t k_pack_stride_b, k_params_stride_b, v_pack_stride_b;
    int64_t v_params_stride_b, v_params_stride_g, v_params_stride_h;
    const int32_t *cache_seqlens;   /* optional (b): quantized tokens valid per sequence */
    const void *k_res;        /* optional (b, res_len, h_k, d), same dtype as q; with k_new the step also
                                 WRITES row res_lens[ib] of k_res and v_res (see k_new below) */
    const void *v_res;
    int64_t res_stride_b, res_stride_s, res_stride_h;
    const int32_t *res_lens;  /* optional (b): tail tokens valid per sequence */
    int32_t res_len;          /* token rows of the tail buffers (at most 256): the tail length of every
                                 sequence when res_lens is null, the bound of res_lens[ib] otherwise */
    int32_t b, h, h_k, d;
    int32_t s;                /* quantized tokens (upper bound when cache_seqlens is given) */
    int32_t s_cap;            /* token capacity of the pack buffers, a multiple of NB */
    int32_t bits, group;
    int32_t dtype;            /* of q and the tail: BD_FP16 / BD_BF16 */
    int32_t out_dtype;        /* BD_FP16 / BD_BF16 / BD_FP32 */
    float softmax_scale;
    int32_t num_splits;       /* 0 = choose (bd_plan_splits); n > 0 = about n ranges per sequence */
    /* Paged cache (reference: block_table, decode_api.cpp:328-352): when block_table is not null
     * the four packed buffers hold `num_pages` pages of `page_size` tokens each instead of b
     * sequences of s_cap tokens (same layout, the *_stride_b fields step from page to page,
     * s_cap must equal page_size), and tokens [i*page_size, (i+1)*page_size) of sequence ib
     * live in page block_table[ib * block_table_stride + i].  page_size is a multiple of 256. */
    /* Fused append (no counterpart in the reference snapshot; the scheme of its imgs/scheme.png):
     * k_new / v_new (b, 1, h_k, d) hold the K/V rows of the token decoded in this step.  The step
     * attends over them as tail row res_lens[ib] and stores them at that row of k_res / v_res, so
     * the caller only has to add one to its res_lens afterwards.  Needs res_lens and room in the
     * tail (res_lens[ib] < res_len, the rows of the tail buffers). */
    const void *k_new, *v_new;
    int64_t new_stride_b, new_stride_h;
    const int32_t *block_table;
    int32_t block_table_stride; /* entries per sequence (>= ceil(s / page_size)) */
    int32_t num_pages;
    void *workspace;
    size_t workspace_bytes;
    int32_t advance;          /* with k_new: after the step, advance the sequences on the device, so that a
                                 decoder loop needs no host-side bookkeeping and the whole step can be captured
                                 in a CUDA graph: res_lens[ib] += 1, and a tail that has reached one pack block
                                 (NB tokens) is quantize-packed as block cache_seqlens[ib] / NB of the packed
                                 buffers (same bytes as bd_pack on those rows), cache_seqlens[ib] += NB,
                                 res_lens[ib] = 0.  This is the roll-over of the reference's residual scheme
                                 (its imgs/scheme.png; residual_block_size in kernel_traits.h:76-85, not wired up
                                 in its snapshot).  Needs cache_seqlens and res_lens (both are then WRITTEN), a tail
                                 buffer of at least NB rows, no block_table.  Runs as two small kernels behind the
                                 decode kernel on the same stream.  No room left for the block: BD_ERR_CAPACITY in
                                 the status word, the tail stays full. */
    uint32_t spin_limit;      /* polls a device-side wait on a copy may take before it gives up with
                                 BD_ERR_TIMEOUT; 0 = the default (about 2^22, seconds) */
    int32_t test_starve;      /* test hook, leave 0.  1: the warps of the first CTA expect 16 bytes more
                                 than their first copy delivers, so their bounded waits run out (nothing
                                 faults or hangs: the kernel sets BD_ERR_TIMEOUT and returns) */
    /* Rotary embedding of the step's token (the reference carries this for its append path, dead in its
     * snapshot: rotary_cos_ptr / rotary_sin_ptr / rotary_dim in src/include/flash.h:121, 149-151, 189,
     * is_rotary_interleaved in decode_api.cpp:316, rotary_dim = 0 at decode_api.cpp:418;
     * src/include/rotary.h).  With k_new: q and k_new are rotated at the token's position
     * cache_seqlens[ib] + res_lens[ib] (or s, res_len) before anything else happens, so the step attends
     * with the rotated query over the rotated new key and files the rotated key in the tail.  cos / sin:
     * (rotary_positions, rotary_dim / 2) in q's dtype, contiguous.  The first rotary_dim dims of every
     * head are rotated, in fp32, pairs (2i, 2i+1) when interleaved, else (i, i + rotary_dim/2):
     * x0' = x0 cos - x1 sin, x1' = x0 sin + x1 cos.  rotary_dim: a multiple of 16, at most d; 0: none.
     * One small kernel in front of the decode kernel; its rotated copies live in the workspace. */
    const void *rotary_cos, *rotary_sin;
    int32_t rotary_dim;
    int32_t rotary_interleaved;
    int32_t rotary_positions; /* rows of the tables; a position beyond them uses the last row and sets
                                 BD_ERR_POSITION in the status word */
    int32_t reserved0;
} bd_decode_args;

int bd_decode(const bd_decode_args *args, bd_stream_t stream);

/* Bytes of workspace bd_decode needs for these arguments (0 on invalid input). */
size_t bd_decode_workspace_bytes(const bd_decode_args *args);

/*
 * bd_decode for callers that cannot allocate device memory.  (No counterpart in
 * the reference, whose decode call allocates its split buffers itself on every
 * call.)
 *
 * bd_decode needs a caller-allocated workspace.  Some callers have nowhere to
 * get one at the point of the call: a serving runtime that has already given
 * every free byte of HBM to its KV-cache pool, a latency path that must never
 * enter the allocator, a plugin host that forbids cudaMalloc after start-up.
 * bd_decode_noalloc takes the same arguments (args->workspace and
 * args->workspace_bytes are ignored) and keeps the partial results, arrival
 * counters and sequence table in a fixed area of BD_NOALLOC_SCRATCH_BYTES that is
 * part of the library image: every GPU that loads the library carries those
 * bytes until the process exits, whether this entry point is used or not.
 *
 *  - It calls no cudaMalloc / cudaFree and no allocating library routine; per
 *    call it queues one small memset (the arrival counters) and the decode
 *    kernel(s) on `stream`.  The status word is left alone, so an error code a
 *    step wrote stays until bd_read_status(NULL, stream) fetches and clears it.
 *  - The first call on each device looks up the area's device address (with
 *    that device current).  Make that first call outside any stream capture.
 *  - A call whose shapes need more than BD_NOALLOC_SCRATCH_BYTES (large batch *
 *    head counts; bd_decode_workspace_bytes tells) fails with
 *    BD_ERR_SCRATCH_LIMIT and launches nothing; use bd_decode for those.
 *  - There is one area per device, shared by every call and every stream, and it
 *    keeps what the last call left.  Two calls that can overlap on the same
 *    device race on it: serialise them (same stream, or events).
 */
#define BD_NOALLOC_SCRATCH_BYTES (8u << 20)
int bd_decode_noalloc(const bd_decode_args *args, bd_stream_t stream);
size_t bd_noalloc_scratch_bytes(void);

/*
 * How bd_decode splits the sequence dimension when num_splits == 0; takes the
 * place of num_splits_heuristic (reference: csrc/bit_decode/decode_api.cpp:234-268).
 * Per KV head the pack blocks of all sequences form one list; the list is cut
 * into this many equal ranges ("rows"), one CTA per (row, KV head), so the grid
 * fills every SM with `ctas_per_sm` resident CTAs of equal work whatever the
 * batch size and lengths.  A caller-given num_splits > 0 asks for
 * num_splits * b rows instead.  `ctas_per_sm` <= 0 selects what the decode kernel of this build
 * keeps resident (one CTA of up to twelve streaming warps per SM).
 */
int bd_plan_splits(int b, int h_k, int64_t max_s, int bits, int sm_count, int ctas_per_sm);

/*
 * What bd_decode will do with these arguments on the current device: out[0] = rows (ranges per KV
 * head; the grid is rows * h_k CTAs), out[1] = CTAs resident per SM (2: the variant with two smaller
 * CTAs, taken where whole rows of KV heads would leave more than a tenth of the SMs without a CTA),
 * out[2] = streaming warps per CTA, out[3] = kernels launched per call (prefix table of a ragged
 * batch, rotary embedding, decode, parts merge, roll-over).  No counterpart in the reference (its grid is
 * (1, num_splits, b * h_k), csrc/bit_decode/src/flash_fwd_launch_template.h:110).
 */
int bd_decode_plan(const bd_decode_args *args, int32_t out[4]);

/*
 * Host-side view of that partition, for tests and debugging (pure integer
 * arithmetic, no device work, no counterpart in the reference).  A unit is one
 * pack block or one 32-token chunk of the unquantized tail; a sequence's units are
 * its blocks, then its tail chunks.  `table` is null for equal lengths (then every
 * sequence has n_uniform units) or points to HOST memory holding (first unit, unit
 * count) per sequence followed by (total, 0).  bd_partition_segments writes up to
 * max_segments tuples (sequence, first unit, end unit, owns_empty) covered by
 * `row`; owns_empty marks a sequence without units that this row answers for.
 * bd_partition_parts writes the rows that hold a part of sequence `ib` (none for
 * a sequence without units).  Both return the number of entries found.  The decode
 * kernel applies the partition twice: `rows` CTAs per KV head, and rows * W warps
 * (W warps per CTA), warp w of CTA c being row c * W + w.
 */
int bd_partition_segments(const int32_t *table, int b, int n_uniform, int rows, int row,
                          int32_t *out, int max_segments);
int bd_partition_parts(const int32_t *table, int b, int n_uniform, int rows, int ib,
                       int32_t *out, int max_parts);

/*
 * Merge n partial results (each normalised within its part) with their
 * log-sum-exp: LSE = log sum_i exp(lse_i), out = sum_i exp(lse_i - LSE) * out_i.
 * Same arithmetic as the reference's split combine (reference:
 * csrc/bit_decode/src/flash_fwd_kernel.h:1217-1231, 1280-1298), usable on
 * partials that came from other GPUs: the pointer arrays live in HOST memory
 * and hold device pointers (local, or peer pointers mapped into this process).
 */
#define BD_MAX_PARTS 16
typedef struct bd_combine_args {
    int32_t n_parts;                      /* 1 .. BD_MAX_PARTS */
    const float *const *part_out;         /* host array of n device pointers, each (rows, d) fp32 */
    const float *const *part_lse;         /* host array of n device pointers, each (rows) fp32 */
    int64_t rows;                         /* b * h */
    int32_t d;
    void *out;                            /* (rows, d) in out_dtype, contiguous */
    float *lse;                           /* optional (rows) */
    int32_t out_dtype;
} bd_combine_args;

int bd_combine(const bd_combine_args *args, bd_stream_t stream);

/*
 * Sequence split over GPUs: exchange of the per-GPU partial results and their merge in ONE kernel per
 * rank and step, over peer-mapped memory (no counterpart in the reference, which is single-GPU; the
 * merge is its split combine applied across GPUs).  One process per GPU.
 *
 * Set-up (allocates; never on the step): every rank allocates an exchange area of
 * bd_exchange_area_bytes(world, rows) with bd_peer_alloc (zero-filled device memory that can be
 * shared), exports it with bd_peer_export (a 64-byte handle to pass to the other processes by any
 * host-side means) and maps the others' with bd_peer_open.  rows = batch * query heads.
 *
 * Step, fused with the decode (the fast path): bd_decode_exchange(decode args, exchange args) runs this
 * rank's decode over its shard of the tokens with every CTA leaving its part in the workspace, and then
 * ONE more kernel, a warp per (sequence, query head) row: it merges this rank's parts of the row, stores
 * the row (128 fp32 values and the log-sum-exp, every 8 bytes carrying the step's epoch beside the
 * value, so that no fence or separate flag is needed) into every peer's area with plain 16-byte stores,
 * polls (bounded) for the peers' rows in its own area, merges the `world` partials and writes `out`
 * (and `lse`) of the decode args: the full result on every rank.  part_out, part_lse, out, lse,
 * out_dtype of the exchange args are not used; rows must be b * h.
 * Step, as a call of its own: bd_exchange_combine does the same for a partial that is already there
 * (part_out fp32 (rows, 128), part_lse (rows), normalised within this rank's tokens; e.g. from bd_decode
 * with out_dtype = BD_FP32 and lse).
 * Neither allocates or synchronises on the host, both can be captured in a CUDA graph: the step counter
 * ("epoch") lives in the area.  All ranks must make the same number of calls on an area; the areas
 * hold two steps, so ranks may be up to one step apart.
 *
 * A row whose peers do not publish within `spin_limit` polls (0 = the default, seconds) is not written;
 * the kernel puts BD_ERR_TIMEOUT into the area's status word and returns normally.
 * bd_exchange_state waits for `stream`, returns that word (and clears it) and the area's epoch.
 * After a timeout the ranks are out of step: zero all areas (with the ranks quiesced) before going on.
 *
 * bd_exchange_put publishes a partial into an area from the HOST side (copies + flag), standing in for
 * a peer's kernel (records built on the host, one copy): for tests on one GPU and for partials that
 * arrive by other means.  Synchronises.
 */
typedef struct bd_exchange_args {
    int32_t rank, world;                  /* world <= BD_MAX_PARTS */
    void *const *areas;                   /* host array of `world` device pointers: rank r's area as mapped
                                             into this process; areas[rank] is this rank's own */
    const float *part_out;                /* (rows, d) fp32, normalised within this rank's tokens */
    const float *part_lse;                /* (rows) */
    int64_t rows;                         /* b * h */
    int32_t d;                            /* 128 */
    void *out;                            /* (rows, d) in out_dtype */
    float *lse;                           /* optional (rows) */
    int32_t out_dtype;
    uint32_t spin_limit;
} bd_exchange_args;

size_t bd_exchange_area_bytes(int world, int64_t rows);
int bd_peer_alloc(size_t bytes, void **ptr);
int bd_peer_free(void *ptr);
int bd_peer_export(const void *ptr, void *handle64);
int bd_peer_open(const void *handle64, void **ptr);
int bd_peer_close(void *ptr);
int bd_exchange_combine(const bd_exchange_args *args, bd_stream_t stream);
int bd_decode_exchange(const bd_decode_args *decode, const bd_exchange_args *exchange, bd_stream_t stream);
int bd_exchange_put(void *area, int world, int64_t rows, int from_rank, uint32_t epoch, const float *part_out,
                    const float *part_lse, bd_stream_t stream);
int bd_exchange_state(const void *area, bd_stream_t stream, uint32_t *epoch_out);

/*
 * Blocks until the work queued on `stream` is done, returns the status word the decode calls on
 * that workspace left (BD_OK, BD_ERR_TIMEOUT if a bounded wait inside a kernel ran out,
 * BD_ERR_PAGE for a bad block_table entry) and sets the word back to zero.  workspace == NULL
 * reads the fixed area bd_decode_noalloc uses on the current device.  Synchronises: for tests,
 * debugging and callers that check every n-th step, not for the hot path.
 */
int bd_read_status(const void *workspace, bd_stream_t stream);

const char *bd_strerror(int code);
int bd_version(void);

#ifdef __cplusplus
}
#endif
#endif /* BITDECODE_H_ */
