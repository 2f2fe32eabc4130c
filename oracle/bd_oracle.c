/*
 * CPU oracle, C restatement (test infrastructure only — never linked into or
 * called from the shipped library; used by the tests as a second, independent
 * statement of the formulas and by the benchmark's cpu_baseline leg).
 *
 * Parity status: pinned for 4-bit, group 128 and 32.  The reference has no CPU path and no
 * golden vectors of its own, but its CUDA kernels compile for sm_100a (oracle/build_ref.py);
 * what they write on seeded inputs is committed as tests/golden/ref_i4.npz
 * (tests/golden/make_ref_golden.py) and this restatement reproduces the packed codes, scales and
 * zeros of the reference built WITHOUT --use_fast_math byte for byte (tests/test_ref_golden.py).
 * The reference as shipped (--use_fast_math, setup.py:149) divides with the GPU's approximate
 * reciprocal; its scale_inv differs by one ulp in about a quarter of the groups, which moves a
 * code by one step where (x - min) * 15 / range is exactly k + 0.5 (a few codes in 10^5).
 * 2-bit, group 64 and bf16 have no runnable reference kernel: defined by this build.
 *
 * Restates (paths relative to the reference project):
 *   quantizer        csrc/bit_decode/src/include/qpack.h:219-300, :110-217
 *   group geometry   csrc/bit_decode/src/flash_fwd_kernel.h:919-957
 *   dequantisation   csrc/bit_decode/src/include/dequantize.h:253-384
 *   softmax / LSE    csrc/bit_decode/src/include/softmax.h:188-309
 *   GQA mapping      csrc/bit_decode/decode_api.cpp:360-368
 *
 * Build: see oracle/Makefile (gcc -O2 -fopenmp -ffp-contract=off, no -ffast-math,
 * baseline x86-64 so the shared object runs on any host).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

static inline float h2f(uint16_t bits) {
    _Float16 h;
    memcpy(&h, &bits, 2);
    return (float)h;
}
static inline uint16_t f2h(float x) {            /* round to nearest even */
    _Float16 h = (_Float16)x;
    uint16_t bits;
    memcpy(&bits, &h, 2);
    return bits;
}
static inline uint16_t d2h(double x) {           /* one rounding, double -> half */
    _Float16 h = (_Float16)x;
    uint16_t bits;
    memcpy(&bits, &h, 2);
    return bits;
}
static inline float bf2f(uint16_t bits) {
    uint32_t u = (uint32_t)bits << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static inline uint16_t f2bf(float x) {           /* round to nearest even */
    uint32_t u;
    memcpy(&u, &x, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static inline float in2f(uint16_t bits, int is_bf16) { return is_bf16 ? bf2f(bits) : h2f(bits); }

/* Threads the parallel loops will use from now on (n <= 0: leave as is).  A launcher that
   exports OMP_NUM_THREADS=1 for its ranks would otherwise pin the timed CPU baseline to one core. */
void bdo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int bdo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/*
 * Where the scale of (group g of a pack block or 128-token run, element c of 0..127) is stored:
 * `row` among the block's / run's parameter rows and fp16 column `col` (the zero sits 128 columns
 * on).  For K, g is the token group and c the channel; for V, g is the dim group and c the token
 * within its run of 128, and "row" selects the dim-group plane of v_params.
 * Natural order everywhere except 4-bit with group 32, where the reference stores the parameters
 * in the order its MMA fragments hold them (flash_fwd_kernel.h:939-957 with num_params = 4).
 */
static inline void param_slot(int bits, int group, int g, int c, int *row, int *col) {
    if (bits == 4 && group == 32) {
        *row = 2 * (g & 1) + ((c >> 3) & 1);
        *col = 16 * (c >> 4) + 8 * (g >> 1) + (c & 7);
    } else {
        *row = g;
        *col = c;
    }
}

/* One group: min/max -> scale_inv, stored scale and zero -> codes (qpack.h:241-281). */
static void quantize_group(const float *x, int n, int bits, uint8_t *codes,
                           uint16_t *scale_h, uint16_t *zero_h) {
    const float maxv = (float)((1 << bits) - 1);
    float mx = x[0], mn = x[0];
    for (int i = 1; i < n; ++i) {
        mx = x[i] > mx ? x[i] : mx;
        mn = x[i] < mn ? x[i] : mn;
    }
    const float range = mx - mn;
    const float scale_inv = (range > 0.0f) ? (maxv / range) : 0.0f;
    const float scale = (scale_inv == 0.0f) ? 0.0f : 1.0f / scale_inv;
    *scale_h = f2h(scale);
    *zero_h = f2h(mn);
    for (int i = 0; i < n; ++i) {
        float v = x[i] - mn;
        v = v * scale_inv;
        v = fminf(fmaxf(roundf(v), 0.0f), maxv);
        codes[i] = (uint8_t)v;
    }
}

/*
 * Quantize-pack of contiguous (b, s, h, d) K and V into the four buffers.
 *   k_pack   (b, s/P, h, d)   u16      k_params (b, s/G, h, 2d) fp16 bits
 *   v_pack   (b, s, h, d/P)   u16      v_params (b, d/G, h, 2s) fp16 bits
 * Layouts as documented in oracle/oracle.py.  Returns 0, or -1 on bad sizes.
 */
int bdo_quantize_pack(const uint16_t *k, const uint16_t *v, int is_bf16,
                      int b, int s, int h, int d, int bits, int group,
                      uint16_t *k_pack, uint16_t *k_params,
                      uint16_t *v_pack, uint16_t *v_params) {
    if (bits != 2 && bits != 4) return -1;
    const int P = 16 / bits, NB = 32 * P;
    if (s % NB || NB % group || d % group || d % P || group > 256) return -1;
    const int ngk = s / group, ngd = d / group, dP = d / P;
    const int64_t nblk = (int64_t)b * (s / NB) * h;

#pragma omp parallel for schedule(static)
    for (int64_t it = 0; it < nblk; ++it) {
        const int ih = (int)(it % h);
        const int blk = (int)((it / h) % (s / NB));
        const int ib = (int)(it / ((int64_t)h * (s / NB)));
        float xs[256];
        uint8_t cs[256];
        /* ---- K: per channel, groups of `group` consecutive tokens ---- */
        for (int c = 0; c < d; ++c) {
            uint8_t codes_blk[256];
            for (int g0 = 0; g0 < NB; g0 += group) {
                for (int i = 0; i < group; ++i) {
                    const int64_t t = (int64_t)blk * NB + g0 + i;
                    xs[i] = in2f(k[(((int64_t)ib * s + t) * h + ih) * d + c], is_bf16);
                }
                uint16_t sc, ze;
                quantize_group(xs, group, bits, cs, &sc, &ze);
                int prow, pcol;
                param_slot(bits, group, g0 / group, c, &prow, &pcol);
                const int64_t gi = (int64_t)blk * (NB / group) + prow;
                uint16_t *prm = k_params + (((int64_t)ib * ngk + gi) * h + ih) * 2 * d;
                prm[pcol] = sc;
                prm[d + pcol] = ze;
                memcpy(codes_blk + g0, cs, group);
            }
            for (int p = 0; p < 32; ++p) {
                uint16_t w = 0;
                for (int j = 0; j < P; ++j) w |= (uint16_t)(codes_blk[p + 32 * j] << (bits * j));
                k_pack[(((int64_t)ib * (s / P) + (int64_t)blk * 32 + p) * h + ih) * d + c] = w;
            }
        }
        /* ---- V: per token, groups of `group` consecutive dims ---- */
        for (int tt = 0; tt < NB; ++tt) {
            const int64_t t = (int64_t)blk * NB + tt;
            uint8_t codes_tok[256];
            for (int gd = 0; gd < ngd; ++gd) {
                for (int i = 0; i < group; ++i)
                    xs[i] = in2f(v[(((int64_t)ib * s + t) * h + ih) * d + gd * group + i], is_bf16);
                uint16_t sc, ze;
                quantize_group(xs, group, bits, cs, &sc, &ze);
                memcpy(codes_tok + gd * group, cs, group);
                int prow, pcol;
                param_slot(bits, group, gd, (int)(t % 128), &prow, &pcol);
                uint16_t *prm = v_params + (((int64_t)ib * ngd + prow) * h + ih) * 2 * (int64_t)s;
                const int64_t tb = t / 128;
                prm[256 * tb + pcol] = sc;
                prm[256 * tb + 128 + pcol] = ze;
            }
            for (int p = 0; p < dP; ++p) {
                uint16_t w = 0;
                for (int j = 0; j < P; ++j) w |= (uint16_t)(codes_tok[p + dP * j] << (bits * j));
                v_pack[(((int64_t)ib * s + t) * h + ih) * dP + p] = w;
            }
        }
    }
    return 0;
}

/*
 * Dequantize-then-attention for one decode step (one query token).
 *   q (b, h, d) fp16/bf16 bits; packed buffers as above; optional residual tail
 *   k_res/v_res (b, res_cap, h_k, d) in the same dtype as q.
 *   cache_seqlens / res_lens may be NULL (then s / res_len apply to every row).
 * Dequantised values are code*scale+zero rounded once to fp16 (and once more to
 * bf16 when is_bf16).  Softmax and the weighted sum run in double.
 *   out (b, h, d) double, lse (b, h) double (natural log; -inf for an empty row).
 */
int bdo_decode(const uint16_t *q, int is_bf16,
               const uint16_t *k_pack, const uint16_t *k_params,
               const uint16_t *v_pack, const uint16_t *v_params,
               int b, int h, int h_k, int d, int s, int bits, int group, float softmax_scale,
               const int32_t *cache_seqlens,
               const uint16_t *k_res, const uint16_t *v_res, int res_cap,
               const int32_t *res_lens, int res_len,
               double *out, double *lse) {
    if (bits != 2 && bits != 4) return -1;
    const int P = 16 / bits, NB = 32 * P;
    if (h % h_k || d > 256 || d % group || (s % NB)) return -1;
    const int gq = h / h_k, ngk = s / group, ngd = d / group, dP = d / P;
    const unsigned mask = (1u << bits) - 1u;
    const int64_t nwork = (int64_t)b * h_k;

#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t it = 0; it < nwork; ++it) {
        const int ib = (int)(it / h_k), ih = (int)(it % h_k);
        const int n = cache_seqlens ? cache_seqlens[ib] : s;
        const int r = (k_res && v_res) ? (res_lens ? res_lens[ib] : res_len) : 0;
        double *m = (double *)malloc(sizeof(double) * gq);
        double *l = (double *)malloc(sizeof(double) * gq);
        double *acc = (double *)calloc((size_t)gq * d, sizeof(double));
        float *qf = (float *)malloc(sizeof(float) * gq * d);
        float krow[256], vrow[256];
        for (int g = 0; g < gq; ++g) {
            m[g] = -INFINITY;
            l[g] = 0.0;
            for (int c = 0; c < d; ++c)
                qf[g * d + c] = in2f(q[((int64_t)ib * h + (int64_t)ih * gq + g) * d + c], is_bf16);
        }
        for (int t = 0; t < n + r; ++t) {
            if (t < n) {
                const int blk = t / NB, tt = t % NB, p = tt % 32, j = tt / 32;
                const uint16_t *kp = k_pack + (((int64_t)ib * (s / P) + (int64_t)blk * 32 + p) * h_k + ih) * d;
                for (int c = 0; c < d; ++c) {
                    const unsigned code = (kp[c] >> (bits * j)) & mask;
                    int prow, pcol;
                    param_slot(bits, group, tt / group, c, &prow, &pcol);
                    const uint16_t *kprm = k_params +
                        (((int64_t)ib * ngk + (int64_t)blk * (NB / group) + prow) * h_k + ih) * 2 * d;
                    uint16_t hv = d2h((double)code * (double)h2f(kprm[pcol]) + (double)h2f(kprm[d + pcol]));
                    krow[c] = is_bf16 ? bf2f(f2bf(h2f(hv))) : h2f(hv);
                }
                const uint16_t *vp = v_pack + (((int64_t)ib * s + t) * h_k + ih) * dP;
                for (int c = 0; c < d; ++c) {
                    const unsigned code = (vp[c % dP] >> (bits * (c / dP))) & mask;
                    int prow, pcol;
                    param_slot(bits, group, c / group, t % 128, &prow, &pcol);
                    const uint16_t *vprm = v_params + (((int64_t)ib * ngd + prow) * h_k + ih) * 2 * (int64_t)s;
                    const int64_t tb = t / 128;
                    uint16_t hv = d2h((double)code * (double)h2f(vprm[256 * tb + pcol]) +
                                      (double)h2f(vprm[256 * tb + 128 + pcol]));
                    vrow[c] = is_bf16 ? bf2f(f2bf(h2f(hv))) : h2f(hv);
                }
            } else {
                const int64_t off = (((int64_t)ib * res_cap + (t - n)) * h_k + ih) * d;
                for (int c = 0; c < d; ++c) {
                    krow[c] = in2f(k_res[off + c], is_bf16);
                    vrow[c] = in2f(v_res[off + c], is_bf16);
                }
            }
            for (int g = 0; g < gq; ++g) {
                double sc = 0.0;
                for (int c = 0; c < d; ++c) sc += (double)qf[g * d + c] * (double)krow[c];
                sc *= (double)softmax_scale;
                double *a = acc + (size_t)g * d;
                if (sc > m[g]) {
                    const double f = exp(m[g] - sc);       /* exp(-inf) = 0 on the first token */
                    l[g] *= f;
                    for (int c = 0; c < d; ++c) a[c] *= f;
                    m[g] = sc;
                }
                const double pw = exp(sc - m[g]);
                l[g] += pw;
                for (int c = 0; c < d; ++c) a[c] += pw * (double)vrow[c];
            }
        }
        for (int g = 0; g < gq; ++g) {
            const int64_t o = ((int64_t)ib * h + (int64_t)ih * gq + g);
            if (l[g] > 0.0) {
                for (int c = 0; c < d; ++c) out[o * d + c] = acc[(size_t)g * d + c] / l[g];
                lse[o] = m[g] + log(l[g]);
            } else {
                for (int c = 0; c < d; ++c) out[o * d + c] = 0.0;
                lse[o] = -INFINITY;
            }
        }
        free(m); free(l); free(acc); free(qf);
    }
    return 0;
}
