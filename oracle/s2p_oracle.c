/* TEST INFRASTRUCTURE — CPU restatement of the s2pro-native token loop.
 *
 * This file is the parity checker, never the product: only tests, the smoke
 * check and the CPU-baseline leg of the benchmark may load it.  It restates,
 * in plain C11, the arithmetic of the reference's decode tick so that the CUDA
 * library can be compared with it on the same seeded inputs.  Every function
 * cites the reference file:line it follows (paths relative to the reference
 * project root).
 *
 * Pinning: the integer/byte functions (quantize, pack, unpack, dequant, GEMV
 * accumulation order, argmax, greedy sampler, KV8 quantize, VQ sum, residual
 * add, INT8 embedding) are built only from IEEE f32 add/mul/div/fma, integer
 * ops and RNE bf16/f16 conversions, so they are bit-reproducible on a CPU and
 * are pinned (a) on the GPU against the reference's own CUDA kernels rebuilt
 * for sm_100a and (b) on the CPU against the reference's host sampler and the
 * committed golden vectors.  Functions that go through rsqrtf / expf / powf /
 * cosf / sinf follow the same operation order but use the host libm, so they
 * agree with the GPU only to a stated tolerance.
 *
 * Build: gcc -O2 -std=c11 -ffp-contract=off (every fused multiply-add below is
 * an explicit fmaf, mirroring nvcc's default contraction of a*b+c in the
 * reference's kernels).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define S2PO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------ conversions */

static inline float bf2f(uint16_t h) {
    union { uint32_t u; float f; } v;
    v.u = (uint32_t)h << 16;
    return v.f;
}

/* round-to-nearest-even f32 -> bf16 (what __float2bfloat16 does) */
static inline uint16_t f2bf(float f) {
    union { uint32_t u; float f; } v;
    v.f = f;
    if ((v.u & 0x7fffffffu) > 0x7f800000u) return 0x7fff; /* NaN */
    uint32_t lsb = (v.u >> 16) & 1u;
    v.u += 0x7fffu + lsb;
    return (uint16_t)(v.u >> 16);
}

/* IEEE binary16 <-> f32, RNE (what __float2half_rn / __half2float do) */
static inline float h2f(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    union { uint32_t u; float f; } v;
    if (exp == 0) {
        if (man == 0) { v.u = sign; return v.f; }
        /* subnormal: value = man * 2^-24 */
        float f = (float)man * 5.9604644775390625e-8f;
        return sign ? -f : f;
    }
    if (exp == 31) { v.u = sign | 0x7f800000u | (man << 13); return v.f; }
    v.u = sign | ((exp + 112u) << 23) | (man << 13);
    return v.f;
}

static inline uint16_t f2h(float f) {
    union { uint32_t u; float f; } v;
    v.f = f;
    uint32_t sign = (v.u >> 16) & 0x8000u;
    uint32_t a = v.u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);      /* NaN */
    if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);     /* >= 65520 -> inf */
    if (a < 0x33000001u) return (uint16_t)sign;                  /* <= 2^-25 -> 0 */
    int32_t e = (int32_t)(a >> 23) - 127;
    uint32_t m = (a & 0x7fffffu) | 0x800000u;
    if (e < -14) {
        /* subnormal half: shift so that the unit is 2^-24 */
        int shift = -e - 14 + 13; /* 13 = 23-10 */
        uint32_t r = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (r & 1u))) r++;
        return (uint16_t)(sign | r);
    }
    uint32_t r = ((uint32_t)(e + 15) << 10) | ((m >> 13) & 0x3ffu);
    uint32_t rem = m & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) r++;
    return (uint16_t)(sign | r);
}

S2PO_API float s2po_bf2f(uint16_t h) { return bf2f(h); }
S2PO_API uint16_t s2po_f2bf(float f) { return f2bf(f); }
S2PO_API float s2po_h2f(uint16_t h) { return h2f(h); }
S2PO_API uint16_t s2po_f2h(float f) { return f2h(f); }

static inline int rn_int(float v) { return (int)lrintf(v); } /* __float2int_rn */

static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* --------------------------------------------------------------- quantizers */

/* Per-output-channel INT8: src/sched/int8_gemv.cu:32-58 (k_quant).
 * scale = amax/levels (1.0 when the row is all zero), inv = 1.0f/scale,
 * q = rint(w*inv) clamped to +-levels. */
S2PO_API void s2po_quant_int8(int8_t* q, float* scales, const uint16_t* w,
                              int N, int K) {
    const int levels = 127;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        const uint16_t* row = w + (size_t)n * K;
        float amax = 0.f;
        for (int k = 0; k < K; k++) amax = fmaxf(amax, fabsf(bf2f(row[k])));
        const float scale = amax > 0.f ? amax / (float)levels : 1.0f;
        const float inv = 1.0f / scale;
        scales[n] = scale;
        for (int k = 0; k < K; k++)
            q[(size_t)n * K + k] =
                (int8_t)clampi(rn_int(bf2f(row[k]) * inv), -levels, levels);
    }
}

/* Group-wise symmetric quantizer with the 32-candidate MSE clip search:
 * src/sched/int8_gemv.cu:135-195 (k_quant_g), launched with min(G,256)
 * threads (:760).  Thread t accumulates err over k = t, t+T, ... as an fma
 * chain starting from 0; the T partials are merged by a halving tree
 * (red[t] += red[t+r], r = T/2 .. 1); strict '<' keeps the first minimum. */
S2PO_API void s2po_quant_g(int8_t* q, uint16_t* scales_f16, const uint16_t* w,
                           int N, int K, int G, int levels, int mse) {
    const int ng = K / G;
    const int T = G < 256 ? G : 256;
#pragma omp parallel for schedule(static)
    for (int64_t blk = 0; blk < (int64_t)N * ng; blk++) {
        const int n = (int)(blk / ng), g = (int)(blk % ng);
        const uint16_t* wp = w + (size_t)n * K + (size_t)g * G;
        float red[256];
        float amax = 0.f;
        for (int k = 0; k < G; k++) amax = fmaxf(amax, fabsf(bf2f(wp[k])));
        const float base = amax > 0.f ? amax / (float)levels : 1.0f;
        float scale = h2f(f2h(base));
        if (mse && amax > 0.f) {
            float best_err = 3.4e38f, best_s = scale;
            for (int c = 0; c < 32; c++) {
                const float s = h2f(f2h(base * (1.0f - (float)c / 64.0f)));
                const float inv = 1.0f / s;
                for (int t = 0; t < T; t++) {
                    float err = 0.f;
                    for (int k = t; k < G; k += T) {
                        const float v = bf2f(wp[k]);
                        const int qi = clampi(rn_int(v * inv), -levels, levels);
                        const float d = fmaf(-(float)qi, s, v); /* v - qi*s */
                        err = fmaf(d, d, err);
                    }
                    red[t] = err;
                }
                for (int r = T / 2; r > 0; r >>= 1)
                    for (int t = 0; t < r; t++) red[t] += red[t + r];
                if (red[0] < best_err) { best_err = red[0]; best_s = s; }
            }
            scale = best_s;
        }
        scales_f16[(size_t)n * ng + g] = f2h(scale);
        const float inv = 1.0f / scale;
        int8_t* qp = q + (size_t)n * K + (size_t)g * G;
        for (int k = 0; k < G; k++)
            qp[k] = (int8_t)clampi(rn_int(bf2f(wp[k]) * inv), -levels, levels);
    }
}

/* Two 4-bit codes per byte, low nibble = even K index:
 * src/sched/int8_gemv.cu:265-269 (k_pack_nib). */
S2PO_API void s2po_pack(uint8_t* p, const int8_t* q, size_t n_bytes) {
    for (size_t i = 0; i < n_bytes; i++)
        p[i] = (uint8_t)((q[2 * i] & 0xF) | ((q[2 * i + 1] & 0xF) << 4));
}

/* Sign-extending unpack: src/sched/int8_gemv.cu:271-277 (unpack16). */
static inline int8_t nib_lo(uint8_t b) { return (int8_t)((int8_t)(b << 4) >> 4); }
static inline int8_t nib_hi(uint8_t b) { return (int8_t)((int8_t)b >> 4); }

S2PO_API void s2po_unpack(int8_t* q, const uint8_t* p, size_t n_bytes) {
    for (size_t i = 0; i < n_bytes; i++) {
        q[2 * i] = nib_lo(p[i]);
        q[2 * i + 1] = nib_hi(p[i]);
    }
}

/* Dequant to bf16: src/sched/int8_gemv.cu:106-114, 244-253, 731-744. */
S2PO_API void s2po_dequant_int8(uint16_t* o, const int8_t* w, const float* scales,
                                int N, int K) {
    for (int n = 0; n < N; n++)
        for (int k = 0; k < K; k++)
            o[(size_t)n * K + k] = f2bf((float)w[(size_t)n * K + k] * scales[n]);
}
S2PO_API void s2po_dequant_g(uint16_t* o, const int8_t* w, const uint16_t* sc,
                             int N, int K, int G) {
    const int ng = K / G;
    for (int n = 0; n < N; n++)
        for (int k = 0; k < K; k++)
            o[(size_t)n * K + k] =
                f2bf((float)w[(size_t)n * K + k] * h2f(sc[(size_t)n * ng + k / G]));
}
S2PO_API void s2po_dequant_p(uint16_t* o, const uint8_t* w, const uint16_t* sc,
                             int N, int K, int G) {
    const int ng = K / G;
    for (int n = 0; n < N; n++)
        for (int k = 0; k < K; k++) {
            const uint8_t b = w[(size_t)n * (K / 2) + k / 2];
            const int8_t v = (k & 1) ? nib_hi(b) : nib_lo(b);
            o[(size_t)n * K + k] = f2bf((float)v * h2f(sc[(size_t)n * ng + k / G]));
        }
}

/* ---------------------------------------------------------------- GEMVs --- */

/* The shuffle-down tree of the reference GEMVs (acc += shfl_down(acc, off),
 * off = 16,8,4,2,1); only lane 0's value is used. */
static inline float lane_tree(float* a) {
    for (int off = 16; off > 0; off >>= 1)
        for (int l = 0; l < off; l++) a[l] += a[l + off];
    return a[0];
}

/* INT8 per-channel GEMV: src/sched/int8_gemv.cu:60-104 (k_gemv).  One warp
 * per row; lane l owns k = 512 i + 16 l .. +15: a 16-term fma chain from 0,
 * then acc += s; tree; y = bf16(acc * scale[n]).  Requires K % 512 == 0. */
S2PO_API void s2po_gemv_int8(uint16_t* y, const uint16_t* x, const int8_t* w,
                             const float* scales, int M, int N, int K) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        const int8_t* wr = w + (size_t)n * K;
        for (int m = 0; m < M; m++) {
            const uint16_t* xr = x + (size_t)m * K;
            float acc[32];
            for (int l = 0; l < 32; l++) {
                float a = 0.f;
                for (int k0 = l * 16; k0 < K; k0 += 512) {
                    float s = 0.f;
                    for (int j = 0; j < 16; j++)
                        s = fmaf((float)wr[k0 + j], bf2f(xr[k0 + j]), s);
                    a += s;
                }
                acc[l] = a;
            }
            y[(size_t)m * N + n] = f2bf(lane_tree(acc) * scales[n]);
        }
    }
}

/* Group-scaled GEMV on the int8 container: src/sched/int8_gemv.cu:197-242
 * (k_gemv_g): acc = fma(s, gs, acc) with gs the f16 scale of the tile's group. */
S2PO_API void s2po_gemv_g(uint16_t* y, const uint16_t* x, const int8_t* w,
                          const uint16_t* sc, int M, int N, int K, int G) {
    const int ng = K / G;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        const int8_t* wr = w + (size_t)n * K;
        const uint16_t* sr = sc + (size_t)n * ng;
        for (int m = 0; m < M; m++) {
            const uint16_t* xr = x + (size_t)m * K;
            float acc[32];
            for (int l = 0; l < 32; l++) {
                float a = 0.f;
                for (int k0 = l * 16; k0 < K; k0 += 512) {
                    float s = 0.f;
                    for (int j = 0; j < 16; j++)
                        s = fmaf((float)wr[k0 + j], bf2f(xr[k0 + j]), s);
                    a = fmaf(s, h2f(sr[k0 / G]), a);
                }
                acc[l] = a;
            }
            y[(size_t)m * N + n] = f2bf(lane_tree(acc));
        }
    }
}

/* Packed INT4 GEMV: src/sched/int8_gemv.cu:279-324 (k_gemv_p); identical
 * order to the container kernel after the sign-extending unpack. */
S2PO_API void s2po_gemv_p(uint16_t* y, const uint16_t* x, const uint8_t* w,
                          const uint16_t* sc, int M, int N, int K, int G) {
    const int ng = K / G;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        const uint8_t* wr = w + (size_t)n * (K / 2);
        const uint16_t* sr = sc + (size_t)n * ng;
        for (int m = 0; m < M; m++) {
            const uint16_t* xr = x + (size_t)m * K;
            float acc[32];
            for (int l = 0; l < 32; l++) {
                float a = 0.f;
                for (int k0 = l * 16; k0 < K; k0 += 512) {
                    float s = 0.f;
                    for (int j = 0; j < 8; j++) {
                        const uint8_t b = wr[(k0 >> 1) + j];
                        s = fmaf((float)nib_lo(b), bf2f(xr[k0 + 2 * j]), s);
                        s = fmaf((float)nib_hi(b), bf2f(xr[k0 + 2 * j + 1]), s);
                    }
                    a = fmaf(s, h2f(sr[k0 / G]), a);
                }
                acc[l] = a;
            }
            y[(size_t)m * N + n] = f2bf(lane_tree(acc));
        }
    }
}

/* ------------------------------------------------------ row primitives ---- */

/* Halving tree over T values in place (red[t] op= red[t+off]). */
static inline float tree_sum(float* red, int T) {
    for (int off = T >> 1; off > 0; off >>= 1)
        for (int t = 0; t < off; t++) red[t] += red[t + off];
    return red[0];
}

/* GPU rsqrtf is not the correctly rounded 1/sqrt; the host value differs by
 * at most a few ulp, which is why everything downstream of a norm is compared
 * to tolerance and not bitwise. */
static inline float host_rsqrtf(float v) { return 1.0f / sqrtf(v); }

/* RMSNorm: src/slowar/kernels.cu:46-68 (k_rms_norm, `threads` = 256) and
 * :81-101 (k_qk_norm, 128 threads over head_dim).  Partials s_t = fma chain
 * over i = t, t+T, ...; halving tree; inv = rsqrtf(sum/width + eps);
 * y = bf16((v*inv)*w). */
S2PO_API void s2po_rms_norm(const uint16_t* x, const uint16_t* w, uint16_t* y,
                            int rows, int width, float eps, int threads) {
    float red[256];
    for (int r = 0; r < rows; r++) {
        const uint16_t* xr = x + (size_t)r * width;
        for (int t = 0; t < threads; t++) {
            float s = 0.f;
            for (int i = t; i < width; i += threads) {
                const float v = bf2f(xr[i]);
                s = fmaf(v, v, s);
            }
            red[t] = s;
        }
        const float inv = host_rsqrtf(tree_sum(red, threads) / (float)width + eps);
        for (int i = 0; i < width; i++)
            y[(size_t)r * width + i] = f2bf(bf2f(xr[i]) * inv * bf2f(w[i]));
    }
}

/* RoPE on one tensor [rows, heads, head_dim], interleaved pairs, cos/sin
 * rounded through bf16, no fma in the butterfly: src/slowar/kernels.cu:114-139. */
S2PO_API void s2po_rope(uint16_t* x, int rows, int heads, int head_dim,
                        const int32_t* pos, float rope_base) {
    for (int r = 0; r < rows; r++)
        for (int h = 0; h < heads; h++)
            for (int i = 0; i < head_dim / 2; i++) {
                const float ex = (float)(2 * i) / (float)head_dim;
                const float inv = 1.0f / powf(rope_base, ex);
                const float ang = (float)pos[r] * inv;
                const float c = bf2f(f2bf(cosf(ang)));
                const float s = bf2f(f2bf(sinf(ang)));
                uint16_t* p = x + ((size_t)r * heads + h) * head_dim + 2 * i;
                const float x0 = bf2f(p[0]), x1 = bf2f(p[1]);
                p[0] = f2bf(x0 * c - x1 * s);
                p[1] = f2bf(x1 * c + x0 * s);
            }
}

/* INT8 KV quantize of one 128-vector (4 groups of 32):
 * src/slowar/kernels.cu:521-581 (k_kv_append8<8>). */
S2PO_API void s2po_kv8_quant(int8_t* q, uint16_t* sc_f16, const uint16_t* v,
                             int head_dim) {
    for (int g = 0; g < head_dim / 32; g++) {
        float a = 0.f;
        for (int e = 0; e < 32; e++) a = fmaxf(a, fabsf(bf2f(v[g * 32 + e])));
        const uint16_t hsc = f2h(a / 127.0f);
        const float sc = h2f(hsc);
        sc_f16[g] = hsc;
        for (int e = 0; e < 32; e++) {
            const float xv = bf2f(v[g * 32 + e]);
            q[g * 32 + e] =
                (int8_t)clampi(sc > 0.f ? rn_int(xv / sc) : 0, -127, 127);
        }
    }
}

/* SwiGLU with two bf16 roundings: src/slowar/kernels.cu:1216-1229. */
S2PO_API void s2po_silu_mul(const uint16_t* gu, uint16_t* h, int rows, int ffn) {
    for (int r = 0; r < rows; r++)
        for (int c = 0; c < ffn; c++) {
            const float g = bf2f(gu[(size_t)r * 2 * ffn + c]);
            const float u = bf2f(gu[(size_t)r * 2 * ffn + ffn + c]);
            const float sig = 1.0f / (1.0f + expf(-g));
            const float sil = bf2f(f2bf(g * sig));
            h[(size_t)r * ffn + c] = f2bf(sil * u);
        }
}

/* Residual add: src/slowar/kernels.cu:1242-1247. */
S2PO_API void s2po_add(uint16_t* y, const uint16_t* x, int64_t n) {
    for (int64_t i = 0; i < n; i++) y[i] = f2bf(bf2f(y[i]) + bf2f(x[i]));
}

/* Embedding from the INT8 sidecar: src/slowar/kernels.cu:1281-1291. */
S2PO_API void s2po_embed_i8(const int8_t* table, const float* scales,
                            const int64_t* ids, uint16_t* out, int rows, int dim) {
    for (int r = 0; r < rows; r++)
        for (int d = 0; d < dim; d++)
            out[(size_t)r * dim + d] =
                f2bf((float)table[(size_t)ids[r] * dim + d] * scales[ids[r]]);
}

/* Sum of the 10 codebook embeddings added to a row:
 * src/fastar/fastar.cu:104-127 (k_vq_embed_add); codes cb-major [10*T]. */
S2PO_API void s2po_vq_embed_add(const uint16_t* table, const int32_t* codes, int T,
                                uint16_t* rows, int dim, int ncb, int cbsize) {
    for (int t = 0; t < T; t++)
        for (int d = 0; d < dim; d++) {
            float acc = 0.f;
            for (int cb = 0; cb < ncb; cb++) {
                int c = clampi(codes[(size_t)cb * T + t], 0, cbsize - 1);
                acc += bf2f(table[((size_t)cb * cbsize + c) * dim + d]);
            }
            const uint16_t s = f2bf(acc);
            uint16_t* o = rows + (size_t)t * dim + d;
            *o = f2bf(bf2f(*o) + bf2f(s));
        }
}

/* Argmax with lowest index on ties: src/slowar/kernels.cu:1326-1357. */
S2PO_API void s2po_argmax(const uint16_t* logits, int32_t* ids, int rows, int vocab) {
    for (int r = 0; r < rows; r++) {
        float bv = -INFINITY;
        int bi = 0;
        for (int i = 0; i < vocab; i++) {
            const float v = bf2f(logits[(size_t)r * vocab + i]);
            if (v > bv) { bv = v; bi = i; }
        }
        ids[r] = bi;
    }
}

/* -------------------------------------------------------------- attention -- */

/* Split-K flash decode over a bf16 cache followed by the ascending-split
 * combine: src/slowar/kernels.cu:351-489.  One query row, all q heads.
 * kc/vc: [kv_heads, max_seq, 128]; len positions are visible. */
#define HD 128
#define SPLIT 64

static void combine_splits(const float* part, int n_splits, uint16_t* out_head) {
    /* part: [n_splits][HD+2] = (m, l, acc[HD]) — kernels.cu:469-489 */
    float M = -INFINITY;
    for (int s = 0; s < n_splits; s++) M = fmaxf(M, part[(size_t)s * (HD + 2)]);
    for (int t = 0; t < HD; t++) {
        float l = 0.f, acc = 0.f;
        for (int s = 0; s < n_splits; s++) {
            const float* ph = part + (size_t)s * (HD + 2);
            if (ph[1] == 0.f) continue;
            const float w = expf(ph[0] - M);
            l = fmaf(ph[1], w, l);
            acc = fmaf(ph[2 + t], w, acc);
        }
        out_head[t] = f2bf(acc / l);
    }
}

static float tree_max128(const float* v, int cnt) {
    float red[128];
    for (int t = 0; t < 128; t++) red[t] = t < cnt ? v[t] : -INFINITY;
    for (int off = 64; off > 0; off >>= 1)
        for (int t = 0; t < off; t++) red[t] = fmaxf(red[t], red[t + off]);
    return red[0];
}
static float tree_sum128(const float* v, int cnt) {
    float red[128];
    for (int t = 0; t < 128; t++) red[t] = t < cnt ? v[t] : 0.f;
    return tree_sum(red, 128);
}

S2PO_API void s2po_attn_decode_bf16(const uint16_t* q, const uint16_t* kc,
                                    const uint16_t* vc, uint16_t* out, int q_heads,
                                    int kv_heads, int len, int max_seq) {
    const int group = q_heads / kv_heads;
    const int n_splits = (len + SPLIT - 1) / SPLIT;
    const float scale = host_rsqrtf((float)HD);
    float* part = (float*)malloc((size_t)n_splits * (HD + 2) * sizeof(float));
    for (int h = 0; h < q_heads; h++) {
        const int kvh = h / group;
        float sq[HD];
        for (int e = 0; e < HD; e++) sq[e] = bf2f(q[(size_t)h * HD + e]) * scale;
        for (int sp = 0; sp < n_splits; sp++) {
            const int start = sp * SPLIT;
            const int cnt = len - start < SPLIT ? len - start : SPLIT;
            float sc[SPLIT];
            for (int t = 0; t < cnt; t++) {
                const uint16_t* kr = kc + ((size_t)kvh * max_seq + start + t) * HD;
                float d = 0.f;
                for (int e = 0; e < HD; e++) d = fmaf(sq[e], bf2f(kr[e]), d);
                sc[t] = d;
            }
            const float m = tree_max128(sc, cnt);
            for (int t = 0; t < cnt; t++) sc[t] = expf(sc[t] - m);
            const float l = tree_sum128(sc, cnt);
            float* ph = part + (size_t)sp * (HD + 2);
            ph[0] = m;
            ph[1] = l;
            for (int t = 0; t < HD; t++) {
                float acc = 0.f;
                for (int j = 0; j < cnt; j++)
                    acc = fmaf(sc[j],
                               bf2f(vc[((size_t)kvh * max_seq + start + j) * HD + t]),
                               acc);
                ph[2 + t] = acc;
            }
        }
        combine_splits(part, n_splits, out + (size_t)h * HD);
    }
    free(part);
}

/* Same over the INT8 cache (payload i8 + f16 scale per 32):
 * src/slowar/kernels.cu:759-918 (k_attn_split8<8>). */
S2PO_API void s2po_attn_decode_kv8(const uint16_t* q, const int8_t* kc,
                                   const int8_t* vc, const uint16_t* ks,
                                   const uint16_t* vs, uint16_t* out, int q_heads,
                                   int kv_heads, int len, int max_seq) {
    const int group = q_heads / kv_heads;
    const int n_splits = (len + SPLIT - 1) / SPLIT;
    const int NG = HD / 32;
    const float scale = host_rsqrtf((float)HD);
    float* part = (float*)malloc((size_t)n_splits * (HD + 2) * sizeof(float));
    for (int h = 0; h < q_heads; h++) {
        const int kvh = h / group;
        float sq[HD];
        for (int e = 0; e < HD; e++) sq[e] = bf2f(q[(size_t)h * HD + e]) * scale;
        for (int sp = 0; sp < n_splits; sp++) {
            const int start = sp * SPLIT;
            const int cnt = len - start < SPLIT ? len - start : SPLIT;
            float sc[SPLIT];
            for (int t = 0; t < cnt; t++) {
                const size_t p = (size_t)kvh * max_seq + start + t;
                float d = 0.f;
                for (int g = 0; g < NG; g++) {
                    float pp = 0.f;
                    for (int e = 0; e < 32; e++)
                        pp = fmaf(sq[g * 32 + e], (float)kc[p * HD + g * 32 + e], pp);
                    d = fmaf(pp, h2f(ks[p * NG + g]), d);
                }
                sc[t] = d;
            }
            const float m = tree_max128(sc, cnt);
            for (int t = 0; t < cnt; t++) sc[t] = expf(sc[t] - m);
            const float l = tree_sum128(sc, cnt);
            float* ph = part + (size_t)sp * (HD + 2);
            ph[0] = m;
            ph[1] = l;
            for (int t = 0; t < HD; t++) {
                float acc = 0.f;
                for (int j = 0; j < cnt; j++) {
                    const size_t p = (size_t)kvh * max_seq + start + j;
                    acc = fmaf(sc[j] * h2f(vs[p * NG + (t >> 5)]),
                               (float)vc[p * HD + t], acc);
                }
                ph[2 + t] = acc;
            }
        }
        combine_splits(part, n_splits, out + (size_t)h * HD);
    }
    free(part);
}

/* Single-pass online-softmax attention, tiles of 128 positions; used by
 * prefill, the fast-AR (depth <= 10) and the legacy path:
 * src/slowar/kernels.cu:234-309 (k_attention) and :625-728 (k_attention8<8>).
 * kv8 != 0 selects the INT8 cache (kc/vc are int8, ks/vs f16 scales). */
S2PO_API void s2po_attn_single(const uint16_t* q, const void* kc_, const void* vc_,
                               const uint16_t* ks, const uint16_t* vs, uint16_t* out,
                               int q_heads, int kv_heads, int len, int max_seq,
                               int kv8) {
    const int group = q_heads / kv_heads;
    const int NG = HD / 32;
    const float scale = host_rsqrtf((float)HD);
    for (int h = 0; h < q_heads; h++) {
        const int kvh = h / group;
        float sq[HD], acc[HD];
        for (int e = 0; e < HD; e++) {
            sq[e] = bf2f(q[(size_t)h * HD + e]) * scale;
            acc[e] = 0.f;
        }
        float m = -INFINITY, l = 0.f;
        for (int t0 = 0; t0 < len; t0 += 128) {
            const int lim = len - t0 < 128 ? len - t0 : 128;
            float s[128];
            for (int t = 0; t < lim; t++) {
                const size_t p = (size_t)kvh * max_seq + t0 + t;
                float d = 0.f;
                if (!kv8) {
                    const uint16_t* kr = (const uint16_t*)kc_ + p * HD;
                    for (int e = 0; e < HD; e++) d = fmaf(sq[e], bf2f(kr[e]), d);
                } else {
                    const int8_t* kr = (const int8_t*)kc_ + p * HD;
                    for (int g = 0; g < NG; g++) {
                        float pp = 0.f;
                        for (int e = 0; e < 32; e++)
                            pp = fmaf(sq[g * 32 + e], (float)kr[g * 32 + e], pp);
                        d = fmaf(pp, h2f(ks[p * NG + g]), d);
                    }
                }
                s[t] = d;
            }
            const float m_new = fmaxf(m, tree_max128(s, lim));
            const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
            float pr[128];
            for (int t = 0; t < lim; t++) pr[t] = expf(s[t] - m_new);
            l = fmaf(l, corr, tree_sum128(pr, lim));
            for (int e = 0; e < HD; e++) {
                float a = acc[e] * corr;
                for (int j = 0; j < lim; j++) {
                    const size_t p = (size_t)kvh * max_seq + t0 + j;
                    if (!kv8)
                        a = fmaf(pr[j], bf2f(((const uint16_t*)vc_)[p * HD + e]), a);
                    else
                        a = fmaf(pr[j] * h2f(vs[p * NG + (e >> 5)]),
                                 (float)((const int8_t*)vc_)[p * HD + e], a);
                }
                acc[e] = a;
            }
            m = m_new;
        }
        for (int e = 0; e < HD; e++) out[(size_t)h * HD + e] = f2bf(acc[e] / l);
    }
}

/* ----------------------------------------------------------------- sampler -- */

/* Sampler state and algorithm: src/slowar/sampling.c:95-112 (init) and
 * :119-282 (s2ps_sample); device twin src/slowar/kernels.cu:979-1181.
 * Order: repetition penalty (gather, then scatter) -> top-30 (value desc,
 * index asc) -> un-temperatured top-p keeping rank 0 -> temperature softmax
 * -> seeded hash-Gumbel draw (counter = uncapped step) or xoshiro inverse CDF. */
typedef struct {
    float temperature, top_p, rep_penalty;
    int32_t window, seeded;
    uint32_t seed31;
    int64_t prev[64];
    uint64_t count;
    uint64_t rng[4];
} s2po_sampler;

static uint64_t splitmix64(uint64_t* s) {
    uint64_t z = (*s += 0x9E3779B97F4A7C15ULL);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}
static inline uint64_t rotl64(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }
static uint64_t xoshiro_next(uint64_t s[4]) {
    const uint64_t result = rotl64(s[1] * 5, 7) * 9;
    const uint64_t t = s[1] << 17;
    s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3];
    s[2] ^= t;
    s[3] = rotl64(s[3], 45);
    return result;
}

S2PO_API size_t s2po_sampler_size(void) { return sizeof(s2po_sampler); }

S2PO_API void s2po_sampler_init(s2po_sampler* sp, float temperature, float top_p,
                                float rep_penalty, int window, uint64_t seed,
                                uint64_t entropy) {
    memset(sp, 0, sizeof(*sp));
    sp->temperature = temperature < 0.f ? 0.f : temperature;
    sp->top_p = (top_p <= 0.f || top_p > 1.f) ? 1.f : top_p;
    sp->rep_penalty = rep_penalty > 0.f ? rep_penalty : 1.f;
    sp->window = window > 0 ? window : 16;
    if (sp->window > 64) sp->window = 64;
    sp->seeded = seed != 0;
    sp->seed31 = (uint32_t)(seed & 0x7FFFFFFFULL);
    uint64_t sm = entropy ^ 0xD1B54A32D192ED03ULL;
    for (int i = 0; i < 4; i++) sp->rng[i] = splitmix64(&sm);
}

/* cand: n_sem semantic logits + 1 EOS logit (bf16).  Returns the raw vocab id;
 * *out_sem = candidate index (0 on EOS), *out_eos = 1 on EOS. */
S2PO_API int64_t s2po_sample(s2po_sampler* sp, const uint16_t* sem_bf16,
                             uint16_t eos_bf16, int n_sem, int64_t sem_start,
                             int64_t eos_id, int32_t* out_sem, int32_t* out_eos) {
    const int n_cand = n_sem + 1;
    float* cand = (float*)malloc((size_t)n_cand * sizeof(float));
    for (int i = 0; i < n_sem; i++) cand[i] = bf2f(sem_bf16[i]);
    cand[n_sem] = bf2f(eos_bf16);

    const int greedy = sp->temperature == 0.0f;
    const int capped = sp->count < (uint64_t)sp->window ? (int)sp->count : sp->window;
    int use_ras = 0;
    if (!greedy && capped >= 4) {
        int64_t last4[4];
        for (int r = 0; r < 4; r++) {
            int idx = capped - (4 - r);
            if (idx < 0) idx = 0;
            last4[r] = sp->prev[idx];
        }
        for (int a = 0; a < 4 && !use_ras; a++)
            for (int b = a + 1; b < 4; b++)
                if (last4[a] == last4[b]) use_ras = 1;
    }
    const float temp = use_ras ? 1.0f : sp->temperature;
    const float topp = use_ras ? 0.9f : sp->top_p;

    if (capped > 0) {
        int ridx[64], rn = 0;
        float rval[64];
        for (int j = 0; j < capped; j++) {
            const int64_t tok = sp->prev[j];
            int ci;
            if (tok >= sem_start && tok < sem_start + n_sem) ci = (int)(tok - sem_start);
            else if (tok == eos_id) ci = n_sem;
            else continue;
            const float v = cand[ci];
            ridx[rn] = ci;
            rval[rn] = v < 0.f ? v * sp->rep_penalty : v / sp->rep_penalty;
            rn++;
        }
        for (int j = 0; j < rn; j++) cand[ridx[j]] = rval[j];
    }

    /* top-30 by 30 passes of "largest value, lowest index" (the device form,
     * kernels.cu:1067-1096; equal to the host insertion form sampling.c:177-192) */
    enum { TOPK = 30 };
    float tv[TOPK];
    int ti[TOPK];
    for (int k = 0; k < TOPK; k++) {
        float bv = -INFINITY;
        int bi = n_cand;
        for (int i = 0; i < n_cand; i++)
            if (cand[i] > bv || (cand[i] == bv && i < bi)) { bv = cand[i]; bi = i; }
        if (bi >= n_cand) bi = n_cand - 1; /* all -inf: never with finite logits */
        tv[k] = bv;
        ti[k] = bi;
        cand[bi] = -INFINITY;
    }

    int choice = 0;
    if (!greedy) {
        float e[TOPK], sum = 0.f;
        const float m = tv[0];
        for (int j = 0; j < TOPK; j++) { e[j] = expf(tv[j] - m); sum += e[j]; }
        int masked[TOPK] = {0};
        float cum = 0.f;
        for (int j = 0; j < TOPK; j++) {
            cum += e[j] / sum;
            if (j > 0 && cum > topp) masked[j] = 1;
        }
        const float t = temp < 1e-5f ? 1e-5f : temp;
        float p2[TOPK], s2 = 0.f;
        const float m2 = tv[0] / t;
        for (int j = 0; j < TOPK; j++) {
            p2[j] = masked[j] ? 0.f : expf(tv[j] / t - m2);
            s2 += p2[j];
        }
        for (int j = 0; j < TOPK; j++) p2[j] /= s2;
        if (sp->seeded) {
            const uint64_t step_seed = ((uint64_t)sp->seed31 * 19349663ULL) ^
                                       (sp->count * 73856093ULL);
            float best = -INFINITY;
            for (int j = 0; j < TOPK; j++) {
                const uint64_t hashed = (step_seed * 8589934591ULL) ^
                                        ((uint64_t)j * 479001599ULL);
                float u = (float)(uint32_t)(hashed & 0xFFFFFFULL) / 16777216.0f;
                if (u < 1e-10f) u = 1e-10f;
                const float g = -logf(-logf(u));
                const float pert = logf(p2[j] + 1e-10f) + g;
                if (pert > best) { best = pert; choice = j; }
            }
        } else {
            const double r = (double)(xoshiro_next(sp->rng) >> 11) * 0x1.0p-53;
            double cum2 = 0.0;
            int lastnz = 0;
            choice = -1;
            for (int j = 0; j < TOPK; j++) {
                if (p2[j] <= 0.f) continue;
                lastnz = j;
                cum2 += (double)p2[j];
                if (r < cum2) { choice = j; break; }
            }
            if (choice < 0) choice = lastnz;
        }
    }
    free(cand);

    const int ci = ti[choice];
    const int64_t tok = ci == n_sem ? eos_id : sem_start + ci;
    if (tok == eos_id) {
        *out_sem = 0;
        *out_eos = 1;
        return tok;
    }
    *out_sem = ci;
    *out_eos = 0;
    if (sp->count < (uint64_t)sp->window) {
        sp->prev[sp->count] = tok;
    } else {
        memmove(sp->prev, sp->prev + 1, (size_t)(sp->window - 1) * sizeof(int64_t));
        sp->prev[sp->window - 1] = tok;
    }
    sp->count++;
    return tok;
}

/* ------------------------------------------------------------ whole model -- */

/* A linear layer in one of the reference's storage forms
 * (include/s2pro/gemm.h:42-62).  kind: 0 bf16, 1 per-channel INT8,
 * 2 group INT4 in an int8 container, 3 group INT4 packed. */
typedef struct {
    int N, K, kind, G;
    uint16_t* w_bf16;
    int8_t* q;
    uint8_t* pack;
    float* scale_f32;
    uint16_t* scale_f16;
} s2po_linear;

static void lin_free(s2po_linear* l) {
    free(l->w_bf16); free(l->q); free(l->pack); free(l->scale_f32); free(l->scale_f16);
    memset(l, 0, sizeof(*l));
}

/* Load-time conversion following src/sched/gemm.c:267-373: per-channel INT8,
 * or g32 INT4 with MSE search and nibble packing when int4 != 0. */
static void lin_prepare(s2po_linear* l, const uint16_t* w, int N, int K, int quant,
                        int int4) {
    memset(l, 0, sizeof(*l));
    l->N = N; l->K = K;
    if (!quant) {
        l->kind = 0;
        l->w_bf16 = (uint16_t*)malloc((size_t)N * K * 2);
        memcpy(l->w_bf16, w, (size_t)N * K * 2);
        return;
    }
    l->q = (int8_t*)malloc((size_t)N * K);
    if (!int4) {
        l->kind = 1;
        l->scale_f32 = (float*)malloc((size_t)N * sizeof(float));
        s2po_quant_int8(l->q, l->scale_f32, w, N, K);
        return;
    }
    l->kind = 3; l->G = 32;
    l->scale_f16 = (uint16_t*)malloc((size_t)N * (K / 32) * 2);
    s2po_quant_g(l->q, l->scale_f16, w, N, K, 32, 7, 1);
    l->pack = (uint8_t*)malloc((size_t)N * K / 2);
    s2po_pack(l->pack, l->q, (size_t)N * K / 2);
    free(l->q);
    l->q = NULL;
}

/* y[M,N] = x[M,K] W^T following src/sched/gemm.c:424-501: M <= 16 takes the
 * exact-order GEMV; larger M (prefill) multiplies by the weights dequantized
 * to bf16 with f32 accumulation (the reference calls cuBLAS there, whose
 * summation order is not specified: tolerance class). */
static void lin_forward(const s2po_linear* l, const uint16_t* x, uint16_t* y, int M) {
    const int N = l->N, K = l->K;
    if (l->kind != 0 && M <= 16) {
        if (l->kind == 1) s2po_gemv_int8(y, x, l->q, l->scale_f32, M, N, K);
        else if (l->kind == 2) s2po_gemv_g(y, x, l->q, l->scale_f16, M, N, K, l->G);
        else s2po_gemv_p(y, x, l->pack, l->scale_f16, M, N, K, l->G);
        return;
    }
    float* xf = (float*)malloc((size_t)M * K * sizeof(float));
    for (size_t i = 0; i < (size_t)M * K; i++) xf[i] = bf2f(x[i]);
#pragma omp parallel
    {
        float* wf = (float*)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
        for (int n = 0; n < N; n++) {
            for (int k = 0; k < K; k++) {
                float v;
                if (l->kind == 0) v = bf2f(l->w_bf16[(size_t)n * K + k]);
                else if (l->kind == 1)
                    v = bf2f(f2bf((float)l->q[(size_t)n * K + k] * l->scale_f32[n]));
                else {
                    int8_t qv;
                    if (l->kind == 2) qv = l->q[(size_t)n * K + k];
                    else {
                        const uint8_t b = l->pack[(size_t)n * (K / 2) + k / 2];
                        qv = (k & 1) ? nib_hi(b) : nib_lo(b);
                    }
                    v = bf2f(f2bf((float)qv *
                                  h2f(l->scale_f16[(size_t)n * (K / l->G) + k / l->G])));
                }
                wf[k] = v;
            }
            for (int m = 0; m < M; m++) {
                const float* xr = xf + (size_t)m * K;
                float a = 0.f;
                for (int k = 0; k < K; k++) a = fmaf(wf[k], xr[k], a);
                y[(size_t)m * N + n] = f2bf(a);
            }
        }
        free(wf);
    }
    free(xf);
}

typedef struct {
    s2po_linear wqkv, wo, gate_up, w2;
    uint16_t *attn_norm, *ffn_norm, *q_norm, *k_norm; /* q/k_norm NULL in fast-AR */
} s2po_layer;

typedef struct {
    /* dimensions (reference values: include/s2pro/config.h:16-53) */
    int dim, q_heads, kv_heads, ffn, vocab, n_slow, n_fast, cb_size, n_cb, fast_seq;
    int64_t sem_start, eos_id;
    float eps, rope_base;
    /* modes (src/slowar/model.c:185-215, 243-271; src/sched/gemm.c:252-265) */
    int quant, int4_backbone, int4_fast, kv8, embed_i8_only, ctx_len;
    /* weights */
    uint16_t* embed;       /* bf16 table, kept when !embed_i8_only */
    int8_t* embed_i8;      /* INT8 sidecar of the tied head */
    float* embed_scale;
    s2po_layer* slow;
    uint16_t* final_norm;
    s2po_layer* fast;
    uint16_t* fast_norm;
    s2po_linear fast_out;
    uint16_t* cb_emb;      /* [n_cb*cb_size, dim] */
    uint16_t* fast_emb;    /* [cb_size, dim] */
} s2po_model;

typedef struct {
    s2po_model* m;
    int state; /* 0 new, 1 prefilled, 2 decoding, 3 finished */
    int kv_len;
    void* kv;        /* [n_slow][2*kv_heads][ctx][128] bf16 or i8 */
    uint16_t* kvs;   /* kv8: [n_slow][2*kv_heads][ctx][4] f16 */
    uint16_t* pending_hidden;
    int64_t prev_token;
    int32_t prev_codes[16];
    s2po_sampler samp;
} s2po_session;

S2PO_API s2po_model* s2po_model_new(int dim, int q_heads, int kv_heads, int ffn,
                                    int vocab, int n_slow, int n_fast, int cb_size,
                                    int n_cb, int64_t sem_start, int64_t eos_id,
                                    int quant, int int4_backbone, int int4_fast,
                                    int kv8, int embed_i8_only, int ctx_len) {
    s2po_model* m = (s2po_model*)calloc(1, sizeof(*m));
    m->dim = dim; m->q_heads = q_heads; m->kv_heads = kv_heads; m->ffn = ffn;
    m->vocab = vocab; m->n_slow = n_slow; m->n_fast = n_fast; m->cb_size = cb_size;
    m->n_cb = n_cb; m->fast_seq = n_cb + 1; m->sem_start = sem_start; m->eos_id = eos_id;
    m->eps = 1e-6f; m->rope_base = 1000000.0f;
    m->quant = quant; m->int4_backbone = int4_backbone; m->int4_fast = int4_fast;
    m->kv8 = kv8; m->embed_i8_only = quant && embed_i8_only; m->ctx_len = ctx_len;
    m->slow = (s2po_layer*)calloc((size_t)n_slow, sizeof(s2po_layer));
    m->fast = (s2po_layer*)calloc((size_t)n_fast, sizeof(s2po_layer));
    return m;
}

static uint16_t* dup16(const uint16_t* p, size_t n) {
    uint16_t* o = (uint16_t*)malloc(n * 2);
    memcpy(o, p, n * 2);
    return o;
}

/* Tensor intake by checkpoint role.  which: 0 wqkv, 1 wo, 2 w1(gate), 3 w3(up),
 * 4 w2, 5 attn_norm, 6 ffn_norm, 7 q_norm, 8 k_norm.  w1 must arrive before w3:
 * the two are fused row-wise into gate_up (src/slowar/model.c:55-92). */
S2PO_API void s2po_model_set_layer(s2po_model* m, int fast, int layer, int which,
                                   const uint16_t* w) {
    s2po_layer* L = fast ? &m->fast[layer] : &m->slow[layer];
    const int D = m->dim, QW = m->q_heads * HD, KVW = m->kv_heads * HD, F = m->ffn;
    const int i4 = fast ? m->int4_fast : m->int4_backbone;
    static __thread uint16_t* gate_tmp = NULL;
    switch (which) {
    case 0: lin_prepare(&L->wqkv, w, QW + 2 * KVW, D, m->quant, i4); break;
    case 1: lin_prepare(&L->wo, w, D, QW, m->quant, i4); break;
    case 2: free(gate_tmp); gate_tmp = dup16(w, (size_t)F * D); break;
    case 3: {
        uint16_t* gu = (uint16_t*)malloc((size_t)2 * F * D * 2);
        memcpy(gu, gate_tmp, (size_t)F * D * 2);
        memcpy(gu + (size_t)F * D, w, (size_t)F * D * 2);
        lin_prepare(&L->gate_up, gu, 2 * F, D, m->quant, i4);
        free(gu); free(gate_tmp); gate_tmp = NULL;
        break;
    }
    case 4: lin_prepare(&L->w2, w, D, F, m->quant, i4); break;
    case 5: L->attn_norm = dup16(w, (size_t)D); break;
    case 6: L->ffn_norm = dup16(w, (size_t)D); break;
    case 7: L->q_norm = dup16(w, HD); break;
    case 8: L->k_norm = dup16(w, HD); break;
    }
}

/* which: 0 embeddings (+INT8 sidecar), 1 final norm, 2 fast norm, 3 fast output
 * head, 4 codebook_embeddings, 5 fast embeddings. */
S2PO_API void s2po_model_set_global(s2po_model* m, int which, const uint16_t* w) {
    const int D = m->dim;
    switch (which) {
    case 0:
        if (m->quant) {
            m->embed_i8 = (int8_t*)malloc((size_t)m->vocab * D);
            m->embed_scale = (float*)malloc((size_t)m->vocab * sizeof(float));
            s2po_quant_int8(m->embed_i8, m->embed_scale, w, m->vocab, D);
        }
        if (!m->embed_i8_only) m->embed = dup16(w, (size_t)m->vocab * D);
        break;
    case 1: m->final_norm = dup16(w, (size_t)D); break;
    case 2: m->fast_norm = dup16(w, (size_t)D); break;
    case 3: lin_prepare(&m->fast_out, w, m->cb_size, D, m->quant, m->int4_fast); break;
    case 4: m->cb_emb = dup16(w, (size_t)m->n_cb * m->cb_size * D); break;
    case 5: m->fast_emb = dup16(w, (size_t)m->cb_size * D); break;
    }
}

static void layer_free(s2po_layer* L) {
    lin_free(&L->wqkv); lin_free(&L->wo); lin_free(&L->gate_up); lin_free(&L->w2);
    free(L->attn_norm); free(L->ffn_norm); free(L->q_norm); free(L->k_norm);
}

S2PO_API void s2po_model_free(s2po_model* m) {
    if (!m) return;
    for (int l = 0; l < m->n_slow; l++) layer_free(&m->slow[l]);
    for (int l = 0; l < m->n_fast; l++) layer_free(&m->fast[l]);
    free(m->slow); free(m->fast); free(m->embed); free(m->embed_i8);
    free(m->embed_scale); free(m->final_norm); free(m->fast_norm);
    lin_free(&m->fast_out); free(m->cb_emb); free(m->fast_emb);
    free(m);
}

S2PO_API s2po_session* s2po_session_new(s2po_model* m, float temperature, float top_p,
                                        float rep_penalty, int window, uint64_t seed) {
    s2po_session* s = (s2po_session*)calloc(1, sizeof(*s));
    s->m = m;
    const size_t planes = (size_t)m->n_slow * 2 * m->kv_heads;
    s->kv = calloc(planes * m->ctx_len * HD, m->kv8 ? 1 : 2);
    if (m->kv8) s->kvs = (uint16_t*)calloc(planes * m->ctx_len * (HD / 32), 2);
    s->pending_hidden = (uint16_t*)calloc((size_t)m->dim, 2);
    s2po_sampler_init(&s->samp, temperature, top_p, rep_penalty, window, seed, 0);
    return s;
}

S2PO_API void s2po_session_free(s2po_session* s) {
    if (!s) return;
    free(s->kv); free(s->kvs); free(s->pending_hidden); free(s);
}

static void embed_rows(const s2po_model* m, const int64_t* ids, uint16_t* out, int rows) {
    const int D = m->dim;
    if (m->embed_i8_only) { s2po_embed_i8(m->embed_i8, m->embed_scale, ids, out, rows, D); return; }
    for (int r = 0; r < rows; r++)
        memcpy(out + (size_t)r * D, m->embed + (size_t)ids[r] * D, (size_t)D * 2);
}

/* One pre-norm transformer layer over `rows` rows at positions pos0..pos0+rows-1
 * against one session's cache: src/slowar/slowar.c:156-260 (run_layer).
 * decode != 0 selects the split-K decode attention (batch path), else the
 * single-pass kernel used by prefill.  For the fast-AR (src/fastar/fastar.cu:
 * 655-724) kbase/vbase point at the per-layer bf16 slab of depth fast_seq. */
static void run_layer(const s2po_model* m, const s2po_layer* L, uint16_t* x, int rows,
                      int pos0, void* kc, void* vc, uint16_t* ks, uint16_t* vs,
                      int max_seq, int kv8, int decode) {
    const int D = m->dim, QH = m->q_heads, KVH = m->kv_heads, F = m->ffn;
    const int QW = QH * HD, KVW = KVH * HD;
    uint16_t* norm = (uint16_t*)malloc((size_t)rows * D * 2);
    uint16_t* qkv = (uint16_t*)malloc((size_t)rows * (QW + 2 * KVW) * 2);
    uint16_t* q = (uint16_t*)malloc((size_t)rows * QW * 2);
    uint16_t* k = (uint16_t*)malloc((size_t)rows * KVW * 2);
    uint16_t* v = (uint16_t*)malloc((size_t)rows * KVW * 2);
    uint16_t* attn = (uint16_t*)malloc((size_t)rows * QW * 2);
    uint16_t* proj = (uint16_t*)malloc((size_t)rows * D * 2);
    uint16_t* gu = (uint16_t*)malloc((size_t)rows * 2 * F * 2);
    uint16_t* hff = (uint16_t*)malloc((size_t)rows * F * 2);
    int32_t* pos = (int32_t*)malloc((size_t)rows * sizeof(int32_t));
    for (int r = 0; r < rows; r++) pos[r] = pos0 + r;

    s2po_rms_norm(x, L->attn_norm, norm, rows, D, m->eps, 256);
    lin_forward(&L->wqkv, norm, qkv, rows);
    for (int r = 0; r < rows; r++) {
        const uint16_t* src = qkv + (size_t)r * (QW + 2 * KVW);
        memcpy(q + (size_t)r * QW, src, (size_t)QW * 2);
        memcpy(k + (size_t)r * KVW, src + QW, (size_t)KVW * 2);
        memcpy(v + (size_t)r * KVW, src + QW + KVW, (size_t)KVW * 2);
    }
    if (L->q_norm) {
        s2po_rms_norm(q, L->q_norm, q, rows * QH, HD, m->eps, 128);
        s2po_rms_norm(k, L->k_norm, k, rows * KVH, HD, m->eps, 128);
    }
    s2po_rope(q, rows, QH, HD, pos, m->rope_base);
    s2po_rope(k, rows, KVH, HD, pos, m->rope_base);
    for (int r = 0; r < rows; r++)
        for (int h = 0; h < KVH; h++) {
            const size_t dst = (size_t)h * max_seq + pos[r];
            const uint16_t* kr = k + ((size_t)r * KVH + h) * HD;
            const uint16_t* vr = v + ((size_t)r * KVH + h) * HD;
            if (kv8) {
                s2po_kv8_quant((int8_t*)kc + dst * HD, ks + dst * (HD / 32), kr, HD);
                s2po_kv8_quant((int8_t*)vc + dst * HD, vs + dst * (HD / 32), vr, HD);
            } else {
                memcpy((uint16_t*)kc + dst * HD, kr, HD * 2);
                memcpy((uint16_t*)vc + dst * HD, vr, HD * 2);
            }
        }
#pragma omp parallel for schedule(dynamic)
    for (int r = 0; r < rows; r++) {
        const int len = pos[r] + 1;
        if (decode && kv8)
            s2po_attn_decode_kv8(q + (size_t)r * QW, (int8_t*)kc, (int8_t*)vc, ks, vs,
                                 attn + (size_t)r * QW, QH, KVH, len, max_seq);
        else if (decode)
            s2po_attn_decode_bf16(q + (size_t)r * QW, (uint16_t*)kc, (uint16_t*)vc,
                                  attn + (size_t)r * QW, QH, KVH, len, max_seq);
        else
            s2po_attn_single(q + (size_t)r * QW, kc, vc, ks, vs, attn + (size_t)r * QW,
                             QH, KVH, len, max_seq, kv8);
    }
    lin_forward(&L->wo, attn, proj, rows);
    s2po_add(x, proj, (int64_t)rows * D);
    s2po_rms_norm(x, L->ffn_norm, norm, rows, D, m->eps, 256);
    lin_forward(&L->gate_up, norm, gu, rows);
    s2po_silu_mul(gu, hff, rows, F);
    lin_forward(&L->w2, hff, proj, rows);
    s2po_add(x, proj, (int64_t)rows * D);

    free(norm); free(qkv); free(q); free(k); free(v); free(attn); free(proj);
    free(gu); free(hff); free(pos);
}

static void* kv_plane(const s2po_session* s, int layer, int v) {
    const s2po_model* m = s->m;
    const size_t per = (size_t)m->kv_heads * m->ctx_len * HD;
    const size_t off = ((size_t)layer * 2 + (size_t)v) * per;
    return m->kv8 ? (void*)((int8_t*)s->kv + off) : (void*)((uint16_t*)s->kv + off);
}
static uint16_t* kvs_plane(const s2po_session* s, int layer, int v) {
    const s2po_model* m = s->m;
    if (!m->kv8) return NULL;
    const size_t per = (size_t)m->kv_heads * m->ctx_len * (HD / 32);
    return s->kvs + ((size_t)layer * 2 + (size_t)v) * per;
}

/* Prompt prefill without VQ parts: src/slowar/slowar.c:264-379.  hid_dump, if
 * not NULL, receives [n_slow+1][dim] f32: the residual of the last prompt row
 * after every layer, then the final-normed hidden (the S2P_DUMP_DIR hooks). */
S2PO_API int s2po_prefill(s2po_session* s, const int64_t* ids, int n_ids,
                          float* hid_dump) {
    s2po_model* m = s->m;
    if (s->state > 1 || n_ids <= 0 || s->kv_len + n_ids > m->ctx_len - 1) return -1;
    const int D = m->dim, pos0 = s->kv_len;
    uint16_t* x = (uint16_t*)malloc((size_t)n_ids * D * 2);
    embed_rows(m, ids, x, n_ids);
    for (int l = 0; l < m->n_slow; l++) {
        run_layer(m, &m->slow[l], x, n_ids, pos0, kv_plane(s, l, 0), kv_plane(s, l, 1),
                  kvs_plane(s, l, 0), kvs_plane(s, l, 1), m->ctx_len, m->kv8, 0);
        if (hid_dump)
            for (int d = 0; d < D; d++)
                hid_dump[(size_t)l * D + d] = bf2f(x[(size_t)(n_ids - 1) * D + d]);
    }
    s2po_rms_norm(x + (size_t)(n_ids - 1) * D, m->final_norm, s->pending_hidden, 1, D,
                  m->eps, 256);
    if (hid_dump)
        for (int d = 0; d < D; d++)
            hid_dump[(size_t)m->n_slow * D + d] = bf2f(s->pending_hidden[d]);
    free(x);
    s->kv_len = pos0 + n_ids;
    s->state = 1;
    return 0;
}

/* Fast-AR frame: src/fastar/fastar.cu:726-788.  hidden = final-normed slow
 * hidden; sem = sampled semantic code; out9 receives codebooks 1..9. */
static void fast_frame(const s2po_model* m, const uint16_t* hidden, int sem,
                       int32_t* out9, float* logits_dump) {
    const int D = m->dim, KVH = m->kv_heads;
    const size_t per = (size_t)KVH * m->fast_seq * HD;
    uint16_t* slab = (uint16_t*)calloc((size_t)m->n_fast * 2 * per, 2);
    uint16_t* x = (uint16_t*)malloc((size_t)D * 2);
    uint16_t* t = (uint16_t*)malloc((size_t)D * 2);
    uint16_t* logits = (uint16_t*)malloc((size_t)m->cb_size * 2);
    memcpy(x, hidden, (size_t)D * 2);
    for (int l = 0; l < m->n_fast; l++)
        run_layer(m, &m->fast[l], x, 1, 0, slab + (size_t)l * 2 * per,
                  slab + ((size_t)l * 2 + 1) * per, NULL, NULL, m->fast_seq, 0, 0);
    int code = clampi(sem, 0, m->cb_size - 1);
    for (int cb = 1; cb < m->n_cb; cb++) {
        memcpy(x, m->fast_emb + (size_t)code * D, (size_t)D * 2);
        for (int l = 0; l < m->n_fast; l++)
            run_layer(m, &m->fast[l], x, 1, cb, slab + (size_t)l * 2 * per,
                      slab + ((size_t)l * 2 + 1) * per, NULL, NULL, m->fast_seq, 0, 0);
        s2po_rms_norm(x, m->fast_norm, t, 1, D, m->eps, 256);
        lin_forward(&m->fast_out, t, logits, 1);
        if (logits_dump)
            for (int i = 0; i < m->cb_size; i++)
                logits_dump[(size_t)(cb - 1) * m->cb_size + i] = bf2f(logits[i]);
        int32_t id;
        s2po_argmax(logits, &id, 1, m->cb_size);
        out9[cb - 1] = id;
        code = clampi(id, 0, m->cb_size - 1);
    }
    free(slab); free(x); free(t); free(logits);
}

/* One frame for one session: src/slowar/slowar.c:463-606 and :609-826 at n = 1.
 * out_codes[n_cb]; returns 1 on EOS, 0 otherwise, <0 on misuse.  hidden_out
 * (optional, [dim] f32) receives the final-normed hidden the frame sampled from;
 * sem_logits_out (optional, [n_sem+1] f32) the candidate logits. */
S2PO_API int s2po_next_frame(s2po_session* s, int32_t* out_codes, float* hidden_out,
                             float* sem_logits_out) {
    s2po_model* m = s->m;
    const int D = m->dim, n_sem = 4096;
    memset(out_codes, 0, (size_t)m->n_cb * sizeof(int32_t));
    if (s->state == 0) return -6;
    if (s->state == 3) return 1;
    uint16_t* hidden = (uint16_t*)malloc((size_t)D * 2);
    if (s->state == 2) {
        if (s->kv_len >= m->ctx_len) { s->state = 3; free(hidden); return 1; }
        uint16_t* x = (uint16_t*)malloc((size_t)D * 2);
        embed_rows(m, &s->prev_token, x, 1);
        const int sem_tok = s->prev_token >= m->sem_start &&
                            s->prev_token < m->sem_start + n_sem;
        if (sem_tok) {
            /* slowar.c:491-498: VQ sum of the previous frame, then * f32(1/sqrt(11)) */
            s2po_vq_embed_add(m->cb_emb, s->prev_codes, 1, x, D, m->n_cb, m->cb_size);
            const float sc = (float)(1.0 / 3.3166247903554);
            for (int d = 0; d < D; d++) x[d] = f2bf(bf2f(x[d]) * sc);
        }
        for (int l = 0; l < m->n_slow; l++)
            run_layer(m, &m->slow[l], x, 1, s->kv_len, kv_plane(s, l, 0),
                      kv_plane(s, l, 1), kvs_plane(s, l, 0), kvs_plane(s, l, 1),
                      m->ctx_len, m->kv8, 1);
        s2po_rms_norm(x, m->final_norm, hidden, 1, D, m->eps, 256);
        free(x);
    } else {
        memcpy(hidden, s->pending_hidden, (size_t)D * 2);
    }
    if (hidden_out) for (int d = 0; d < D; d++) hidden_out[d] = bf2f(hidden[d]);

    /* tied head on the 4096 semantic rows + the EOS row: slowar.c:519-541 */
    uint16_t* lg = (uint16_t*)malloc((size_t)(n_sem + 1) * 2);
    if (m->quant) {
        s2po_gemv_int8(lg, hidden, m->embed_i8 + (size_t)m->sem_start * D,
                       m->embed_scale + m->sem_start, 1, n_sem, D);
        s2po_gemv_int8(lg + n_sem, hidden, m->embed_i8 + (size_t)m->eos_id * D,
                       m->embed_scale + m->eos_id, 1, 1, D);
    } else {
        for (int i = 0; i <= n_sem; i++) {
            const int64_t row = i < n_sem ? m->sem_start + i : m->eos_id;
            float a = 0.f;
            for (int d = 0; d < D; d++)
                a = fmaf(bf2f(m->embed[(size_t)row * D + d]), bf2f(hidden[d]), a);
            lg[i] = f2bf(a);
        }
    }
    if (sem_logits_out) for (int i = 0; i <= n_sem; i++) sem_logits_out[i] = bf2f(lg[i]);
    int32_t sem = 0, eos = 0;
    const int64_t tok = s2po_sample(&s->samp, lg, lg[n_sem], n_sem, m->sem_start,
                                    m->eos_id, &sem, &eos);
    free(lg);
    int32_t res[16];
    fast_frame(m, hidden, sem, res, NULL);
    free(hidden);
    if (s->state == 2) s->kv_len++;
    if (eos) { s->state = 3; return 1; }
    out_codes[0] = sem;
    for (int cb = 1; cb < m->n_cb; cb++) out_codes[cb] = res[cb - 1];
    s->prev_token = tok;
    memcpy(s->prev_codes, out_codes, (size_t)m->n_cb * sizeof(int32_t));
    s->state = 2;
    return 0;
}

/* Fast-AR frame alone, for golden-vector pinning against the reference's torch
 * model (tools/qat_fastar.py:204-232): hidden bf16 [dim], sem -> 9 codes and,
 * optionally, the 9x4096 head logits as f32. */
S2PO_API void s2po_fast_frame(const s2po_model* m, const uint16_t* hidden, int sem,
                              int32_t* out9, float* logits_dump) {
    fast_frame(m, hidden, sem, out9, logits_dump);
}

/* ------------------------------------------------- CPU baseline sample ---- */

#ifdef _OPENMP
#include <omp.h>
#endif
/* Threads the row loops use from now on (0: leave the OpenMP default); returns the count in
 * force.  A launcher may have exported OMP_NUM_THREADS=1 for its children; a timing that
 * reports "cores" sets the number itself. */
S2PO_API int s2po_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

static void fill_bytes(uint8_t* p, size_t n, uint64_t seed) {
#pragma omp parallel for schedule(static)
    for (int64_t blk = 0; blk < (int64_t)((n + 4095) / 4096); blk++) {
        uint64_t z = seed + 0x9E3779B97F4A7C15ull * (uint64_t)(blk + 1);
        const size_t lo = (size_t)blk * 4096, hi = lo + 4096 < n ? lo + 4096 : n;
        for (size_t i = lo; i < hi; i++) {
            z = z * 6364136223846793005ull + 1442695040888963407ull;
            p[i] = (uint8_t)(z >> 56);
        }
    }
}
static void lin_synthetic(s2po_linear* l, int N, int K, int int4, uint64_t seed) {
    memset(l, 0, sizeof(*l));
    l->N = N; l->K = K;
    if (int4) {
        l->kind = 3; l->G = 32;
        l->pack = (uint8_t*)malloc((size_t)N * K / 2);
        fill_bytes(l->pack, (size_t)N * K / 2, seed);
        l->scale_f16 = (uint16_t*)malloc((size_t)N * (K / 32) * 2);
        for (size_t i = 0; i < (size_t)N * (K / 32); i++) l->scale_f16[i] = f2h(0.003f);
    } else {
        l->kind = 1;
        l->q = (int8_t*)malloc((size_t)N * K);
        fill_bytes((uint8_t*)l->q, (size_t)N * K, seed);
        l->scale_f32 = (float*)malloc((size_t)N * sizeof(float));
        for (int i = 0; i < N; i++) l->scale_f32[i] = 1.6e-4f;
    }
}
static uint16_t* ones16(size_t n) {
    uint16_t* p = (uint16_t*)malloc(n * 2);
    for (size_t i = 0; i < n; i++) p[i] = 0x3F80; /* bf16 1.0 */
    return p;
}
static uint16_t* small16(size_t n, uint64_t seed) { /* bf16 values of magnitude ~0.02, either sign */
    uint16_t* p = (uint16_t*)malloc(n * 2);
    fill_bytes((uint8_t*)p, n * 2, seed);
    for (size_t i = 0; i < n; i++) p[i] = (uint16_t)((p[i] & 0x807F) | 0x3C80);
    return p;
}

/* Timing aid: give a model quantised weights of the right shapes and storage forms without the
 * load-time quantisers (seeded pseudo-random codes, constant scales, unit gains) - the frame
 * functions then do exactly the work of a real checkpoint; the values carry no meaning.
 * Requires quant != 0 and embed_i8_only. */
S2PO_API void s2po_model_fill_synthetic(s2po_model* m, uint64_t seed) {
    const int D = m->dim, QW = m->q_heads * HD, KVW = m->kv_heads * HD, F = m->ffn;
    for (int f = 0; f < 2; f++) {
        const int n = f ? m->n_fast : m->n_slow, i4 = f ? m->int4_fast : m->int4_backbone;
        for (int l = 0; l < n; l++) {
            s2po_layer* L = f ? &m->fast[l] : &m->slow[l];
            const uint64_t s0 = seed + 1000u * (uint64_t)(f * 64 + l);
            lin_synthetic(&L->wqkv, QW + 2 * KVW, D, i4, s0 + 1);
            lin_synthetic(&L->wo, D, QW, i4, s0 + 2);
            lin_synthetic(&L->gate_up, 2 * F, D, i4, s0 + 3);
            lin_synthetic(&L->w2, D, F, i4, s0 + 4);
            L->attn_norm = ones16((size_t)D); L->ffn_norm = ones16((size_t)D);
            if (!f) { L->q_norm = ones16(HD); L->k_norm = ones16(HD); }
        }
    }
    m->embed_i8 = (int8_t*)malloc((size_t)m->vocab * D);
    fill_bytes((uint8_t*)m->embed_i8, (size_t)m->vocab * D, seed + 7);
    m->embed_scale = (float*)malloc((size_t)m->vocab * sizeof(float));
    for (int i = 0; i < m->vocab; i++) m->embed_scale[i] = 1.6e-4f;
    m->final_norm = ones16((size_t)D); m->fast_norm = ones16((size_t)D);
    lin_synthetic(&m->fast_out, m->cb_size, D, m->int4_fast, seed + 8);
    m->cb_emb = small16((size_t)m->n_cb * m->cb_size * D, seed + 9);
    m->fast_emb = small16((size_t)m->cb_size * D, seed + 10);
}


/* Weight-streaming work of `reps` backbone-shaped layers at batch 1 (the four
 * GEMVs of one layer: 6144x2560, 2560x4096, 19456x2560, 2560x9728) on packed
 * INT4 (int4 != 0) or per-channel INT8 weights.  Used only to time the CPU port
 * of the hot loop on a bounded sample; buffers are caller-provided. */
S2PO_API void s2po_layer_gemv_sample(const uint8_t* w, const uint16_t* sc_f16,
                                     const float* sc_f32, const uint16_t* x,
                                     uint16_t* y, int int4, int reps) {
    static const int shp[4][2] = {{6144, 2560}, {2560, 4096}, {19456, 2560}, {2560, 9728}};
    for (int r = 0; r < reps; r++)
        for (int i = 0; i < 4; i++) {
            if (int4) s2po_gemv_p(y, x, w, sc_f16, 1, shp[i][0], shp[i][1], 32);
            else s2po_gemv_int8(y, x, (const int8_t*)w, sc_f32, 1, shp[i][0], shp[i][1]);
        }
}
