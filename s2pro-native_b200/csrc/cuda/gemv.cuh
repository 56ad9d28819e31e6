/* Weight-streaming dequant GEMV for batch-1 decode, as a device-side stage
 * that both the stand-alone launchers (gemv.cu) and the fused decode tick
 * (tick.cu) instantiate.
 *
 * Arithmetic contract (bit-exact with the reference GEMVs,
 * src/sched/int8_gemv.cu:60-104 per-channel INT8, :197-242 group scale on an
 * int8 container, :279-324 packed INT4): output row n is the sum of 32 lane
 * partials; lane l owns the 16 weights k = 512 i + 16 l .. +15 of every K-tile
 * i; inside a tile the products are accumulated as one fma chain starting from
 * 0 (j ascending); tiles are folded in ascending i as acc += s (INT8) or
 * acc = fma(s, group_scale, acc) (INT4); the 32 lane values are merged by the
 * 16/8/4/2/1 tree; INT8 multiplies by the row scale; one bf16 rounding.
 *
 * Mapping to B200 (what is NOT the reference's): the unit of work is a
 * (row-group, K-tile) job, so a 2560-row matrix still offers thousands of
 * independent jobs to the 148 SMs; a CTA owns a contiguous block of rows, i.e.
 * one contiguous span of HBM; every lane keeps two jobs of 8-byte (INT4) or
 * 16-byte (INT8) loads in flight; codes are widened to f32 with one byte-permute
 * and one exact subtraction (no int->float converts); two rows advance per
 * instruction through the packed f32x2 fma of sm_100, each half being its own
 * IEEE fma chain; the activation vector is staged once per CTA in shared
 * memory in the lane order the jobs read it; per-tile partials cross warps
 * through shared memory and one warp per row folds them in the fixed order.
 */
#pragma once
#include "common.cuh"

namespace s2p {

enum WeightKind { WK_INT8_CH = 0, WK_INT8_GRP = 1, WK_INT4_PACK = 2 };
enum Prologue {
    PRO_VEC = 0,  /* x is a bf16 vector */
    PRO_NORM = 1  /* x = bf16(rmsnorm(src) * norm_w), the reference's k_rms_norm order */
};
enum Epilogue {
    EPI_STORE = 0,  /* y[n] = bf16(acc) */
    EPI_RESID = 1,  /* dst[n] = bf16(f32(src[n]) + f32(bf16(acc)))  (GEMV store, then the residual add) */
    EPI_SWIGLU = 2, /* rows come as (gate n, up n+F): h[n] = bf16(f32(bf16(g*sigmoid(g))) * u) */
    EPI_ARGMAX = 3  /* y[n] = bf16(acc) and a packed (value, lowest index) atomic max */
};

struct GemvStage {
    /* weights */
    const void* w;       /* int8 [N,K] or nibbles [N,K/2] */
    const void* scales;  /* f32 [N] (WK_INT8_CH) or f16 [N, K>>gshift] */
    int N, K, gshift;
    /* input */
    const __nv_bfloat16* x;       /* [K]; with x_index / x_key: a row of a [*,K] table */
    const int32_t* x_index;       /* optional device index selecting the input row */
    const unsigned long long* x_key; /* optional packed arg-max key selecting the input row */
    const __nv_bfloat16* norm_w;  /* PRO_NORM gain [K] */
    float eps;
    /* output */
    __nv_bfloat16* y;                 /* EPI_STORE/ARGMAX: [N]; EPI_SWIGLU: [N/2]; EPI_RESID: destination [N] */
    const __nv_bfloat16* resid_src;   /* EPI_RESID: vector the product is added to */
    const int32_t* resid_index;       /* optional device index: resid_src is row *resid_index of a [*,N] table */
    const unsigned long long* resid_key; /* same, from a packed arg-max key */
    unsigned long long* argmax_key;   /* EPI_ARGMAX */
    int rows_per_pass;                /* rows (row pairs for EPI_SWIGLU) the shared partial buffer holds */
};

constexpr int GEMV_THREADS = 512;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;

/* rows advanced together by one job */
template <int WK> struct JobRows { static constexpr int value = (WK == WK_INT4_PACK) ? 8 : 4; };

__host__ __device__ inline size_t gemv_smem_bytes(int wk, int rows_per_cta, int K, int gshift) {
    const int T = K / 512;
    size_t b = (size_t)K * 8;                             /* x, duplicated f32 pairs */
    b += (size_t)rows_per_cta * T * 32 * sizeof(float);   /* per-tile lane partials */
    if (wk != WK_INT8_CH) b += ((size_t)rows_per_cta * (K >> gshift) * 2 + 15) & ~(size_t)15;
    return b + 1024 /* reduction scratch */;
}

/* Shared-memory slot of activation k as a duplicated pair (x_k, x_k).  A lane
 * reads its 16 activations of a tile as eight 16-byte words, consecutive lanes
 * touching consecutive words (no bank conflicts). */
__device__ __forceinline__ int xs_slot(int k) {
    const int i = k >> 9, l = (k >> 4) & 31, j = k & 15;
    return (((i * 8 + (j >> 1)) * 32 + l) << 2) + ((j & 1) << 1);
}

/* index held in a packed arg-max key (see EPI_ARGMAX) */
__device__ __forceinline__ uint32_t key_index(unsigned long long key) { return 0xFFFFFFFFu - (uint32_t)key; }

__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }

/* 8 nibbles of two rows (same columns) -> 8 steps of the two fma chains. */
__device__ __forceinline__ void chain_int4_word(uint32_t wa, uint32_t wb, const float4* xq, float2& s) {
    const uint32_t a = wa ^ 0x88888888u, b = wb ^ 0x88888888u;
    const uint32_t ae = a & 0x0F0F0F0Fu, ao = (a >> 4) & 0x0F0F0F0Fu;
    const uint32_t be = b & 0x0F0F0F0Fu, bo = (b >> 4) & 0x0F0F0F0Fu;
    const float2 bias = make_float2(-8388616.0f, -8388616.0f); /* -(2^23 + 8) */
#pragma unroll
    for (int t = 0; t < 4; t++) {
        const float4 xv = xq[t]; /* (x_2t, x_2t, x_2t+1, x_2t+1) */
        float2 f;
        f.x = __uint_as_float(__byte_perm(ae, 0x4B000000u, 0x7540u | t));
        f.y = __uint_as_float(__byte_perm(be, 0x4B000000u, 0x7540u | t));
        s = ffma2(__fadd2_rn(f, bias), make_float2(xv.x, xv.y), s);
        f.x = __uint_as_float(__byte_perm(ao, 0x4B000000u, 0x7540u | t));
        f.y = __uint_as_float(__byte_perm(bo, 0x4B000000u, 0x7540u | t));
        s = ffma2(__fadd2_rn(f, bias), make_float2(xv.z, xv.w), s);
    }
}

/* 4 int8 codes of two rows -> 4 steps. xq: two 16-byte words = 4 duplicated pairs. */
__device__ __forceinline__ void chain_int8_word(uint32_t wa, uint32_t wb, const float4* xq, float2& s) {
    const uint32_t a = wa ^ 0x80808080u, b = wb ^ 0x80808080u;
    const float2 bias = make_float2(-8388736.0f, -8388736.0f); /* -(2^23 + 128) */
#pragma unroll
    for (int t = 0; t < 2; t++) {
        const float4 xv = xq[t];
        float2 f;
        f.x = __uint_as_float(__byte_perm(a, 0x4B000000u, 0x7540u | (2 * t)));
        f.y = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7540u | (2 * t)));
        s = ffma2(__fadd2_rn(f, bias), make_float2(xv.x, xv.y), s);
        f.x = __uint_as_float(__byte_perm(a, 0x4B000000u, 0x7540u | (2 * t + 1)));
        f.y = __uint_as_float(__byte_perm(b, 0x4B000000u, 0x7540u | (2 * t + 1)));
        s = ffma2(__fadd2_rn(f, bias), make_float2(xv.z, xv.w), s);
    }
}

template <int WK> struct LaneTile;  /* the bytes one lane owns of one (row, tile) */
template <> struct LaneTile<WK_INT4_PACK> { typedef uint2 type; };
template <> struct LaneTile<WK_INT8_CH> { typedef uint4 type; };
template <> struct LaneTile<WK_INT8_GRP> { typedef uint4 type; };

template <int WK>
__device__ __forceinline__ void chain_tile(const typename LaneTile<WK>::type& a, const typename LaneTile<WK>::type& b,
                                           const float4* xq, float2& s);
template <>
__device__ __forceinline__ void chain_tile<WK_INT4_PACK>(const uint2& a, const uint2& b, const float4* xq, float2& s) {
    chain_int4_word(a.x, b.x, xq, s);
    chain_int4_word(a.y, b.y, xq + 4, s);
}
template <>
__device__ __forceinline__ void chain_tile<WK_INT8_CH>(const uint4& a, const uint4& b, const float4* xq, float2& s) {
    chain_int8_word(a.x, b.x, xq, s);
    chain_int8_word(a.y, b.y, xq + 2, s);
    chain_int8_word(a.z, b.z, xq + 4, s);
    chain_int8_word(a.w, b.w, xq + 6, s);
}
template <>
__device__ __forceinline__ void chain_tile<WK_INT8_GRP>(const uint4& a, const uint4& b, const float4* xq, float2& s) {
    chain_tile<WK_INT8_CH>(a, b, xq, s);
}

/* ---- prologue: stage the activation vector ------------------------------- */
template <int PRO>
__device__ __forceinline__ void stage_activation(const GemvStage& g, float* xs, float* red) {
    const int K = g.K;
    const __nv_bfloat16* x = g.x;
    if (g.x_index) x += (size_t)(*g.x_index) * K;
    else if (g.x_key) x += (size_t)key_index(*g.x_key) * K;
    if (PRO == PRO_VEC) {
        for (int k = threadIdx.x; k < K; k += blockDim.x) {
            const float v = bf2f(x[k]);
            const int s = xs_slot(k);
            xs[s] = v;
            xs[s + 1] = v;
        }
    } else {
        /* 256 strided partial sums of squares, halving tree, rsqrtf(mean + eps):
         * src/slowar/kernels.cu:46-68 */
        float ss = 0.f;
        if (threadIdx.x < 256)
            for (int i = threadIdx.x; i < K; i += 256) {
                const float v = bf2f(x[i]);
                ss = __fmaf_rn(v, v, ss);
            }
        const float tot = block_tree<256, false>(ss, red);
        const float inv = rsqrtf(__fdiv_rn(tot, (float)K) + g.eps);
        for (int k = threadIdx.x; k < K; k += blockDim.x) {
            const float v = bf16_round(__fmul_rn(__fmul_rn(bf2f(x[k]), inv), bf2f(g.norm_w[k])));
            const int s = xs_slot(k);
            xs[s] = v;
            xs[s + 1] = v;
        }
    }
}

/* ---- the stage ------------------------------------------------------------
 * Rows [row0, row0+cnt) of the matrix belong to this CTA; with EPI_SWIGLU the
 * CTA owns gate rows [row0, row0+cnt) and up rows [F+row0, F+row0+cnt), F = N/2.
 * The rows are walked in passes of at most g.rows_per_pass (what the partial
 * buffer in shared memory holds).  smem: dynamic shared memory base, sized by
 * gemv_smem_bytes(wk, rows_per_pass * (swiglu ? 2 : 1), K, gshift).
 * All threads of the CTA (GEMV_THREADS) must call this. */
template <int WK, int PRO, int EPI>
__device__ void gemv_stage_cta(const GemvStage& g, int row0, int cnt_total, unsigned char* smem) {
    typedef typename LaneTile<WK>::type tile_t;
    constexpr int R = JobRows<WK>::value;
    constexpr int SW = (EPI == EPI_SWIGLU) ? 2 : 1;
    const int K = g.K, T = K >> 9;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int F = g.N >> 1;
    const size_t row_bytes = (WK == WK_INT4_PACK) ? (size_t)(K >> 1) : (size_t)K;
    const int sc_per_row = (WK == WK_INT8_CH) ? 0 : (K >> g.gshift);
    const int cap_rows = g.rows_per_pass * SW;

    float* xs = reinterpret_cast<float*>(smem);
    float* part = xs + 2 * K;
    __half* sc_s = reinterpret_cast<__half*>(part + (size_t)cap_rows * T * 32);
    float* red = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(sc_s) +
                                          (((size_t)cap_rows * sc_per_row * 2 + 15) & ~(size_t)15));
    const unsigned char* wbase = static_cast<const unsigned char*>(g.w);
    const float4* xs4 = reinterpret_cast<const float4*>(xs);
    unsigned long long best = 0ull;

    if (cnt_total <= 0) return; /* uniform over the CTA */
    for (int done = 0; done < cnt_total; done += g.rows_per_pass) {
        const int cnt = min(g.rows_per_pass, cnt_total - done);
        const int r0 = row0 + done;
        const int local_rows = cnt * SW;
        auto global_row = [&](int lr) -> int {
            if (EPI == EPI_SWIGLU) return lr < cnt ? r0 + lr : F + r0 + (lr - cnt);
            return r0 + lr;
        };
        const int n_jobs = ((local_rows + R - 1) / R) * T;
        auto load_job = [&](int job, tile_t* buf) {
            const int oct = job / T, tile = job - oct * T;
#pragma unroll
            for (int r = 0; r < R; r++) {
                int lr = oct * R + r;
                lr = lr < local_rows ? lr : local_rows - 1;
                const unsigned char* p = wbase + (size_t)global_row(lr) * row_bytes +
                                         (size_t)tile * (sizeof(tile_t) * 32) + (size_t)lane * sizeof(tile_t);
                buf[r] = *reinterpret_cast<const tile_t*>(p);
            }
        };

        /* weight and scale traffic does not depend on the activations: start it first */
        tile_t cur[R], nxt[R];
        int job = warp;
        if (job < n_jobs) load_job(job, cur);
        if constexpr (WK != WK_INT8_CH) {
            const __half* sg = static_cast<const __half*>(g.scales);
            for (int idx = threadIdx.x; idx < local_rows * sc_per_row; idx += blockDim.x) {
                const int lr = idx / sc_per_row, c = idx - lr * sc_per_row;
                sc_s[idx] = sg[(size_t)global_row(lr) * sc_per_row + c];
            }
        }
        if (done == 0) stage_activation<PRO>(g, xs, red);
        __syncthreads();

        for (; job < n_jobs; job += GEMV_WARPS) {
            const int njob = job + GEMV_WARPS;
            if (njob < n_jobs) load_job(njob, nxt);
            const int oct = job / T, tile = job - oct * T;
            float4 xq[8];
#pragma unroll
            for (int q = 0; q < 8; q++) xq[q] = xs4[(tile * 8 + q) * 32 + lane];
#pragma unroll
            for (int p = 0; p < R / 2; p++) {
                float2 s = make_float2(0.f, 0.f);
                chain_tile<WK>(cur[2 * p], cur[2 * p + 1], xq, s);
                const int lr = oct * R + 2 * p;
                if (lr < local_rows) part[((size_t)lr * T + tile) * 32 + lane] = s.x;
                if (lr + 1 < local_rows) part[((size_t)(lr + 1) * T + tile) * 32 + lane] = s.y;
            }
#pragma unroll
            for (int r = 0; r < R; r++) cur[r] = nxt[r];
        }
        __syncthreads();

        /* fold the tiles of one row in ascending order, merge lanes, finish */
        auto fold_row = [&](int lr) -> float {
            float acc = 0.f;
            const float* pr = part + (size_t)lr * T * 32 + lane;
            if (WK == WK_INT8_CH) {
                for (int i = 0; i < T; i++) acc += pr[i * 32];
            } else {
                const __half* sr = sc_s + (size_t)lr * sc_per_row;
                for (int i = 0; i < T; i++)
                    acc = __fmaf_rn(pr[i * 32], __half2float(sr[(i * 512 + lane * 16) >> g.gshift]), acc);
            }
            acc = warp_tree_sum(acc);
            if (WK == WK_INT8_CH) acc = __fmul_rn(acc, static_cast<const float*>(g.scales)[global_row(lr)]);
            return acc;
        };

        if (EPI == EPI_SWIGLU) {
            for (int r = warp; r < cnt; r += GEMV_WARPS) {
                const float gate = bf16_round(fold_row(r));
                const float up = bf16_round(fold_row(r + cnt));
                if (lane == 0) {
                    /* src/slowar/kernels.cu:1216-1229: silu rounds to bf16 before the up-multiply */
                    const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-gate)));
                    const float sil = bf16_round(__fmul_rn(gate, sig));
                    g.y[r0 + r] = f2bf(__fmul_rn(sil, up));
                }
            }
        } else {
            for (int r = warp; r < cnt; r += GEMV_WARPS) {
                const float acc = fold_row(r);
                const int n = r0 + r;
                if (lane == 0) {
                    const __nv_bfloat16 yb = f2bf(acc);
                    if (EPI == EPI_RESID) {
                        const __nv_bfloat16* src = g.resid_src;
                        if (g.resid_index) src += (size_t)(*g.resid_index) * g.N;
                        else if (g.resid_key) src += (size_t)key_index(*g.resid_key) * g.N;
                        g.y[n] = f2bf(__fadd_rn(bf2f(src[n]), bf2f(yb)));
                    } else {
                        g.y[n] = yb;
                    }
                    if (EPI == EPI_ARGMAX) {
                        /* order-preserving key: larger value first, then lower index
                         * (src/slowar/kernels.cu:1326-1357); -0 counts as +0 */
                        uint32_t u = __float_as_uint(bf2f(yb));
                        if (u == 0x80000000u) u = 0u;
                        u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
                        const unsigned long long key = ((unsigned long long)u << 32) | (0xFFFFFFFFu - (uint32_t)n);
                        best = key > best ? key : best;
                    }
                }
            }
        }
        __syncthreads(); /* partials and scales are overwritten by the next pass */
    }
    if (EPI == EPI_ARGMAX && lane == 0 && best) atomicMax(g.argmax_key, best);
}

}  // namespace s2p
