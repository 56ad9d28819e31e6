/* Weight-streaming dequant GEMV for batch-1 decode, as a device-side stage
 * that the stand-alone launchers (gemv.cu), the fused per-stage tick (tick.cu)
 * and the persistent tick kernel (mega.cu) all instantiate.
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
 * Mapping to B200 (what is NOT the reference's):
 *  - the unit of work is one (row, K-tile) pair; the units of a CTA's row block
 *    are laid out tile-major and cut into 16 equal contiguous ranges, one per
 *    warp, so a 2560-row matrix loads all 148 x 16 warps evenly; per-tile
 *    partials cross warps through shared memory and one warp per row folds
 *    them in the fixed order;
 *  - INT4: a packed word becomes four bf16x2 registers with one shift and one
 *    logic op each (nibble | 0x4300 = 128 + code) and one packed bf16
 *    subtraction of 136; the products run on the mixed-precision fma of sm_100
 *    (fma.rn.f32.bf16: bf16 x bf16 exact product, f32 accumulate), which is
 *    bit-identical to fmaf((float)w, (float)x, s) because codes and
 *    activations are exactly representable in bf16.  Measured 3.25
 *    instructions per weight against 3.9 for byte-permute + packed f32x2 fma
 *    and 4.7 for the scalar int->float route;
 *  - INT8: byte-permute into the mantissa of 2^23, one exact subtraction, f32 fma;
 *  - the activation vector is staged once per CTA in shared memory in the lane
 *    order the units read it (bf16 pairs for INT4, f32 for INT8);
 *  - activations, residuals and indices written by other SMs are read with
 *    L1-bypassing loads, so the same code is correct inside a persistent kernel.
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
    __nv_bfloat16* normed_out;        /* PRO_NORM, optional: CTA 0 also writes the normalised vector here */
    int rows_per_pass;                /* rows (row pairs for EPI_SWIGLU) the shared partial buffer holds */
};

constexpr int GEMV_THREADS = 512;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;
constexpr int GEMV_GROUP = 4; /* units a warp keeps in flight together */

__host__ __device__ inline size_t gemv_x_bytes(int wk, int K) { return (size_t)K * (wk == WK_INT4_PACK ? 2 : 4); }

__host__ __device__ inline size_t gemv_smem_bytes(int wk, int rows_local, int K, int gshift) {
    const int T = K / 512;
    size_t b = gemv_x_bytes(wk, K);
    b += (size_t)rows_local * T * 32 * sizeof(float);   /* per-tile lane partials */
    if (wk != WK_INT8_CH) b += ((size_t)rows_local * (K >> gshift) * 2 + 15) & ~(size_t)15;
    return b + 2048 /* reduction scratch */;
}

/* index held in a packed arg-max key (see EPI_ARGMAX) */
__device__ __forceinline__ uint32_t key_index(unsigned long long key) { return 0xFFFFFFFFu - (uint32_t)key; }

/* L1-bypassing loads for data other SMs may have written during this kernel */
__device__ __forceinline__ float ldcg_bf16(const __nv_bfloat16* p) {
    return bf_bits_to_f32(__ldcg(reinterpret_cast<const unsigned short*>(p)));
}

/* mixed-precision fma: s + w * x with bf16 w, x (exact product), f32 s, one rounding */
__device__ __forceinline__ float fma_bf16(unsigned short w, unsigned short x, float s) {
    asm("fma.rn.f32.bf16 %0, %1, %2, %0;" : "+f"(s) : "h"(w), "h"(x));
    return s;
}

/* 8 packed nibbles (weights j = 0..7 of a half tile) against 8 bf16 activations */
__device__ __forceinline__ void chain_int4_word(uint32_t w, const unsigned short* xh, float& s) {
    const uint32_t a = w ^ 0x88888888u; /* two's complement nibble -> code + 8 */
    unsigned short lo[4], hi[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        uint32_t m = ((a >> (4 * k)) & 0x000F000Fu) | 0x43004300u; /* bf16x2 (128 + n_k, 128 + n_{k+4}) */
        __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&m);
        const uint32_t c = 0x43084308u;                            /* (136, 136) */
        h = __hsub2(h, *reinterpret_cast<const __nv_bfloat162*>(&c));
        const uint32_t p = *reinterpret_cast<uint32_t*>(&h);
        asm("mov.b32 {%0,%1}, %2;" : "=h"(lo[k]), "=h"(hi[k]) : "r"(p));
    }
#pragma unroll
    for (int j = 0; j < 4; j++) s = fma_bf16(lo[j], xh[j], s);
#pragma unroll
    for (int j = 0; j < 4; j++) s = fma_bf16(hi[j], xh[4 + j], s);
}

/* 4 int8 codes (weights j = 0..3 of a quarter tile) against 4 f32 activations */
__device__ __forceinline__ void chain_int8_word(uint32_t w, const float4& xv, float& s) {
    const uint32_t a = w ^ 0x80808080u;
    const float bias = 8388736.0f; /* 2^23 + 128 */
    s = __fmaf_rn(__uint_as_float(__byte_perm(a, 0x4B000000u, 0x7540u)) - bias, xv.x, s);
    s = __fmaf_rn(__uint_as_float(__byte_perm(a, 0x4B000000u, 0x7541u)) - bias, xv.y, s);
    s = __fmaf_rn(__uint_as_float(__byte_perm(a, 0x4B000000u, 0x7542u)) - bias, xv.z, s);
    s = __fmaf_rn(__uint_as_float(__byte_perm(a, 0x4B000000u, 0x7543u)) - bias, xv.w, s);
}

template <int WK> struct LaneTile;  /* the bytes one lane owns of one (row, tile) unit */
template <> struct LaneTile<WK_INT4_PACK> { typedef uint2 type; };
template <> struct LaneTile<WK_INT8_CH> { typedef uint4 type; };
template <> struct LaneTile<WK_INT8_GRP> { typedef uint4 type; };

/* The activations one lane needs for one tile, held in registers while the warp
 * walks the rows of that tile. */
template <int WK> struct LaneX;
template <> struct LaneX<WK_INT4_PACK> {
    unsigned short h[16];
    __device__ __forceinline__ void load(const unsigned char* xs, int tile, int lane) {
        const uint4* p = reinterpret_cast<const uint4*>(xs);
        const uint4 a = p[(tile * 2) * 32 + lane], b = p[(tile * 2 + 1) * 32 + lane];
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; i++) asm("mov.b32 {%0,%1}, %2;" : "=h"(h[2 * i]), "=h"(h[2 * i + 1]) : "r"(w[i]));
    }
    __device__ __forceinline__ float unit(const uint2& t) const {
        float s = 0.f;
        chain_int4_word(t.x, h, s);
        chain_int4_word(t.y, h + 8, s);
        return s;
    }
};
template <> struct LaneX<WK_INT8_CH> {
    float4 v[4];
    __device__ __forceinline__ void load(const unsigned char* xs, int tile, int lane) {
        const float4* p = reinterpret_cast<const float4*>(xs);
#pragma unroll
        for (int q = 0; q < 4; q++) v[q] = p[(tile * 4 + q) * 32 + lane];
    }
    __device__ __forceinline__ float unit(const uint4& t) const {
        float s = 0.f;
        chain_int8_word(t.x, v[0], s);
        chain_int8_word(t.y, v[1], s);
        chain_int8_word(t.z, v[2], s);
        chain_int8_word(t.w, v[3], s);
        return s;
    }
};
template <> struct LaneX<WK_INT8_GRP> : LaneX<WK_INT8_CH> {};

/* ---- the staged activation vector -------------------------------------------
 * Element k = 512 i + 16 l + j sits where lane l reads it for tile i: INT4 keeps
 * bf16, eight to a uint4 at index (i*2 + (j>>3))*32 + l; INT8 keeps f32, four to a
 * float4 at index (i*4 + (j>>2))*32 + l.  Eight consecutive k (one 16-byte vector
 * of the source) therefore land in one uint4 or two float4. */

template <int WK>
__device__ __forceinline__ void xs_store_vec8(unsigned char* xs, int v, const uint4& q) {
    const int i = v >> 6, l = (v >> 1) & 31, h = v & 1;
    if (WK == WK_INT4_PACK) {
        reinterpret_cast<uint4*>(xs)[(i * 2 + h) * 32 + l] = q;
    } else {
        float4* p = reinterpret_cast<float4*>(xs) + (i * 4 + h * 2) * 32 + l;
        p[0] = make_float4(bf_lo(q.x), bf_hi(q.x), bf_lo(q.y), bf_hi(q.y));
        p[32] = make_float4(bf_lo(q.z), bf_hi(q.z), bf_lo(q.w), bf_hi(q.w));
    }
}
/* one element into the staged layout */
template <int WK>
__device__ __forceinline__ void xs_store(unsigned char* xs, int k, __nv_bfloat16 v) {
    const int i = k >> 9, l = (k >> 4) & 31, j = k & 15;
    if (WK == WK_INT4_PACK)
        reinterpret_cast<__nv_bfloat16*>(xs)[(((i * 2 + (j >> 3)) * 32 + l) << 3) + (j & 7)] = v;
    else
        reinterpret_cast<float*>(xs)[(((i * 4 + (j >> 2)) * 32 + l) << 2) + (j & 3)] = bf2f(v);
}
template <int WK>
__device__ __forceinline__ float xs_load(const unsigned char* xs, int k) {
    const int i = k >> 9, l = (k >> 4) & 31, j = k & 15;
    if (WK == WK_INT4_PACK)
        return bf_bits_to_f32(reinterpret_cast<const unsigned short*>(xs)[(((i * 2 + (j >> 3)) * 32 + l) << 3) + (j & 7)]);
    return reinterpret_cast<const float*>(xs)[(((i * 4 + (j >> 2)) * 32 + l) << 2) + (j & 3)];
}

/* ---- prologue: stage the activation vector -------------------------------
 * `nthreads` threads (threadIdx.x < nthreads, a multiple of 32, >= 256) call this
 * together.  x, norm_w and normed_out must be 16-byte aligned.  `red`: 257 floats. */
__device__ __forceinline__ uint4 norm_vec8(const uint4& xq, const uint4& wq, float inv) {
    const uint32_t xw[4] = {xq.x, xq.y, xq.z, xq.w};
    const uint32_t ww[4] = {wq.x, wq.y, wq.z, wq.w};
    uint32_t o[4];
#pragma unroll
    for (int c = 0; c < 4; c++) {
        const __nv_bfloat16 lo = f2bf(__fmul_rn(__fmul_rn(bf_lo(xw[c]), inv), bf_lo(ww[c])));
        const __nv_bfloat16 hi = f2bf(__fmul_rn(__fmul_rn(bf_hi(xw[c]), inv), bf_hi(ww[c])));
        o[c] = (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

/* barrier over the threads that stage the activation: the whole CTA unless the caller passes its own */
struct CtaSyncFn {
    __device__ __forceinline__ void operator()() const { S2P_CTA_SYNC(); }
};

/* `load(v)` returns the eight consecutive bf16 activations 8v .. 8v+7 as a uint4; `sync` is a barrier
 * over exactly the `nthreads` calling threads */
template <int WK, int PRO, class LoadVec, class SyncFn = CtaSyncFn>
__device__ __forceinline__ void stage_activation_from(const GemvStage& g, LoadVec load, unsigned char* xs, float* red,
                                                      int nthreads, SyncFn sync = SyncFn()) {
    const int K = g.K, NVEC = K >> 3;
    const uint4* wsrc = reinterpret_cast<const uint4*>(g.norm_w);
    /* the first two vectors of a thread stay in registers for the normalisation (the model's
     * normed widths need no more with 256 threads), and their gains are fetched before the
     * activations, which may have to be waited for */
    const int v0 = threadIdx.x, v1 = threadIdx.x + nthreads;
    uint4 x0 = make_uint4(0, 0, 0, 0), w0 = x0, x1 = x0, w1 = x0;
    if (PRO == PRO_NORM) {
        if (v0 < NVEC) w0 = wsrc[v0];
        if (v1 < NVEC) w1 = wsrc[v1];
    }
    if (v0 < NVEC) {
        x0 = load(v0);
        xs_store_vec8<WK>(xs, v0, x0);
    }
    if (v1 < NVEC) {
        x1 = load(v1);
        xs_store_vec8<WK>(xs, v1, x1);
    }
    for (int v = v1 + nthreads; v < NVEC; v += nthreads) xs_store_vec8<WK>(xs, v, load(v));
    if (PRO == PRO_VEC) return;
    sync();
    /* 256 strided partial sums of squares, halving tree, rsqrtf(mean + eps):
     * src/slowar/kernels.cu:46-68 */
    float ss = 0.f;
    if (threadIdx.x < 256)
        for (int i = threadIdx.x; i < K; i += 256) {
            const float v = xs_load<WK>(xs, i);
            ss = __fmaf_rn(v, v, ss);
        }
    const float tot = tree256_sum(ss, red, sync); /* its first barrier also orders the reads above before the rewrite below */
    const float inv = rsqrtf(__fdiv_rn(tot, (float)K) + g.eps);
    const bool emit = g.normed_out != nullptr && blockIdx.x == 0;
    if (v0 < NVEC) {
        const uint4 q = norm_vec8(x0, w0, inv);
        xs_store_vec8<WK>(xs, v0, q);
        if (emit) reinterpret_cast<uint4*>(g.normed_out)[v0] = q;
    }
    if (v1 < NVEC) {
        const uint4 q = norm_vec8(x1, w1, inv);
        xs_store_vec8<WK>(xs, v1, q);
        if (emit) reinterpret_cast<uint4*>(g.normed_out)[v1] = q;
    }
    for (int v = v1 + nthreads; v < NVEC; v += nthreads) {
        const uint4 q = norm_vec8(load(v), wsrc[v], inv);
        xs_store_vec8<WK>(xs, v, q);
        if (emit) reinterpret_cast<uint4*>(g.normed_out)[v] = q;
    }
}

template <int WK, int PRO>
__device__ __forceinline__ void stage_activation(const GemvStage& g, unsigned char* xs, float* red, int nthreads) {
    const __nv_bfloat16* x = g.x;
    if (g.x_index) x += (size_t)__ldcg(g.x_index) * g.K;
    else if (g.x_key) x += (size_t)key_index(__ldcg(g.x_key)) * g.K;
    const uint4* xsrc = reinterpret_cast<const uint4*>(x);
    stage_activation_from<WK, PRO>(g, [xsrc](int v) { return __ldcg(xsrc + v); }, xs, red, nthreads);
}

/* ---- the stage ------------------------------------------------------------
 * Rows [row0, row0+cnt_total) of the matrix belong to this CTA; with EPI_SWIGLU
 * the CTA owns gate rows [row0, ..) and up rows [F+row0, ..), F = N/2.  The rows
 * are walked in passes of at most g.rows_per_pass (what the partial buffer in
 * shared memory holds).  smem: dynamic shared memory base, sized by
 * gemv_smem_bytes(wk, rows_per_pass * (swiglu ? 2 : 1), K, gshift).
 * All threads of the CTA (GEMV_THREADS) must call this. */
template <int WK, int PRO, int EPI>
__device__ void gemv_stage_cta(const GemvStage& g, int row0, int cnt_total, unsigned char* smem) {
    typedef typename LaneTile<WK>::type tile_t;
    constexpr int SW = (EPI == EPI_SWIGLU) ? 2 : 1;
    constexpr int R = GEMV_GROUP;
    if (cnt_total <= 0) return; /* uniform over the CTA */
    const int K = g.K, T = K >> 9;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int F = g.N >> 1;
    const size_t row_bytes = (WK == WK_INT4_PACK) ? (size_t)(K >> 1) : (size_t)K;
    const int sc_per_row = (WK == WK_INT8_CH) ? 1 : (K >> g.gshift);
    const int cap_rows = g.rows_per_pass * SW;

    unsigned char* xs = smem;
    float* part = reinterpret_cast<float*>(smem + ((gemv_x_bytes(WK, K) + 15) & ~(size_t)15));
    __half* sc_s = reinterpret_cast<__half*>(part + (size_t)cap_rows * T * 32);
    float* red = reinterpret_cast<float*>(
        reinterpret_cast<unsigned char*>(sc_s) +
        ((WK == WK_INT8_CH) ? 0 : (((size_t)cap_rows * sc_per_row * 2 + 15) & ~(size_t)15)));
    const unsigned char* wbase = static_cast<const unsigned char*>(g.w) + (size_t)lane * sizeof(tile_t);
    unsigned long long best = 0ull;

    for (int done = 0; done < cnt_total; done += g.rows_per_pass) {
        const int cnt = min(g.rows_per_pass, cnt_total - done);
        const int r0 = row0 + done;
        const int local_rows = cnt * SW;
        auto global_row = [&](int lr) -> int {
            if (EPI == EPI_SWIGLU) return lr < cnt ? r0 + lr : F + r0 + (lr - cnt);
            return r0 + lr;
        };
        /* this warp's contiguous range of (tile-major) units */
        const int U = local_rows * T;
        int u = (int)((long long)U * warp / GEMV_WARPS);
        const int u_end = (int)((long long)U * (warp + 1) / GEMV_WARPS);
        int tile = u / local_rows, lr = u - tile * local_rows;

        /* a group = up to R consecutive rows of one tile */
        auto group_size = [&](int uu, int l) { return min(R, min(u_end - uu, local_rows - l)); };
        auto load_group = [&](int t, int l, int n, tile_t* buf) {
#pragma unroll
            for (int r = 0; r < R; r++)
                if (r < n)
                    buf[r] = *reinterpret_cast<const tile_t*>(wbase + (size_t)global_row(l + r) * row_bytes +
                                                              (size_t)t * (sizeof(tile_t) * 32));
        };
        tile_t cur[R], nxt[R];
        int n_cur = (u < u_end) ? group_size(u, lr) : 0;
        if (n_cur) load_group(tile, lr, n_cur, cur); /* weights do not depend on the activations: first */
        if constexpr (WK != WK_INT8_CH) {
            const __half* sg = static_cast<const __half*>(g.scales);
            for (int idx = threadIdx.x; idx < local_rows * sc_per_row; idx += blockDim.x) {
                const int l = idx / sc_per_row, c = idx - l * sc_per_row;
                sc_s[idx] = sg[(size_t)global_row(l) * sc_per_row + c];
            }
        }
        if (done == 0) stage_activation<WK, PRO>(g, xs, red, GEMV_THREADS);
        S2P_CTA_SYNC();

        LaneX<WK> lx;
        int x_tile = -1;
        while (n_cur) {
            /* next group: same tile while rows remain, else the first rows of the next tile */
            int u2 = u + n_cur, lr2 = lr + n_cur, tile2 = tile;
            if (lr2 == local_rows) { lr2 = 0; tile2++; }
            const int n_nxt = (u2 < u_end) ? group_size(u2, lr2) : 0;
            if (n_nxt) load_group(tile2, lr2, n_nxt, nxt);
            if (tile != x_tile) { lx.load(xs, tile, lane); x_tile = tile; }
#pragma unroll
            for (int r = 0; r < R; r++)
                if (r < n_cur) part[((size_t)(lr + r) * T + tile) * 32 + lane] = lx.unit(cur[r]);
#pragma unroll
            for (int r = 0; r < R; r++) cur[r] = nxt[r];
            u = u2; lr = lr2; tile = tile2; n_cur = n_nxt;
        }
        S2P_CTA_SYNC();

        /* fold the tiles of one row in ascending order, merge lanes, finish */
        auto fold_row = [&](int l) -> float {
            float acc = 0.f;
            const float* pr = part + (size_t)l * T * 32 + lane;
            if (WK == WK_INT8_CH) {
                for (int i = 0; i < T; i++) acc += pr[i * 32];
            } else {
                const __half* sr = sc_s + (size_t)l * sc_per_row;
                for (int i = 0; i < T; i++)
                    acc = __fmaf_rn(pr[i * 32], __half2float(sr[(i * 512 + lane * 16) >> g.gshift]), acc);
            }
            acc = warp_tree_sum(acc);
            if (WK == WK_INT8_CH) acc = __fmul_rn(acc, static_cast<const float*>(g.scales)[global_row(l)]);
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
                        if (g.resid_index) src += (size_t)__ldcg(g.resid_index) * g.N;
                        else if (g.resid_key) src += (size_t)key_index(__ldcg(g.resid_key)) * g.N;
                        g.y[n] = f2bf(__fadd_rn(ldcg_bf16(src + n), bf2f(yb)));
                    } else {
                        g.y[n] = yb;
                    }
                    if (EPI == EPI_ARGMAX) {
                        /* order-preserving key: larger value first, then lower index
                         * (src/slowar/kernels.cu:1326-1357); -0 counts as +0 */
                        uint32_t uu = __float_as_uint(bf2f(yb));
                        if (uu == 0x80000000u) uu = 0u;
                        uu = (uu & 0x80000000u) ? ~uu : (uu | 0x80000000u);
                        const unsigned long long key = ((unsigned long long)uu << 32) | (0xFFFFFFFFu - (uint32_t)n);
                        best = key > best ? key : best;
                    }
                }
            }
        }
        S2P_CTA_SYNC(); /* partials and scales are overwritten by the next pass */
    }
    if (EPI == EPI_ARGMAX && lane == 0 && best) atomicMax(g.argmax_key, best);
}

/* rows of the stage owned by CTA `cta` of `n_cta` */
template <int EPI>
__device__ __forceinline__ void gemv_cta_rows(const GemvStage& g, int cta, int n_cta, int& row0, int& cnt) {
    const int units = (EPI == EPI_SWIGLU) ? (g.N >> 1) : g.N;
    row0 = (int)((long long)units * cta / n_cta);
    cnt = (int)((long long)units * (cta + 1) / n_cta) - row0;
}

}  // namespace s2p
