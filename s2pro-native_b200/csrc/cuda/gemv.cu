/* Stand-alone GEMV entry points of the C ABI (include/s2p_b200_abi.h):
 * s2p_int8_gemv, s2p_intq_gemv, s2p_int4p_gemv — the reference's
 * src/sched/int8_gemv.cu:964-986, :773-799, :836-902.
 *
 * M == 1 runs the batch-1 streaming stage of gemv.cuh.  2 <= M <= 16 runs the
 * exact-order small-batch kernel below: every row of x is an independent
 * product with the same summation order as M == 1 (the reference's batched
 * GEMV computes rows independently, int8_gemv.cu:77-91), codes are widened
 * once per tile and reused for all M rows.
 */
#include <stdio.h>
#include "gemv.cuh"
#include "s2p_b200_abi.h"

namespace s2p {

int device_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int WK, int PRO, int EPI>
__global__ void __launch_bounds__(GEMV_THREADS, 1) k_gemv_stage(GemvStage g) {
    extern __shared__ __align__(16) unsigned char smem[];
    int row0, cnt;
    gemv_cta_rows<EPI>(g, blockIdx.x, gridDim.x, row0, cnt);
    gemv_stage_cta<WK, PRO, EPI>(g, row0, cnt, smem);
}

/* Rows per pass that keep the CTA's shared memory within `limit` bytes. */
int gemv_rows_per_pass(int wk, int rows_per_cta, int K, int gshift, int swiglu, size_t limit) {
    int r = rows_per_cta;
    while (r > 8 && gemv_smem_bytes(wk, r * (swiglu ? 2 : 1), K, gshift) > limit) r = (r + 1) / 2;
    return r < 1 ? 1 : r;
}

constexpr size_t GEMV_SMEM_LIMIT = 200 * 1024;

/* Opt the kernel in to large dynamic shared memory, once per device. */
template <int WK, int PRO, int EPI>
cudaError_t gemv_stage_setup() {
    static int done_mask = 0; /* bit per device ordinal */
    int dev = 0;
    cudaGetDevice(&dev);
    if (done_mask & (1 << (dev & 31))) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(k_gemv_stage<WK, PRO, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)GEMV_SMEM_LIMIT);
    if (e == cudaSuccess) done_mask |= 1 << (dev & 31);
    return e;
}

template <int WK, int PRO, int EPI>
cudaError_t launch_gemv_stage(GemvStage g, cudaStream_t stream) {
    const size_t limit = GEMV_SMEM_LIMIT;
    {
        const cudaError_t e = gemv_stage_setup<WK, PRO, EPI>();
        if (e != cudaSuccess) return e;
    }
    const int units = (EPI == EPI_SWIGLU) ? (g.N >> 1) : g.N;
    int grid = device_sm_count();
    if (grid > units) grid = units;
    const int rows_per_cta = (units + grid - 1) / grid;
    g.rows_per_pass = gemv_rows_per_pass(WK, rows_per_cta, g.K, g.gshift, EPI == EPI_SWIGLU, limit);
    const size_t smem = gemv_smem_bytes(WK, g.rows_per_pass * (EPI == EPI_SWIGLU ? 2 : 1), g.K, g.gshift);
    k_gemv_stage<WK, PRO, EPI><<<grid, GEMV_THREADS, smem, stream>>>(g);
    return cudaGetLastError();
}

/* instantiations used by the tick live here so that every kernel is compiled once */
template cudaError_t launch_gemv_stage<WK_INT8_CH, PRO_VEC, EPI_STORE>(GemvStage, cudaStream_t);
template cudaError_t launch_gemv_stage<WK_INT8_GRP, PRO_VEC, EPI_STORE>(GemvStage, cudaStream_t);
template cudaError_t launch_gemv_stage<WK_INT4_PACK, PRO_VEC, EPI_STORE>(GemvStage, cudaStream_t);
#define S2P_INST(WK)                                                                         \
    template cudaError_t launch_gemv_stage<WK, PRO_NORM, EPI_STORE>(GemvStage, cudaStream_t); \
    template cudaError_t launch_gemv_stage<WK, PRO_VEC, EPI_RESID>(GemvStage, cudaStream_t);  \
    template cudaError_t launch_gemv_stage<WK, PRO_NORM, EPI_SWIGLU>(GemvStage, cudaStream_t);\
    template cudaError_t launch_gemv_stage<WK, PRO_NORM, EPI_ARGMAX>(GemvStage, cudaStream_t);
S2P_INST(WK_INT8_CH)
S2P_INST(WK_INT8_GRP)
S2P_INST(WK_INT4_PACK)
#undef S2P_INST

/* Attribute set-up for every instantiation, to be called once before any stream
 * capture (function attributes are not stream operations). */
extern "C" cudaError_t gemv_setup_all(void) {
    cudaError_t e = cudaSuccess;
#define S2P_SETUP(WK, PRO, EPI) if (e == cudaSuccess) e = gemv_stage_setup<WK, PRO, EPI>();
#define S2P_SETUP_WK(WK)               \
    S2P_SETUP(WK, PRO_VEC, EPI_STORE)  \
    S2P_SETUP(WK, PRO_NORM, EPI_STORE) \
    S2P_SETUP(WK, PRO_VEC, EPI_RESID)  \
    S2P_SETUP(WK, PRO_NORM, EPI_SWIGLU) \
    S2P_SETUP(WK, PRO_NORM, EPI_ARGMAX)
    S2P_SETUP_WK(WK_INT8_CH)
    S2P_SETUP_WK(WK_INT8_GRP)
    S2P_SETUP_WK(WK_INT4_PACK)
#undef S2P_SETUP_WK
#undef S2P_SETUP
    return e;
}

/* ---- exact-order small batch (2 <= M <= 16) -------------------------------
 * One warp per output row; lane l owns k = 512 i + 16 l .. +15.  The 16 codes
 * of a tile are widened once, then each of the M activation rows runs its own
 * 16-term fma chain and tile fold, exactly as for M == 1. */
template <int WK>
__device__ __forceinline__ void widen16(const typename LaneTile<WK>::type& t, float* w16);
template <>
__device__ __forceinline__ void widen16<WK_INT4_PACK>(const uint2& t, float* w16) {
    const uint32_t u[2] = {t.x ^ 0x88888888u, t.y ^ 0x88888888u};
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const uint32_t e = u[h] & 0x0F0F0F0Fu, o = (u[h] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            w16[h * 8 + 2 * b] = biased_byte_to_f32(e, b, 8388616.0f);
            w16[h * 8 + 2 * b + 1] = biased_byte_to_f32(o, b, 8388616.0f);
        }
    }
}
template <>
__device__ __forceinline__ void widen16<WK_INT8_CH>(const uint4& t, float* w16) {
    const uint32_t u[4] = {t.x ^ 0x80808080u, t.y ^ 0x80808080u, t.z ^ 0x80808080u, t.w ^ 0x80808080u};
#pragma unroll
    for (int h = 0; h < 4; h++)
#pragma unroll
        for (int b = 0; b < 4; b++) w16[h * 4 + b] = biased_byte_to_f32(u[h], b, 8388736.0f);
}
template <>
__device__ __forceinline__ void widen16<WK_INT8_GRP>(const uint4& t, float* w16) { widen16<WK_INT8_CH>(t, w16); }

template <int WK, int MM>
__global__ void __launch_bounds__(256) k_gemv_batch(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ x,
                                                    const void* __restrict__ w, const void* __restrict__ scales,
                                                    int M, int N, int K, int gshift) {
    typedef typename LaneTile<WK>::type tile_t;
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const size_t row_bytes = (WK == WK_INT4_PACK) ? (size_t)(K >> 1) : (size_t)K;
    const int T = K >> 9;
    /* the grid's y dimension walks groups of MM activation rows (see k_gemv_batch_i4) */
    x += (size_t)blockIdx.y * MM * K;
    y += (size_t)blockIdx.y * MM * N;
    M = min(MM, M - (int)blockIdx.y * MM);
    for (int n = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; n < N; n += warps) {
        const unsigned char* wrow = static_cast<const unsigned char*>(w) + (size_t)n * row_bytes;
        float acc[MM];
#pragma unroll
        for (int m = 0; m < MM; m++) acc[m] = 0.f;
        tile_t nxt = *reinterpret_cast<const tile_t*>(wrow + (size_t)lane * sizeof(tile_t));
        for (int i = 0; i < T; i++) {
            const tile_t cur = nxt;
            if (i + 1 < T)
                nxt = *reinterpret_cast<const tile_t*>(wrow + (size_t)(i + 1) * 32 * sizeof(tile_t) +
                                                       (size_t)lane * sizeof(tile_t));
            const int k0 = i * 512 + lane * 16;
            float gs = 1.f;
            if (WK != WK_INT8_CH)
                gs = __half2float(static_cast<const __half*>(scales)[(size_t)n * (K >> gshift) + (k0 >> gshift)]);
            float w16[16];
            widen16<WK>(cur, w16);
#pragma unroll
            for (int m = 0; m < MM; m++) {
                if (m < M) {
                    const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)m * K + k0);
                    const uint4 xa = xp[0], xb = xp[1];
                    const uint32_t xu[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
                    float s = 0.f;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        s = __fmaf_rn(w16[2 * j], bf_bits_to_f32(xu[j] & 0xffffu), s);
                        s = __fmaf_rn(w16[2 * j + 1], __uint_as_float(xu[j] & 0xffff0000u), s);
                    }
                    if (WK == WK_INT8_CH) acc[m] += s;
                    else acc[m] = __fmaf_rn(s, gs, acc[m]);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MM; m++) {
            float a = warp_tree_sum(acc[m]);
            if (WK == WK_INT8_CH) a = __fmul_rn(a, static_cast<const float*>(scales)[n]);
            if (lane == 0 && m < M) y[(size_t)m * N + n] = f2bf(a);
        }
    }
}

/* The same for packed INT4, R weight rows per warp: the 16 codes of each row's tile become bf16 once
 * (exact), an activation row's 16 values are loaded once for the R rows, and every (row, activation row)
 * pair runs its own chain of mixed-precision fmas (bf16 x bf16 exact, f32 accumulate: bit for bit
 * fmaf((float)w, (float)x, s)).  Loading the activations once per R rows is what matters: a lockstep
 * batch reads M x 32 bytes per lane and tile, which otherwise bounds the kernel by L1 bandwidth. */
template <int MM, int R>
__global__ void __launch_bounds__(256) k_gemv_batch_i4(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ x,
                                                       const unsigned char* __restrict__ w, const __half* __restrict__ scales,
                                                       int M, int N, int K, int gshift) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const size_t row_bytes = (size_t)(K >> 1);
    const int T = K >> 9, spr = K >> gshift;
    /* the grid's y dimension walks groups of MM activation rows: a matrix of few rows gets enough warps that way
     * while every warp still carries R weight rows per activation load (each (m, n) chain is untouched by it) */
    x += (size_t)blockIdx.y * MM * K;
    y += (size_t)blockIdx.y * MM * N;
    M = min(MM, M - (int)blockIdx.y * MM);
    for (int n0 = ((blockIdx.x * blockDim.x + threadIdx.x) >> 5) * R; n0 < N; n0 += warps * R) {
        const unsigned char* wrow[R];
        const __half* srow[R];
#pragma unroll
        for (int r = 0; r < R; r++) { /* rows beyond N repeat row N - 1 and are not stored */
            const int n = min(n0 + r, N - 1);
            wrow[r] = w + (size_t)n * row_bytes + (size_t)lane * sizeof(uint2);
            srow[r] = scales + (size_t)n * spr;
        }
        float acc[R][MM];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int m = 0; m < MM; m++) acc[r][m] = 0.f;
        /* each row's next PD tiles are in registers: with few warps per SM the loads of one tile ahead
         * would leave the weight stream bound by DRAM latency */
        constexpr int PD = 4;
        uint2 pf[R][PD];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int d = 0; d < PD; d++)
                pf[r][d] = d < T ? *reinterpret_cast<const uint2*>(wrow[r] + (size_t)d * 32 * sizeof(uint2)) : make_uint2(0, 0);
        for (int i0 = 0; i0 < T; i0 += PD) {
#pragma unroll
          for (int d = 0; d < PD; d++) {
            const int i = i0 + d;
            if (i >= T) break;
            const int k0 = i * 512 + lane * 16;
            unsigned short wl[R][16];
            float gs[R];
#pragma unroll
            for (int r = 0; r < R; r++) {
                const uint2 cur = pf[r][d];
                if (i + PD < T) pf[r][d] = *reinterpret_cast<const uint2*>(wrow[r] + (size_t)(i + PD) * 32 * sizeof(uint2));
                gs[r] = __half2float(srow[r][k0 >> gshift]);
                const uint32_t tw[2] = {cur.x, cur.y};
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const uint32_t a = tw[h] ^ 0x88888888u; /* two's complement nibble -> code + 8 */
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        uint32_t mg = ((a >> (4 * k)) & 0x000F000Fu) | 0x43004300u; /* bf16x2 (128 + n_k, 128 + n_{k+4}) */
                        __nv_bfloat162 hv = *reinterpret_cast<__nv_bfloat162*>(&mg);
                        const uint32_t c136 = 0x43084308u;
                        hv = __hsub2(hv, *reinterpret_cast<const __nv_bfloat162*>(&c136));
                        const uint32_t pr = *reinterpret_cast<uint32_t*>(&hv);
                        asm("mov.b32 {%0,%1}, %2;" : "=h"(wl[r][h * 8 + k]), "=h"(wl[r][h * 8 + 4 + k]) : "r"(pr));
                    }
                }
            }
#pragma unroll
            for (int m = 0; m < MM; m++) {
                if (m < M) {
                    const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)m * K + k0);
                    const uint4 xa = xp[0], xb = xp[1];
                    const uint32_t xu[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
                    unsigned short xh[16];
#pragma unroll
                    for (int j = 0; j < 8; j++) asm("mov.b32 {%0,%1}, %2;" : "=h"(xh[2 * j]), "=h"(xh[2 * j + 1]) : "r"(xu[j]));
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        float sm_ = 0.f;
#pragma unroll
                        for (int j = 0; j < 16; j++) sm_ = fma_bf16(wl[r][j], xh[j], sm_);
                        acc[r][m] = __fmaf_rn(sm_, gs[r], acc[r][m]);
                    }
                }
            }
          }
        }
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int m = 0; m < MM; m++) {
                const float a = warp_tree_sum(acc[r][m]);
                if (lane == 0 && m < M && n0 + r < N) y[(size_t)m * N + n0 + r] = f2bf(a);
            }
    }
}

template <int WK>
cudaError_t launch_gemv_batch(void* y, const void* x, const void* w, const void* scales, int M, int N, int K,
                              int gshift, cudaStream_t stream) {
    const int cap = device_sm_count() * 8;
    if (WK == WK_INT4_PACK) { /* two or four weight rows per warp, 8 warps per CTA */
#define S2P_GB4(MM, R)                                                                                     \
    do {                                                                                                   \
        int g4 = (N + 8 * R - 1) / (8 * R);                                                                \
        if (g4 > cap) g4 = cap;                                                                            \
        k_gemv_batch_i4<MM, R><<<dim3((unsigned)g4, (unsigned)((M + MM - 1) / MM)), 256, 0, stream>>>(     \
            (__nv_bfloat16*)y, (const __nv_bfloat16*)x, (const unsigned char*)w, (const __half*)scales, M, N, K, gshift); \
    } while (0)
        /* A warp carries R weight rows and a group of MM activation rows: R x MM x 16 fmas per tile against MM
         * 32-byte activation loads per lane, so R is what keeps the kernel off the L1 bandwidth bound (R = 1: two
         * cycles of L1 per cycle of fma issue), and the accumulators (R x MM) are what decides how many warps an SM
         * holds: 8 rows x 4 rows is 158 registers (8 warps per SM), 4 x 4 is 128 (16 warps), 4 x 2 is 80.  Measured on
         * the lockstep tick: beyond 4 activation rows, groups of 4 over the grid's y dimension with R = 4 on the large
         * matrices and R = 2 on those of few rows (2560: twice the warps) beat 8-row groups by a quarter (batch 8:
         * 13.9 -> 10.6 ms per tick, batch 16: 23.0 -> 17.5).  With 4 rows or fewer the kernel is bound by latency and
         * warps count for more than reuse.  Per-row results do not depend on any of this. */
        const int sms = device_sm_count();
        const int ctas4 = (N + 31) / 32, ctas2 = (N + 15) / 16; /* CTAs of 8 warps at R = 4 / R = 2 */
        if (M <= 4) {
            const int R = ctas4 >= 2 * sms ? 4 : (ctas2 >= 2 * sms ? 2 : 1);
            if (M <= 2) { if (R == 4) S2P_GB4(2, 4); else if (R == 2) S2P_GB4(2, 2); else S2P_GB4(2, 1); }
            else { if (R == 4) S2P_GB4(4, 4); else if (R == 2) S2P_GB4(4, 2); else S2P_GB4(4, 1); }
        }
        else if (ctas4 >= sms) S2P_GB4(4, 4);
        else S2P_GB4(4, 2);
#undef S2P_GB4
        return cudaGetLastError();
    }
    int grid = (N + 7) / 8;
    if (grid > cap) grid = cap;
#define S2P_GB(MM)                                                                                      \
    k_gemv_batch<WK, MM><<<dim3((unsigned)grid, (unsigned)((M + MM - 1) / MM)), 256, 0, stream>>>(      \
        (__nv_bfloat16*)y, (const __nv_bfloat16*)x, w, scales, M, N, K, gshift)
    /* beyond four activation rows: groups of four over the grid's y dimension (twice to four times the warps at half
     * the registers; INT8 lockstep tick at 16 rows 34.7 -> 22.9 ms, at 8 rows 15.4 -> 13.9) */
    if (M <= 2) S2P_GB(2);
    else S2P_GB(4);
#undef S2P_GB
    return cudaGetLastError();
}

int gshift_of(int G) {
    if (G < 16 || (G & (G - 1))) return -1;
    int s = 0;
    while ((1 << s) < G) s++;
    return s;
}

template <int WK>
s2p_status gemv_entry(const char* what, void* y, const void* x, const void* w, const void* scales, int M, int N,
                      int K, int gshift, cudaStream_t stream) {
    /* 16-byte loads of activations and weight tiles */
    if (((uintptr_t)x | (uintptr_t)w) & 15) return S2P_ERR_INVALID;
    cudaError_t ce;
    if (M == 1) {
        GemvStage g = {};
        g.w = w; g.scales = scales; g.N = N; g.K = K; g.gshift = gshift;
        g.x = (const __nv_bfloat16*)x; g.y = (__nv_bfloat16*)y;
        ce = launch_gemv_stage<WK, PRO_VEC, EPI_STORE>(g, stream);
    } else {
        ce = launch_gemv_batch<WK>(y, x, w, scales, M, N, K, gshift, stream);
    }
    if (ce != cudaSuccess) {
        fprintf(stderr, "[s2pro] %s launch (M=%d,N=%d,K=%d): %s\n", what, M, N, K, cudaGetErrorString(ce));
        return S2P_ERR_CUDA;
    }
    return S2P_OK;
}

}  // namespace s2p

using namespace s2p;

extern "C" s2p_status s2p_int8_gemv(void* y_bf16, const void* x_bf16, const void* w_i8, const float* scales, int M,
                                    int N, int K, cudaStream_t stream) {
    if (!y_bf16 || !x_bf16 || !w_i8 || !scales || M <= 0 || N <= 0 || K <= 0) return S2P_ERR_INVALID;
    if (M > S2P_INT8_GEMV_MAX_M || K % 512 != 0) return S2P_ERR_INVALID;
    return gemv_entry<WK_INT8_CH>("int8 gemv", y_bf16, x_bf16, w_i8, scales, M, N, K, 0, stream);
}

extern "C" s2p_status s2p_intq_gemv(void* y_bf16, const void* x_bf16, const void* w_i8, const void* scales_f16,
                                    int M, int N, int K, int G, cudaStream_t stream) {
    if (!y_bf16 || !x_bf16 || !w_i8 || !scales_f16 || M <= 0 || N <= 0 || K <= 0) return S2P_ERR_INVALID;
    const int gs = gshift_of(G);
    if (M > S2P_INT8_GEMV_MAX_M || K % 512 != 0 || gs < 0 || K % G != 0) return S2P_ERR_INVALID;
    return gemv_entry<WK_INT8_GRP>("intq gemv", y_bf16, x_bf16, w_i8, scales_f16, M, N, K, gs, stream);
}

extern "C" s2p_status s2p_int4p_gemv(void* y_bf16, const void* x_bf16, const void* w_pack, const void* scales_f16,
                                     int M, int N, int K, int G, cudaStream_t stream) {
    if (!y_bf16 || !x_bf16 || !w_pack || !scales_f16 || M <= 0 || N <= 0 || K <= 0) return S2P_ERR_INVALID;
    const int gs = gshift_of(G);
    if (M > S2P_INT8_GEMV_MAX_M || K % 512 != 0 || gs < 0 || K % G != 0) return S2P_ERR_INVALID;
    return gemv_entry<WK_INT4_PACK>("int4p gemv", y_bf16, x_bf16, w_pack, scales_f16, M, N, K, gs, stream);
}
