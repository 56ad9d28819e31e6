/* Batched decode linear on the 5th-generation tensor cores: y[M, N] = x[M, K] · Wq^T for the
 * lockstep batches the exact-order GEMV cannot serve well (M > 16 rows; the reference's own
 * kernels stop at 16 rows, src/sched/int8_gemv.cu:964-986, so there is no bit-exact contract
 * beyond that: results agree with the exact path to f32-accumulation-order tolerance).
 *
 * One CTA owns 128 weight rows (the MMA's M; the batch is its N, padded to a multiple of 16):
 *   - all 256 threads dequantise a [128 rows x 128 k] slab of packed INT4 / INT8 codes into f16
 *     in shared memory (INT4: code x f16 group scale, one rounding of a 15-bit product; INT8
 *     per-channel: the exact code, the row scale is applied to the accumulator), in the
 *     K-major, unswizzled core-matrix layout the instruction reads: 16-byte units
 *     [k / 8][row], i.e. 8 rows x 16 B core matrices, 128 B apart along rows (SBO) and
 *     one [k/8] plane apart along K (LBO);
 *   - the activations (bf16 -> f16, exact in the normal range) go beside them as [k / 8][batch row];
 *   - one thread issues eight tcgen05.mma (M 128, N = padded batch, K 16, f16 x f16 -> f32 in
 *     TMEM) per slab and commits them to an mbarrier; two slabs are in flight, so the
 *     dequantisation of slab i+1 overlaps the MMAs of slab i;
 *   - epilogue: tcgen05.ld of the accumulator (lane = weight row, column = batch row), row
 *     scale, bf16, stores coalesced over weight rows.
 * Every mbarrier wait is bounded; on a time-out the kernel records a status code, skips the
 * epilogue, frees its TMEM and returns.
 */
#include <stdio.h>
#include "common.cuh"
#include "gemv.cuh"
#include "ops.h"
#include "pipe.cuh"
#include "s2p_b200_abi.h"

namespace s2p {

constexpr int SK_BM = 128;
constexpr int SK_KC = 128;
constexpr int SK_THREADS = 256;
constexpr int SK_A_BYTES = SK_BM * SK_KC * 2; /* 32 KB per stage */

/* 0 unless a bounded wait inside a launch gave up (read back by skinny_status) */
__device__ int g_sk_status;

__device__ __forceinline__ uint64_t sk_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    /* start address, leading (K) and stride (rows) byte offsets in 16-byte units; descriptor version 1;
     * base offset 0, no swizzle */
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}

/* 8 packed nibbles -> 8 f16 (code x scale) in ascending k, as one 16-byte unit */
__device__ __forceinline__ uint4 sk_int4_chunk(uint32_t w, __half2 sc2) {
    const uint32_t a = w ^ 0x88888888u;
    uint32_t p[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const uint32_t m = ((a >> (4 * k)) & 0x000F000Fu) | 0x64006400u; /* (1024 + n_k, 1024 + n_{k+4}) */
        const uint32_t c = 0x64086408u;                                  /* (1032, 1032) */
        __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&m), *reinterpret_cast<const __half2*>(&c));
        h = __hmul2(h, sc2);
        p[k] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(__byte_perm(p[0], p[1], 0x5410), __byte_perm(p[2], p[3], 0x5410), __byte_perm(p[0], p[1], 0x7632),
                      __byte_perm(p[2], p[3], 0x7632));
}
/* 8 int8 codes (two words) -> 8 f16, optionally x group scale */
template <bool SCALE>
__device__ __forceinline__ uint4 sk_int8_chunk(uint32_t w0, uint32_t w1, __half2 sc2) {
    const uint32_t c = 0x64806480u; /* (1152, 1152) = 1024 + 128 */
    uint32_t o[4];
    const uint32_t ws[2] = {w0 ^ 0x80808080u, w1 ^ 0x80808080u};
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const uint32_t lo = __byte_perm(ws[i], 0x64646464u, 0x4140), hi = __byte_perm(ws[i], 0x64646464u, 0x4342);
        __half2 hl = __hsub2(*reinterpret_cast<const __half2*>(&lo), *reinterpret_cast<const __half2*>(&c));
        __half2 hh = __hsub2(*reinterpret_cast<const __half2*>(&hi), *reinterpret_cast<const __half2*>(&c));
        if (SCALE) { hl = __hmul2(hl, sc2); hh = __hmul2(hh, sc2); }
        o[2 * i] = *reinterpret_cast<uint32_t*>(&hl);
        o[2 * i + 1] = *reinterpret_cast<uint32_t*>(&hh);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

template <int WK>
__global__ void __launch_bounds__(SK_THREADS, 2) k_skinny_tc(const void* __restrict__ w, const void* __restrict__ scales, int N,
                                                             int K, int gshift, const __nv_bfloat16* __restrict__ x, int M,
                                                             int NB, __nv_bfloat16* y, const __nv_bfloat16* resid,
                                                             float* __restrict__ partial, unsigned* __restrict__ arrivals) {
    /* resid (may alias y): y = bf16(f32(resid) + f32(bf16(product))), the residual add of the decode layers */
    /* gridDim.y > 1: the K range is split over gridDim.y CTAs per row tile; each leaves its f32 partial in
     * `partial`[split][batch row][weight row] and the last one to arrive adds them in split order */
    int* status = &g_sk_status;
    extern __shared__ __align__(1024) unsigned char smem[];
    const int b_bytes = NB * SK_KC * 2;
    unsigned char* stage_a[2] = {smem, smem + SK_A_BYTES + b_bytes};
    unsigned char* stage_b[2] = {smem + SK_A_BYTES, smem + 2 * SK_A_BYTES + b_bytes};
    uint64_t* done = reinterpret_cast<uint64_t*>(smem + 2 * (SK_A_BYTES + b_bytes));
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 2);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * SK_BM;
    const size_t row_bytes = (WK == WK_INT4_PACK) ? (size_t)(K >> 1) : (size_t)K;
    int ncols = 32;
    while (ncols < NB) ncols <<= 1;

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        mbar_init(done, 1);
        mbar_init(done + 1, 1);
        mbar_init_fence();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    /* instruction descriptor: D f32, A and B f16, both K-major, N = NB, M = 128 */
    const uint32_t idesc = (1u << 4) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(SK_BM >> 4) << 24);

    const int nk_all = K / SK_KC, KS = gridDim.y, ks = blockIdx.y;
    const int it_first = (int)((long long)nk_all * ks / KS), nk = (int)((long long)nk_all * (ks + 1) / KS) - it_first;
    bool ok = true;
    /* this thread's packed words and scales of a slab, fetched one slab ahead (the global loads of
     * slab i + 1 are in flight while slab i is converted and multiplied) */
    constexpr int NLD = (WK == WK_INT4_PACK) ? 2 : 4;          /* 16-byte loads per thread per slab */
    constexpr int WPL = (WK == WK_INT4_PACK) ? 32 : 16;        /* weights per load */
    uint4 pk[NLD];
    __half2 sc[NLD];
    auto fetch = [&](int it) {
        const int k0 = (it_first + it) * SK_KC;
#pragma unroll
        for (int i = 0; i < NLD; i++) {
            const int idx = tid + SK_THREADS * i, row = idx & (SK_BM - 1), q = idx >> 7;
            const int grow = n0 + row;
            pk[i] = make_uint4(0, 0, 0, 0);
            sc[i] = __float2half2_rn(WK == WK_INT4_PACK ? 0.f : 1.f);
            if (grow < N) {
                const int kq = k0 + q * WPL;
                pk[i] = *reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(w) + (size_t)grow * row_bytes +
                                                        (WK == WK_INT4_PACK ? (kq >> 1) : kq));
                if (WK != WK_INT8_CH)
                    sc[i] = __half2half2(static_cast<const __half*>(scales)[(size_t)grow * (K >> gshift) + (kq >> gshift)]);
            }
        }
    };
    /* the first two 16-byte units of this thread's share of the activation slab travel with them
     * (that is the whole share for batches up to 32 rows) */
    uint4 xb[2];
    auto fetch_x = [&](int it) {
        const int k0 = (it_first + it) * SK_KC;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int c = tid + SK_THREADS * i, n = c % NB, kc = c / NB;
            xb[i] = make_uint4(0, 0, 0, 0);
            if (c < NB * (SK_KC / 8) && n < M) xb[i] = *reinterpret_cast<const uint4*>(x + (size_t)n * K + k0 + kc * 8);
        }
    };
    auto to_f16 = [](const uint4& v) -> uint4 {
        const uint32_t vs[4] = {v.x, v.y, v.z, v.w};
        uint32_t os[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const __half2 h = __floats2half2_rn(bf_lo(vs[j]), bf_hi(vs[j]));
            os[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        return make_uint4(os[0], os[1], os[2], os[3]);
    };
    fetch(0);
    fetch_x(0);
    for (int it = 0; it < nk && ok; it++) {
        const int s = it & 1;
        if (it >= 2) ok = mbar_wait_bounded(done + s, ((unsigned)(it >> 1) - 1u) & 1u, status); /* the MMAs that read this stage */
        if (!ok) break;
        const int k0 = (it_first + it) * SK_KC;
        uint4* A = reinterpret_cast<uint4*>(stage_a[s]);
        uint4* B = reinterpret_cast<uint4*>(stage_b[s]);
        /* weights: A[k / 8][row] (rows beyond N: zero scale / zero codes) */
#pragma unroll
        for (int i = 0; i < NLD; i++) {
            const int idx = tid + SK_THREADS * i, row = idx & (SK_BM - 1), q = idx >> 7;
            if (WK == WK_INT4_PACK) {
                const uint32_t ws[4] = {pk[i].x, pk[i].y, pk[i].z, pk[i].w};
#pragma unroll
                for (int j = 0; j < 4; j++) A[(q * 4 + j) * SK_BM + row] = sk_int4_chunk(ws[j], sc[i]);
            } else {
                A[(q * 2) * SK_BM + row] = sk_int8_chunk<WK == WK_INT8_GRP>(pk[i].x, pk[i].y, sc[i]);
                A[(q * 2 + 1) * SK_BM + row] = sk_int8_chunk<WK == WK_INT8_GRP>(pk[i].z, pk[i].w, sc[i]);
            }
        }
        if (it + 1 < nk) fetch(it + 1);
        /* activations: B[k / 8][batch row], rows beyond the batch are zero (bf16 zero = f16 zero) */
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int c = tid + SK_THREADS * i;
            if (c < NB * (SK_KC / 8)) B[(c / NB) * NB + (c % NB)] = to_f16(xb[i]);
        }
        for (int c = tid + 2 * SK_THREADS; c < NB * (SK_KC / 8); c += SK_THREADS) {
            const int n = c % NB, kc = c / NB;
            uint4 o = make_uint4(0, 0, 0, 0);
            if (n < M) o = to_f16(*reinterpret_cast<const uint4*>(x + (size_t)n * K + k0 + kc * 8));
            B[kc * NB + n] = o;
        }
        if (it + 1 < nk) fetch_x(it + 1);
        fence_proxy_async_smem(); /* these generic-proxy stores are read by the tensor core (async proxy) */
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a0 = smem_u32(stage_a[s]), b0 = smem_u32(stage_b[s]);
#pragma unroll
            for (int kk = 0; kk < SK_KC / 16; kk++) {
                const uint64_t da = sk_smem_desc(a0 + (uint32_t)(kk * 2 * SK_BM * 16), SK_BM * 16, 128);
                const uint64_t db = sk_smem_desc(b0 + (uint32_t)(kk * 2 * NB * 16), (uint32_t)NB * 16, 128);
                const uint32_t accumulate = (it > 0 || kk > 0) ? 1u : 0u;
                asm volatile(
                    "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                    ::"r"(tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
            }
            /* arrives on the barrier once every MMA issued so far has completed */
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(done + s)) : "memory");
        }
    }
    /* the last commit covers every MMA before it */
    if (ok) ok = mbar_wait_bounded(done + ((nk - 1) & 1), (unsigned)((nk - 1) >> 1) & 1u, status);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok && warp < 4) { /* warp w reads TMEM lanes 32 w .. 32 w + 31 = weight rows */
        const int grow = n0 + warp * 32 + lane;
        float rs = 1.f;
        if (WK == WK_INT8_CH && grow < N) rs = static_cast<const float*>(scales)[grow];
        for (int col0 = 0; col0 < NB; col0 += 32) {
            uint32_t v[32];
            const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)col0;
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                  "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                  "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                  "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                : "r"(taddr)
                : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (grow < N) {
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const int m = col0 + j;
                    if (m < M) {
                        if (KS == 1) {
                            __nv_bfloat16 o = f2bf(__fmul_rn(__uint_as_float(v[j]), rs));
                            if (resid) o = f2bf(__fadd_rn(bf2f(resid[(size_t)m * N + grow]), bf2f(o)));
                            y[(size_t)m * N + grow] = o;
                        }
                        else partial[((size_t)ks * M + m) * N + grow] = __uint_as_float(v[j]);
                    }
                }
            }
        }
    }
    if (KS > 1) {
        __shared__ int s_last;
        __threadfence();
        __syncthreads();
        if (tid == 0) s_last = ok && (atomicAdd(arrivals + blockIdx.x, 1u) == (unsigned)(KS - 1));
        __syncthreads();
        if (s_last) {
            __threadfence();
            for (int e = tid; e < SK_BM * M; e += SK_THREADS) {
                const int m = e / SK_BM, grow = n0 + (e % SK_BM);
                if (grow >= N) continue;
                float acc = 0.f;
                for (int q = 0; q < KS; q++) acc += __ldcg(partial + ((size_t)q * M + m) * N + grow);
                if (WK == WK_INT8_CH) acc = __fmul_rn(acc, static_cast<const float*>(scales)[grow]);
                __nv_bfloat16 o = f2bf(acc);
                if (resid) o = f2bf(__fadd_rn(bf2f(resid[(size_t)m * N + grow]), bf2f(o)));
                y[(size_t)m * N + grow] = o;
            }
            if (tid == 0) arrivals[blockIdx.x] = 0u;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(ncols) : "memory");
}

static size_t sk_smem_bytes(int NB) { return 2 * ((size_t)SK_A_BYTES + (size_t)NB * SK_KC * 2) + 64; }

/* scratch for split-K launches: partials [SK_MAX_SPLIT][rows][SK_SPLIT_MAX_N] f32 and one arrival counter per row tile */
constexpr int SK_MAX_SPLIT = 8;
constexpr int SK_SPLIT_MAX_N = 6144;
static float* g_partial[64];
static unsigned* g_arrivals[64];
static int g_partial_rows[64];

/* once per device, outside stream capture: room for split-K launches with up to `max_rows` batch rows */
extern "C" cudaError_t skinny_setup(int max_rows) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || max_rows < 1) return cudaErrorInvalidValue;
    if (g_partial_rows[dev] >= max_rows) return cudaSuccess;
    if (g_partial[dev]) cudaFree(g_partial[dev]);
    g_partial[dev] = nullptr;
    g_partial_rows[dev] = 0;
    if ((e = cudaMalloc((void**)&g_partial[dev], (size_t)SK_MAX_SPLIT * max_rows * SK_SPLIT_MAX_N * sizeof(float))) != cudaSuccess) return e;
    if (!g_arrivals[dev]) {
        if ((e = cudaMalloc((void**)&g_arrivals[dev], 256 * sizeof(unsigned))) != cudaSuccess) return e;
        if ((e = cudaMemset(g_arrivals[dev], 0, 256 * sizeof(unsigned))) != cudaSuccess) return e;
    }
    g_partial_rows[dev] = max_rows;
    return cudaSuccess;
}

template <int WK>
static cudaError_t sk_launch(const LinRef* lin, const void* x, int M, void* y, const void* resid, cudaStream_t st) {
    const int NB = (M + 15) & ~15;
    const size_t smem = sk_smem_bytes(NB);
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(k_skinny_tc<WK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sk_smem_bytes(256));
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    const int tiles = (lin->N + SK_BM - 1) / SK_BM;
    int dev = 0, split = 1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    /* few row tiles and a long K: split K over several CTAs so the whole GPU streams the matrix */
    if (dev >= 0 && dev < 64 && g_partial_rows[dev] >= M && lin->N <= SK_SPLIT_MAX_N && tiles <= 74 && tiles <= 256) {
        split = 148 / tiles;
        if (split > SK_MAX_SPLIT) split = SK_MAX_SPLIT;
        if (split > lin->K / SK_KC) split = lin->K / SK_KC;
        if (split < 1) split = 1;
    }
    k_skinny_tc<WK><<<dim3((unsigned)tiles, (unsigned)split), SK_THREADS, smem, st>>>(
        lin->w, lin->scales, lin->N, lin->K, lin->gshift, (const __nv_bfloat16*)x, M, NB, (__nv_bfloat16*)y,
        (const __nv_bfloat16*)resid, split > 1 ? g_partial[dev] : nullptr, split > 1 ? g_arrivals[dev] : nullptr);
    return cudaGetLastError();
}

/* y[M, N] (bf16) = x[M, K] (bf16) · W^T for 1 <= M <= 256, plus `resid` [M, N] when given (it may be y
 * itself).  K must be a multiple of 128, the group size of grouped kinds at least 32 (INT4) / 16 (INT8 codes). */
extern "C" cudaError_t skinny_gemm_tc(const LinRef* lin, const void* x, int M, void* y, const void* resid, cudaStream_t st) {
    if (!lin || !x || !y || M < 1 || M > 256 || lin->K % SK_KC) return cudaErrorInvalidValue;
    if (((uintptr_t)x | (uintptr_t)lin->w) & 15) return cudaErrorInvalidValue;
    switch (lin->kind) {
    case WK_INT8_CH: return sk_launch<WK_INT8_CH>(lin, x, M, y, resid, st);
    case WK_INT8_GRP: return lin->gshift >= 4 ? sk_launch<WK_INT8_GRP>(lin, x, M, y, resid, st) : cudaErrorInvalidValue;
    case WK_INT4_PACK: return lin->gshift >= 5 ? sk_launch<WK_INT4_PACK>(lin, x, M, y, resid, st) : cudaErrorInvalidValue;
    }
    return cudaErrorInvalidValue;
}

/* status word of the launches so far on the current device (0 = no wait ever gave up); synchronises */
extern "C" cudaError_t skinny_status(int* out) { return cudaMemcpyFromSymbol(out, g_sk_status, sizeof(int)); }

}  // namespace s2p
