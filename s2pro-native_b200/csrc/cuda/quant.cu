/* Load-time weight conversion: per-channel INT8, group-wise INT4 with the MSE
 * clip search, nibble packing and the three dequantisers.
 *
 * Results are bit-identical to the reference quantisers
 * (src/sched/int8_gemv.cu:32-58 k_quant, :135-195 k_quant_g, :265-269
 * k_pack_nib, :106-114 / :244-253 / :731-744 dequant); what differs is the
 * mapping to the machine: rows and groups are handled by warps with shuffle
 * trees and 16-byte loads, grids are sized to the SM count and walk the matrix
 * with a grid stride, so one launch streams the whole tensor at HBM rate.
 *
 * Entry points (C ABI, include/s2p_b200_abi.h): s2p_int8_quant,
 * s2p_intq_quant, s2p_int4_pack, s2p_int8_dequant, s2p_intq_dequant,
 * s2p_int4p_dequant.
 */
#include <stdio.h>
#include "common.cuh"
#include "s2p_b200_abi.h"

namespace {

int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

__device__ __forceinline__ int clamp_q(int v, int levels) { return max(-levels, min(levels, v)); }

/* One warp per row.  amax is order-free (max), so any traversal is exact. */
__global__ void __launch_bounds__(256) k_quant_rows(int8_t* __restrict__ q, float* __restrict__ scales,
                                                    const __nv_bfloat16* __restrict__ w, int N, int K, int levels,
                                                    int vec_ok) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int n = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; n < N; n += warps) {
        const __nv_bfloat16* row = w + (size_t)n * K;
        float amax = 0.f;
        if (vec_ok) {
            const uint4* r4 = reinterpret_cast<const uint4*>(row);
            for (int i = lane; i < (K >> 3); i += 32) {
                const uint4 v = r4[i];
                const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    amax = fmaxf(amax, fabsf(bf_bits_to_f32(u[j] & 0xffffu)));
                    amax = fmaxf(amax, fabsf(__uint_as_float(u[j] & 0xffff0000u)));
                }
            }
        } else {
            for (int k = lane; k < K; k += 32) amax = fmaxf(amax, fabsf(bf2f(row[k])));
        }
        amax = warp_tree_max(amax);
        const float scale = amax > 0.f ? __fdiv_rn(amax, (float)levels) : 1.0f;
        const float inv = __fdiv_rn(1.0f, scale);
        if (lane == 0) scales[n] = scale;
        int8_t* qrow = q + (size_t)n * K;
        for (int k = lane; k < K; k += 32)
            qrow[k] = (int8_t)clamp_q(__float2int_rn(__fmul_rn(bf2f(row[k]), inv)), levels);
    }
}

/* Tree over GL consecutive lanes (GL = 16 or 32), off = GL/2 .. 1. */
template <int GL, bool IS_MAX>
__device__ __forceinline__ float seg_tree(float v, unsigned mask) {
#pragma unroll
    for (int off = GL >> 1; off > 0; off >>= 1) {
        const float o = __shfl_xor_sync(mask, v, off);
        v = IS_MAX ? fmaxf(v, o) : v + o;
    }
    return v;
}

/* G == 16 or 32: GL lanes per group, lane == element.  The per-candidate error
 * is d*d of one element per lane (an fma onto 0), merged by the GL/2..1 tree;
 * the first strict minimum wins.  n_groups must be a multiple of 32/GL (it is:
 * K % 512 == 0 for every served layer; checked by the launcher). */
template <int GL>
__global__ void __launch_bounds__(256) k_quant_gw(int8_t* __restrict__ q, __half* __restrict__ scales,
                                                  const __nv_bfloat16* __restrict__ w, size_t n_groups,
                                                  int levels, int mse) {
    const int lane = threadIdx.x & (GL - 1);
    /* the two 16-lane groups of a warp may diverge on amax == 0: each syncs only its own lanes */
    const unsigned mask = GL == 32 ? S2P_FULL_MASK : (0xffffu << (threadIdx.x & 16));
    const size_t segs = ((size_t)gridDim.x * blockDim.x) / GL;
    for (size_t g = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) / GL; g < n_groups; g += segs) {
        const float v = bf2f(w[g * GL + lane]);
        const float amax = seg_tree<GL, true>(fabsf(v), mask);
        const float base = amax > 0.f ? __fdiv_rn(amax, (float)levels) : 1.0f;
        float scale = __half2float(__float2half_rn(base));
        if (mse && amax > 0.f) {
            float best_err = 3.4e38f, best_s = scale;
#pragma unroll 4
            for (int c = 0; c < 32; c++) {
                const float s = __half2float(__float2half_rn(__fmul_rn(base, 1.0f - (float)c / 64.0f)));
                const float inv = __fdiv_rn(1.0f, s);
                const int qi = clamp_q(__float2int_rn(__fmul_rn(v, inv)), levels);
                const float d = __fmaf_rn(-(float)qi, s, v);
                const float err = seg_tree<GL, false>(__fmaf_rn(d, d, 0.f), mask);
                if (err < best_err) { best_err = err; best_s = s; }
            }
            scale = best_s;
        }
        if (lane == 0) scales[g] = __float2half_rn(scale);
        const float inv = __fdiv_rn(1.0f, scale);
        q[g * GL + lane] = (int8_t)clamp_q(__float2int_rn(__fmul_rn(v, inv)), levels);
    }
}

/* Any other legal G (power of two >= 16): a block of T = min(G,256) threads
 * per group, thread t owning elements t, t+T, ... (fma chain), halving tree in
 * shared memory — the structure the reference's launch fixes (int8_gemv.cu:760). */
template <int T>
__global__ void k_quant_g_generic(int8_t* __restrict__ q, __half* __restrict__ scales,
                                  const __nv_bfloat16* __restrict__ w, int K, int G, int levels, int mse) {
    __shared__ float red[T];
    const int ng = K / G;
    const int n = blockIdx.x / ng, g = blockIdx.x - n * ng;
    const __nv_bfloat16* wp = w + (size_t)n * K + (size_t)g * G;
    const int t = threadIdx.x;
    float amax = 0.f;
    for (int k = t; k < G; k += T) amax = fmaxf(amax, fabsf(bf2f(wp[k])));
    amax = block_tree<T, true>(amax, red);
    const float base = amax > 0.f ? __fdiv_rn(amax, (float)levels) : 1.0f;
    float scale = __half2float(__float2half_rn(base));
    if (mse && amax > 0.f) {
        float best_err = 3.4e38f, best_s = scale;
        for (int c = 0; c < 32; c++) {
            const float s = __half2float(__float2half_rn(__fmul_rn(base, 1.0f - (float)c / 64.0f)));
            const float inv = __fdiv_rn(1.0f, s);
            float err = 0.f;
            for (int k = t; k < G; k += T) {
                const float v = bf2f(wp[k]);
                const int qi = clamp_q(__float2int_rn(__fmul_rn(v, inv)), levels);
                const float d = __fmaf_rn(-(float)qi, s, v);
                err = __fmaf_rn(d, d, err);
            }
            err = block_tree<T, false>(err, red);
            if (err < best_err) { best_err = err; best_s = s; }
        }
        scale = best_s;
    }
    if (t == 0) scales[(size_t)n * ng + g] = __float2half_rn(scale);
    const float inv = __fdiv_rn(1.0f, scale);
    int8_t* qp = q + (size_t)n * K + (size_t)g * G;
    for (int k = t; k < G; k += T) qp[k] = (int8_t)clamp_q(__float2int_rn(__fmul_rn(bf2f(wp[k]), inv)), levels);
}

/* 8 codes -> 4 bytes per thread; low nibble = even column. */
__global__ void __launch_bounds__(256) k_pack(uint8_t* __restrict__ p, const int8_t* __restrict__ q, size_t n_bytes,
                                              int vec_ok) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t n4 = vec_ok ? (n_bytes >> 2) : 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const uint2 v = reinterpret_cast<const uint2*>(q)[i];
        uint32_t out = 0;
        const uint32_t u[2] = {v.x, v.y};
#pragma unroll
        for (int j = 0; j < 2; j++)
#pragma unroll
            for (int b = 0; b < 2; b++) {
                const uint32_t lo = (u[j] >> (16 * b)) & 0xFu, hi = (u[j] >> (16 * b + 8)) & 0xFu;
                out |= (lo | (hi << 4)) << (8 * (2 * j + b));
            }
        reinterpret_cast<uint32_t*>(p)[i] = out;
    }
    /* tail (n_bytes not a multiple of 4) */
    for (size_t i = (n4 << 2) + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_bytes; i += stride)
        p[i] = (uint8_t)((q[2 * i] & 0xF) | ((q[2 * i + 1] & 0xF) << 4));
}

/* mode 0: per-channel f32 scale; 1: f16 group scale on int8 codes; 2: packed nibbles. */
template <int MODE>
__global__ void __launch_bounds__(256) k_dequant(__nv_bfloat16* __restrict__ o, const void* __restrict__ wq,
                                                 const void* __restrict__ sc, int N, int K, int gshift) {
    const size_t total = (size_t)N * K;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t n = i / K;
        const int k = (int)(i - n * K);
        float v, s;
        if (MODE == 2) {
            const uint8_t b = static_cast<const uint8_t*>(wq)[i >> 1];
            v = (float)((k & 1) ? (int8_t)((int8_t)b >> 4) : (int8_t)((int8_t)(b << 4) >> 4));
        } else {
            v = (float)static_cast<const int8_t*>(wq)[i];
        }
        if (MODE == 0) s = static_cast<const float*>(sc)[n];
        else s = __half2float(static_cast<const __half*>(sc)[n * (size_t)(K >> gshift) + (k >> gshift)]);
        o[i] = f2bf(__fmul_rn(v, s));
    }
}

/* The same, eight consecutive elements of a row per thread (K a multiple of 8; a group of 16 or more codes shares a
 * scale, so the eight share one): one 4- or 8-byte load of codes, one scale, one 16-byte store, no division per
 * element.  Element values are formed exactly as above: bf16(code x scale), one f32 multiply. */
template <int MODE>
__global__ void __launch_bounds__(256) k_dequant8(uint4* __restrict__ o, const void* __restrict__ wq,
                                                  const void* __restrict__ sc, unsigned n_units, unsigned k8n, int K, int gshift) {
    const unsigned stride = gridDim.x * blockDim.x;
    for (unsigned u = blockIdx.x * blockDim.x + threadIdx.x; u < n_units; u += stride) {
        const unsigned n = u / k8n, k = (u - n * k8n) * 8;
        float s;
        if (MODE == 0) s = static_cast<const float*>(sc)[n];
        else s = __half2float(static_cast<const __half*>(sc)[(size_t)n * (unsigned)(K >> gshift) + (k >> gshift)]);
        float v[8];
        if (MODE == 2) {
            const uint32_t w = static_cast<const uint32_t*>(wq)[u]; /* byte j: codes 2j (low nibble), 2j + 1 (high) */
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int8_t b = (int8_t)((w >> (8 * j)) & 0xFFu);
                v[2 * j] = (float)(int8_t)((int8_t)(b << 4) >> 4);
                v[2 * j + 1] = (float)(int8_t)(b >> 4);
            }
        } else {
            const uint2 w = static_cast<const uint2*>(wq)[u];
            const uint32_t ws[2] = {w.x, w.y};
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = (float)(int8_t)((ws[j >> 2] >> (8 * (j & 3))) & 0xFFu);
        }
        uint32_t pk[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const __nv_bfloat162 h = __halves2bfloat162(f2bf(__fmul_rn(v[2 * j], s)), f2bf(__fmul_rn(v[2 * j + 1], s)));
            pk[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        o[u] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
}
/* true when the 8-per-thread form serves the shape and the pointers */
static bool dequant8_ok(const void* o, const void* wq, int N, int K) {
    return K % 8 == 0 && ((uintptr_t)o & 15) == 0 && ((uintptr_t)wq & 7) == 0 && (size_t)N * K / 8 < 0xFFFFFFFFull;
}

int gshift_of(int G) {
    if (G < 16 || (G & (G - 1))) return -1;
    int s = 0;
    while ((1 << s) < G) s++;
    return s;
}

s2p_status launched(const char* what, int N, int K) {
    const cudaError_t ce = cudaGetLastError();
    if (ce == cudaSuccess) return S2P_OK;
    fprintf(stderr, "[s2pro] %s launch (N=%d,K=%d): %s\n", what, N, K, cudaGetErrorString(ce));
    return S2P_ERR_CUDA;
}

int stream_grid(size_t work_items, int per_block) {
    size_t b = (work_items + per_block - 1) / per_block;
    const size_t cap = (size_t)sm_count() * 8;
    if (b > cap) b = cap;
    return b < 1 ? 1 : (int)b;
}

}  // namespace

extern "C" s2p_status s2p_int8_quant(void* w_i8, float* scales, const void* w_bf16, int N, int K,
                                     cudaStream_t stream) {
    if (!w_i8 || !scales || !w_bf16 || N <= 0 || K <= 0) return S2P_ERR_INVALID;
    k_quant_rows<<<stream_grid((size_t)N, 8), 256, 0, stream>>>((int8_t*)w_i8, scales,
                                                                (const __nv_bfloat16*)w_bf16, N, K, 127,
                                                                (K % 8 == 0) && ((uintptr_t)w_bf16 % 16 == 0));
    return launched("int8 quant", N, K);
}

extern "C" s2p_status s2p_intq_quant(void* w_i8, void* scales_f16, const void* w_bf16, int N, int K, int G,
                                     int levels, int mse, cudaStream_t stream) {
    if (!w_i8 || !scales_f16 || !w_bf16 || N <= 0 || K <= 0 || levels <= 0) return S2P_ERR_INVALID;
    if (gshift_of(G) < 0 || K % G != 0) return S2P_ERR_INVALID;
    const size_t n_groups = (size_t)N * (K / G);
    if (G == 32) {
        k_quant_gw<32><<<stream_grid(n_groups, 8), 256, 0, stream>>>((int8_t*)w_i8, (__half*)scales_f16,
                                                                     (const __nv_bfloat16*)w_bf16, n_groups, levels, mse);
    } else if (G == 16 && n_groups % 2 == 0) {
        k_quant_gw<16><<<stream_grid(n_groups, 16), 256, 0, stream>>>((int8_t*)w_i8, (__half*)scales_f16,
                                                                      (const __nv_bfloat16*)w_bf16, n_groups, levels, mse);
    } else {
        if (n_groups > 0x7fffffffull) return S2P_ERR_INVALID;
        const unsigned blocks = (unsigned)n_groups;
#define S2P_QG(T) k_quant_g_generic<T><<<blocks, T, 0, stream>>>((int8_t*)w_i8, (__half*)scales_f16, \
                                                                 (const __nv_bfloat16*)w_bf16, K, G, levels, mse)
        if (G == 16) return S2P_ERR_UNSUPPORTED; /* odd group count at G=16: no served layer has it */
        else if (G == 64) S2P_QG(64);
        else if (G == 128) S2P_QG(128);
        else S2P_QG(256);
#undef S2P_QG
    }
    return launched("intq quant", N, K);
}

extern "C" s2p_status s2p_int4_pack(void* w_pack, const void* w_i8, int N, int K, cudaStream_t stream) {
    if (!w_pack || !w_i8 || N <= 0 || K <= 0 || (K & 1)) return S2P_ERR_INVALID;
    const size_t n = (size_t)N * (K >> 1);
    k_pack<<<stream_grid((n >> 2) + 1, 256), 256, 0, stream>>>((uint8_t*)w_pack, (const int8_t*)w_i8, n,
                                                         ((uintptr_t)w_i8 % 8 == 0) && ((uintptr_t)w_pack % 4 == 0));
    return launched("int4 pack", N, K);
}

extern "C" s2p_status s2p_int8_dequant(void* w_bf16, const void* w_i8, const float* scales, int N, int K,
                                       cudaStream_t stream) {
    if (!w_bf16 || !w_i8 || !scales || N <= 0 || K <= 0) return S2P_ERR_INVALID;
    if (dequant8_ok(w_bf16, w_i8, N, K))
        k_dequant8<0><<<stream_grid((size_t)N * K / 8, 1024), 256, 0, stream>>>((uint4*)w_bf16, w_i8, scales, (unsigned)((size_t)N * K / 8),
                                                                              (unsigned)(K / 8), K, 0);
    else
        k_dequant<0><<<stream_grid((size_t)N * K, 1024), 256, 0, stream>>>((__nv_bfloat16*)w_bf16, w_i8, scales, N, K, 0);
    return launched("int8 dequant", N, K);
}

extern "C" s2p_status s2p_intq_dequant(void* w_bf16, const void* w_i8, const void* scales_f16, int N, int K, int G,
                                       cudaStream_t stream) {
    if (!w_bf16 || !w_i8 || !scales_f16 || N <= 0 || K <= 0) return S2P_ERR_INVALID;
    const int gs = gshift_of(G);
    if (gs < 0 || K % G != 0) return S2P_ERR_INVALID;
    if (dequant8_ok(w_bf16, w_i8, N, K))
        k_dequant8<1><<<stream_grid((size_t)N * K / 8, 1024), 256, 0, stream>>>((uint4*)w_bf16, w_i8, scales_f16, (unsigned)((size_t)N * K / 8),
                                                                              (unsigned)(K / 8), K, gs);
    else
        k_dequant<1><<<stream_grid((size_t)N * K, 1024), 256, 0, stream>>>((__nv_bfloat16*)w_bf16, w_i8, scales_f16, N, K, gs);
    return launched("intq dequant", N, K);
}

extern "C" s2p_status s2p_int4p_dequant(void* w_bf16, const void* w_pack, const void* scales_f16, int N, int K, int G,
                                        cudaStream_t stream) {
    if (!w_bf16 || !w_pack || !scales_f16 || N <= 0 || K <= 0 || (K & 1)) return S2P_ERR_INVALID;
    const int gs = gshift_of(G);
    if (gs < 0 || K % G != 0) return S2P_ERR_INVALID;
    if (dequant8_ok(w_bf16, w_pack, N, K) && ((uintptr_t)w_pack & 3) == 0)
        k_dequant8<2><<<stream_grid((size_t)N * K / 8, 1024), 256, 0, stream>>>((uint4*)w_bf16, w_pack, scales_f16, (unsigned)((size_t)N * K / 8),
                                                                              (unsigned)(K / 8), K, gs);
    else
        k_dequant<2><<<stream_grid((size_t)N * K, 1024), 256, 0, stream>>>((__nv_bfloat16*)w_bf16, w_pack, scales_f16, N, K, gs);
    return launched("int4p dequant", N, K);
}
