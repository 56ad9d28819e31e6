/* Split-K GQA decode attention over per-session KV caches, with the merge of
 * the partials done by the last CTA to finish (no second launch).
 *
 * Arithmetic: the reference's flash-decode pair k_attn_split / k_attn_combine
 * (src/slowar/kernels.cu:351-489) and its INT8-cache twin k_attn_split8<8>
 * (:759-918): 64-position splits; per position a 128-term fma chain against the
 * pre-scaled query (INT8: four 32-term chains folded with the f16 group scale);
 * split max and exp-sum by halving trees; PV as a sequential fma over the
 * split; partial = (m, l, acc[128]); merge in ascending split order with
 * w = expf(m_s - M), l = fma(l_s, w, l), acc = fma(acc_s, w, acc), out = acc / l.
 *
 * Mapping: a fixed grid (rows, kv heads, workers) independent of the sequence
 * length, so one captured CUDA graph serves every frame; each worker walks the
 * splits s = worker, worker + workers, ...; 512 threads score the four q heads
 * of the kv head concurrently (one chain per thread) from a K tile staged in
 * shared memory with a skewed stride.  With PREP the kernel also performs what
 * precedes attention in the decode tick — per-head RMSNorm of q and k, RoPE,
 * and the append (bf16 copy or INT8 quantise) of the new k/v vectors — so the
 * fused tick needs no separate launches for them.
 */
#include <math.h>
#include "common.cuh"
#include "headops.cuh"
#include "ops.h"
#include "attn.cuh"

namespace s2p {


template <bool KV8, bool PREP>
__global__ void __launch_bounds__(512) k_attn_decode(AttnArgs a, AttnPrep pz) {
    constexpr int VB = KV8 ? 128 : 256;  /* payload bytes per cached vector */
    constexpr int TS = VB + 4;           /* staged row stride (skewed) */
    __shared__ __align__(16) unsigned char tile[64 * TS];
    __shared__ __half ssc[64 * 4];
    __shared__ float sq[4][128];
    __shared__ float sc[4][64];
    __shared__ float red[4][128];
    __shared__ float hm[4], hs[4];
    __shared__ int s_last;

    const int row = blockIdx.x, kvh = blockIdx.y, wk = blockIdx.z, workers = gridDim.z;
    const int tid = threadIdx.x;
    const int QH = a.q_heads, KVH = a.kv_heads;
    const int pos = a.pos_arr ? a.pos_arr[row] : a.pos0 + row * a.pos_row_step;
    const int len = pos + 1;
    const int n_active = (len + 63) >> 6;
    const size_t plane = (size_t)kvh * a.max_seq;
    unsigned char* kc = kv_payload(a.kv, row) + a.kv.k_off;
    unsigned char* vc = kv_payload(a.kv, row) + a.kv.v_off;
    __half* ks = KV8 ? reinterpret_cast<__half*>(kv_scales(a.kv, row) + a.kv.ks_off) : nullptr;
    __half* vs = KV8 ? reinterpret_cast<__half*>(kv_scales(a.kv, row) + a.kv.vs_off) : nullptr;
    const float scale = rsqrtf(128.0f);

    {   /* queries of the four heads sharing this kv head, pre-scaled */
        const int g = tid >> 7, t = tid & 127;
        const int h = kvh * 4 + g;
        float v;
        if (PREP) {
            v = bf2f(pz.qkv[(size_t)row * (QH + 2 * KVH) * 128 + (size_t)h * 128 + t]);
            if (pz.q_norm) {
                const float tot = head_tree_sum(__fmaf_rn(v, v, 0.f), red, g, t);
                const float inv = rsqrtf(__fdiv_rn(tot, 128.0f) + pz.eps);
                v = bf16_round(__fmul_rn(__fmul_rn(v, inv), bf2f(pz.q_norm[t])));
            }
            float c, s;
            rope_cs(t >> 1, pos, pz.rope_base, c, s);
            const float other = __shfl_xor_sync(S2P_FULL_MASK, v, 1);
            v = rope_elem(t, v, other, c, s);
        } else {
            v = bf2f(a.q[((size_t)row * QH + h) * 128 + t]);
        }
        sq[g][t] = __fmul_rn(v, scale);
    }
    if (PREP) {
        /* the worker that owns the split holding the new position appends k and v */
        const bool owner = ((n_active - 1) % workers) == wk;
        if (owner) { /* uniform over the CTA */
            const int g = tid >> 7, t = tid & 127; /* g 0: k, g 1: v, g 2,3 idle but join the barriers */
            const size_t src = (size_t)row * (QH + 2 * KVH) * 128 + (size_t)(QH + (g == 1 ? KVH : 0) + kvh) * 128 + t;
            float v = bf2f(pz.qkv[g < 2 ? src : 0]);
            if (pz.k_norm) { /* uniform */
                const float tot = head_tree_sum(__fmaf_rn(v, v, 0.f), red, g, t);
                if (g == 0) {
                    const float inv = rsqrtf(__fdiv_rn(tot, 128.0f) + pz.eps);
                    v = bf16_round(__fmul_rn(__fmul_rn(v, inv), bf2f(pz.k_norm[t])));
                }
            }
            if (g == 0) {
                float c, s;
                rope_cs(t >> 1, pos, pz.rope_base, c, s);
                const float other = __shfl_xor_sync(S2P_FULL_MASK, v, 1);
                v = rope_elem(t, v, other, c, s);
            }
            if (g < 2) {
                unsigned char* cache = g == 0 ? kc : vc;
                const size_t vec = plane + pos;
                if (!KV8) {
                    reinterpret_cast<__nv_bfloat16*>(cache)[vec * 128 + t] = f2bf(v);
                } else {
                    __half hsc;
                    const int8_t q8 = kv8_quant(v, hsc);
                    reinterpret_cast<int8_t*>(cache)[vec * 128 + t] = q8;
                    if ((t & 31) == 0) (g == 0 ? ks : vs)[vec * 4 + (t >> 5)] = hsc;
                }
            }
        }
    }
    __syncthreads();

    for (int spl = wk; spl < n_active; spl += workers) {
        const int start = spl << 6;
        const int cnt = min(64, len - start);
        /* K tile */
        for (int i = tid; i < cnt * (VB / 4); i += 512) {
            const int rr = i / (VB / 4), cw = i - rr * (VB / 4);
            *reinterpret_cast<uint32_t*>(tile + rr * TS + cw * 4) =
                *reinterpret_cast<const uint32_t*>(kc + (plane + start + rr) * VB + cw * 4);
        }
        if (KV8)
            for (int i = tid; i < cnt * 4; i += 512) ssc[i] = ks[(plane + start) * 4 + i];
        __syncthreads();

        /* scores: thread (head g4, position t4), one chain each */
        const int g4 = (tid >> 6) & 3, t4 = tid & 63;
        float d = -INFINITY;
        if (tid < 256 && t4 < cnt) {
            d = 0.f;
            if (!KV8) {
                const __nv_bfloat162* kr = reinterpret_cast<const __nv_bfloat162*>(tile + t4 * TS);
#pragma unroll 8
                for (int e = 0; e < 64; e++) {
                    const float2 kf = __bfloat1622float2(kr[e]);
                    d = __fmaf_rn(sq[g4][2 * e], kf.x, d);
                    d = __fmaf_rn(sq[g4][2 * e + 1], kf.y, d);
                }
            } else {
                const int8_t* kr = reinterpret_cast<const int8_t*>(tile + t4 * TS);
#pragma unroll
                for (int gi = 0; gi < 4; gi++) {
                    float pp = 0.f;
#pragma unroll 8
                    for (int e = 0; e < 32; e++) pp = __fmaf_rn(sq[g4][gi * 32 + e], (float)kr[gi * 32 + e], pp);
                    d = __fmaf_rn(pp, __half2float(ssc[t4 * 4 + gi]), d);
                }
            }
        }
        if (tid < 256) { /* split max per head: two warps of 32 slots each */
            const float mx = warp_tree_max(d);
            if ((tid & 31) == 0) red[0][tid >> 5] = mx;
        }
        __syncthreads();
        float m = 0.f;
        if (tid < 256) {
            m = fmaxf(red[0][2 * g4], red[0][2 * g4 + 1]);
            sc[g4][t4] = (t4 < cnt) ? expf(d - m) : 0.f;
        }
        __syncthreads();
        if (tid < 256 && t4 < 32) { /* exp-sum: pairs (t, t+32), then 16..1 */
            const float x = warp_tree_sum(sc[g4][t4] + sc[g4][t4 + 32]);
            if (t4 == 0) { hm[g4] = m; hs[g4] = x; }
        }
        /* V tile replaces K */
        for (int i = tid; i < cnt * (VB / 4); i += 512) {
            const int rr = i / (VB / 4), cw = i - rr * (VB / 4);
            *reinterpret_cast<uint32_t*>(tile + rr * TS + cw * 4) =
                *reinterpret_cast<const uint32_t*>(vc + (plane + start + rr) * VB + cw * 4);
        }
        if (KV8)
            for (int i = tid; i < cnt * 4; i += 512) ssc[i] = vs[(plane + start) * 4 + i];
        __syncthreads();
        {
            const int g = tid >> 7, dd = tid & 127;
            float acc = 0.f;
            if (!KV8) {
                for (int j = 0; j < cnt; j++)
                    acc = __fmaf_rn(sc[g][j], bf2f(reinterpret_cast<const __nv_bfloat16*>(tile + j * TS)[dd]), acc);
            } else {
                for (int j = 0; j < cnt; j++)
                    acc = __fmaf_rn(__fmul_rn(sc[g][j], __half2float(ssc[j * 4 + (dd >> 5)])),
                                    (float)reinterpret_cast<const int8_t*>(tile + j * TS)[dd], acc);
            }
            float* ph = a.part + (((size_t)row * QH + kvh * 4 + g) * a.n_split_slots + spl) * 130;
            if (dd == 0) { ph[0] = hm[g]; ph[1] = hs[g]; }
            ph[2 + dd] = acc;
        }
        __syncthreads(); /* tile, sc, hm/hs are rewritten by the next split */
    }

    /* the last worker of this (row, kv head) to finish merges the partials */
    __threadfence();
    __syncthreads();
    unsigned int* ctr = a.counters + (size_t)row * KVH + kvh;
    if (tid == 0) s_last = (atomicAdd(ctr, 1u) == (unsigned)(workers - 1));
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    {
        const int g = tid >> 7, dd = tid & 127, h = kvh * 4 + g;
        const float* pb = a.part + ((size_t)row * QH + h) * a.n_split_slots * 130;
        float M = -INFINITY;
        for (int s = 0; s < n_active; s++) M = fmaxf(M, __ldcg(pb + (size_t)s * 130));
        float l = 0.f, acc = 0.f;
        for (int s = 0; s < n_active; s++) {
            const float* ph = pb + (size_t)s * 130;
            const float ls = __ldcg(ph + 1);
            if (ls == 0.f) continue;
            const float w = expf(__ldcg(ph) - M);
            l = __fmaf_rn(ls, w, l);
            acc = __fmaf_rn(__ldcg(ph + 2 + dd), w, acc);
        }
        a.out[((size_t)row * QH + h) * 128 + dd] = f2bf(__fdiv_rn(acc, l));
    }
    if (tid == 0) *ctr = 0u;
}

cudaError_t launch_attn_decode(const AttnArgs& a, const AttnPrep* prep, int rows, cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    if (a.q_heads != a.kv_heads * 4 || !a.part || !a.counters || a.workers < 1) return cudaErrorInvalidValue;
    dim3 grid((unsigned)rows, (unsigned)a.kv_heads, (unsigned)a.workers);
    AttnPrep pz = {};
    if (prep) {
        pz = *prep;
        if (a.kv8) k_attn_decode<true, true><<<grid, 512, 0, st>>>(a, pz);
        else k_attn_decode<false, true><<<grid, 512, 0, st>>>(a, pz);
    } else {
        if (a.kv8) k_attn_decode<true, false><<<grid, 512, 0, st>>>(a, pz);
        else k_attn_decode<false, false><<<grid, 512, 0, st>>>(a, pz);
    }
    return cudaGetLastError();
}

extern "C" cudaError_t attn_decode(const AttnArgs* a, int rows, cudaStream_t st) {
    return launch_attn_decode(*a, nullptr, rows, st);
}

/* ---- allocation-free variant (include/s2p_b200_ext.h) --------------------------
 * Split-K decode attention for one query row whose scratch (the per-split partials
 * and the arrival counters) lives in a fixed array inside the library image instead
 * of memory obtained from the driver.  Every GPU that loads the library carries the
 * array (about 2.1 MB) until the process exits. */
constexpr int NOALLOC_MAX_POSITIONS = 8192;                       /* cached positions a call may attend over */
constexpr int NOALLOC_SLOTS = NOALLOC_MAX_POSITIONS / 64;          /* 64-position splits */
constexpr size_t NOALLOC_PART_BYTES = (size_t)32 * NOALLOC_SLOTS * 130 * sizeof(float);
constexpr size_t NOALLOC_CTR_BYTES = 8 * sizeof(unsigned int);
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_PART_BYTES + NOALLOC_CTR_BYTES];

}  // namespace s2p

#include <stdio.h>
#include "s2p_b200_ext.h"

extern "C" s2p_status s2p_b200_attention_decode_noalloc(const s2p_bf16* q, const s2p_bf16* k_cache,
                                                        const s2p_bf16* v_cache, s2p_bf16* out, int q_heads,
                                                        int kv_heads, int head_dim, int pos, int max_seq,
                                                        cudaStream_t stream) {
    using namespace s2p;
    if (!q || !k_cache || !v_cache || !out) return S2P_ERR_INVALID;
    if (q_heads != 32 || kv_heads != 8 || head_dim != 128) {
        fprintf(stderr, "[s2pro] attention_decode_noalloc: only 32 query / 8 kv heads of width 128 are served\n");
        return S2P_ERR_INVALID;
    }
    if (pos < 0 || pos >= max_seq || pos + 1 > NOALLOC_MAX_POSITIONS) {
        fprintf(stderr, "[s2pro] attention_decode_noalloc: position %d outside the cache (%d) or beyond the built-in "
                        "scratch limit of %d positions\n", pos, max_seq, NOALLOC_MAX_POSITIONS);
        return S2P_ERR_INVALID;
    }
    /* The array's name is only a host-side handle; the kernel needs its device address.
     * It is looked up once per device, with that device current. */
    static void* dev_addr[64] = {0};
    int dev = -1;
    S2P_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return S2P_ERR_UNSUPPORTED;
    if (!dev_addr[dev]) {
        void* p = NULL;
        S2P_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        dev_addr[dev] = p;
    }
    unsigned char* base = static_cast<unsigned char*>(dev_addr[dev]);
    unsigned int* counters = reinterpret_cast<unsigned int*>(base + NOALLOC_PART_BYTES);
    /* the array keeps whatever the previous call left: the arrival counters must start at zero */
    S2P_CUDA_TRY(cudaMemsetAsync(counters, 0, NOALLOC_CTR_BYTES, stream));
    AttnArgs a = {};
    a.q = reinterpret_cast<const __nv_bfloat16*>(q);
    a.out = reinterpret_cast<__nv_bfloat16*>(out);
    a.q_heads = q_heads; a.kv_heads = kv_heads; a.max_seq = max_seq; a.kv8 = 0; a.head_dim = head_dim;
    a.pos0 = pos; a.pos_row_step = 0;
    a.kv.base0 = (void*)k_cache;
    a.kv.k_off = 0;
    a.kv.v_off = (size_t)((const char*)v_cache - (const char*)k_cache);
    a.part = reinterpret_cast<float*>(base);
    a.counters = counters;
    a.n_split_slots = NOALLOC_SLOTS;
    a.workers = 16;
    S2P_CUDA_TRY(launch_attn_decode(a, nullptr, 1, stream));
    return S2P_OK;
}

namespace s2p {

}  // namespace s2p
