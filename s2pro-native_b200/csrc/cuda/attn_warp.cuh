/* Split-K decode attention for lockstep batches: one WARP per 64-position split.
 *
 * Same arithmetic as attn_body.cuh (the reference's k_attn_split / k_attn_split8<8> and
 * k_attn_combine, src/slowar/kernels.cu:351-489 and :759-918): per position a 128-term fma chain
 * against the pre-scaled query (INT8 cache: four 32-term chains folded with the f16 group scale),
 * split max, exp, exp-sum pairs (t, t+32) then the 16..1 tree, the value sum as one fma per
 * position in ascending order, partial = (m, l, acc[128]) per (head, split), merge in ascending
 * split order by the last CTA of the (row, kv head) to finish.
 *
 * What differs is who does what.  The 512-thread body gives every (position, head) chain its own
 * thread, converts each cached key four times (once per query head of the kv head), and crosses six
 * CTA barriers per split, three quarters of the CTA idle in the value phase; on a lockstep batch
 * of 32 rows x 8192 positions it issues about twice the instructions the arithmetic needs and
 * reads the cache at under a fifth of the HBM rate.  Here a warp owns a split from the copy to the
 * partial:
 *   scores   lane l carries positions l and l+32 for all four heads (8 chains): a key word is
 *            converted once for the four heads, a query float4 serves two positions;
 *   softmax  the split max and the exp-sum are warp shuffles (lane l holds exactly the pair
 *            (l, l+32) the sum tree starts with);
 *   values   lane l carries dimensions 4l..4l+3 for the four heads (16 chains): one 32-bit word
 *            of the value row per position, one float4 of weights;
 * and nothing but __syncwarp orders it.  The K and V tiles of a warp are single-buffered: the
 * next split's keys are copied (cp.async, 16 bytes per lane and request) while the values of this
 * one are summed, the next values while the next scores are formed.  Key rows are staged with a
 * 16-byte pad per row, which makes the per-lane 16-byte reads of 32 different rows conflict-free.
 *
 * Requirements checked by the launcher: every per-row offset a multiple of 16 bytes and an even
 * number of cache slots (the scales of two positions share a 16-byte request).  A cache whose base
 * address is not 16-byte aligned is copied with 4-byte requests instead.
 */
#pragma once
#include <math.h>
#include "common.cuh"
#include "headops.cuh"
#include "ops.h"

namespace s2p {

template <bool KV8> struct AttnWarpTile {
    static constexpr int VB = KV8 ? 128 : 256;  /* payload bytes per cached vector */
    static constexpr int KS = VB + 16;          /* staged key row stride */
    alignas(16) unsigned char k[64 * KS];
    alignas(16) unsigned char v[64 * VB];
    alignas(16) __half ksc[KV8 ? 64 * 4 : 8];   /* group scales of the keys / values (INT8 cache) */
    alignas(16) __half vsc[KV8 ? 64 * 4 : 8];
    alignas(16) float w[KV8 ? 64 * 4 * 4 : 64 * 4]; /* value-sum weights: [position][value group][head] or [position][head] */
};

template <bool KV8, int NW> struct AttnWarpSmem {
    AttnWarpTile<KV8> tile[NW];
    alignas(16) float sq[4][128];
    int s_last;
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

/* `rows` cached vectors of `vb` bytes each, contiguous in global memory, to rows `stride` bytes apart */
template <int VB, int STRIDE>
__device__ __forceinline__ void warp_copy_rows(unsigned char* dst, const unsigned char* src, int rows, bool al16, int lane) {
    if (al16) {
        constexpr int CPR = VB / 16; /* requests per row */
        const int r0 = lane / CPR, c = lane % CPR;
#pragma unroll 4
        for (int r = r0; r < rows; r += 32 / CPR) cp_async16(dst + r * STRIDE + c * 16, src + (size_t)r * VB + c * 16);
    } else {
        for (int i = lane; i < rows * (VB / 4); i += 32) {
            const int r = i / (VB / 4), c = i - r * (VB / 4);
            cp_async4(dst + r * STRIDE + c * 4, src + (size_t)r * VB + c * 4);
        }
    }
}
/* the f16 group scales of `rows` positions (8 bytes each, contiguous) */
__device__ __forceinline__ void warp_copy_scales(__half* dst, const __half* src, int rows, bool al16, int lane) {
    if (al16) {
        for (int i = lane; i < (rows + 1) / 2; i += 32) cp_async16(dst + i * 8, src + i * 8); /* an odd count reads one slot more; the cache has an even number */
    } else {
        for (int i = lane; i < rows * 2; i += 32) cp_async4(dst + i * 2, src + i * 2);
    }
}

constexpr int ATTN_WARP_RUN = 4;

template <bool KV8, int NW>
__global__ void __launch_bounds__(NW * 32) k_attn_decode_warp(AttnArgs a) {
    extern __shared__ __align__(16) unsigned char attn_warp_smem[];
    AttnWarpSmem<KV8, NW>& sm = *reinterpret_cast<AttnWarpSmem<KV8, NW>*>(attn_warp_smem);
    constexpr int VB = AttnWarpTile<KV8>::VB;
    constexpr int KS = AttnWarpTile<KV8>::KS;
    const int row = blockIdx.x, kvh = blockIdx.y, wk = blockIdx.z, workers = gridDim.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int QH = a.q_heads, KVH = a.kv_heads;
    const int pos = a.pos_arr ? __ldg(a.pos_arr + row) : a.pos0 + row * a.pos_row_step;
    const int len = pos + 1;
    const int n_active = (len + 63) >> 6;
    const size_t plane = (size_t)kvh * a.max_seq;
    const unsigned char* kc = kv_payload(a.kv, row) + a.kv.k_off;
    const unsigned char* vc = kv_payload(a.kv, row) + a.kv.v_off;
    const __half* ks = KV8 ? reinterpret_cast<const __half*>(kv_scales(a.kv, row) + a.kv.ks_off) : nullptr;
    const __half* vs = KV8 ? reinterpret_cast<const __half*>(kv_scales(a.kv, row) + a.kv.vs_off) : nullptr;
    const bool al16 = ((((uintptr_t)kc) | ((uintptr_t)vc) | ((uintptr_t)ks) | ((uintptr_t)vs)) & 15u) == 0;

    AttnWarpTile<KV8>& T = sm.tile[warp];
    /* The grid is fixed per batch size (one captured graph serves every context length), so the CTAs
     * decide here how many of the `workers` per (row, kv head) take part: enough warps for about
     * ATTN_WARP_RUN splits each, so that the copies of one split overlap the arithmetic of another,
     * but never so few CTAs that SMs stay empty.  The others go straight to the arrival counter. */
    const int fill = (2 * 148 + (int)(gridDim.x * gridDim.y) - 1) / (int)(gridDim.x * gridDim.y);
    const int eff = min(workers, max(max(n_active / (NW * ATTN_WARP_RUN), fill), 1));
    /* this warp's splits: first, first + step, ... */
    const int first = wk < eff ? wk + eff * warp : n_active, step = eff * NW;

    auto fetch_k = [&](int spl) {
        if (spl < n_active) {
            const int start = spl << 6, cnt = min(64, len - start);
            warp_copy_rows<VB, KS>(T.k, kc + (plane + start) * VB, cnt, al16, lane);
            if (KV8) warp_copy_scales(T.ksc, ks + (plane + start) * 4, cnt, al16, lane);
        }
        cp_async_commit(); /* also when empty: the waits below count groups */
    };
    auto fetch_v = [&](int spl) {
        if (spl < n_active) {
            const int start = spl << 6, cnt = min(64, len - start);
            warp_copy_rows<VB, VB>(T.v, vc + (plane + start) * VB, cnt, al16, lane);
            if (KV8) warp_copy_scales(T.vsc, vs + (plane + start) * 4, cnt, al16, lane);
        }
        cp_async_commit();
    };
    fetch_k(first);
    fetch_v(first);

    {   /* queries of the four heads sharing this kv head, pre-scaled */
        const float scale = rsqrtf(128.0f);
        for (int i = tid; i < 512; i += NW * 32) {
            const int g = i >> 7, t = i & 127;
            const float v = bf2f(a.q[((size_t)row * QH + kvh * 4 + g) * 128 + t]);
            sm.sq[g][t] = __fmul_rn(v, scale);
        }
    }
    __syncthreads();

    for (int spl = first; spl < n_active; spl += step) {
        const int start = spl << 6;
        const int cnt = min(64, len - start);
        cp_async_wait<1>(); /* this split's keys have landed (its values may still be on the way) */
        __syncwarp();

        /* ---- scores: positions lane and lane + 32, four heads each ---- */
        float d[2][4];
#pragma unroll
        for (int p = 0; p < 2; p++)
#pragma unroll
            for (int h = 0; h < 4; h++) d[p][h] = 0.f;
        const uint4* k0p = reinterpret_cast<const uint4*>(T.k + lane * KS);
        const uint4* k1p = reinterpret_cast<const uint4*>(T.k + (lane + 32) * KS);
        if (KV8) {
            const uint2 s0 = *reinterpret_cast<const uint2*>(T.ksc + lane * 4);
            const uint2 s1 = *reinterpret_cast<const uint2*>(T.ksc + (lane + 32) * 4);
            const __half2 s0a = *reinterpret_cast<const __half2*>(&s0.x), s0b = *reinterpret_cast<const __half2*>(&s0.y);
            const __half2 s1a = *reinterpret_cast<const __half2*>(&s1.x), s1b = *reinterpret_cast<const __half2*>(&s1.y);
            const float ksf[2][4] = {{__low2float(s0a), __high2float(s0a), __low2float(s0b), __high2float(s0b)},
                                     {__low2float(s1a), __high2float(s1a), __low2float(s1b), __high2float(s1b)}};
#pragma unroll
            for (int gi = 0; gi < 4; gi++) {
                float pp[2][4];
#pragma unroll
                for (int p = 0; p < 2; p++)
#pragma unroll
                    for (int h = 0; h < 4; h++) pp[p][h] = 0.f;
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const uint4 ka = k0p[gi * 2 + c], kb = k1p[gi * 2 + c];
                    const uint32_t wa[4] = {ka.x, ka.y, ka.z, ka.w}, wb[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
                    for (int wi = 0; wi < 4; wi++) {
                        const uint32_t ua = s8x4_bias(wa[wi]), ub = s8x4_bias(wb[wi]);
                        const float ka0 = s8_biased_to_f32<0>(ua), ka1 = s8_biased_to_f32<1>(ua), ka2 = s8_biased_to_f32<2>(ua), ka3 = s8_biased_to_f32<3>(ua);
                        const float kb0 = s8_biased_to_f32<0>(ub), kb1 = s8_biased_to_f32<1>(ub), kb2 = s8_biased_to_f32<2>(ub), kb3 = s8_biased_to_f32<3>(ub);
#pragma unroll
                        for (int h = 0; h < 4; h++) {
                            const float4 qv = reinterpret_cast<const float4*>(sm.sq[h])[gi * 8 + c * 4 + wi];
                            pp[0][h] = __fmaf_rn(qv.x, ka0, pp[0][h]);
                            pp[0][h] = __fmaf_rn(qv.y, ka1, pp[0][h]);
                            pp[0][h] = __fmaf_rn(qv.z, ka2, pp[0][h]);
                            pp[0][h] = __fmaf_rn(qv.w, ka3, pp[0][h]);
                            pp[1][h] = __fmaf_rn(qv.x, kb0, pp[1][h]);
                            pp[1][h] = __fmaf_rn(qv.y, kb1, pp[1][h]);
                            pp[1][h] = __fmaf_rn(qv.z, kb2, pp[1][h]);
                            pp[1][h] = __fmaf_rn(qv.w, kb3, pp[1][h]);
                        }
                    }
                }
#pragma unroll
                for (int p = 0; p < 2; p++)
#pragma unroll
                    for (int h = 0; h < 4; h++) d[p][h] = __fmaf_rn(pp[p][h], ksf[p][gi], d[p][h]);
            }
        } else {
#pragma unroll 2
            for (int c = 0; c < 16; c++) { /* 8 bf16 per 16-byte request */
                const uint4 ka = k0p[c], kb = k1p[c];
                const uint32_t wa[4] = {ka.x, ka.y, ka.z, ka.w}, wb[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
                for (int wi = 0; wi < 4; wi += 2) {
                    const float ka0 = bf_lo(wa[wi]), ka1 = bf_hi(wa[wi]), ka2 = bf_lo(wa[wi + 1]), ka3 = bf_hi(wa[wi + 1]);
                    const float kb0 = bf_lo(wb[wi]), kb1 = bf_hi(wb[wi]), kb2 = bf_lo(wb[wi + 1]), kb3 = bf_hi(wb[wi + 1]);
#pragma unroll
                    for (int h = 0; h < 4; h++) {
                        const float4 qv = reinterpret_cast<const float4*>(sm.sq[h])[c * 2 + (wi >> 1)];
                        d[0][h] = __fmaf_rn(qv.x, ka0, d[0][h]);
                        d[0][h] = __fmaf_rn(qv.y, ka1, d[0][h]);
                        d[0][h] = __fmaf_rn(qv.z, ka2, d[0][h]);
                        d[0][h] = __fmaf_rn(qv.w, ka3, d[0][h]);
                        d[1][h] = __fmaf_rn(qv.x, kb0, d[1][h]);
                        d[1][h] = __fmaf_rn(qv.y, kb1, d[1][h]);
                        d[1][h] = __fmaf_rn(qv.z, kb2, d[1][h]);
                        d[1][h] = __fmaf_rn(qv.w, kb3, d[1][h]);
                    }
                }
            }
        }
        __syncwarp();          /* every lane is through with the key tile */
        fetch_k(spl + step);   /* the next split's keys travel during the value sum */

        /* ---- split max, probabilities, exp-sum ---- */
        const bool in0 = lane < cnt, in1 = lane + 32 < cnt;
        float m[4], l[4], pr[2][4];
#pragma unroll
        for (int h = 0; h < 4; h++) {
            const float d0 = in0 ? d[0][h] : -INFINITY, d1 = in1 ? d[1][h] : -INFINITY;
            m[h] = warp_tree_max(fmaxf(d0, d1));
            pr[0][h] = in0 ? expf(d0 - m[h]) : 0.f;
            pr[1][h] = in1 ? expf(d1 - m[h]) : 0.f;
            l[h] = warp_tree_sum(pr[0][h] + pr[1][h]);
        }
        cp_async_wait<1>(); /* this split's values (and their scales) have landed */
        __syncwarp();
        /* weights of the value sum: the probability, for the INT8 cache times the value group's scale */
#pragma unroll
        for (int p = 0; p < 2; p++) {
            const int j = lane + 32 * p;
            if (KV8) {
                const uint2 sv = *reinterpret_cast<const uint2*>(T.vsc + j * 4);
                const __half2 sva = *reinterpret_cast<const __half2*>(&sv.x), svb = *reinterpret_cast<const __half2*>(&sv.y);
                const float vsf[4] = {__low2float(sva), __high2float(sva), __low2float(svb), __high2float(svb)};
#pragma unroll
                for (int grp = 0; grp < 4; grp++)
                    reinterpret_cast<float4*>(T.w)[j * 4 + grp] =
                        make_float4(__fmul_rn(pr[p][0], vsf[grp]), __fmul_rn(pr[p][1], vsf[grp]), __fmul_rn(pr[p][2], vsf[grp]),
                                    __fmul_rn(pr[p][3], vsf[grp]));
            } else {
                reinterpret_cast<float4*>(T.w)[j] = make_float4(pr[p][0], pr[p][1], pr[p][2], pr[p][3]);
            }
        }
        __syncwarp();

        /* ---- value sum: dimensions 4 lane .. 4 lane + 3, four heads ---- */
        float acc[4][4];
#pragma unroll
        for (int h = 0; h < 4; h++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[h][i] = 0.f;
        const float4* wp = reinterpret_cast<const float4*>(T.w) + (KV8 ? (lane >> 3) : 0);
#pragma unroll 4
        for (int j = 0; j < cnt; j++) {
            float v0, v1, v2, v3;
            if (KV8) {
                const uint32_t u = s8x4_bias(*reinterpret_cast<const uint32_t*>(T.v + j * VB + lane * 4));
                v0 = s8_biased_to_f32<0>(u); v1 = s8_biased_to_f32<1>(u); v2 = s8_biased_to_f32<2>(u); v3 = s8_biased_to_f32<3>(u);
            } else {
                const uint2 u = *reinterpret_cast<const uint2*>(T.v + j * VB + lane * 8);
                v0 = bf_lo(u.x); v1 = bf_hi(u.x); v2 = bf_lo(u.y); v3 = bf_hi(u.y);
            }
            const float4 wj = wp[KV8 ? j * 4 : j];
            const float wh[4] = {wj.x, wj.y, wj.z, wj.w};
#pragma unroll
            for (int h = 0; h < 4; h++) {
                acc[h][0] = __fmaf_rn(wh[h], v0, acc[h][0]);
                acc[h][1] = __fmaf_rn(wh[h], v1, acc[h][1]);
                acc[h][2] = __fmaf_rn(wh[h], v2, acc[h][2]);
                acc[h][3] = __fmaf_rn(wh[h], v3, acc[h][3]);
            }
        }
        __syncwarp();          /* every lane is through with the value tile and the weights */
        fetch_v(spl + step);   /* the next split's values travel during its scores */

#pragma unroll
        for (int h = 0; h < 4; h++) {
            float* ph = a.part + (((size_t)row * QH + kvh * 4 + h) * a.n_split_slots + spl) * 130;
            if (lane == 0) *reinterpret_cast<float2*>(ph) = make_float2(m[h], l[h]);
            *reinterpret_cast<float2*>(ph + 2 + 4 * lane) = make_float2(acc[h][0], acc[h][1]);
            *reinterpret_cast<float2*>(ph + 4 + 4 * lane) = make_float2(acc[h][2], acc[h][3]);
        }
    }
    cp_async_wait<0>();

    /* the last CTA of this (row, kv head) to finish merges the partials in ascending split order */
    __threadfence();
    __syncthreads();
    unsigned int* ctr = a.counters + (size_t)row * KVH + kvh;
    if (tid == 0) sm.s_last = (atomicAdd(ctr, 1u) == (unsigned)(workers - 1));
    __syncthreads();
    if (sm.s_last) {
        __threadfence();
        /* The tiles are idle now: they take, per (head, split), the split's max (then its merge weight)
         * and its exp-sum, so that each weight's expf is evaluated once instead of once per dimension. */
        float* wm = reinterpret_cast<float*>(attn_warp_smem); /* [4][n_active] */
        float* wl = wm + 4 * n_active;                        /* [4][n_active] */
        float* hmax = wl + 4 * n_active;                      /* [4] */
        const float* pb0 = a.part + ((size_t)row * QH + kvh * 4) * a.n_split_slots * 130;
        for (int i = tid; i < 4 * n_active; i += NW * 32) {
            const int g = i / n_active, sidx = i - g * n_active;
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(pb0 + ((size_t)g * a.n_split_slots + sidx) * 130));
            wm[i] = ml.x; wl[i] = ml.y;
        }
        __syncthreads();
        for (int g = warp; g < 4; g += NW) {
            float M = -INFINITY;
            for (int sidx = lane; sidx < n_active; sidx += 32) M = fmaxf(M, wm[g * n_active + sidx]);
            M = warp_tree_max(M);
            if (lane == 0) hmax[g] = M;
        }
        __syncthreads();
        for (int i = tid; i < 4 * n_active; i += NW * 32) wm[i] = expf(wm[i] - hmax[i / n_active]);
        __syncthreads();
        /* one thread per dimension carries the four heads' chains side by side: four independent loads per
         * split, eight splits ahead, instead of four passes of dependent L2 round trips */
        for (int dd = tid; dd < 128; dd += NW * 32) {
            const float* pa = pb0 + 2 + dd;
            const size_t hs = (size_t)a.n_split_slots * 130;
            float l[4] = {0.f, 0.f, 0.f, 0.f}, acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
            for (int sidx = 0; sidx < n_active; sidx++) {
#pragma unroll
                for (int g = 0; g < 4; g++) {
                    const float av = __ldcg(pa + g * hs + (size_t)sidx * 130);
                    const float ls = wl[g * n_active + sidx], w = wm[g * n_active + sidx];
                    if (ls != 0.f) { /* an empty split leaves the sums untouched */
                        l[g] = __fmaf_rn(ls, w, l[g]);
                        acc[g] = __fmaf_rn(av, w, acc[g]);
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < 4; g++) a.out[((size_t)row * QH + kvh * 4 + g) * 128 + dd] = f2bf(__fdiv_rn(acc[g], l[g]));
        }
        if (tid == 0) *ctr = 0u;
    }
}

}  // namespace s2p
