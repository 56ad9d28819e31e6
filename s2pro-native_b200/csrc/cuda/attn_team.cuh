/* Split-K decode attention for lockstep batches: a TEAM of two warps per 64-position split.
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
 * CTA barriers per split with three quarters of the CTA idle in the value phase; on a lockstep batch
 * of 32 rows x 8192 positions it issues about twice the instructions the arithmetic needs and reads
 * the cache at a fifth of the HBM rate.  Here two warps own a split from the copy to the partial:
 *   scores   warp 0 carries positions 0..31, warp 1 positions 32..63: one position per lane with the
 *            four heads' chains side by side, so a key word is converted once for the four heads;
 *   softmax  each warp reduces its half by shuffles (the four heads' trees packed into one: 6 shuffles
 *            instead of 20); the halves meet through eight floats in shared
 *            memory.  The exp-sum starts with the pairs (t, t+32), i.e. one value of either warp:
 *            the probabilities go through a 1 KB buffer and every lane adds its pair itself;
 *   values   warp 0 carries dimensions 0..63, warp 1 dimensions 64..127 (two per lane, four heads):
 *            a value is converted once for the four heads.
 * Four 64-thread named barriers per split order the hand-overs.  The K and V tiles of a team are
 * single-buffered: the next split's keys are copied (cp.async, 16 bytes per request) while the
 * values of this one are summed, the next values while the next scores are formed.  Key rows are
 * staged with a 16-byte pad per row, which makes the per-lane 16-byte reads of 32 different rows
 * conflict-free.  Two CTAs of four teams fit an SM (16 warps); the kernel is bound by instruction
 * issue on dependent chains, not by HBM, so warps per SM and instructions per split are what count
 * (one warp per split with twice the tiles per warp measured 6 % slower on INT8, 24 % on bf16).
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

template <bool KV8> struct AttnSplitTile {
    static constexpr int VB = KV8 ? 128 : 256;  /* payload bytes per cached vector */
    static constexpr int KS = VB + 16;          /* staged key row stride */
    alignas(16) unsigned char k[64 * KS];
    alignas(16) unsigned char v[64 * VB];
    alignas(16) __half ksc[KV8 ? 64 * 4 : 8];   /* group scales of the keys / values (INT8 cache) */
    alignas(16) __half vsc[KV8 ? 64 * 4 : 8];
    alignas(16) float w[KV8 ? 64 * 4 * 4 : 64 * 4]; /* value-sum weights: [position][value group][head] or [position][head] */
};


__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }


/* Merge of the per-split partials of one (row, kv head) in ascending split order, by the CTA that
 * arrived last: w = expf(m_s - M), l = fma(l_s, w, l), acc = fma(acc_s, w, acc), out = acc / l.
 * `scratch` (the CTA's idle tiles) takes, per (head, split), the split's max (then its merge weight)
 * and its exp-sum, so that each weight's expf is evaluated once instead of once per dimension; it
 * needs 8 floats per split and 4 more. */
template <int THREADS>
__device__ __forceinline__ void attn_merge_partials(const AttnArgs& a, int row, int kvh, int n_active, float* scratch) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int QH = a.q_heads;
    __threadfence();
    float* wm = scratch;              /* [4][n_active] */
    float* wl = wm + 4 * n_active;    /* [4][n_active] */
    float* hmax = wl + 4 * n_active;  /* [4] */
    const float* pb0 = a.part + ((size_t)row * QH + kvh * 4) * a.n_split_slots * 130;
    for (int i = tid; i < 4 * n_active; i += THREADS) {
        const int g = i / n_active, sidx = i - g * n_active;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(pb0 + ((size_t)g * a.n_split_slots + sidx) * 130));
        wm[i] = ml.x; wl[i] = ml.y;
    }
    __syncthreads();
    for (int g = warp; g < 4; g += THREADS / 32) {
        float M = -INFINITY;
        for (int sidx = lane; sidx < n_active; sidx += 32) M = fmaxf(M, wm[g * n_active + sidx]);
        M = warp_tree_max(M);
        if (lane == 0) hmax[g] = M;
    }
    __syncthreads();
    for (int i = tid; i < 4 * n_active; i += THREADS) wm[i] = expf(wm[i] - hmax[i / n_active]);
    __syncthreads();
    /* a thread carries the chains of HP heads of one dimension side by side: independent loads, eight
     * splits ahead, instead of passes of dependent L2 round trips */
    constexpr int HP = THREADS >= 256 ? 2 : 4;
    for (int i = tid; i < 128 * (4 / HP); i += THREADS) {
        const int dd = i & 127, g0 = (i >> 7) * HP;
        const size_t hs = (size_t)a.n_split_slots * 130;
        const float* pa = pb0 + g0 * hs + 2 + dd;
        float l[HP], acc[HP];
#pragma unroll
        for (int g = 0; g < HP; g++) { l[g] = 0.f; acc[g] = 0.f; }
#pragma unroll 8
        for (int sidx = 0; sidx < n_active; sidx++) {
#pragma unroll
            for (int g = 0; g < HP; g++) {
                const float av = __ldcg(pa + g * hs + (size_t)sidx * 130);
                const float ls = wl[(g0 + g) * n_active + sidx], w = wm[(g0 + g) * n_active + sidx];
                if (ls != 0.f) { /* an empty split leaves the sums untouched */
                    l[g] = __fmaf_rn(ls, w, l[g]);
                    acc[g] = __fmaf_rn(av, w, acc[g]);
                }
            }
        }
#pragma unroll
        for (int g = 0; g < HP; g++) a.out[((size_t)row * QH + kvh * 4 + g0 + g) * 128 + dd] = f2bf(__fdiv_rn(acc[g], l[g]));
    }
}

constexpr int ATTN_SPLITS_PER_TEAM = 4; /* splits a team should get before more workers join */

template <bool KV8> struct AttnTeamTile {
    AttnSplitTile<KV8> t;
    alignas(16) float p[64 * 4];  /* probabilities [position][head] */
    alignas(16) float xm[2][4];   /* split max of either half, per head */
};

template <bool KV8, int NT> struct AttnTeamSmem {
    AttnTeamTile<KV8> tile[NT];
    alignas(16) float sq[4][128];
    int s_last;
};

__device__ __forceinline__ void team_sync(int team) {
    asm volatile("bar.sync %0, 64;" ::"r"(team + 1) : "memory");
}

/* `rows` cached vectors to rows `STRIDE` bytes apart, by the 64 threads of a team */
template <int VB, int STRIDE>
__device__ __forceinline__ void team_copy_rows(unsigned char* dst, const unsigned char* src, int rows, bool al16, int t64) {
    if (al16) {
        constexpr int CPR = VB / 16; /* requests per row */
        const int r0 = t64 / CPR, c = t64 % CPR;
#pragma unroll 4
        for (int r = r0; r < rows; r += 64 / CPR) cp_async16(dst + r * STRIDE + c * 16, src + (size_t)r * VB + c * 16);
    } else {
        for (int i = t64; i < rows * (VB / 4); i += 64) {
            const int r = i / (VB / 4), c = i - r * (VB / 4);
            cp_async4(dst + r * STRIDE + c * 4, src + (size_t)r * VB + c * 4);
        }
    }
}
__device__ __forceinline__ void team_copy_scales(__half* dst, const __half* src, int rows, bool al16, int t64) {
    if (al16) {
        if (t64 < (rows + 1) / 2) cp_async16(dst + t64 * 8, src + t64 * 8); /* an odd count reads one slot more; the cache has an even number */
    } else {
        for (int i = t64; i < rows * 2; i += 64) cp_async4(dst + i * 2, src + i * 2);
    }
}

template <bool KV8, int NT>
__global__ void __launch_bounds__(NT * 64) k_attn_decode_team(AttnArgs a) {
    extern __shared__ __align__(16) unsigned char attn_team_smem[];
    AttnTeamSmem<KV8, NT>& sm = *reinterpret_cast<AttnTeamSmem<KV8, NT>*>(attn_team_smem);
    constexpr int VB = AttnSplitTile<KV8>::VB;
    constexpr int KS = AttnSplitTile<KV8>::KS;
    const int row = blockIdx.x, kvh = blockIdx.y, wk = blockIdx.z, workers = gridDim.z;
    const int tid = threadIdx.x, lane = tid & 31, team = tid >> 6, half = (tid >> 5) & 1, t64 = tid & 63;
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

    AttnTeamTile<KV8>& TT = sm.tile[team];
    AttnSplitTile<KV8>& T = TT.t;
    /* The grid is fixed per batch size (one captured graph serves every context length), so the CTAs
     * decide here how many of the `workers` per (row, kv head) take part: enough teams for about
     * ATTN_SPLITS_PER_TEAM splits each, so that the copies of one split overlap the arithmetic of
     * another, but never so few CTAs that SMs stay empty.  The others go straight to the arrival counter. */
    const int fill = (2 * 148 + (int)(gridDim.x * gridDim.y) - 1) / (int)(gridDim.x * gridDim.y);
    const int eff = min(workers, max(max(n_active / (NT * ATTN_SPLITS_PER_TEAM), fill), 1));
    const int first = wk < eff ? wk + eff * team : n_active, step = eff * NT;

    auto fetch_k = [&](int spl) {
        if (spl < n_active) {
            const int start = spl << 6, cnt = min(64, len - start);
            team_copy_rows<VB, KS>(T.k, kc + (plane + start) * VB, cnt, al16, t64);
            if (KV8) team_copy_scales(T.ksc, ks + (plane + start) * 4, cnt, al16, t64);
        }
        cp_async_commit(); /* also when empty: the waits below count groups */
    };
    auto fetch_v = [&](int spl) {
        if (spl < n_active) {
            const int start = spl << 6, cnt = min(64, len - start);
            team_copy_rows<VB, VB>(T.v, vc + (plane + start) * VB, cnt, al16, t64);
            if (KV8) team_copy_scales(T.vsc, vs + (plane + start) * 4, cnt, al16, t64);
        }
        cp_async_commit();
    };
    fetch_k(first);
    fetch_v(first);

    {   /* queries of the four heads sharing this kv head, pre-scaled */
        const float scale = rsqrtf(128.0f);
        for (int i = tid; i < 512; i += NT * 64) {
            const int g = i >> 7, t = i & 127;
            const float v = bf2f(a.q[((size_t)row * QH + kvh * 4 + g) * 128 + t]);
            sm.sq[g][t] = __fmul_rn(v, scale);
        }
    }
    __syncthreads();

    const int j_own = lane + 32 * half;            /* the position this lane scores */
    const int d_own = 64 * half + 2 * lane;        /* the first of the two dimensions this lane sums */
    for (int spl = first; spl < n_active; spl += step) {
        const int start = spl << 6;
        const int cnt = min(64, len - start);
        cp_async_wait<1>(); /* own requests for this split's keys are through ... */
        team_sync(team);    /* ... and so are the other threads' */

        /* ---- scores: one position, four heads ---- */
        float d[4] = {0.f, 0.f, 0.f, 0.f};
        const uint4* kp = reinterpret_cast<const uint4*>(T.k + j_own * KS);
        if (KV8) {
            const uint2 s0 = *reinterpret_cast<const uint2*>(T.ksc + j_own * 4);
            const __half2 s0a = *reinterpret_cast<const __half2*>(&s0.x), s0b = *reinterpret_cast<const __half2*>(&s0.y);
            const float ksf[4] = {__low2float(s0a), __high2float(s0a), __low2float(s0b), __high2float(s0b)};
#pragma unroll
            for (int gi = 0; gi < 4; gi++) {
                float pp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const uint4 ka = kp[gi * 2 + c];
                    const uint32_t wa[4] = {ka.x, ka.y, ka.z, ka.w};
#pragma unroll
                    for (int wi = 0; wi < 4; wi++) {
                        const uint32_t ua = s8x4_bias(wa[wi]);
                        const float k0 = s8_biased_to_f32<0>(ua), k1 = s8_biased_to_f32<1>(ua), k2 = s8_biased_to_f32<2>(ua), k3 = s8_biased_to_f32<3>(ua);
#pragma unroll
                        for (int h = 0; h < 4; h++) {
                            const float4 qv = reinterpret_cast<const float4*>(sm.sq[h])[gi * 8 + c * 4 + wi];
                            pp[h] = __fmaf_rn(qv.x, k0, pp[h]);
                            pp[h] = __fmaf_rn(qv.y, k1, pp[h]);
                            pp[h] = __fmaf_rn(qv.z, k2, pp[h]);
                            pp[h] = __fmaf_rn(qv.w, k3, pp[h]);
                        }
                    }
                }
#pragma unroll
                for (int h = 0; h < 4; h++) d[h] = __fmaf_rn(pp[h], ksf[gi], d[h]);
            }
        } else {
#pragma unroll 4
            for (int c = 0; c < 16; c++) { /* 8 bf16 per 16-byte request */
                const uint4 ka = kp[c];
                const uint32_t wa[4] = {ka.x, ka.y, ka.z, ka.w};
#pragma unroll
                for (int wi = 0; wi < 4; wi += 2) {
                    const float k0 = bf_lo(wa[wi]), k1 = bf_hi(wa[wi]), k2 = bf_lo(wa[wi + 1]), k3 = bf_hi(wa[wi + 1]);
#pragma unroll
                    for (int h = 0; h < 4; h++) {
                        const float4 qv = reinterpret_cast<const float4*>(sm.sq[h])[c * 2 + (wi >> 1)];
                        d[h] = __fmaf_rn(qv.x, k0, d[h]);
                        d[h] = __fmaf_rn(qv.y, k1, d[h]);
                        d[h] = __fmaf_rn(qv.z, k2, d[h]);
                        d[h] = __fmaf_rn(qv.w, k3, d[h]);
                    }
                }
            }
        }
        const bool in = j_own < cnt;
#pragma unroll
        for (int h = 0; h < 4; h++) d[h] = in ? d[h] : -INFINITY;
        {   /* the four heads' maxima over this warp's 32 positions in one packed tree: lane 8 h holds head h's */
            const float mx = warp_tree4<true>(d[0], d[1], d[2], d[3], lane);
            if ((lane & 7) == 0) TT.xm[half][lane >> 3] = mx;
        }
        cp_async_wait<0>(); /* own requests for this split's values are through */
        team_sync(team);    /* the halves' maxima are out, nobody reads the key tile any more, the value tile is complete */
        fetch_k(spl + step);

        /* ---- probabilities and the weights of the value sum ---- */
        float m[4], pr[4];
#pragma unroll
        for (int h = 0; h < 4; h++) {
            m[h] = fmaxf(TT.xm[0][h], TT.xm[1][h]);
            pr[h] = in ? expf(d[h] - m[h]) : 0.f;
        }
        reinterpret_cast<float4*>(TT.p)[j_own] = make_float4(pr[0], pr[1], pr[2], pr[3]);
        if (KV8) {
            const uint2 sv = *reinterpret_cast<const uint2*>(T.vsc + j_own * 4);
            const __half2 sva = *reinterpret_cast<const __half2*>(&sv.x), svb = *reinterpret_cast<const __half2*>(&sv.y);
            const float vsf[4] = {__low2float(sva), __high2float(sva), __low2float(svb), __high2float(svb)};
#pragma unroll
            for (int grp = 0; grp < 4; grp++)
                reinterpret_cast<float4*>(T.w)[j_own * 4 + grp] =
                    make_float4(__fmul_rn(pr[0], vsf[grp]), __fmul_rn(pr[1], vsf[grp]), __fmul_rn(pr[2], vsf[grp]), __fmul_rn(pr[3], vsf[grp]));
        }
        team_sync(team);

        /* exp-sum: the pair (lane, lane + 32), then the 16..1 tree of the four heads packed into one; the first
         * warp does it and its lane 8 h stores head h's (max, sum) */
        if (half == 0) {
            const float4 pa = reinterpret_cast<const float4*>(TT.p)[lane], pb = reinterpret_cast<const float4*>(TT.p)[lane + 32];
            const float lsum = warp_tree4<false>(pa.x + pb.x, pa.y + pb.y, pa.z + pb.z, pa.w + pb.w, lane);
            if ((lane & 7) == 0) {
                const int h = lane >> 3;
                const float mh = h == 0 ? m[0] : h == 1 ? m[1] : h == 2 ? m[2] : m[3];
                *reinterpret_cast<float2*>(a.part + (((size_t)row * QH + kvh * 4 + h) * a.n_split_slots + spl) * 130) = make_float2(mh, lsum);
            }
        }

        /* ---- value sum: two dimensions, four heads ---- */
        float acc[4][2];
#pragma unroll
        for (int h = 0; h < 4; h++) { acc[h][0] = 0.f; acc[h][1] = 0.f; }
        const float4* wp = KV8 ? reinterpret_cast<const float4*>(T.w) + (d_own >> 5) : reinterpret_cast<const float4*>(TT.p);
#pragma unroll 8
        for (int j = 0; j < cnt; j++) {
            float v0, v1;
            if (KV8) {
                const uint32_t u = (uint32_t)*reinterpret_cast<const unsigned short*>(T.v + j * VB + d_own) ^ 0x8080u;
                v0 = s8_biased_to_f32<0>(u); v1 = s8_biased_to_f32<1>(u);
            } else {
                const uint32_t u = *reinterpret_cast<const uint32_t*>(T.v + j * VB + d_own * 2);
                v0 = bf_lo(u); v1 = bf_hi(u);
            }
            const float4 wj = wp[KV8 ? j * 4 : j];
            acc[0][0] = __fmaf_rn(wj.x, v0, acc[0][0]); acc[0][1] = __fmaf_rn(wj.x, v1, acc[0][1]);
            acc[1][0] = __fmaf_rn(wj.y, v0, acc[1][0]); acc[1][1] = __fmaf_rn(wj.y, v1, acc[1][1]);
            acc[2][0] = __fmaf_rn(wj.z, v0, acc[2][0]); acc[2][1] = __fmaf_rn(wj.z, v1, acc[2][1]);
            acc[3][0] = __fmaf_rn(wj.w, v0, acc[3][0]); acc[3][1] = __fmaf_rn(wj.w, v1, acc[3][1]);
        }
        team_sync(team);       /* the value tile, the weights and the probabilities are free */
        fetch_v(spl + step);

#pragma unroll
        for (int h = 0; h < 4; h++) {
            float* ph = a.part + (((size_t)row * QH + kvh * 4 + h) * a.n_split_slots + spl) * 130;
            *reinterpret_cast<float2*>(ph + 2 + d_own) = make_float2(acc[h][0], acc[h][1]);
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
        attn_merge_partials<NT * 64>(a, row, kvh, n_active, reinterpret_cast<float*>(attn_team_smem));
        if (tid == 0) *ctr = 0u;
    }
}

}  // namespace s2p
