/* Single-pass causal attention for a prompt slice: a block of RB consecutive query rows of ONE session per CTA.
 *
 * Arithmetic per (row, head): that of the single-row kernel in prims.cu (the reference's k_attention /
 * k_attention8, src/slowar/kernels.cu:234-309 and :625-728) - tiles of 128 cached positions, per position one
 * 128-term fma chain against the pre-scaled query (INT8 cache: four 32-term chains folded with the f16 group scale),
 * tile max and sum by 128-wide halving trees, l = fma(l, corr, tile_sum), acc *= corr, then one fma per position in
 * ascending order - so the outputs are the same bits.
 *
 * What the row block buys.  The single-row kernel stages a K and a V tile per (row, kv head), converts every cached
 * value for that one row and crosses ~20 CTA barriers per tile: a 512-token prompt spends 13 of its 29 ms there, an
 * 8192-token prompt 2.8 of 2.9 s.  Here a tile is staged once for RB rows, a cached key or value is read and
 * converted once and feeds RB chains held side by side in registers, and the trees of the RB rows share their
 * barriers.  (RB = 4 in the product: 64 registers, two CTAs per SM.)  Rows of a block differ only in how far they may look: row i of the block sees positions below
 * len0 + i, which only matters in the block's last one or two tiles; there the chains of positions a row may not see
 * yield -inf / probability 0 and its value sum skips them, exactly as the single-row loop ends earlier.
 *
 * Thread (g, t) of 512: head g of the kv head's four; t is a cached position of the tile in the score phase and a
 * head dimension in the value phase.
 */
#pragma once
#include <math.h>
#include "common.cuh"
#include "headops.cuh"
#include "ops.h"

namespace s2p {

template <bool KV8, int RB> struct AttnPrefillSmem {
    static constexpr int VB = KV8 ? 128 : 256; /* payload bytes per cached vector */
    static constexpr int TS = VB + 4;          /* staged row stride: word reads of 32 different rows hit 32 banks */
    alignas(16) unsigned char tile[128 * TS];  /* K rows of the tile, then its V rows */
    alignas(16) __half ssc[128 * 4];           /* group scales of the keys (INT8 cache) */
    alignas(16) __half vssc[128 * 4];          /* ... and of the values, staged with the keys */
    alignas(16) float sq[RB][4][128];          /* pre-scaled queries */
    alignas(16) float red[RB][4][128];         /* tree scratch */
    /* weights of the value sum: [row][head][value group][position] = probability x the group's scale (INT8 cache),
     * or [row][head][0][position] = probability (bf16 cache) */
    alignas(16) float spv[RB][4][KV8 ? 4 : 1][128];
};

template <bool KV8, int RB>
__global__ void __launch_bounds__(512) k_attn_prefill(AttnArgs a, int rows) {
    extern __shared__ __align__(16) unsigned char attn_prefill_smem[];
    AttnPrefillSmem<KV8, RB>& sm = *reinterpret_cast<AttnPrefillSmem<KV8, RB>*>(attn_prefill_smem);
    constexpr int VB = AttnPrefillSmem<KV8, RB>::VB, TS = AttnPrefillSmem<KV8, RB>::TS;
    /* the last rows of the slice look furthest back: their blocks start first, the short ones fill in behind them */
    const int r0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * RB, kvh = blockIdx.y;
    const int rb = min(RB, rows - r0);
    const int g = threadIdx.x >> 7, t = threadIdx.x & 127;
    const int QH = a.q_heads, h = kvh * 4 + g;
    const int len0 = a.pos0 + r0 + 1;   /* positions row r0 attends over; row r0 + i: len0 + i */
    const int len_max = len0 + rb - 1;
    const size_t plane = (size_t)kvh * a.max_seq;
    const unsigned char* kc = kv_payload(a.kv, r0) + a.kv.k_off; /* one cache for all rows of the block */
    const unsigned char* vc = kv_payload(a.kv, r0) + a.kv.v_off;
    const __half* ks = KV8 ? reinterpret_cast<const __half*>(kv_scales(a.kv, r0) + a.kv.ks_off) : nullptr;
    const __half* vs = KV8 ? reinterpret_cast<const __half*>(kv_scales(a.kv, r0) + a.kv.vs_off) : nullptr;

    const float scale = rsqrtf((float)a.head_dim); /* run-time value on purpose, see AttnArgs */
#pragma unroll
    for (int i = 0; i < RB; i++)
        sm.sq[i][g][t] = i < rb ? __fmul_rn(bf2f(a.q[((size_t)(r0 + i) * QH + h) * 128 + t]), scale) : 0.f;

    float m[RB], l[RB], acc[RB];
#pragma unroll
    for (int i = 0; i < RB; i++) { m[i] = -INFINITY; l[i] = 0.f; acc[i] = 0.f; }

    for (int t0 = 0; t0 < len_max; t0 += 128) {
        const int lim_max = min(128, len_max - t0);
        __syncthreads(); /* previous tile fully consumed; sq visible */
        for (int i = threadIdx.x; i < lim_max * (VB / 4); i += 512) {
            const int rr = i / (VB / 4), cw = i - rr * (VB / 4);
            *reinterpret_cast<uint32_t*>(sm.tile + rr * TS + cw * 4) =
                __ldg(reinterpret_cast<const uint32_t*>(kc + (plane + t0 + rr) * VB + cw * 4));
        }
        if (KV8)
            for (int i = threadIdx.x; i < lim_max * 4; i += 512) {
                sm.ssc[i] = ks[(plane + t0) * 4 + i];
                sm.vssc[i] = vs[(plane + t0) * 4 + i];
            }
        __syncthreads();

        /* ---- scores: the key of position t, converted once, against the RB rows' queries ---- */
        float d[RB];
#pragma unroll
        for (int i = 0; i < RB; i++) d[i] = 0.f;
        if (t < lim_max) {
            const uint32_t* kw = reinterpret_cast<const uint32_t*>(sm.tile + t * TS);
            if (KV8) {
#pragma unroll 1
                for (int gi = 0; gi < 4; gi++) {
                    float pp[RB];
#pragma unroll
                    for (int i = 0; i < RB; i++) pp[i] = 0.f;
#pragma unroll
                    for (int w = 0; w < 8; w++) {
                        const uint32_t u = s8x4_bias(kw[gi * 8 + w]);
                        const float k0 = s8_biased_to_f32<0>(u), k1 = s8_biased_to_f32<1>(u), k2 = s8_biased_to_f32<2>(u), k3 = s8_biased_to_f32<3>(u);
#pragma unroll
                        for (int i = 0; i < RB; i++) {
                            const float4 qv = reinterpret_cast<const float4*>(sm.sq[i][g])[gi * 8 + w];
                            pp[i] = __fmaf_rn(qv.x, k0, pp[i]);
                            pp[i] = __fmaf_rn(qv.y, k1, pp[i]);
                            pp[i] = __fmaf_rn(qv.z, k2, pp[i]);
                            pp[i] = __fmaf_rn(qv.w, k3, pp[i]);
                        }
                    }
                    const float ksf = __half2float(sm.ssc[t * 4 + gi]);
#pragma unroll
                    for (int i = 0; i < RB; i++) d[i] = __fmaf_rn(pp[i], ksf, d[i]);
                }
            } else {
#pragma unroll 4
                for (int w = 0; w < 64; w += 2) { /* two words = four bf16 */
                    const uint32_t w0 = kw[w], w1 = kw[w + 1];
                    const float k0 = bf_lo(w0), k1 = bf_hi(w0), k2 = bf_lo(w1), k3 = bf_hi(w1);
#pragma unroll
                    for (int i = 0; i < RB; i++) {
                        const float4 qv = reinterpret_cast<const float4*>(sm.sq[i][g])[w >> 1];
                        d[i] = __fmaf_rn(qv.x, k0, d[i]);
                        d[i] = __fmaf_rn(qv.y, k1, d[i]);
                        d[i] = __fmaf_rn(qv.z, k2, d[i]);
                        d[i] = __fmaf_rn(qv.w, k3, d[i]);
                    }
                }
            }
        }
        /* row i of the block sees positions below len0 + i */
        float s[RB];
#pragma unroll
        for (int i = 0; i < RB; i++) s[i] = (i < rb && t0 + t < len0 + i) ? d[i] : -INFINITY;

        /* ---- tile max per (row, head): the 128-wide halving tree, the rows' trees side by side ---- */
#pragma unroll
        for (int i = 0; i < RB; i++) sm.red[i][g][t] = s[i];
        __syncthreads();
        if (t < 64) {
#pragma unroll
            for (int i = 0; i < RB; i++) sm.red[i][g][t] = fmaxf(sm.red[i][g][t], sm.red[i][g][t + 64]);
        }
        __syncthreads();
        if (t < 32) {
#pragma unroll
            for (int i = 0; i < RB; i++) sm.red[i][g][t] = fmaxf(sm.red[i][g][t], sm.red[i][g][t + 32]);
        }
        __syncthreads();
        float corr[RB], mn[RB];
#pragma unroll
        for (int i = 0; i < RB; i++) {
            const float tmax = warp_tree_max(sm.red[i][g][t & 31]);
            mn[i] = fmaxf(m[i], tmax);
            corr[i] = (m[i] == -INFINITY) ? 0.f : expf(m[i] - mn[i]);
        }
        __syncthreads();
        {
            float vsf[4] = {1.f, 1.f, 1.f, 1.f};
            if (KV8 && t < lim_max) {
                const uint2 sv = *reinterpret_cast<const uint2*>(sm.vssc + t * 4);
                const __half2 sva = *reinterpret_cast<const __half2*>(&sv.x), svb = *reinterpret_cast<const __half2*>(&sv.y);
                vsf[0] = __low2float(sva); vsf[1] = __high2float(sva); vsf[2] = __low2float(svb); vsf[3] = __high2float(svb);
            }
#pragma unroll
            for (int i = 0; i < RB; i++) {
                const float p = (s[i] == -INFINITY) ? 0.f : expf(s[i] - mn[i]);
                sm.red[i][g][t] = p;
                if (KV8) {
#pragma unroll
                    for (int grp = 0; grp < 4; grp++) sm.spv[i][g][grp][t] = __fmul_rn(p, vsf[grp]);
                } else {
                    sm.spv[i][g][0][t] = p;
                }
            }
        }
        __syncthreads();
        if (t < 64) {
#pragma unroll
            for (int i = 0; i < RB; i++) sm.red[i][g][t] += sm.red[i][g][t + 64];
        }
        __syncthreads();
        if (t < 32) {
#pragma unroll
            for (int i = 0; i < RB; i++) sm.red[i][g][t] += sm.red[i][g][t + 32];
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < RB; i++) {
            const float tsum = warp_tree_sum(sm.red[i][g][t & 31]);
            if (i < rb && t0 < len0 + i) { /* the row reaches into this tile (uniform over the CTA) */
                l[i] = __fmaf_rn(l[i], corr[i], tsum);
                acc[i] = __fmul_rn(acc[i], corr[i]);
                m[i] = mn[i];
            }
        }
        __syncthreads(); /* K tile no longer needed: the buffer takes V */
        for (int i = threadIdx.x; i < lim_max * (VB / 4); i += 512) {
            const int rr = i / (VB / 4), cw = i - rr * (VB / 4);
            *reinterpret_cast<uint32_t*>(sm.tile + rr * TS + cw * 4) =
                __ldg(reinterpret_cast<const uint32_t*>(vc + (plane + t0 + rr) * VB + cw * 4));
        }
        __syncthreads();

        /* ---- value sums: the value of (position j, dimension t), converted once, into the RB rows' chains; the
         * weights of four positions come with one 16-byte read per row ---- */
        const int full = min(lim_max, max(0, len0 - t0)); /* positions every row of the block sees */
        const int grp = KV8 ? (t >> 5) : 0;
        auto value_at = [&](int j) -> float {
            return KV8 ? s8_to_f32(reinterpret_cast<const int8_t*>(sm.tile + j * TS)[t])
                       : bf2f(reinterpret_cast<const __nv_bfloat16*>(sm.tile + j * TS)[t]);
        };
        int j = 0;
        for (; j + 4 <= full; j += 4) {
            const float v0 = value_at(j), v1 = value_at(j + 1), v2 = value_at(j + 2), v3 = value_at(j + 3);
#pragma unroll
            for (int i = 0; i < RB; i++) {
                const float4 w = *reinterpret_cast<const float4*>(&sm.spv[i][g][grp][j]);
                acc[i] = __fmaf_rn(w.x, v0, acc[i]);
                acc[i] = __fmaf_rn(w.y, v1, acc[i]);
                acc[i] = __fmaf_rn(w.z, v2, acc[i]);
                acc[i] = __fmaf_rn(w.w, v3, acc[i]);
            }
        }
        for (; j < lim_max; j++) { /* the rest, and the diagonal: row i sees position t0 + j only if it lies below len0 + i */
            const float vf = value_at(j);
#pragma unroll
            for (int i = 0; i < RB; i++)
                if (i < rb && t0 + j < len0 + i) acc[i] = __fmaf_rn(sm.spv[i][g][grp][j], vf, acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < RB; i++)
        if (i < rb) a.out[((size_t)(r0 + i) * QH + h) * 128 + t] = f2bf(__fdiv_rn(acc[i], l[i]));
}

}  // namespace s2p
