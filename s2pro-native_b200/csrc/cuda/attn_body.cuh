/* Device body of the split-K decode attention (see attn.cu for the arithmetic
 * contract), callable from a stand-alone kernel (one CTA per (row, kv head,
 * worker)) and from the persistent tick kernel.  512 threads.  Everything
 * another SM may have produced earlier in the same kernel (the qkv projection,
 * the per-split partials) is read with L1-bypassing loads. */
#pragma once
#include <math.h>
#include "common.cuh"
#include "headops.cuh"
#include "ops.h"
#include "attn.cuh"
#include "pipe.cuh"

namespace s2p {

template <bool KV8> struct AttnSmem {
    static constexpr int VB = KV8 ? 128 : 256; /* payload bytes per cached vector */
    static constexpr int TS = VB + 4;          /* staged row stride (skewed) */
    static constexpr int NBUF = KV8 ? 2 : 1;   /* INT8 cache: the next split is copied while this one is worked on */
    alignas(16) unsigned char tile[NBUF][64 * TS];   /* K rows of a split */
    alignas(16) unsigned char vtile[NBUF][64 * TS];  /* V rows of a split */
    alignas(8) __half ssc[NBUF][64 * 4];             /* their group scales (INT8 cache) */
    alignas(8) __half vssc[NBUF][64 * 4];
    alignas(16) float sq[4][128];
    float sc[4][64];
    alignas(16) float scv[64 * 4 * 4];         /* [position][value group][head]: probability x value scale */
    float red[4][128];
    float hm[4], hs[4];
    int s_last;
};

__device__ __forceinline__ float ldcg_bf(const __nv_bfloat16* p) {
    return bf_bits_to_f32(__ldcg(reinterpret_cast<const unsigned short*>(p)));
}
/* element idx of the raw qkv projection: plain bf16, or a flagged word to wait for */
__device__ __forceinline__ float prep_load(const AttnPrep& pz, size_t idx) {
    if (pz.qkv_ll) {
        uint32_t w;
        if (!flag_wait1(pz.qkv_ll + idx, pz.qkv_tag, pz.status, w)) return 0.f; /* status is set; the kernel winds down */
        return flag_payload(w);
    }
    return ldcg_bf(pz.qkv + idx);
}

template <bool KV8, bool PREP, int HPT>
__device__ void attn_decode_cta(const AttnArgs& a, const AttnPrep& pz, int row, int kvh, int wk, int workers,
                                AttnSmem<KV8>& sm) {
    constexpr int VB = AttnSmem<KV8>::VB;
    constexpr int TS = AttnSmem<KV8>::TS;

    constexpr int NBUF = AttnSmem<KV8>::NBUF;
    unsigned char* tile = sm.tile[0]; /* buffer 0 takes the worker's first split (and the appended row) */
    unsigned char* vtile = sm.vtile[0];
    __half* ssc = sm.ssc[0];
    __half* vssc = sm.vssc[0];
    float (*sq)[128] = sm.sq;
    float (*sc)[64] = sm.sc;
    float (*red)[128] = sm.red;
    float* hm = sm.hm;
    float* hs = sm.hs;
    const int tid = threadIdx.x;
    const int QH = a.q_heads, KVH = a.kv_heads;
    const int pos = a.pos_arr ? __ldcg(a.pos_arr + row) : a.pos0 + row * a.pos_row_step;
    const int len = pos + 1;
    const int n_active = (len + 63) >> 6;
    const size_t plane = (size_t)kvh * a.max_seq;
    unsigned char* kc = kv_payload(a.kv, row) + a.kv.k_off;
    unsigned char* vc = kv_payload(a.kv, row) + a.kv.v_off;
    __half* ks = KV8 ? reinterpret_cast<__half*>(kv_scales(a.kv, row) + a.kv.ks_off) : nullptr;
    __half* vs = KV8 ? reinterpret_cast<__half*>(kv_scales(a.kv, row) + a.kv.vs_off) : nullptr;
    const float scale = rsqrtf(128.0f);

    /* Start the copies of a split's K and V rows (and scales) into shared memory; they run
     * while the caller does something else.  `skip` (or -1): a row the caller writes itself. */
    auto fetch_split = [&](int spl, int skip, int buf) {
        unsigned char* tile = sm.tile[buf];
        unsigned char* vtile = sm.vtile[buf];
        __half* ssc = sm.ssc[buf];
        __half* vssc = sm.vssc[buf];
        const int start = spl << 6;
        const int cnt = min(64, len - start);
        for (int i = tid; i < cnt * (VB / 4); i += 512) {
            const int rr = i / (VB / 4), cw = i - rr * (VB / 4);
            if (start + rr == skip) continue;
            const size_t off = (plane + start + rr) * VB + cw * 4;
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(tile + rr * TS + cw * 4)), "l"(kc + off) : "memory");
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(vtile + rr * TS + cw * 4)), "l"(vc + off) : "memory");
        }
        if (KV8)
            for (int rr = tid; rr < cnt; rr += 512) {
                if (start + rr == skip) continue;
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((uint32_t)__cvta_generic_to_shared(ssc + rr * 4)), "l"(ks + (plane + start + rr) * 4) : "memory");
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((uint32_t)__cvta_generic_to_shared(vssc + rr * 4)), "l"(vs + (plane + start + rr) * 4) : "memory");
            }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    /* the first split of this worker is on its way before the query is prepared; the new
     * position's row, if it falls into that split, is written below by this CTA itself */
    const bool pre_has_new = PREP && wk == n_active - 1;
    if (wk < n_active) fetch_split(wk, pre_has_new ? pos : -1, 0);

    {   /* queries of the four heads sharing this kv head, pre-scaled */
        const int g = tid >> 7, t = tid & 127;
        const int h = kvh * 4 + g;
        float v;
        if (PREP) {
            v = prep_load(pz, (size_t)row * (QH + 2 * KVH) * 128 + (size_t)h * 128 + t);
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
            v = ldcg_bf(a.q + ((size_t)row * QH + h) * 128 + t);
        }
        sq[g][t] = __fmul_rn(v, scale);
    }
    if (PREP) {
        /* the worker that owns the split holding the new position appends k and v */
        const bool owner = ((n_active - 1) % workers) == wk;
        if (owner) { /* uniform over the CTA */
            const int g = tid >> 7, t = tid & 127; /* g 0: k, g 1: v, g 2,3 idle but join the barriers */
            const size_t src = (size_t)row * (QH + 2 * KVH) * 128 + (size_t)(QH + (g == 1 ? KVH : 0) + kvh) * 128 + t;
            float v = prep_load(pz, g < 2 ? src : 0);
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
                unsigned char* trow = (g == 0 ? tile : vtile) + (pos & 63) * TS; /* its row of the staged split */
                if (!KV8) {
                    const __nv_bfloat16 vb = f2bf(v);
                    reinterpret_cast<__nv_bfloat16*>(cache)[vec * 128 + t] = vb;
                    if (pre_has_new) reinterpret_cast<__nv_bfloat16*>(trow)[t] = vb;
                } else {
                    __half hsc;
                    const int8_t q8 = kv8_quant(v, hsc);
                    reinterpret_cast<int8_t*>(cache)[vec * 128 + t] = q8;
                    if (pre_has_new) reinterpret_cast<int8_t*>(trow)[t] = q8;
                    if ((t & 31) == 0) {
                        (g == 0 ? ks : vs)[vec * 4 + (t >> 5)] = hsc;
                        if (pre_has_new) (g == 0 ? ssc : vssc)[(pos & 63) * 4 + (t >> 5)] = hsc;
                    }
                }
            }
        }
    }
    S2P_CTA_SYNC();

    int cur = 0;
    for (int spl = wk; spl < n_active; spl += workers) {
        const int start = spl << 6;
        const int cnt = min(64, len - start);
        /* later splits: this CTA's own append, if any, is already visible */
        if (NBUF == 2) {
            /* the other buffer was last read before the barrier that ended the previous round */
            if (spl + workers < n_active) {
                fetch_split(spl + workers, -1, cur ^ 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_all;" ::: "memory");
            }
            tile = sm.tile[cur]; vtile = sm.vtile[cur]; ssc = sm.ssc[cur]; vssc = sm.vssc[cur];
            cur ^= 1;
        } else {
            if (spl != wk) fetch_split(spl, -1, 0);
            asm volatile("cp.async.wait_all;" ::: "memory");
        }
        S2P_CTA_SYNC();

        /* scores: thread (head group, position t4) carries the chains of HPT heads of its position, so a
         * cached key is read and converted once for them (HPT 1: lowest latency; 4: fewest instructions) */
        constexpr int QT = 256 / HPT;
        const int g4 = (tid >> 6) & 3, t4 = tid & 63, gq = (tid >> 6) * HPT;
        float d[HPT];
#pragma unroll
        for (int h = 0; h < HPT; h++) d[h] = -INFINITY;
        if (tid < QT && t4 < cnt) {
#pragma unroll
            for (int h = 0; h < HPT; h++) d[h] = 0.f;
            const uint32_t* kw = reinterpret_cast<const uint32_t*>(tile + t4 * TS);
            if (!KV8) {
#pragma unroll 4
                for (int e = 0; e < 32; e++) {
                    const uint32_t w0 = kw[2 * e], w1 = kw[2 * e + 1];
                    const float k0 = bf_lo(w0), k1 = bf_hi(w0), k2 = bf_lo(w1), k3 = bf_hi(w1);
#pragma unroll
                    for (int h = 0; h < HPT; h++) {
                        const float4 qv = reinterpret_cast<const float4*>(sq[gq + h])[e];
                        d[h] = __fmaf_rn(qv.x, k0, d[h]);
                        d[h] = __fmaf_rn(qv.y, k1, d[h]);
                        d[h] = __fmaf_rn(qv.z, k2, d[h]);
                        d[h] = __fmaf_rn(qv.w, k3, d[h]);
                    }
                }
            } else {
                /* four codes per shared-memory word, four query values per load; the chain order is unchanged */
#pragma unroll
                for (int gi = 0; gi < 4; gi++) {
                    float pp[HPT];
#pragma unroll
                    for (int h = 0; h < HPT; h++) pp[h] = 0.f;
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const uint32_t w = s8x4_bias(kw[gi * 8 + e]);
                        const float k0 = s8_biased_to_f32<0>(w), k1 = s8_biased_to_f32<1>(w);
                        const float k2 = s8_biased_to_f32<2>(w), k3 = s8_biased_to_f32<3>(w);
#pragma unroll
                        for (int h = 0; h < HPT; h++) {
                            const float4 qv = reinterpret_cast<const float4*>(sq[gq + h])[gi * 8 + e];
                            pp[h] = __fmaf_rn(qv.x, k0, pp[h]);
                            pp[h] = __fmaf_rn(qv.y, k1, pp[h]);
                            pp[h] = __fmaf_rn(qv.z, k2, pp[h]);
                            pp[h] = __fmaf_rn(qv.w, k3, pp[h]);
                        }
                    }
                    const float ks = __half2float(ssc[t4 * 4 + gi]);
#pragma unroll
                    for (int h = 0; h < HPT; h++) d[h] = __fmaf_rn(pp[h], ks, d[h]);
                }
            }
        }
        if (tid < QT) { /* split max per head: two warps of 32 slots each */
#pragma unroll
            for (int h = 0; h < HPT; h++) {
                const float mx = warp_tree_max(d[h]);
                if ((tid & 31) == 0) red[0][(gq + h) * 2 + ((tid >> 5) & 1)] = mx;
            }
        }
        S2P_CTA_SYNC();
        if (tid < QT) {
#pragma unroll
            for (int h = 0; h < HPT; h++) {
                const float mh = fmaxf(red[0][2 * (gq + h)], red[0][2 * (gq + h) + 1]);
                sc[gq + h][t4] = (t4 < cnt) ? expf(d[h] - mh) : 0.f;
            }
        }
        float m = 0.f;
        if (tid < 256) m = fmaxf(red[0][2 * g4], red[0][2 * g4 + 1]);
        S2P_CTA_SYNC();
        if (tid < 256 && t4 < 32) { /* exp-sum: pairs (t, t+32), then 16..1 */
            const float x = warp_tree_sum(sc[g4][t4] + sc[g4][t4 + 32]);
            if (t4 == 0) { hm[g4] = m; hs[g4] = x; }
        }
        /* meanwhile the weights of the value sum, per (position, value group, head): the probability,
         * for the INT8 cache times the group's scale (the product the value chain multiplies by) */
        for (int i = tid; i < 64 * 4 * 4; i += 512) {
            const int g = i & 3, grp = (i >> 2) & 3, j = i >> 4;
            sm.scv[i] = KV8 ? __fmul_rn(sc[g][j], __half2float(vssc[j * 4 + grp])) : sc[g][j];
        }
        S2P_CTA_SYNC();
        if (tid < 128) { /* one thread per value dimension carries the chains of the four heads: a value is read and converted once */
            const int dd = tid;
            const float4* wv = reinterpret_cast<const float4*>(sm.scv) + (dd >> 5);
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 4
            for (int j = 0; j < cnt; j++) {
                const float vf = KV8 ? s8_to_f32(reinterpret_cast<const int8_t*>(vtile + j * TS)[dd])
                                     : bf2f(reinterpret_cast<const __nv_bfloat16*>(vtile + j * TS)[dd]);
                const float4 wj = wv[j * 4];
                a0 = __fmaf_rn(wj.x, vf, a0);
                a1 = __fmaf_rn(wj.y, vf, a1);
                a2 = __fmaf_rn(wj.z, vf, a2);
                a3 = __fmaf_rn(wj.w, vf, a3);
            }
            const float accs[4] = {a0, a1, a2, a3};
#pragma unroll
            for (int g = 0; g < 4; g++) {
                float* ph = a.part + (((size_t)row * QH + kvh * 4 + g) * a.n_split_slots + spl) * 130;
                if (dd == 0) { ph[0] = hm[g]; ph[1] = hs[g]; }
                ph[2 + dd] = accs[g];
            }
        }
        S2P_CTA_SYNC(); /* tile, sc, hm/hs are rewritten by the next split */
    }

    /* the last worker of this (row, kv head) to finish merges the partials */
    __threadfence();
    S2P_CTA_SYNC();
    unsigned int* ctr = a.counters + (size_t)row * KVH + kvh;
    if (tid == 0) sm.s_last = (atomicAdd(ctr, 1u) == (unsigned)(workers - 1));
    S2P_CTA_SYNC();
    const bool last = sm.s_last != 0;
    if (last) {
        __threadfence();
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
        const __nv_bfloat16 ob = f2bf(__fdiv_rn(acc, l));
        const size_t oi = ((size_t)row * QH + h) * 128 + dd;
        if (a.out_ll) {
            uint32_t* ow = reinterpret_cast<uint32_t*>(a.out) + oi;
            const uint32_t word = flag_word(ob, a.out_ll_tag);
            *ow = word;
            for (int p = 0; p < a.n_out_peers; p++)
                *reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(ow) + a.out_peer_delta[p]) = word;
        } else {
            a.out[oi] = ob;
            for (int p = 0; p < a.n_out_peers; p++)
                *reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<unsigned char*>(a.out + oi) + a.out_peer_delta[p]) = ob;
        }
    }
    if (last && tid == 0) *ctr = 0u;
    S2P_CTA_SYNC(); /* the shared block may be reused by the caller right away */
}


}  // namespace s2p
