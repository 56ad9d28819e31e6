/* Device body of the semantic sampler (see sampler.cu for the algorithm), for a
 * CTA of NT threads: the stand-alone kernel runs it with 256, the persistent tick
 * kernel with its 512.  The top-30 selection is a total order, so the thread
 * count does not change the result. */
#pragma once
#include <math.h>
#include "common.cuh"
#include "ops.h"
#include "s2p_b200_abi.h"

namespace s2p {

constexpr int SMP_N_SEM = 4096;
constexpr int SMP_N_CAND = 4097;
constexpr int SMP_TOPK = 30;

template <int NT> struct SamplerSmem {
    float cand[SMP_N_CAND];
    float wtop_v[(NT / 32) * SMP_TOPK];  /* every warp's own top-30 */
    int wtop_i[(NT / 32) * SMP_TOPK];
    float tv[SMP_TOPK];
    int ti[SMP_TOPK];
    float sh_temp, sh_topp;
    int64_t hist[64];   /* the history window, read once */
    int64_t fin_tok;    /* the sampled token */
    int fin_mode;       /* 0 EOS (state untouched), 1 append at `count`, 2 shift the full window */
};

__device__ __forceinline__ uint64_t rotl64(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }
static __device__ __forceinline__ uint64_t xoshiro_next(uint64_t* s) {
    const uint64_t result = rotl64(s[1] * 5, 7) * 9;
    const uint64_t t = s[1] << 17;
    s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3];
    s[2] ^= t;
    s[3] = rotl64(s[3], 45);
    return result;
}

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

/* logits: 4096 semantic logits of the row; eos_logit: its EOS logit; sp: its state;
 * outputs are the row's own slots. */
template <int NT>
__device__ void sampler_cta(const __nv_bfloat16* lrow, const __nv_bfloat16* eos_logit, SamplerState* sp,
                            int64_t* out_tok, int32_t* out_sem, int32_t* out_code0, uint8_t* out_eos,
                            SamplerSmem<NT>& sm) {
    constexpr int SMP_THREADS = NT;
    constexpr int SMP_PER_THREAD = (SMP_N_CAND + NT - 1) / NT;
    float* cand = sm.cand;
    float* tv = sm.tv;
    int* ti = sm.ti;
    float& sh_temp = sm.sh_temp;
    float& sh_topp = sm.sh_topp;
    const int tid = threadIdx.x;
    for (int i = tid; i < SMP_N_SEM; i += SMP_THREADS) cand[i] = bf_bits_to_f32(__ldcg(reinterpret_cast<const unsigned short*>(lrow + i)));
    if (tid == 0) cand[SMP_N_SEM] = bf_bits_to_f32(__ldcg(reinterpret_cast<const unsigned short*>(eos_logit)));
    int64_t* hist = sm.hist;
    if (tid < 64) hist[tid] = sp->prev[tid];
    const uint64_t count0 = sp->count;
    const int window = sp->window;
    S2P_CTA_SYNC();

    const bool greedy = sp->temperature == 0.0f;
    const int capped = count0 < (uint64_t)window ? (int)count0 : window;
    if (tid == 0) {
        bool ras = false;
        if (!greedy && capped >= 4) {
            int64_t last4[4];
            for (int r = 0; r < 4; r++) {
                int idx = capped - (4 - r);
                last4[r] = hist[idx < 0 ? 0 : idx];
            }
            for (int x = 0; x < 4; x++)
                for (int y = x + 1; y < 4; y++) ras |= (last4[x] == last4[y]);
        }
        sh_temp = ras ? 1.0f : sp->temperature;
        sh_topp = ras ? 0.9f : sp->top_p;
        if (capped > 0) {
            int ridx[64];
            float rval[64];
            int rn = 0;
            const float rep_penalty = sp->rep_penalty;
            for (int j = 0; j < capped; j++) {
                const int64_t tok = hist[j];
                int ci;
                if (tok >= S2P_TOK_SEMANTIC_START && tok <= S2P_TOK_SEMANTIC_END) ci = (int)(tok - S2P_TOK_SEMANTIC_START);
                else if (tok == S2P_TOK_EOS) ci = SMP_N_SEM;
                else continue;
                const float v = cand[ci];
                ridx[rn] = ci;
                rval[rn] = v < 0.f ? __fmul_rn(v, rep_penalty) : __fdiv_rn(v, rep_penalty);
                rn++;
            }
            for (int j = 0; j < rn; j++) cand[ridx[j]] = rval[j];
        }
    }
    S2P_CTA_SYNC();

    /* top-30 in two warp-level passes without block-wide rounds: every warp selects the 30 best of
     * its own candidates (i = tid + NT j, held in registers) with shuffles only; warp 0 then selects
     * the 30 best of the warps' winners.  (value desc, index asc) is a total order, so the result
     * is the block-wide top-30 in order. */
    const int lane = tid & 31, warp = tid >> 5;
    constexpr int NW = SMP_THREADS / 32;
    float* wtv = sm.wtop_v;
    int* wti = sm.wtop_i;
    {
        float mine[SMP_PER_THREAD];
#pragma unroll
        for (int j = 0; j < SMP_PER_THREAD; j++) {
            const int i = tid + j * SMP_THREADS;
            mine[j] = i < SMP_N_CAND ? cand[i] : -INFINITY;
        }
        for (int k = 0; k < SMP_TOPK; k++) {
            float bv = -INFINITY;
            int bi = SMP_N_CAND;
#pragma unroll
            for (int j = 0; j < SMP_PER_THREAD; j++) {
                const int i = tid + j * SMP_THREADS;
                if (i < SMP_N_CAND && better(mine[j], i, bv, bi)) { bv = mine[j]; bi = i; }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float ov = __shfl_xor_sync(S2P_FULL_MASK, bv, off);
                const int oi = __shfl_xor_sync(S2P_FULL_MASK, bi, off);
                if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
            }
            if (lane == 0) { wtv[warp * SMP_TOPK + k] = bv; wti[warp * SMP_TOPK + k] = bi; }
            if (bi < SMP_N_CAND && (bi % SMP_THREADS) == tid) { /* the owner retires the winner */
#pragma unroll
                for (int j = 0; j < SMP_PER_THREAD; j++)
                    if (tid + j * SMP_THREADS == bi) mine[j] = -INFINITY;
            }
        }
    }
    S2P_CTA_SYNC();
    if (warp == 0) {
        constexpr int PER2 = (NW * SMP_TOPK + 31) / 32;
        float v2[PER2];
        int i2[PER2];
#pragma unroll
        for (int j = 0; j < PER2; j++) {
            const int e = lane + 32 * j;
            v2[j] = e < NW * SMP_TOPK ? wtv[e] : -INFINITY;
            i2[j] = e < NW * SMP_TOPK ? wti[e] : SMP_N_CAND;
        }
        for (int k = 0; k < SMP_TOPK; k++) {
            float bv = -INFINITY;
            int bi = SMP_N_CAND;
#pragma unroll
            for (int j = 0; j < PER2; j++)
                if (i2[j] < SMP_N_CAND && better(v2[j], i2[j], bv, bi)) { bv = v2[j]; bi = i2[j]; }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float ov = __shfl_xor_sync(S2P_FULL_MASK, bv, off);
                const int oi = __shfl_xor_sync(S2P_FULL_MASK, bi, off);
                if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
            }
            if (lane == 0) { tv[k] = bv; ti[k] = bi; }
#pragma unroll
            for (int j = 0; j < PER2; j++)
                if (i2[j] == bi) i2[j] = SMP_N_CAND; /* retired: an index never matches again */
        }
    }
    S2P_CTA_SYNC();
    if (tid == 0) {
    int choice = 0;
    if (!greedy) {
        float e[SMP_TOPK], sum = 0.f;
        const float m = tv[0];
        for (int j = 0; j < SMP_TOPK; j++) {
            e[j] = expf(tv[j] - m);
            sum = __fadd_rn(sum, e[j]);
        }
        bool masked[SMP_TOPK];
        float cum = 0.f;
        for (int j = 0; j < SMP_TOPK; j++) {
            cum = __fadd_rn(cum, __fdiv_rn(e[j], sum));
            masked[j] = (j > 0 && cum > sh_topp);
        }
        const float t = sh_temp < 1e-5f ? 1e-5f : sh_temp;
        float p2[SMP_TOPK], s2 = 0.f;
        const float m2 = __fdiv_rn(tv[0], t);
        for (int j = 0; j < SMP_TOPK; j++) {
            p2[j] = masked[j] ? 0.f : expf(__fsub_rn(__fdiv_rn(tv[j], t), m2));
            s2 = __fadd_rn(s2, p2[j]);
        }
        for (int j = 0; j < SMP_TOPK; j++) p2[j] = __fdiv_rn(p2[j], s2);

        if (sp->seeded) {
            const uint64_t step_seed = ((uint64_t)sp->seed31 * 19349663ULL) ^ (count0 * 73856093ULL);
            float best = -INFINITY;
            for (int j = 0; j < SMP_TOPK; j++) {
                const uint64_t hashed = (step_seed * 8589934591ULL) ^ ((uint64_t)j * 479001599ULL);
                float u = __fdiv_rn((float)(uint32_t)(hashed & 0xFFFFFFULL), 16777216.0f);
                if (u < 1e-10f) u = 1e-10f;
                const float g = -logf(-logf(u));
                const float pert = __fadd_rn(logf(__fadd_rn(p2[j], 1e-10f)), g);
                if (pert > best) { best = pert; choice = j; }
            }
        } else {
            const double r = (double)(xoshiro_next(sp->rng) >> 11) * 0x1.0p-53;
            double cum2 = 0.0;
            int lastnz = 0;
            choice = -1;
            for (int j = 0; j < SMP_TOPK; j++) {
                if (p2[j] <= 0.f) continue;
                lastnz = j;
                cum2 += (double)p2[j];
                if (r < cum2) { choice = j; break; }
            }
            if (choice < 0) choice = lastnz;
        }
    }

    const int ci = ti[choice];
    if (ci == SMP_N_SEM) { /* EOS: semantic code forced to 0, sampler state untouched */
        *out_tok = S2P_TOK_EOS;
        *out_sem = 0;
        *out_code0 = 0;
        *out_eos = 1;
        sm.fin_mode = 0;
    } else {
        const int64_t tok = (int64_t)S2P_TOK_SEMANTIC_START + ci;
        *out_tok = tok;
        *out_sem = ci;
        *out_code0 = ci;
        *out_eos = 0;
        sm.fin_tok = tok;
        sm.fin_mode = count0 < (uint64_t)window ? 1 : 2;
        sp->count = count0 + 1;
    }
    } /* tid == 0 */
    S2P_CTA_SYNC();
    /* history update, the shift done by the threads side by side from the staged window */
    if (sm.fin_mode == 1) {
        if (tid == 0) sp->prev[count0] = sm.fin_tok;
    } else if (sm.fin_mode == 2) {
        if (tid < window - 1) sp->prev[tid] = hist[tid + 1];
        else if (tid == window - 1) sp->prev[tid] = sm.fin_tok;
    }
}

}  // namespace s2p
