/* Device-side semantic sampler: one CTA per session row.
 *
 * Algorithm and operation order follow the reference's host sampler and its
 * device twin (src/slowar/sampling.c:119-282, src/slowar/kernels.cu:979-1181):
 * 4096 semantic logits + the EOS logit widened to f32; RAS switch when the last
 * four history tokens hold a duplicate; repetition penalty gathered from the
 * original values and then scattered; top-30 by (value desc, index asc);
 * un-temperatured softmax for the top-p mask (rank 0 always kept); temperature
 * softmax; seeded hash-Gumbel draw keyed by the uncapped step counter, or an
 * xoshiro256** inverse-CDF draw; history/counter update unless EOS.
 *
 * The top-30 selection is a total order, so it is computed here with
 * register-resident candidates and shuffle reductions instead of 30 sweeps of a
 * shared-memory tree; the 30-element tail runs on one thread in the reference's
 * exact expression order (its expf/logf results decide the draw).
 */
#include <math.h>
#include "common.cuh"
#include "ops.h"
#include "s2p_b200_abi.h"

namespace s2p {

constexpr int SMP_THREADS = 256;
constexpr int SMP_N_SEM = 4096;
constexpr int SMP_N_CAND = 4097;
constexpr int SMP_TOPK = 30;
constexpr int SMP_PER_THREAD = (SMP_N_CAND + SMP_THREADS - 1) / SMP_THREADS; /* 17 */

__device__ __forceinline__ uint64_t rotl64(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }
__device__ uint64_t xoshiro_next(uint64_t* s) {
    const uint64_t result = rotl64(s[1] * 5, 7) * 9;
    const uint64_t t = s[1] << 17;
    s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3];
    s[2] ^= t;
    s[3] = rotl64(s[3], 45);
    return result;
}

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

__global__ void __launch_bounds__(SMP_THREADS) k_sample(const __nv_bfloat16* __restrict__ logits, int64_t stride,
                                                        const __nv_bfloat16* __restrict__ eos_logits, int64_t eos_stride,
                                                        SamplerState* const* __restrict__ states,
                                                        int64_t* __restrict__ out_tok, int32_t* __restrict__ out_sem,
                                                        int32_t* __restrict__ out_codes, uint8_t* __restrict__ out_eos) {
    __shared__ float cand[SMP_N_CAND];
    __shared__ float wv[SMP_THREADS / 32];
    __shared__ int wi[SMP_THREADS / 32];
    __shared__ float tv[SMP_TOPK];
    __shared__ int ti[SMP_TOPK];
    __shared__ float sh_temp, sh_topp;
    const int row = blockIdx.x, tid = threadIdx.x;
    SamplerState* sp = states[row];
    const __nv_bfloat16* lrow = logits + (size_t)row * stride;

    for (int i = tid; i < SMP_N_SEM; i += SMP_THREADS) cand[i] = bf2f(lrow[i]);
    if (tid == 0) cand[SMP_N_SEM] = bf2f(eos_logits[(size_t)row * eos_stride]);
    __syncthreads();

    const bool greedy = sp->temperature == 0.0f;
    const int capped = sp->count < (uint64_t)sp->window ? (int)sp->count : sp->window;
    if (tid == 0) {
        bool ras = false;
        if (!greedy && capped >= 4) {
            int64_t last4[4];
            for (int r = 0; r < 4; r++) {
                int idx = capped - (4 - r);
                last4[r] = sp->prev[idx < 0 ? 0 : idx];
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
            for (int j = 0; j < capped; j++) {
                const int64_t tok = sp->prev[j];
                int ci;
                if (tok >= S2P_TOK_SEMANTIC_START && tok <= S2P_TOK_SEMANTIC_END) ci = (int)(tok - S2P_TOK_SEMANTIC_START);
                else if (tok == S2P_TOK_EOS) ci = SMP_N_SEM;
                else continue;
                const float v = cand[ci];
                ridx[rn] = ci;
                rval[rn] = v < 0.f ? __fmul_rn(v, sp->rep_penalty) : __fdiv_rn(v, sp->rep_penalty);
                rn++;
            }
            for (int j = 0; j < rn; j++) cand[ridx[j]] = rval[j];
        }
    }
    __syncthreads();

    /* top-30: candidates i = tid + 256 j live in registers */
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
        if ((tid & 31) == 0) { wv[tid >> 5] = bv; wi[tid >> 5] = bi; }
        __syncthreads();
        bv = wv[0]; bi = wi[0];
#pragma unroll
        for (int w = 1; w < SMP_THREADS / 32; w++)
            if (better(wv[w], wi[w], bv, bi)) { bv = wv[w]; bi = wi[w]; }
        if (tid == 0) { tv[k] = bv; ti[k] = bi; }
        /* the owner retires the winner */
        if (bi < SMP_N_CAND && (bi & (SMP_THREADS - 1)) == tid) {
#pragma unroll
            for (int j = 0; j < SMP_PER_THREAD; j++)
                if (tid + j * SMP_THREADS == bi) mine[j] = -INFINITY;
        }
        __syncthreads();
    }
    if (tid != 0) return;

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
            const uint64_t step_seed = ((uint64_t)sp->seed31 * 19349663ULL) ^ (sp->count * 73856093ULL);
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
        out_tok[row] = S2P_TOK_EOS;
        out_sem[row] = 0;
        out_codes[(size_t)row * 10] = 0;
        out_eos[row] = 1;
        return;
    }
    const int64_t tok = (int64_t)S2P_TOK_SEMANTIC_START + ci;
    out_tok[row] = tok;
    out_sem[row] = ci;
    out_codes[(size_t)row * 10] = ci;
    out_eos[row] = 0;
    if (sp->count < (uint64_t)sp->window) {
        sp->prev[sp->count] = tok;
    } else {
        for (int j = 0; j < sp->window - 1; j++) sp->prev[j] = sp->prev[j + 1];
        sp->prev[sp->window - 1] = tok;
    }
    sp->count++;
}

extern "C" cudaError_t sample_rows(const void* sem_logits, int64_t stride, const void* eos_logits,
                                   int64_t eos_stride, SamplerState* const* states, int rows, int64_t* out_tok, int32_t* out_sem,
                                   int32_t* out_codes, uint8_t* out_eos, cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    k_sample<<<rows, SMP_THREADS, 0, st>>>((const __nv_bfloat16*)sem_logits, stride, (const __nv_bfloat16*)eos_logits,
                                           eos_stride, states, out_tok, out_sem, out_codes, out_eos);
    return cudaGetLastError();
}

}  // namespace s2p
