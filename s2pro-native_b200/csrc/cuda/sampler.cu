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
#include "sampler_body.cuh"

namespace s2p {

__global__ void __launch_bounds__(256) k_sample(const __nv_bfloat16* __restrict__ logits, int64_t stride,
                                                const __nv_bfloat16* __restrict__ eos_logits, int64_t eos_stride,
                                                SamplerState* const* __restrict__ states,
                                                int64_t* __restrict__ out_tok, int32_t* __restrict__ out_sem,
                                                int32_t* __restrict__ out_codes, uint8_t* __restrict__ out_eos) {
    __shared__ SamplerSmem<256> sm;
    const int row = blockIdx.x;
    sampler_cta<256>(logits + (size_t)row * stride, eos_logits + (size_t)row * eos_stride, states[row], out_tok + row,
                     out_sem + row, out_codes + (size_t)row * 10, out_eos + row, sm);
}

extern "C" cudaError_t sample_rows(const void* sem_logits, int64_t stride, const void* eos_logits,
                                   int64_t eos_stride, SamplerState* const* states, int rows, int64_t* out_tok, int32_t* out_sem,
                                   int32_t* out_codes, uint8_t* out_eos, cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    k_sample<<<rows, 256, 0, st>>>((const __nv_bfloat16*)sem_logits, stride, (const __nv_bfloat16*)eos_logits,
                                           eos_stride, states, out_tok, out_sem, out_codes, out_eos);
    return cudaGetLastError();
}

}  // namespace s2p
