/* Per-head helpers shared by the primitive kernels and the fused decode
 * attention: 128-wide head RMSNorm, interleaved-pair RoPE and the INT8 KV
 * quantiser, each in the reference's operation order (src/slowar/kernels.cu:
 * 81-101, 114-139, 547-563). */
#pragma once
#include "common.cuh"
#include "ops.h"

namespace s2p {

/* cos/sin of the pair's angle, rounded through bf16 */
__device__ __forceinline__ void rope_cs(int pair, int pos, float rope_base, float& c, float& s) {
    const float ex = __fdiv_rn((float)(2 * pair), 128.0f);
    const float inv = __fdiv_rn(1.0f, powf(rope_base, ex));
    const float ang = __fmul_rn((float)pos, inv);
    c = bf16_round(cosf(ang));
    s = bf16_round(sinf(ang));
}
/* element t of a head (t even: x0, odd: x1), `other` = its pair partner */
__device__ __forceinline__ float rope_elem(int t, float self, float other, float c, float s) {
    return (t & 1) ? bf16_round(__fadd_rn(__fmul_rn(self, c), __fmul_rn(other, s)))
                   : bf16_round(__fsub_rn(__fmul_rn(self, c), __fmul_rn(other, s)));
}

/* one warp == one 32-element group of a head vector */
__device__ __forceinline__ int8_t kv8_quant(float xv, __half& hsc_out) {
    const float a = warp_tree_max(fabsf(xv));
    const __half hsc = __float2half_rn(__fdiv_rn(a, 127.0f));
    const float sc = __half2float(hsc);
    int q = (sc > 0.f) ? __float2int_rn(__fdiv_rn(xv, sc)) : 0;
    q = max(-127, min(127, q));
    hsc_out = hsc;
    return (int8_t)q;
}

/* Halving tree over the 128 values of one head when a CTA holds G heads side by
 * side (thread = g*128 + t).  red: [G][128] floats.  All threads must call. */
__device__ __forceinline__ float head_tree_sum(float v, float (*red)[128], int g, int t) {
    red[g][t] = v;
    S2P_CTA_SYNC();
    if (t < 64) red[g][t] += red[g][t + 64];
    S2P_CTA_SYNC();
    if (t < 32) red[g][t] += red[g][t + 32];
    S2P_CTA_SYNC();
    const float r = warp_tree_sum(red[g][t & 31]);
    S2P_CTA_SYNC();
    return r;
}


__device__ __forceinline__ unsigned char* kv_payload(const KvRef& kv, int row) {
    return kv.bases ? static_cast<unsigned char*>(kv.bases[row])
                    : static_cast<unsigned char*>(kv.base0) + (size_t)row * kv.row_stride;
}
__device__ __forceinline__ unsigned char* kv_scales(const KvRef& kv, int row) {
    return kv.sbases ? static_cast<unsigned char*>(kv.sbases[row])
                     : static_cast<unsigned char*>(kv.sbase0) + (size_t)row * kv.srow_stride;
}

}  // namespace s2p
