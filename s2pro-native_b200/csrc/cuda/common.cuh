/* Shared device helpers: exact conversions and the reduction trees whose
 * pairing order the reference's kernels fix.
 *
 * Bit-exactness notes.  Floating-point addition and max are commutative, so a
 * reduction is determined by WHICH partial results are paired at each level,
 * not by which thread does it.  The reference reduces with halving trees
 * (value t is combined with value t+off for off = T/2 ... 1).  An xor
 * butterfly over the same off sequence forms exactly the same pairs and leaves
 * the (identical) result in every lane, which is what the helpers here use. */
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define S2P_FULL_MASK 0xffffffffu

/* Barrier over the threads that run the device bodies in these headers.  A kernel
 * whose CTA also holds threads outside that group (the copy-issuing warp of the
 * persistent tick kernel) defines it as a named barrier before including them. */
#ifndef S2P_CTA_SYNC
#define S2P_CTA_SYNC() __syncthreads()
#endif

__device__ __forceinline__ float bf_bits_to_f32(uint32_t hi16) { return __uint_as_float(hi16 << 16); }
/* the two bf16 of a 32-bit word (lower address first) */
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
/* Signed bytes to float without the conversion unit (which runs at a quarter of the arithmetic rate):
 * the byte, offset to unsigned, is placed in the low mantissa bits of 2^23 and the offset subtracted;
 * both steps are exact, so the value equals (float)(int8_t)b. */
__device__ __forceinline__ uint32_t s8x4_bias(uint32_t w) { return w ^ 0x80808080u; }
template <int I> __device__ __forceinline__ float s8_biased_to_f32(uint32_t biased_word) {
    return __fsub_rn(__uint_as_float(__byte_perm(biased_word, 0x4B000000u, 0x7440 + I)), 8388736.0f);
}
/* one sign-extended byte: added to the bit pattern of 2^23 + 2^22, whose mantissa absorbs either sign */
__device__ __forceinline__ float s8_to_f32(int v) { return __fsub_rn(__int_as_float(0x4B400000 + v), 12582912.0f); }
__device__ __forceinline__ float bf2f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ __nv_bfloat16 f2bf(float v) { return __float2bfloat16(v); } /* RNE */
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16(v)); }

/* Warp-level tree over lane values, off = 16,8,4,2,1; result in every lane. */
__device__ __forceinline__ float warp_tree_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(S2P_FULL_MASK, v, off);
    return v;
}
__device__ __forceinline__ float warp_tree_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(S2P_FULL_MASK, v, off));
    return v;
}

/* Four independent warp trees in the shuffles of one and a bit: the same pairs per level as four calls of the
 * helpers above (value l with l^16, then ^8, ^4, ^2, ^1), but at the first level each lane keeps two of the
 * four values and hands the other two to its partner, at the second it keeps one.  Lane l ends up with the
 * result of value index (l >> 3) & 3, the same in the eight lanes of a group.  6 shuffles instead of 20. */
template <bool IS_MAX>
__device__ __forceinline__ float warp_tree4(float v0, float v1, float v2, float v3, int lane) {
    const bool hi16 = (lane & 16) != 0, hi8 = (lane & 8) != 0;
    float k0 = hi16 ? v2 : v0, k1 = hi16 ? v3 : v1;
    const float g0 = __shfl_xor_sync(S2P_FULL_MASK, hi16 ? v0 : v2, 16), g1 = __shfl_xor_sync(S2P_FULL_MASK, hi16 ? v1 : v3, 16);
    k0 = IS_MAX ? fmaxf(k0, g0) : k0 + g0;
    k1 = IS_MAX ? fmaxf(k1, g1) : k1 + g1;
    float k = hi8 ? k1 : k0;
    const float g = __shfl_xor_sync(S2P_FULL_MASK, hi8 ? k0 : k1, 8);
    k = IS_MAX ? fmaxf(k, g) : k + g;
#pragma unroll
    for (int off = 4; off > 0; off >>= 1) {
        const float o = __shfl_xor_sync(S2P_FULL_MASK, k, off);
        k = IS_MAX ? fmaxf(k, o) : k + o;
    }
    return k;
}

/* Halving tree over T values (thread t < T contributes v; T a power of two,
 * T >= 32, T <= blockDim.x).  Levels off >= 32 go through shared memory, the
 * last five through shuffles in warp 0.  `red` needs T floats.  Returns the
 * total in every thread.  All threads of the block must call it. */
template <int T, bool IS_MAX>
__device__ __forceinline__ float block_tree(float v, float* red) {
    const int t = threadIdx.x;
    if (t < T) red[t] = v;
    S2P_CTA_SYNC();
#pragma unroll
    for (int off = T >> 1; off >= 32; off >>= 1) {
        if (t < off) red[t] = IS_MAX ? fmaxf(red[t], red[t + off]) : red[t] + red[t + off];
        S2P_CTA_SYNC();
    }
    if (t < 32) {
        float r = red[t];
        r = IS_MAX ? warp_tree_max(r) : warp_tree_sum(r);
        if (t == 0) red[0] = r;
    }
    S2P_CTA_SYNC();
    const float out = red[0];
    S2P_CTA_SYNC(); /* red may be reused by the caller right away */
    return out;
}

/* The 256-value halving sum tree with two barriers instead of six: warp 0 forms the
 * pairs of the levels 128, 64 and 32 itself (lane t holds the values t + 32 j),
 * then the shuffle levels.  Same pairs as block_tree<256, false>, same result.
 * Thread t < 256 contributes v; `red` needs 256 floats and must not be written
 * again before the caller's next barrier.  All threads of the group must call it; `sync` is a
 * barrier over that group (the whole CTA in the two-argument form). */
template <class SyncFn>
__device__ __forceinline__ float tree256_sum(float v, float* red, SyncFn sync) {
    const int t = threadIdx.x;
    if (t < 256) red[t] = v;
    sync();
    if (t < 32) {
        const float a0 = red[t] + red[t + 128], a1 = red[t + 32] + red[t + 160];
        const float a2 = red[t + 64] + red[t + 192], a3 = red[t + 96] + red[t + 224];
        const float r = warp_tree_sum((a0 + a2) + (a1 + a3));
        if (t == 0) red[256] = r;
    }
    sync();
    return red[256];
}
__device__ __forceinline__ float tree256_sum(float v, float* red) {
    return tree256_sum(v, red, [] { S2P_CTA_SYNC(); });
}

/* Bytes of an int8x4 word (biased by 128) or nibbles of an int4x8 word (biased
 * by 8) to exact f32: the byte is planted in the mantissa of 2^23 and the bias
 * is removed by one exact subtraction. */
__device__ __forceinline__ float biased_byte_to_f32(uint32_t word, int byte_idx, float magic_minus) {
    const uint32_t bits = __byte_perm(word, 0x4B000000u, 0x7540u | (uint32_t)byte_idx);
    return __uint_as_float(bits) - magic_minus;
}
