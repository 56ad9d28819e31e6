/* Launch interface of the split-K decode attention for the fused tick. */
#pragma once
#include "ops.h"

namespace s2p {

/* When given, the kernel itself does q/k head RMSNorm, RoPE and the KV append
 * from the raw qkv projection (see attn.cu). */
struct AttnPrep {
    const __nv_bfloat16* qkv;    /* [rows, (q_heads + 2 kv_heads) * 128] */
    const __nv_bfloat16* q_norm; /* [128] or NULL */
    const __nv_bfloat16* k_norm;
    float eps, rope_base;
    /* persistent tick only: the projection arrives as flagged 32-bit words (bf16 | tag << 16),
     * one per element, and every load waits (bounded) for its word's tag */
    const uint32_t* qkv_ll;
    unsigned qkv_tag;
    int* status;
};

cudaError_t launch_attn_decode(const AttnArgs& a, const AttnPrep* prep, int rows, cudaStream_t st);

}  // namespace s2p
