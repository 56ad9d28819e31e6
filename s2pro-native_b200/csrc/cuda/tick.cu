/* Fused batch-1 decode stages: thin launch wrappers that bind the streaming
 * GEMV stage (gemv.cuh) and the decode attention (attn.cu) to the shapes of the
 * decode tick, plus the frame-start / frame-end glue kernels.
 *
 * One slow-AR layer is five launches instead of the reference's seventeen
 * (src/slowar/slowar.c:162-258):
 *   rmsnorm -> wqkv                       stage_norm_gemv
 *   qk-norm, RoPE, KV append, attention   stage_attn_decode_prep
 *   wo + residual                         stage_gemv_resid
 *   rmsnorm -> gate_up -> SwiGLU          stage_norm_swiglu
 *   w2 + residual                         stage_gemv_resid
 * with every intermediate bf16 rounding of the unfused sequence kept, so the
 * outputs are bit-identical to it.
 */
#include "attn.cuh"
#include "gemv.cuh"
#include "ops.h"
#include "s2p_b200_abi.h"

namespace s2p {

template <int WK, int PRO, int EPI>
cudaError_t launch_gemv_stage(GemvStage g, cudaStream_t stream); /* gemv.cu */

template <int PRO, int EPI>
static cudaError_t dispatch_kind(int kind, const GemvStage& g, cudaStream_t st) {
    switch (kind) {
    case WK_INT8_CH: return launch_gemv_stage<WK_INT8_CH, PRO, EPI>(g, st);
    case WK_INT8_GRP: return launch_gemv_stage<WK_INT8_GRP, PRO, EPI>(g, st);
    case WK_INT4_PACK: return launch_gemv_stage<WK_INT4_PACK, PRO, EPI>(g, st);
    }
    return cudaErrorInvalidValue;
}

static GemvStage base_stage(const LinRef* lin) {
    GemvStage g = {};
    g.w = lin->w; g.scales = lin->scales; g.N = lin->N; g.K = lin->K; g.gshift = lin->gshift;
    return g;
}

extern "C" cudaError_t stage_norm_gemv(const LinRef* lin, const VecRef* x, const __nv_bfloat16* norm_w, float eps,
                                       __nv_bfloat16* y, cudaStream_t st) {
    GemvStage g = base_stage(lin);
    g.x = x->base; g.x_index = x->index; g.x_key = x->key; g.norm_w = norm_w; g.eps = eps; g.y = y;
    return dispatch_kind<PRO_NORM, EPI_STORE>(lin->kind, g, st);
}

extern "C" cudaError_t stage_gemv_resid(const LinRef* lin, const __nv_bfloat16* x, const VecRef* resid,
                                        __nv_bfloat16* dst, cudaStream_t st) {
    GemvStage g = base_stage(lin);
    g.x = x; g.y = dst; g.resid_src = resid->base; g.resid_index = resid->index; g.resid_key = resid->key;
    return dispatch_kind<PRO_VEC, EPI_RESID>(lin->kind, g, st);
}

extern "C" cudaError_t stage_norm_swiglu(const LinRef* lin, const VecRef* x, const __nv_bfloat16* norm_w, float eps,
                                         __nv_bfloat16* h, cudaStream_t st) {
    GemvStage g = base_stage(lin);
    g.x = x->base; g.x_index = x->index; g.x_key = x->key; g.norm_w = norm_w; g.eps = eps; g.y = h;
    return dispatch_kind<PRO_NORM, EPI_SWIGLU>(lin->kind, g, st);
}

extern "C" cudaError_t stage_norm_argmax(const LinRef* lin, const __nv_bfloat16* x, const __nv_bfloat16* norm_w,
                                         float eps, __nv_bfloat16* logits, unsigned long long* key, cudaStream_t st) {
    GemvStage g = base_stage(lin);
    g.x = x; g.norm_w = norm_w; g.eps = eps; g.y = logits; g.argmax_key = key;
    return dispatch_kind<PRO_NORM, EPI_ARGMAX>(lin->kind, g, st);
}

extern "C" cudaError_t stage_attn_decode_prep(const AttnArgs* a, const __nv_bfloat16* qkv,
                                              const __nv_bfloat16* q_norm, const __nv_bfloat16* k_norm, float eps,
                                              float rope_base, int rows, cudaStream_t st) {
    AttnPrep p = {qkv, q_norm, k_norm, eps, rope_base};
    return launch_attn_decode(*a, &p, rows, st);
}

/* ---- frame start (src/slowar/slowar.c:481-498; fastar.cu:104-127) ----------- */
__global__ void __launch_bounds__(256) k_tick_begin(TickBeginArgs a) {
    const int r = blockIdx.x;
    const int64_t id = a.ids[r];
    const bool vq = a.mask[r] != 0;
    int idx[S2P_NUM_CODEBOOKS];
#pragma unroll
    for (int cb = 0; cb < S2P_NUM_CODEBOOKS; cb++) {
        int c = a.codes[r * S2P_NUM_CODEBOOKS + cb];
        c = max(0, min(S2P_CB_SIZE - 1, c));
        idx[cb] = cb * S2P_CB_SIZE + c;
    }
    const float inv_sqrt11 = (float)(1.0 / 3.3166247903554);
    for (int d = threadIdx.x; d < S2P_DIM; d += 256) {
        float v = a.embed ? bf2f(a.embed[(size_t)id * S2P_DIM + d])
                          : bf16_round(__fmul_rn((float)a.embed_i8[(size_t)id * S2P_DIM + d], a.embed_scale[id]));
        if (vq) {
            float acc = 0.f;
#pragma unroll
            for (int cb = 0; cb < S2P_NUM_CODEBOOKS; cb++)
                acc = __fadd_rn(acc, bf2f(a.cb_emb[(size_t)idx[cb] * S2P_DIM + d]));
            v = bf16_round(__fadd_rn(v, bf16_round(acc)));
            v = bf16_round(__fmul_rn(v, inv_sqrt11));
        }
        a.x[(size_t)r * S2P_DIM + d] = f2bf(v);
    }
    if (a.keys && threadIdx.x < 9) a.keys[r * 9 + threadIdx.x] = 0ull;
}

extern "C" cudaError_t tick_begin(const TickBeginArgs* a, int rows, cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    k_tick_begin<<<rows, 256, 0, st>>>(*a);
    return cudaGetLastError();
}

__global__ void k_tick_finish_keys(const unsigned long long* __restrict__ keys, int rows, int32_t* __restrict__ codes) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * 9) return;
    const int r = i / 9, cb = i - r * 9;
    codes[(size_t)r * 10 + cb + 1] = (int32_t)key_index(keys[i]);
}

extern "C" cudaError_t tick_finish_keys(const unsigned long long* keys, int rows, int32_t* codes, cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    k_tick_finish_keys<<<(rows * 9 + 127) / 128, 128, 0, st>>>(keys, rows, codes);
    return cudaGetLastError();
}

}  // namespace s2p
