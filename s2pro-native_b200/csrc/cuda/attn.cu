/* Split-K GQA decode attention over per-session KV caches, with the merge of
 * the partials done by the last CTA to finish (no second launch).
 *
 * Arithmetic: the reference's flash-decode pair k_attn_split / k_attn_combine
 * (src/slowar/kernels.cu:351-489) and its INT8-cache twin k_attn_split8<8>
 * (:759-918): 64-position splits; per position a 128-term fma chain against the
 * pre-scaled query (INT8: four 32-term chains folded with the f16 group scale);
 * split max and exp-sum by halving trees; PV as a sequential fma over the
 * split; partial = (m, l, acc[128]); merge in ascending split order with
 * w = expf(m_s - M), l = fma(l_s, w, l), acc = fma(acc_s, w, acc), out = acc / l.
 *
 * Mapping: a fixed grid (rows, kv heads, workers) independent of the sequence
 * length, so one captured CUDA graph serves every frame; each worker walks the
 * splits s = worker, worker + workers, ...; 512 threads score the four q heads
 * of the kv head concurrently (one chain per thread) from a K tile staged in
 * shared memory with a skewed stride.  With PREP the kernel also performs what
 * precedes attention in the decode tick — per-head RMSNorm of q and k, RoPE,
 * and the append (bf16 copy or INT8 quantise) of the new k/v vectors — so the
 * fused tick needs no separate launches for them.
 */
#include "attn_body.cuh"
#include "attn_team.cuh"

namespace s2p {


template <bool KV8, bool PREP, int HPT>
__global__ void __launch_bounds__(512) k_attn_decode(AttnArgs a, AttnPrep pz) {
    __shared__ AttnSmem<KV8> sm;
    attn_decode_cta<KV8, PREP, HPT>(a, pz, blockIdx.x, blockIdx.y, blockIdx.z, gridDim.z, sm);
}

/* The kernel for lockstep batches on one GPU, no fused prologue: a team of two warps per split
 * (attn_team.cuh). */
template <bool KV8, int NT>
static cudaError_t launch_attn_team(const AttnArgs& a, dim3 grid, cudaStream_t st) {
    static bool attr_set[64] = {false};
    constexpr size_t smem = sizeof(AttnTeamSmem<KV8, NT>);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!attr_set[dev]) {
        e = cudaFuncSetAttribute(k_attn_decode_team<KV8, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    k_attn_decode_team<KV8, NT><<<grid, NT * 64, smem, st>>>(a);
    return cudaGetLastError();
}
constexpr int ATTN_TEAMS_KV8 = 4, ATTN_TEAMS_BF16 = 3; /* two CTAs per SM either way */
static bool attn_team_serves(const AttnArgs& a, int rows) {
    if (rows < 2 || a.out_ll || a.n_out_peers > 0 || (a.max_seq & 1)) return false;
    if ((a.kv.k_off | a.kv.v_off) & 15u) return false;
    if (a.kv8 && ((a.kv.ks_off | a.kv.vs_off) & 15u)) return false;
    if (!a.kv.bases && (a.kv.row_stride & 15u)) return false;
    if (a.kv8 && !a.kv.sbases && (a.kv.srow_stride & 15u)) return false;
    /* the merge keeps two floats per (head, split) in the idle tiles */
    const size_t tiles = a.kv8 ? sizeof(AttnTeamTile<true>) * ATTN_TEAMS_KV8 : sizeof(AttnTeamTile<false>) * ATTN_TEAMS_BF16;
    return (size_t)a.n_split_slots * 32 + 16 <= tiles;
}

cudaError_t launch_attn_decode(const AttnArgs& a, const AttnPrep* prep, int rows, cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    if (a.q_heads != a.kv_heads * 4 || !a.part || !a.counters || a.workers < 1) return cudaErrorInvalidValue;
    dim3 grid((unsigned)rows, (unsigned)a.kv_heads, (unsigned)a.workers);
    if (!prep && attn_team_serves(a, rows))
        return a.kv8 ? launch_attn_team<true, ATTN_TEAMS_KV8>(a, grid, st) : launch_attn_team<false, ATTN_TEAMS_BF16>(a, grid, st);
    AttnPrep pz = {};
    /* one score chain per thread (HPT 1): sharing a key's conversion between the heads of a position
     * (HPT 2 or 4) measured slower on a lockstep batch of 32, fewer warps being busy in the score phase */
    if (prep) {
        pz = *prep;
        if (a.kv8) k_attn_decode<true, true, 1><<<grid, 512, 0, st>>>(a, pz);
        else k_attn_decode<false, true, 1><<<grid, 512, 0, st>>>(a, pz);
    } else {
        if (a.kv8) k_attn_decode<true, false, 1><<<grid, 512, 0, st>>>(a, pz);
        else k_attn_decode<false, false, 1><<<grid, 512, 0, st>>>(a, pz);
    }
    return cudaGetLastError();
}

extern "C" cudaError_t attn_decode(const AttnArgs* a, int rows, cudaStream_t st) {
    return launch_attn_decode(*a, nullptr, rows, st);
}

/* ---- allocation-free variant (include/s2p_b200_ext.h) --------------------------
 * Split-K decode attention for one query row whose scratch (the per-split partials
 * and the arrival counters) lives in a fixed array inside the library image instead
 * of memory obtained from the driver.  Every GPU that loads the library carries the
 * array (about 2.1 MB) until the process exits. */
constexpr int NOALLOC_MAX_POSITIONS = 8192;                       /* cached positions a call may attend over */
constexpr int NOALLOC_SLOTS = NOALLOC_MAX_POSITIONS / 64;          /* 64-position splits */
constexpr size_t NOALLOC_PART_BYTES = (size_t)32 * NOALLOC_SLOTS * 130 * sizeof(float);
constexpr size_t NOALLOC_CTR_BYTES = 8 * sizeof(unsigned int);
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_PART_BYTES + NOALLOC_CTR_BYTES];

}  // namespace s2p

#include <stdio.h>
#include "s2p_b200_ext.h"

extern "C" s2p_status s2p_b200_attention_decode_noalloc(const s2p_bf16* q, const s2p_bf16* k_cache,
                                                        const s2p_bf16* v_cache, s2p_bf16* out, int q_heads,
                                                        int kv_heads, int head_dim, int pos, int max_seq,
                                                        cudaStream_t stream) {
    using namespace s2p;
    if (!q || !k_cache || !v_cache || !out) return S2P_ERR_INVALID;
    if (q_heads != 32 || kv_heads != 8 || head_dim != 128) {
        fprintf(stderr, "[s2pro] attention_decode_noalloc: only 32 query / 8 kv heads of width 128 are served\n");
        return S2P_ERR_INVALID;
    }
    if (pos < 0 || pos >= max_seq || pos + 1 > NOALLOC_MAX_POSITIONS) {
        fprintf(stderr, "[s2pro] attention_decode_noalloc: position %d outside the cache (%d) or beyond the built-in "
                        "scratch limit of %d positions\n", pos, max_seq, NOALLOC_MAX_POSITIONS);
        return S2P_ERR_INVALID;
    }
    /* The array's name is only a host-side handle; the kernel needs its device address.
     * It is looked up once per device, with that device current. */
    static void* dev_addr[64] = {0}; /* filled without a lock: two host threads making their first call at once both look
                                      * the same address up, which is harmless; they must not overlap their launches anyway */
    int dev = -1;
    S2P_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return S2P_ERR_UNSUPPORTED;
    if (!dev_addr[dev]) {
        void* p = NULL;
        S2P_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        dev_addr[dev] = p;
    }
    unsigned char* base = static_cast<unsigned char*>(dev_addr[dev]);
    unsigned int* counters = reinterpret_cast<unsigned int*>(base + NOALLOC_PART_BYTES);
    /* the array keeps whatever the previous call left: the arrival counters must start at zero */
    S2P_CUDA_TRY(cudaMemsetAsync(counters, 0, NOALLOC_CTR_BYTES, stream));
    AttnArgs a = {};
    a.q = reinterpret_cast<const __nv_bfloat16*>(q);
    a.out = reinterpret_cast<__nv_bfloat16*>(out);
    a.q_heads = q_heads; a.kv_heads = kv_heads; a.max_seq = max_seq; a.kv8 = 0; a.head_dim = head_dim;
    a.pos0 = pos; a.pos_row_step = 0;
    /* K and V may be separate allocations in either order: offsets from the lower of the two
     * addresses, computed on integers, so that neither is negative */
    const uintptr_t ka = (uintptr_t)k_cache, va = (uintptr_t)v_cache, lo = ka < va ? ka : va;
    a.kv.base0 = (void*)lo;
    a.kv.k_off = (size_t)(ka - lo);
    a.kv.v_off = (size_t)(va - lo);
    a.part = reinterpret_cast<float*>(base);
    a.counters = counters;
    a.n_split_slots = NOALLOC_SLOTS;
    a.workers = 16;
    S2P_CUDA_TRY(launch_attn_decode(a, nullptr, 1, stream));
    return S2P_OK;
}

namespace s2p {

}  // namespace s2p
