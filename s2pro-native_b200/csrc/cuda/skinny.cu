/* Batched decode linear on the 5th-generation tensor cores: y[M, N] = x[M, K] · Wq^T for the
 * lockstep batches the exact-order GEMV cannot serve well (M > 16 rows; the reference's own
 * kernels stop at 16 rows, src/sched/int8_gemv.cu:964-986, so there is no bit-exact contract
 * beyond that: results agree with the exact path to f32-accumulation-order tolerance).
 *
 * One CTA owns 128 weight rows (the MMA's M; the batch is its N, padded to a power of two from 16
 * to 128; a larger batch takes two launches), or a piece of their K range:
 *   - converting threads (256 or 512) each own one (row, 16-byte unit of packed codes) of every K
 *     slab: they bring the codes and the unit's scales into shared memory with asynchronous copies
 *     that run several slabs ahead (weights in rounds of 256 k, activations slab by slab), convert
 *     them to f16 (INT4: code x f16 group scale, one rounding of a 15-bit product; INT8
 *     per-channel: the exact code, the row scale is applied to the accumulator) and store them in
 *     the K-major, unswizzled core-matrix layout the instruction reads: 16-byte units
 *     [k / 8][row], i.e. 8 rows x 16 B core matrices, 128 B apart along rows (SBO) and one
 *     [k / 8] plane apart along K (LBO);
 *   - the activations (bf16 -> f16, exact in the normal range) go beside them as [k / 8][batch row];
 *   - a separate warp issues the tcgen05.mma of a slab (M 128, N = padded batch, K 16,
 *     f16 x f16 -> f32 in TMEM) when the converting warps have handed the stage over, and commits
 *     them to the mbarrier that gives the stage back; three stages are in flight;
 *   - epilogue: tcgen05.ld of the accumulator (lane = weight row, column = batch row), row
 *     scale, optional residual, bf16, stores coalesced over weight rows; pieces of a split tile
 *     leave f32 partials that the last piece to arrive adds in a fixed order.
 * Every mbarrier wait is bounded; on a time-out the kernel records a status code, skips the
 * epilogue, frees its TMEM and returns.
 */
#include <stdio.h>
#include "common.cuh"
#include "gemv.cuh"
#include "ops.h"
#include "pipe.cuh"
#include "s2p_b200_abi.h"

namespace s2p {

constexpr int SK_BM = 128;
constexpr int SK_MAX_SPLIT = 10;

/* 0 unless a bounded wait inside a launch gave up (read back by skinny_status) */
__device__ int g_sk_status;

__device__ __forceinline__ uint64_t sk_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    /* start address, leading (K) and stride (rows) byte offsets in 16-byte units; descriptor version 1;
     * base offset 0, no swizzle */
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}

/* 8 packed nibbles -> 8 f16 (code x scale) as one 16-byte unit, in the order the extraction yields:
 * nibbles 0,4,1,5,2,6,3,7 (the activations are stored in the same order, see sk_x_unit) */
__device__ __forceinline__ uint4 sk_int4_chunk(uint32_t w, __half2 sc2) {
    const uint32_t a = w ^ 0x88888888u;
    uint32_t p[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const uint32_t m = ((a >> (4 * k)) & 0x000F000Fu) | 0x64006400u; /* (1024 + n_k, 1024 + n_{k+4}) */
        const uint32_t c = 0x64086408u;                                  /* (1032, 1032) */
        __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&m), *reinterpret_cast<const __half2*>(&c));
        h = __hmul2(h, sc2);
        p[k] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(p[0], p[1], p[2], p[3]);
}
/* 8 int8 codes (two words) -> 8 f16, optionally x group scale */
template <bool SCALE>
__device__ __forceinline__ uint4 sk_int8_chunk(uint32_t w0, uint32_t w1, __half2 sc2) {
    const uint32_t c = 0x64806480u; /* (1152, 1152) = 1024 + 128 */
    uint32_t o[4];
    const uint32_t ws[2] = {w0 ^ 0x80808080u, w1 ^ 0x80808080u};
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const uint32_t lo = __byte_perm(ws[i], 0x64646464u, 0x4140), hi = __byte_perm(ws[i], 0x64646464u, 0x4342);
        __half2 hl = __hsub2(*reinterpret_cast<const __half2*>(&lo), *reinterpret_cast<const __half2*>(&c));
        __half2 hh = __hsub2(*reinterpret_cast<const __half2*>(&hi), *reinterpret_cast<const __half2*>(&c));
        if (SCALE) { hl = __hmul2(hl, sc2); hh = __hmul2(hh, sc2); }
        o[2 * i] = *reinterpret_cast<uint32_t*>(&hl);
        o[2 * i + 1] = *reinterpret_cast<uint32_t*>(&hh);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

/* 16-byte asynchronous copy into shared memory, past L1 */
__device__ __forceinline__ void sk_cp16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
/* 4, 8, 16 or 32 bytes of group scales (bytes is uniform over the launch) */
__device__ __forceinline__ void sk_cp_scales(void* dst, const void* src, int bytes) {
    const uint32_t d = smem_u32(dst);
    if (bytes == 4) asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
    else if (bytes == 8) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(src) : "memory");
    else {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
        if (bytes == 32) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d + 16), "l"(static_cast<const char*>(src) + 16) : "memory");
    }
}
/* wait until at most n of this thread's copy groups are pending (n is uniform, 0..7) */
__device__ __forceinline__ void sk_cp_wait(int n) {
    switch (n) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
    }
}

constexpr int SK_SUPER_K = 256; /* K extent of one weight copy round: 128 (INT4) or 256 (INT8) contiguous bytes per row */

constexpr int SK_STAGES = 3; /* converted [A | B] stages between the converting warps and the MMA warp */

template <int WK, int NT, int KCP> struct SkGeom {
    static constexpr int KC = KCP;                                        /* K extent of a converted slab */
    static constexpr int SPS = SK_SUPER_K / KC;                           /* slabs per weight copy round */
    static constexpr int UPR = (WK == WK_INT4_PACK) ? KC / 32 : KC / 16;  /* 16-byte units of packed codes per row and slab */
    static constexpr int PITCHS = UPR * SPS * 16;                         /* bytes of a row per copy round */
    static constexpr int WPU = (WK == WK_INT4_PACK) ? 32 : 16;            /* weights per 16-byte unit */
    static constexpr int NLD = UPR * SK_BM / NT;                          /* units converted per thread and slab */
    static constexpr int NCP = NLD * SPS;                                 /* units copied per thread and round */
    static constexpr int WS_BYTES = NCP * NT * 16;                        /* raw codes of a round: [unit of the thread][thread] */
    static constexpr int SC_BYTES = (WK == WK_INT8_CH) ? 0 : NCP * NT * 4; /* one 4-byte pair of scales per unit */
    static constexpr int SUP_BYTES = WS_BYTES + SC_BYTES;
    static constexpr int A_BYTES = SK_BM * KC * 2;                        /* converted stage */
    static_assert(NT % SK_BM == 0 && NLD >= 1, "thread -> (row, unit) map assumes this");
};

/* bf16 x 8 -> f16 x 8 for the B tile.  INT4 slabs keep the order their conversion produces
 * (elements 0,4,1,5,2,6,3,7 of every eight: no re-interleaving of the nibbles), and the activations
 * follow the same order: the contraction does not care as long as both operands agree. */
template <int WK> __device__ __forceinline__ uint4 sk_x_unit(const uint4& v) {
    __half2 h[4];
    if (WK == WK_INT4_PACK) {
        h[0] = __floats2half2_rn(bf_lo(v.x), bf_lo(v.z));
        h[1] = __floats2half2_rn(bf_hi(v.x), bf_hi(v.z));
        h[2] = __floats2half2_rn(bf_lo(v.y), bf_lo(v.w));
        h[3] = __floats2half2_rn(bf_hi(v.y), bf_hi(v.w));
    } else {
        h[0] = __floats2half2_rn(bf_lo(v.x), bf_hi(v.x));
        h[1] = __floats2half2_rn(bf_lo(v.y), bf_hi(v.y));
        h[2] = __floats2half2_rn(bf_lo(v.z), bf_hi(v.z));
        h[3] = __floats2half2_rn(bf_lo(v.w), bf_hi(v.w));
    }
    return make_uint4(*reinterpret_cast<uint32_t*>(&h[0]), *reinterpret_cast<uint32_t*>(&h[1]), *reinterpret_cast<uint32_t*>(&h[2]),
                      *reinterpret_cast<uint32_t*>(&h[3]));
}

/* weight row behind row r of tile t: plain tiles are 128 consecutive rows; SwiGLU tiles (ffn > 0: the matrix is
 * [gate rows | up rows], ffn of each) pair 64 gate rows with their 64 up rows.  Rows beyond the matrix repeat its
 * last row: their outputs are never stored. */
__device__ __forceinline__ int sk_row(int t, int r, int ffn) {
    if (!ffn) return t * SK_BM + r;
    const int gi = min(t * 64 + (r & 63), ffn - 1);
    return r < 64 ? gi : ffn + gi;
}
/* silu(g) * u with the rounding steps of the unfused kernels (g, u: bf16 values held in f32) */
__device__ __forceinline__ __nv_bfloat16 sk_swiglu(float g, float u) {
    const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g)));
    return f2bf(__fmul_rn(bf16_round(__fmul_rn(g, sig)), u));
}
/* 32 accumulator columns of this warp's 32 TMEM lanes */
__device__ __forceinline__ void sk_tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

/* XT (prompt-sized inputs): the grid's y dimension walks blocks of 256 input rows, and the activations arrive
 * already converted and tiled (k_xt_tile below: f16 units in the order a stage's B tile wants them, one contiguous
 * block per (row block, slab)), so a stage's B tile is ONE bulk copy issued by one thread and the converting threads
 * touch weights only: a weight slab is converted once per 256 input rows instead of once per launch of <= 128.
 * XT == 2: the CTA takes two such blocks (512 rows): two B tiles per stage, two 256-column accumulators side by
 * side in TMEM (all 512 columns), two MMAs per K step on the one converted A tile, and two stages instead of three
 * to make room - a weight slab is converted once per 512 rows. */
template <int WK, int NT, int KCP, int XT>
__global__ void __launch_bounds__(NT + 32, 1) k_skinny_tc(const void* __restrict__ w, const void* __restrict__ scales, int N,
                                                          int K, int gshift, const __nv_bfloat16* __restrict__ x, int M,
                                                          int lgNB, int D, int DW, int n_split_tiles, int KS, int ffn,
                                                          __nv_bfloat16* y, const __nv_bfloat16* resid,
                                                          float* __restrict__ partial, unsigned* __restrict__ arrivals) {
    /* resid (may alias y): y = bf16(f32(resid) + f32(bf16(product))), the residual add of the decode layers */
    /* ffn > 0: W is a [gate | up] pair of ffn rows each and y[M, ffn] = silu(x Wg^T) * (x Wu^T) (see sk_row) */
    /* The last n_split_tiles row tiles have their K range split over KS CTAs each; those CTAs come first
     * in the grid (short pieces first, whole tiles after them: the tail of the grid stays balanced).  Each
     * piece leaves its f32 partial in `partial`[split tile][piece][batch row][128] and the last piece of a
     * tile to arrive adds them in piece order. */
    /* Roles: NT converting threads and one MMA warp, coupled only by mbarriers.
     *  - A converting thread copies, converts and stores its own (row, unit) of every slab: raw codes and
     *    scales travel by asynchronous copies into thread-private places of two rings (DW copy rounds of
     *    weights of 256 k, D slabs of activations), so no thread waits for another's copy; a stage is
     *    handed over by one arrival per warp on full[stage] and taken back on done[stage], which the
     *    tensor core signals when the MMAs that read the stage have completed.
     *  - The MMA warp waits for full[stage], issues the stage's MMAs and commits them to done[stage].
     * Copies, conversion and MMAs of different slabs overlap; nothing in the loop is a CTA-wide barrier. */
    typedef SkGeom<WK, NT, KCP> G;
    constexpr int KC = G::KC, NST = (XT == 2) ? 2 : SK_STAGES;
    constexpr int NBLK = (XT == 2) ? 2 : 1; /* blocks of NB input rows per CTA */
    int* status = &g_sk_status;
    extern __shared__ __align__(1024) unsigned char smem[];
    const int NB = 1 << lgNB;
    const int b_bytes = NB * KC * 2;
    const int x_units = NB * (KC / 8);
    const int x_bytes = x_units * 16;
    unsigned char* stage_b0 = smem + NST * G::A_BYTES;
    unsigned char* xring = stage_b0 + NST * NBLK * b_bytes;
    unsigned char* wring = xring + (XT ? 0 : D * x_bytes); /* XT: no ring of raw activations, B tiles land in the stages */
    uint64_t* full = reinterpret_cast<uint64_t*>(wring + DW * G::SUP_BYTES);
    uint64_t* done = full + NST;
    uint64_t* bx = done + NST; /* XT: the bulk copy of a stage's B tile has landed */
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bx + NST);
    if (XT) { /* this CTA's block(s) of 256 input rows */
        const int tb = (int)blockIdx.y * NBLK;
        x = reinterpret_cast<const __nv_bfloat16*>(reinterpret_cast<const unsigned char*>(x) + (size_t)tb * (size_t)(K / KC) * (size_t)b_bytes);
        y += (size_t)tb * 256 * (size_t)(ffn ? ffn : N);
        if (resid) resid += (size_t)tb * 256 * (size_t)N;
        if (partial) partial += (size_t)blockIdx.y * (size_t)n_split_tiles * KS * (256 * NBLK) * SK_BM;
        if (arrivals) arrivals += (size_t)blockIdx.y * n_split_tiles;
        M = min(256 * NBLK, M - tb * 256);
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool mma_warp = warp == NT / 32;
    const int n_tiles = ffn ? (ffn + 63) / 64 : (N + SK_BM - 1) / SK_BM, n_pieces = n_split_tiles * KS;
    const bool piece = (int)blockIdx.x < n_pieces;
    const int stile = piece ? (int)blockIdx.x / KS : 0;                     /* index among the split tiles */
    const int ks = piece ? (int)blockIdx.x % KS : 0, ksn = piece ? KS : 1;  /* this CTA's piece of how many */
    const int tile = piece ? n_tiles - n_split_tiles + stile : (int)blockIdx.x - n_pieces;
    const int n0 = tile * SK_BM;
    const size_t row_bytes = (WK == WK_INT4_PACK) ? (size_t)(K >> 1) : (size_t)K;
    int ncols = 32;
    while (ncols < NB * NBLK) ncols <<= 1;

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        for (int i = 0; i < NST; i++) {
            mbar_init(full + i, NT / 32);
            mbar_init(done + i, 1);
            mbar_init(bx + i, 1);
        }
        mbar_init_fence();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    /* the K range of this CTA, in whole copy rounds */
    const int nsup_all = K / SK_SUPER_K;
    const int sup_first = nsup_all * ks / ksn, nsup = nsup_all * (ks + 1) / ksn - sup_first;
    const int it_first = sup_first * G::SPS, nk = nsup * G::SPS;
    bool ok = true;

    if (!mma_warp) {
        /* ---- this thread's row and units: unit q0 + i NT / 128 of every slab (i < NLD); rows beyond N (last
         * tile) repeat row N - 1: their outputs are never stored */
        const int cv_row = tid & (SK_BM - 1), cv_q0 = tid >> 7;
        const int grow_c = min(sk_row(tile, cv_row, ffn), N - 1);
        const unsigned char* wsrc = static_cast<const unsigned char*>(w) + (size_t)grow_c * row_bytes + (size_t)sup_first * G::PITCHS;
        const int sc_round = SK_SUPER_K >> gshift; /* scales per row and round */
        const __half* sc_src = nullptr;
        if (WK != WK_INT8_CH) sc_src = static_cast<const __half*>(scales) + (size_t)grow_c * (K >> gshift) + (size_t)sup_first * sc_round;
        int w_wslot = 0, w_issued = 0;
        auto issue_w = [&]() {
            unsigned char* sup = wring + w_wslot + tid * 16;
#pragma unroll
            for (int j = 0; j < G::SPS; j++)
#pragma unroll
                for (int i = 0; i < G::NLD; i++) {
                    const int c = j * G::UPR + cv_q0 + i * (NT / SK_BM), u = j * G::NLD + i;
                    sk_cp16(sup + u * (NT * 16), wsrc + c * 16);
                    if (WK != WK_INT8_CH) /* the aligned pair of scales holding the unit's */
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(wring + w_wslot + G::WS_BYTES + (u * NT + tid) * 4)),
                                     "l"(sc_src + (((c * G::WPU) >> gshift) & ~1)) : "memory");
                }
            wsrc += G::PITCHS;
            if (WK != WK_INT8_CH) sc_src += sc_round;
            w_issued++;
            w_wslot += G::SUP_BYTES;
            if (w_wslot == DW * G::SUP_BYTES) w_wslot = 0;
        };
        /* activations, slab by slab: unit c = [k / 8][batch row] sits in the slot where the B tile wants it;
         * c = tid + NT u; rows beyond the batch repeat row M - 1 (their columns are never stored) */
        const int x_mine = (!XT && tid < x_units) ? (x_units + NT - 1 - tid) / NT : 0; /* units of this thread */
        const int x_step = (NT >> lgNB) * 8;                                   /* elements between them (NB <= NT) */
        const __nv_bfloat16* xsrc = XT ? x : x + (size_t)min(tid & (NB - 1), M - 1) * K + (size_t)it_first * KC + (tid >> lgNB) * 8;
        int b_issued = 0; /* XT, thread 0: bulk copies of B tiles issued */
        int x_wslot = 0, x_issued = 0;
        auto issue_x = [&]() {
            unsigned char* slot = xring + x_wslot + tid * 16;
            for (int u = 0; u < x_mine; u++) sk_cp16(slot + u * (NT * 16), xsrc + u * x_step);
            xsrc += KC;
            x_issued++;
            x_wslot += x_bytes;
            if (x_wslot == D * x_bytes) x_wslot = 0;
        };
        /* One copy group per slab round, empty ones included, so that the group count tells what has landed:
         * round v carries the activations of slab v + D - 1 and, when v is a multiple of SPS, the weights of
         * copy round v / SPS + DW - 1.  With D <= SPS (DW - 1) + 1 (the host's choice), "at most D - 2 groups
         * pending" at the end of round v means this thread's share of slab v + 1 has landed, weights included. */
        for (int v = -G::SPS * (DW - 1); v < 0; v++) {
            if (v + D - 1 >= 0 && x_issued < nk) issue_x();
            if ((-v) % G::SPS == 0 && w_issued < nsup) issue_w();
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        sk_cp_wait(D - 2); /* slab 0 */

        const int a_off0 = (cv_q0 * (G::WPU / 8) * SK_BM + cv_row) * 16;
        int x_rslot = 0, w_rslot = 0; /* read offsets into the rings */
        int s = 0;                              /* stage of slab it, and whether it has been used before */
        unsigned done_parity = 1;               /* parity of the completion of done[s] that frees the stage: it / NST - 1 */
        int it = 0;
        for (int rnd = 0; rnd < nsup && ok; rnd++) {
#pragma unroll
          for (int j_in = 0; j_in < G::SPS; j_in++, it++) { /* the slab's place in its copy round is a constant */
            /* the places the next copies fill were read by this thread one round ago */
            if (x_issued < nk) issue_x();
            if (j_in == 0 && w_issued < nsup) issue_w();
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (it >= NST) ok = mbar_wait_bounded(done + s, done_parity, status); /* the MMAs that read this stage */
            if (!ok) break;
            const unsigned char* sup = wring + w_rslot;
            unsigned char* A = smem + s * G::A_BYTES;
            unsigned char* B = stage_b0 + s * (NBLK * b_bytes);
            if (XT && tid == 0) { /* the stage is free (its MMAs have completed): its B tile(s) travel while the weights are converted */
                mbar_expect_tx(bx + s, (unsigned)(NBLK * b_bytes));
#pragma unroll
                for (int blk = 0; blk < NBLK; blk++) /* the same slab of the next row block lies K / KC tiles further on */
                    tma_load_1d(B + blk * b_bytes,
                                reinterpret_cast<const unsigned char*>(x) + ((size_t)blk * (size_t)(K / KC) + (size_t)(it_first + it)) * (size_t)b_bytes,
                                (unsigned)b_bytes, bx + s);
                b_issued++;
            }
            /* weights: A[k / 8][row] */
#pragma unroll
            for (int i = 0; i < G::NLD; i++) {
                const int u = j_in * G::NLD + i;
                const uint4 pk = *reinterpret_cast<const uint4*>(sup + (u * NT + tid) * 16);
                __half2 sc2 = __float2half2_rn(1.f);
                if (WK != WK_INT8_CH) {
                    const int c = j_in * G::UPR + cv_q0 + i * (NT / SK_BM);
                    sc2 = __half2half2(reinterpret_cast<const __half*>(sup + G::WS_BYTES + (u * NT + tid) * 4)[((c * G::WPU) >> gshift) & 1]);
                }
                uint4* Au = reinterpret_cast<uint4*>(A + a_off0 + i * ((NT / SK_BM) * (G::WPU / 8) * SK_BM * 16));
                if (WK == WK_INT4_PACK) {
                    const uint32_t ws[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
                    for (int j = 0; j < 4; j++) Au[j * SK_BM] = sk_int4_chunk(ws[j], sc2);
                } else {
                    Au[0] = sk_int8_chunk<WK == WK_INT8_GRP>(pk.x, pk.y, sc2);
                    Au[SK_BM] = sk_int8_chunk<WK == WK_INT8_GRP>(pk.z, pk.w, sc2);
                }
            }
            /* activations: B[k / 8][batch row] */
            for (int u = 0; u < x_mine; u++)
                *reinterpret_cast<uint4*>(B + (tid + u * NT) * 16) = sk_x_unit<WK>(*reinterpret_cast<const uint4*>(xring + x_rslot + (tid + u * NT) * 16));
            x_rslot += x_bytes;
            if (x_rslot == D * x_bytes) x_rslot = 0;
            fence_proxy_async_smem(); /* these generic-proxy stores are read by the tensor core (async proxy) */
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(full + s)) : "memory");
            if (++s == NST) { s = 0; done_parity ^= 1u; }
            sk_cp_wait(D - 2); /* this thread's share of slab it + 1 */
          }
          w_rslot += G::SUP_BYTES;
          if (w_rslot == DW * G::SUP_BYTES) w_rslot = 0;
        }
        asm volatile("cp.async.wait_all;" ::: "memory"); /* nothing of this thread's is in flight past here */
        if (XT && tid == 0 && b_issued > 0) {
            /* nor a bulk copy: the last one issued has landed (at once on the normal path, where the MMA warp waited
             * for it; after a give-up, with a fixed generous limit of its own) */
            uint64_t* bar = bx + ((b_issued - 1) % NST);
            const unsigned parity = (unsigned)((b_issued - 1) / NST) & 1u;
            PipeDeadline dl;
            for (unsigned i = 0; i < PIPE_MBAR_TRIES && !mbar_try_wait(bar, parity); i++)
                if ((i & 63u) == 63u && dl.expired(2000000000ull)) break;
        }
    } else {
        /* ---- the MMA warp (its lane 0 issues) */
        /* instruction descriptor: D f32, A and B f16, both K-major, N = NB, M = 128 */
        const uint32_t idesc = (1u << 4) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(SK_BM >> 4) << 24);
        const uint64_t desc_a0 = sk_smem_desc(smem_u32(smem), SK_BM * 16, 128);
        const uint64_t desc_b0 = sk_smem_desc(smem_u32(stage_b0), (uint32_t)NB * 16, 128);
        int s = 0, issued = 0;
        unsigned full_parity = 0;
        for (int it = 0; it < nk; it++) {
            ok = mbar_wait_bounded(full + s, full_parity, status);
            if (ok && XT) ok = mbar_wait_bounded(bx + s, full_parity, status);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                /* the start-address field counts 16-byte units: stage s and K step kk are plain additions */
                const uint64_t da0 = desc_a0 + (uint64_t)((s * G::A_BYTES) >> 4);
                const uint64_t db0 = desc_b0 + (uint64_t)((s * NBLK * b_bytes) >> 4);
#pragma unroll
                for (int kk = 0; kk < KC / 16; kk++) {
                    const uint64_t da = da0 + (uint64_t)(kk * 2 * SK_BM);
                    const uint64_t db = db0 + (uint64_t)(kk * 2 * NB);
                    const uint32_t accumulate = (it > 0 || kk > 0) ? 1u : 0u;
#pragma unroll
                    for (int blk = 0; blk < NBLK; blk++) /* accumulator blk: TMEM columns blk NB .., B tile blk of the stage */
                        asm volatile(
                            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                            ::"r"(tmem + (uint32_t)(blk * NB)), "l"(da), "l"(db + (uint64_t)((blk * b_bytes) >> 4)), "r"(idesc), "r"(accumulate) : "memory");
                }
                /* arrives on the barrier once every MMA issued so far has completed */
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(done + s)) : "memory");
            }
            __syncwarp();
            issued = it + 1;
            if (++s == NST) { s = 0; full_parity ^= 1u; }
        }
        if (!ok && issued > 0) {
            /* giving up with MMAs in flight: they complete by themselves (nothing but the tensor core is
             * waited for), and TMEM must not be freed under them.  Wait for the last commit with a fixed,
             * generous limit, whatever deadline the other waits have. */
            uint64_t* bar = done + ((issued - 1) % NST);
            const unsigned parity = (unsigned)((issued - 1) / NST) & 1u;
            PipeDeadline dl;
            for (unsigned i = 0; i < PIPE_MBAR_TRIES && !mbar_try_wait(bar, parity); i++)
                if ((i & 63u) == 63u && dl.expired(2000000000ull)) break;
        }
    }
    /* the last commit covers every MMA before it */
    if (ok) ok = mbar_wait_bounded(done + ((nk - 1) % NST), (unsigned)((nk - 1) / NST) & 1u, status);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const bool all_ok = __syncthreads_and(ok ? 1 : 0) != 0; /* one verdict for the CTA: the epilogue has barriers */
    /* warp w reads TMEM lanes 32 (w % 4) .. + 31 = the tile's rows; the warps of a lane quarter share the columns */
    const int lrow = (warp & 3) * 32 + lane;
    const int grow = sk_row(tile, lrow, ffn);
    const bool row_live = ffn ? (tile * 64 + (lrow & 63)) < ffn : grow < N;
    float rs = 1.f;
    if (WK == WK_INT8_CH && row_live) rs = static_cast<const float*>(scales)[grow];
    if (all_ok && !mma_warp && (piece || !ffn)) {
        for (int col0 = (warp >> 2) * 32; col0 < NB * NBLK; col0 += (NT / 128) * 32) {
            uint32_t v[32];
            sk_tmem_ld32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)col0, v);
            if (row_live) {
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const int m = col0 + j;
                    if (m < M) {
                        if (!piece) {
                            __nv_bfloat16 o = f2bf(__fmul_rn(__uint_as_float(v[j]), rs));
                            if (resid) o = f2bf(__fadd_rn(bf2f(resid[(size_t)m * N + grow]), bf2f(o)));
                            y[(size_t)m * N + grow] = o;
                        }
                        else partial[(((size_t)stile * KS + ks) * M + m) * SK_BM + lrow] = __uint_as_float(v[j]);
                    }
                }
            }
        }
    }
    if (all_ok && ffn && !piece) {
        /* SwiGLU: lanes 0..63 hold gate rows, lanes 64..127 the matching up rows; the up halves cross to the gate
         * warps through shared memory (the stages are free: every MMA has completed).  Arithmetic of the unfused
         * pair: both products rounded to bf16, sigmoid and silu in f32, silu rounded to bf16, times up, bf16. */
        float* ex = reinterpret_cast<float*>(smem); /* [64 rows][NB + 1] */
        if (!mma_warp && (warp & 3) >= 2) {
            for (int col0 = (warp >> 2) * 32; col0 < NB * NBLK; col0 += (NT / 128) * 32) {
                uint32_t v[32];
                sk_tmem_ld32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)col0, v);
#pragma unroll
                for (int j = 0; j < 32; j++) ex[(lrow - 64) * (NB + 1) + col0 + j] = bf16_round(__fmul_rn(__uint_as_float(v[j]), rs));
            }
        }
        __syncthreads();
        if (!mma_warp && (warp & 3) < 2) {
            const int gi = tile * 64 + lrow;
            for (int col0 = (warp >> 2) * 32; col0 < NB * NBLK; col0 += (NT / 128) * 32) {
                uint32_t v[32];
                sk_tmem_ld32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)col0, v);
                if (row_live) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int m = col0 + j;
                        if (m < M) y[(size_t)m * ffn + gi] = sk_swiglu(bf16_round(__fmul_rn(__uint_as_float(v[j]), rs)), ex[lrow * (NB + 1) + m]);
                    }
                }
            }
        }
    }
    if (piece) {
        __shared__ int s_last;
        __threadfence();
        __syncthreads();
        if (tid == 0) s_last = all_ok && (atomicAdd(arrivals + stile, 1u) == (unsigned)(KS - 1));
        __syncthreads();
        if (s_last && !mma_warp && !ffn) {
            __threadfence();
            /* four outputs per thread and round, the loads of all splits in flight together; the adds keep split order */
            for (int e0 = tid; e0 < SK_BM * M; e0 += NT * 4) {
                float v[4][SK_MAX_SPLIT];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int e = e0 + u * NT, m = e >> 7, er = n0 + (e & (SK_BM - 1));
                    const bool live = e < SK_BM * M && er < N;
#pragma unroll
                    for (int q = 0; q < SK_MAX_SPLIT; q++)
                        v[u][q] = (live && q < KS) ? __ldcg(partial + (((size_t)stile * KS + q) * M + m) * SK_BM + (e & (SK_BM - 1))) : 0.f;
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int e = e0 + u * NT, m = e >> 7, er = n0 + (e & (SK_BM - 1));
                    if (e >= SK_BM * M || er >= N) continue;
                    float acc = 0.f;
#pragma unroll
                    for (int q = 0; q < SK_MAX_SPLIT; q++)
                        if (q < KS) acc += v[u][q];
                    if (WK == WK_INT8_CH) acc = __fmul_rn(acc, static_cast<const float*>(scales)[er]);
                    __nv_bfloat16 o = f2bf(acc);
                    if (resid) o = f2bf(__fadd_rn(bf2f(resid[(size_t)m * N + er]), bf2f(o)));
                    y[(size_t)m * N + er] = o;
                }
            }
        }
        if (s_last && !mma_warp && ffn) {
            __threadfence();
            for (int e = tid; e < 64 * M; e += NT) { /* (batch row, gate row) pairs of the tile */
                const int m = e >> 6, r = e & 63, gi = tile * 64 + r;
                if (gi >= ffn) continue;
                float vg[SK_MAX_SPLIT], vu[SK_MAX_SPLIT];
#pragma unroll
                for (int q = 0; q < SK_MAX_SPLIT; q++) {
                    const float* pp = partial + (((size_t)stile * KS + (q < KS ? q : 0)) * M + m) * SK_BM;
                    vg[q] = q < KS ? __ldcg(pp + r) : 0.f;
                    vu[q] = q < KS ? __ldcg(pp + 64 + r) : 0.f;
                }
                float ag = 0.f, au = 0.f;
#pragma unroll
                for (int q = 0; q < SK_MAX_SPLIT; q++)
                    if (q < KS) { ag += vg[q]; au += vu[q]; }
                if (WK == WK_INT8_CH) {
                    ag = __fmul_rn(ag, static_cast<const float*>(scales)[gi]);
                    au = __fmul_rn(au, static_cast<const float*>(scales)[ffn + gi]);
                }
                y[(size_t)m * ffn + gi] = sk_swiglu(bf16_round(ag), bf16_round(au));
            }
        }
        if (s_last && tid == 0) arrivals[stile] = 0u;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(ncols) : "memory");
}

constexpr size_t SK_SMEM_ONE = 226 * 1024; /* one CTA per SM */
constexpr int SK_MAX_DEPTH = 8;

/* scratch for split-K launches: f32 partials [split tile][piece][batch row][128] and one arrival counter per split tile */
constexpr int SK_SCRATCH_FLOATS_PER_ROW = 8 * 6144; /* per batch row: eight pieces of a 6144-row matrix */
constexpr int SK_MAX_SPLIT_TILES = 256;
static float* g_partial[64];
static unsigned* g_arrivals[64];
static int g_partial_rows[64];

/* Once per device, outside stream capture: room for split-K launches.  The scratch is sized for the largest batch
 * the kernel serves and never freed or moved: captured graphs of any model hold its address.  All models and
 * streams of a device share it (and the arrival counters), so batched ticks of two models must not overlap on
 * the GPU - the library issues every tick of a process from one host thread, as the reference's scheduler does. */
extern "C" cudaError_t skinny_setup(int max_rows) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || max_rows < 1) return cudaErrorInvalidValue;
    if (g_partial[dev]) return cudaSuccess;
    const int rows = 256;
    if ((e = cudaMalloc((void**)&g_partial[dev], (size_t)SK_SCRATCH_FLOATS_PER_ROW * rows * sizeof(float))) != cudaSuccess) return e;
    if (!g_arrivals[dev]) {
        if ((e = cudaMalloc((void**)&g_arrivals[dev], SK_MAX_SPLIT_TILES * sizeof(unsigned))) != cudaSuccess) return e;
        if ((e = cudaMemset(g_arrivals[dev], 0, SK_MAX_SPLIT_TILES * sizeof(unsigned))) != cudaSuccess) return e;
    }
    g_partial_rows[dev] = rows;
    return cudaSuccess;
}

/* After a launch left a status code: clear it and the arrival counters (a CTA that gave up did not count itself in),
 * in stream order, so that later launches start clean. */
extern "C" cudaError_t skinny_reset(cudaStream_t st) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    void* sp = nullptr;
    if ((e = cudaGetSymbolAddress(&sp, g_sk_status)) != cudaSuccess) return e;
    if ((e = cudaMemsetAsync(sp, 0, sizeof(int), st)) != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && g_arrivals[dev])
        e = cudaMemsetAsync(g_arrivals[dev], 0, SK_MAX_SPLIT_TILES * sizeof(unsigned), st);
    return e;
}
extern "C" cudaError_t skinny_set_wait_ns(unsigned long long ns) { return cudaMemcpyToSymbol(c_pipe_wait_ns, &ns, sizeof(ns)); }

/* shared memory of a launch: the converted stages, D slabs of raw activations, DW copy rounds of raw weights, barriers */
template <int WK, int NT, int KCP> static size_t sk_fixed_bytes(int NB) {
    return SK_STAGES * ((size_t)SkGeom<WK, NT, KCP>::A_BYTES + (size_t)NB * SkGeom<WK, NT, KCP>::KC * 2) + 128;
}
/* ring depths that fit `budget` bytes; false if not even the shallowest does */
template <int WK, int NT, int KCP> static bool sk_depths(int NB, size_t budget, int min_d, int* D, int* DW) {
    typedef SkGeom<WK, NT, KCP> G;
    const size_t fixed = sk_fixed_bytes<WK, NT, KCP>(NB), xslot = (size_t)NB * G::KC * 2;
    for (int dw = 3; dw >= 2; dw--) {
        if (fixed + (size_t)dw * G::SUP_BYTES + (size_t)min_d * xslot > budget) continue;
        int d = (int)((budget - fixed - (size_t)dw * G::SUP_BYTES) / xslot);
        if (d > G::SPS * (dw - 1) + 1) d = G::SPS * (dw - 1) + 1; /* what the kernel's group counting needs */
        if (d > SK_MAX_DEPTH) d = SK_MAX_DEPTH;
        if (d < min_d) continue;
        *D = d; *DW = dw;
        return true;
    }
    return false;
}

/* What a launch looks like, decided on the host from the shapes alone (no CUDA call: the CPU tests check it) */
struct SkPlan {
    int lgNB;        /* batch padded to 1 << lgNB */
    int tiles;       /* row tiles of 128 */
    int S, KS;       /* S of them split into KS pieces each (the pieces come first in the grid) */
    int nt, kc;      /* converting threads, K extent of a slab */
    int D, DW;       /* ring depths: activation slabs, weight copy rounds */
    int grid, smem;  /* CTAs, dynamic shared memory */
};

/* launch policy (skinny_tune): CTAs the split aims at, and the kernel shape: 0 = 256 threads, 64-k slabs;
 * 1 = 512 threads, 128-k slabs (the default, fastest measured); 2 = 256 threads, 128-k slabs */
static int g_sk_target_ctas = 148;
static int g_sk_shape = 1;
extern "C" void skinny_tune(int target_ctas, int shape) {
    g_sk_target_ctas = target_ctas < 1 ? 1 : target_ctas;
    g_sk_shape = shape;
}

template <int WK, int NT, int KCP> static bool sk_plan_shape(SkPlan* p) {
    typedef SkGeom<WK, NT, KCP> G;
    const int NB = 1 << p->lgNB;
    if (!sk_depths<WK, NT, KCP>(NB, SK_SMEM_ONE, NT == 256 && KCP == 64 ? 2 : 3, &p->D, &p->DW)) return false;
    p->nt = NT; p->kc = KCP;
    p->smem = (int)(sk_fixed_bytes<WK, NT, KCP>(NB) + (size_t)p->D * NB * G::KC * 2 + (size_t)p->DW * G::SUP_BYTES);
    return true;
}

/* scratch_rows: batch rows the split-K scratch of the device was set up for (0: none) */
template <int WK> static bool sk_plan(int N, int K, int M, int scratch_rows, int ffn, SkPlan* p) {
    p->lgNB = 4; /* the batch is padded to a power of two: the MMA's N */
    while ((1 << p->lgNB) < M) p->lgNB++;
    p->tiles = ffn ? (ffn + 63) / 64 : (N + SK_BM - 1) / SK_BM; /* SwiGLU tiles: 64 gate rows + their 64 up rows */
    /* S of the row tiles have their K range split into KS pieces:
     *  - few tiles: all of them, until the grid fills the GPU;
     *  - a few more tiles than SMs: the surplus ones, so that no SM is left with two whole tiles while the
     *    others idle (the pieces run first, the whole tiles fill in behind them). */
    p->S = 0; p->KS = 1;
    if (scratch_rows >= M) {
        int max_ks = K / SK_SUPER_K;
        if (max_ks > SK_MAX_SPLIT) max_ks = SK_MAX_SPLIT;
        if (p->tiles * 2 <= g_sk_target_ctas) {
            p->S = p->tiles;
            p->KS = g_sk_target_ctas / p->tiles < max_ks ? g_sk_target_ctas / p->tiles : max_ks;
        } else if (p->tiles > 148 && p->tiles < 2 * 148) {
            p->S = p->tiles - 148;
            p->KS = max_ks;
        }
        const size_t cap = (size_t)SK_SCRATCH_FLOATS_PER_ROW * scratch_rows;
        while (p->KS > 1 && (size_t)p->S * p->KS * M * SK_BM > cap) p->KS--;
        if (p->KS <= 1 || p->S > SK_MAX_SPLIT_TILES) { p->S = 0; p->KS = 1; }
    }
    p->grid = p->tiles - p->S + p->S * p->KS;
    if (K % 128 == 0) {
        if (g_sk_shape == 1 && sk_plan_shape<WK, 512, 128>(p)) return true;
        if (g_sk_shape == 2 && sk_plan_shape<WK, 256, 128>(p)) return true;
    }
    return sk_plan_shape<WK, 256, 64>(p);
}

template <int WK, int NT, int KCP>
static cudaError_t sk_launch_nt(const LinRef* lin, const void* x, int M, const SkPlan& p, int ffn, void* y, const void* resid,
                                float* partial, unsigned* arrivals, cudaStream_t st) {
    static bool attr_set[64] = {false}; /* the attribute belongs to the function on one device */
    int dev = 0;
    cudaError_t ed = cudaGetDevice(&dev);
    if (ed != cudaSuccess) return ed;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_skinny_tc<WK, NT, KCP, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SK_SMEM_ONE);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    k_skinny_tc<WK, NT, KCP, 0><<<dim3((unsigned)p.grid), NT + 32, (size_t)p.smem, st>>>(
        lin->w, lin->scales, lin->N, lin->K, lin->gshift, (const __nv_bfloat16*)x, M, p.lgNB, p.D, p.DW, p.S, p.KS, ffn, (__nv_bfloat16*)y,
        (const __nv_bfloat16*)resid, partial, arrivals);
    return cudaGetLastError();
}

template <int WK>
static cudaError_t sk_launch(const LinRef* lin, const void* x, int M, int ffn, void* y, const void* resid, cudaStream_t st) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const bool have = dev >= 0 && dev < 64;
    SkPlan p;
    if (!sk_plan<WK>(lin->N, lin->K, M, have ? g_partial_rows[dev] : 0, ffn, &p)) return cudaErrorInvalidValue;
    float* partial = p.S ? g_partial[dev] : nullptr;
    unsigned* arrivals = p.S ? g_arrivals[dev] : nullptr;
    if (p.nt == 512) return sk_launch_nt<WK, 512, 128>(lin, x, M, p, ffn, y, resid, partial, arrivals, st);
    if (p.kc == 128) return sk_launch_nt<WK, 256, 128>(lin, x, M, p, ffn, y, resid, partial, arrivals, st);
    return sk_launch_nt<WK, 256, 64>(lin, x, M, p, ffn, y, resid, partial, arrivals, st);
}

/* the plan for a shape as 10 ints (SkPlan's fields in order); 0 when the shape cannot be served (tests) */
extern "C" int skinny_plan_probe(int kind, int N, int K, int M, int scratch_rows, int out[10]) {
    SkPlan p = {};
    bool ok = false;
    switch (kind) {
    case WK_INT8_CH: ok = sk_plan<WK_INT8_CH>(N, K, M, scratch_rows, 0, &p); break;
    case WK_INT8_GRP: ok = sk_plan<WK_INT8_GRP>(N, K, M, scratch_rows, 0, &p); break;
    case WK_INT4_PACK: ok = sk_plan<WK_INT4_PACK>(N, K, M, scratch_rows, 0, &p); break;
    }
    const int v[10] = {p.lgNB, p.tiles, p.S, p.KS, p.nt, p.kc, p.D, p.DW, p.grid, p.smem};
    for (int i = 0; i < 10; i++) out[i] = v[i];
    return ok ? 1 : 0;
}

/* y[M, N] (bf16) = x[M, K] (bf16) · W^T for 1 <= M <= 256, plus `resid` [M, N] when given (it may be y
 * itself).  K must be a multiple of 256, the group size of grouped kinds a power of two from 32 (INT4) / 16 (INT8
 * codes) to 128. */
static cudaError_t sk_entry(const LinRef* lin, const void* x, int M, int ffn, void* y, const void* resid, cudaStream_t st) {
    if (!lin || !x || !y || M < 1 || M > 256 || lin->K % SK_SUPER_K) return cudaErrorInvalidValue;
    if (((uintptr_t)x | (uintptr_t)lin->w) & 15) return cudaErrorInvalidValue;
    if (lin->kind != WK_INT8_CH) /* a round's scales (256 / group of them) are copied in aligned 4-byte pairs */
        if (lin->gshift < 4 || lin->gshift > 7 || ((uintptr_t)lin->scales & 15)) return cudaErrorInvalidValue;
    if (lin->kind == WK_INT4_PACK && lin->gshift < 5) return cudaErrorInvalidValue;
    if (ffn && (lin->N != 2 * ffn || resid)) return cudaErrorInvalidValue;
    const int out_cols = ffn ? ffn : lin->N;
    /* the MMA's N is the batch padded to a power of two, at most 128: a larger batch takes two launches */
    for (int m0 = 0; m0 < M; m0 += 128) {
        const int mm = M - m0 < 128 ? M - m0 : 128;
        const void* xs = static_cast<const char*>(x) + (size_t)m0 * lin->K * 2;
        void* ys = static_cast<char*>(y) + (size_t)m0 * out_cols * 2;
        const void* rs = resid ? static_cast<const char*>(resid) + (size_t)m0 * lin->N * 2 : nullptr;
        cudaError_t e = cudaErrorInvalidValue;
        switch (lin->kind) {
        case WK_INT8_CH: e = sk_launch<WK_INT8_CH>(lin, xs, mm, ffn, ys, rs, st); break;
        case WK_INT8_GRP: e = sk_launch<WK_INT8_GRP>(lin, xs, mm, ffn, ys, rs, st); break;
        case WK_INT4_PACK: e = sk_launch<WK_INT4_PACK>(lin, xs, mm, ffn, ys, rs, st); break;
        }
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

extern "C" cudaError_t skinny_gemm_tc(const LinRef* lin, const void* x, int M, void* y, const void* resid, cudaStream_t st) {
    return sk_entry(lin, x, M, 0, y, resid, st);
}

/* h[M, N / 2] (bf16) = silu(x · Wg^T) * (x · Wu^T) for W = [Wg | Wu] stacked along its N rows: the gate/up linear
 * of a decode layer with the SwiGLU kernel's arithmetic in the epilogue */
extern "C" cudaError_t skinny_gemm_tc_swiglu(const LinRef* lin, const void* x, int M, void* h, cudaStream_t st) {
    if (!lin || (lin->N & 1)) return cudaErrorInvalidValue;
    return sk_entry(lin, x, M, lin->N / 2, h, nullptr, st);
}

/* ---- prompt-sized inputs (prefill): M rows in blocks of 256 ------------------------------------------------
 * What this replaces: the reference dequantises the whole layer to bf16 and calls cuBLAS for M > 16
 * (src/sched/gemm.c:467-490; its own S2P_PREFILL_TC path, :458-466, serves M <= 128 only).  Here the packed
 * weights go to the tensor cores directly: a CTA owns 128 weight rows x 256 input rows (one 256-column f32
 * accumulator in TMEM), converts each weight slab once for the 256 rows, and receives the activations as
 * bulk copies of pre-tiled f16 blocks written by k_xt_tile. */
constexpr int XT_ROWS = 256;   /* input rows per block: the MMA's N; a CTA takes one block or (packed INT4, longer prompts) two */
constexpr int XT_NT = 256, XT_KC = 64; /* kernel shape: three stages of 16 KB (A) + 32 KB (B) fit beside the weight ring */

/* x [M, K] bf16 -> f16 units of 8 in the order stage B wants them: [row block][slab][k / 8 within the slab][row][8],
 * each unit in the within-8 element order of the weight conversion (sk_x_unit); rows beyond M are zero */
template <int WK>
__global__ void k_xt_tile(const __nv_bfloat16* __restrict__ x, int M, int K, int rows_pad, uint4* __restrict__ xt) {
    const int k8n = K >> 3;
    const size_t u = (size_t)blockIdx.x * blockDim.x + threadIdx.x; /* (row, k8): consecutive threads read one row */
    const size_t rows_padded = (size_t)rows_pad; /* whole row blocks (an even number of them where a CTA takes two) */
    if (u >= rows_padded * k8n) return;
    const int row = (int)(u / k8n), k8 = (int)(u - (size_t)row * k8n);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < M) v = __ldg(reinterpret_cast<const uint4*>(x + (size_t)row * K) + k8);
    const int tb = row / XT_ROWS, r = row - tb * XT_ROWS;
    const int slab = (k8 * 8) / XT_KC, k8_in = k8 - slab * (XT_KC / 8);
    xt[(((size_t)tb * (K / XT_KC) + slab) * (XT_KC / 8) + k8_in) * XT_ROWS + r] = sk_x_unit<WK>(v);
}

static void* g_xt[64];
static size_t g_xt_bytes[64];

template <int WK>
static cudaError_t xt_launch(const LinRef* lin, const void* x, int M, void* y, cudaStream_t st) {
    typedef SkGeom<WK, XT_NT, XT_KC> G;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    const int N = lin->N, K = lin->K;
    /* two row blocks per CTA where the weight ring leaves room for 64 KB of B tiles per stage (packed INT4) and the
     * slice is long enough that halving the CTAs costs less than converting every weight twice (measured: at 512 rows
     * one block per CTA is 2.5x faster on the 6144-row matrix, at 2048 rows two blocks are 1.25x faster per layer) */
    const bool two = WK == WK_INT4_PACK && M >= 4 * XT_ROWS;
    const int nblk = two ? 2 : 1;
    const int tbs = ((M + XT_ROWS * nblk - 1) / (XT_ROWS * nblk)) * nblk; /* row blocks, padded to whole CTAs */
    const int tiles = (N + SK_BM - 1) / SK_BM, ctas_y = tbs / nblk;
    /* workspace for the tiled activations: grown on demand, never shrunk (not under stream capture: prefill is not captured) */
    const size_t need = (size_t)tbs * XT_ROWS * K * 2;
    if (need > g_xt_bytes[dev]) {
        if ((e = cudaStreamSynchronize(st)) != cudaSuccess) return e;
        if (g_xt[dev]) cudaFree(g_xt[dev]);
        g_xt[dev] = nullptr; g_xt_bytes[dev] = 0;
        if ((e = cudaMalloc(&g_xt[dev], need)) != cudaSuccess) return e;
        g_xt_bytes[dev] = need;
    }
    /* split K where tiles x row blocks leave most SMs idle (short prompts, matrices of few rows) */
    int S = 0, KS = 1;
    if (g_partial_rows[dev] >= XT_ROWS && tiles * ctas_y * 2 <= 148) {
        int max_ks = K / SK_SUPER_K;
        if (max_ks > SK_MAX_SPLIT) max_ks = SK_MAX_SPLIT;
        KS = 148 / (tiles * ctas_y) < max_ks ? 148 / (tiles * ctas_y) : max_ks;
        const size_t cap = (size_t)SK_SCRATCH_FLOATS_PER_ROW * g_partial_rows[dev];
        while (KS > 1 && (size_t)tiles * KS * XT_ROWS * SK_BM * tbs > cap) KS--;
        if (KS > 1 && tiles * ctas_y <= SK_MAX_SPLIT_TILES) S = tiles; else KS = 1;
    }
    const int grid_x = tiles - S + S * KS;
    int DW = 3;
    size_t smem = 0;
    for (; DW >= 2; DW--) {
        smem = (two ? 2 * ((size_t)G::A_BYTES + 2 * (size_t)XT_ROWS * XT_KC * 2) + 128 : sk_fixed_bytes<WK, XT_NT, XT_KC>(XT_ROWS)) +
               (size_t)DW * G::SUP_BYTES;
        if (smem <= SK_SMEM_ONE) break;
    }
    if (DW < 2) return cudaErrorInvalidValue;
    int D = G::SPS * (DW - 1) + 1;
    if (D > SK_MAX_DEPTH) D = SK_MAX_DEPTH;
    static bool attr_set[64] = {false};
    if (!attr_set[dev]) {
        if ((e = cudaFuncSetAttribute(k_skinny_tc<WK, XT_NT, XT_KC, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SK_SMEM_ONE)) != cudaSuccess) return e;
        if (WK == WK_INT4_PACK &&
            (e = cudaFuncSetAttribute(k_skinny_tc<WK_INT4_PACK, XT_NT, XT_KC, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SK_SMEM_ONE)) != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    const size_t units = (size_t)tbs * XT_ROWS * (K >> 3);
    k_xt_tile<WK><<<(unsigned)((units + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)x, M, K, tbs * XT_ROWS, (uint4*)g_xt[dev]);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    if (two)
        k_skinny_tc<WK_INT4_PACK, XT_NT, XT_KC, 2><<<dim3((unsigned)grid_x, (unsigned)ctas_y), XT_NT + 32, smem, st>>>(
            lin->w, lin->scales, N, K, lin->gshift, (const __nv_bfloat16*)g_xt[dev], M, 8, D, DW, S, KS, 0, (__nv_bfloat16*)y, nullptr,
            S ? g_partial[dev] : nullptr, S ? g_arrivals[dev] : nullptr);
    else
        k_skinny_tc<WK, XT_NT, XT_KC, 1><<<dim3((unsigned)grid_x, (unsigned)ctas_y), XT_NT + 32, smem, st>>>(
            lin->w, lin->scales, N, K, lin->gshift, (const __nv_bfloat16*)g_xt[dev], M, 8, D, DW, S, KS, 0, (__nv_bfloat16*)y, nullptr,
            S ? g_partial[dev] : nullptr, S ? g_arrivals[dev] : nullptr);
    return cudaGetLastError();
}

/* y[M, N] (bf16) = x[M, K] (bf16) · W^T for any M >= 1 (prompt slices).  Same constraints on the weights as
 * skinny_gemm_tc.  Not for use under stream capture (the workspace may be allocated here). */
extern "C" cudaError_t skinny_prefill_tc(const LinRef* lin, const void* x, int M, void* y, cudaStream_t st) {
    if (!lin || !x || !y || M < 1 || lin->K % SK_SUPER_K) return cudaErrorInvalidValue;
    if (((uintptr_t)x | (uintptr_t)lin->w) & 15) return cudaErrorInvalidValue;
    if (lin->kind != WK_INT8_CH)
        if (lin->gshift < 4 || lin->gshift > 7 || ((uintptr_t)lin->scales & 15)) return cudaErrorInvalidValue;
    if (lin->kind == WK_INT4_PACK && lin->gshift < 5) return cudaErrorInvalidValue;
    switch (lin->kind) {
    case WK_INT8_CH: return xt_launch<WK_INT8_CH>(lin, x, M, y, st);
    case WK_INT8_GRP: return xt_launch<WK_INT8_GRP>(lin, x, M, y, st);
    case WK_INT4_PACK: return xt_launch<WK_INT4_PACK>(lin, x, M, y, st);
    }
    return cudaErrorInvalidValue;
}

/* status word of the launches so far on the current device (0 = no wait ever gave up); synchronises */
extern "C" cudaError_t skinny_status(int* out) { return cudaMemcpyFromSymbol(out, g_sk_status, sizeof(int)); }

}  // namespace s2p
