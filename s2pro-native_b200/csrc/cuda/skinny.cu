/* Batched decode linear on the 5th-generation tensor cores: y[M, N] = x[M, K] · Wq^T for the
 * lockstep batches the exact-order GEMV cannot serve well (M > 16 rows; the reference's own
 * kernels stop at 16 rows, src/sched/int8_gemv.cu:964-986, so there is no bit-exact contract
 * beyond that: results agree with the exact path to f32-accumulation-order tolerance).
 *
 * One CTA owns 128 weight rows (the MMA's M; the batch is its N, padded to a multiple of 16):
 *   - all 256 threads dequantise a [128 rows x 128 k] slab of packed INT4 / INT8 codes into f16
 *     in shared memory (INT4: code x f16 group scale, one rounding of a 15-bit product; INT8
 *     per-channel: the exact code, the row scale is applied to the accumulator), in the
 *     K-major, unswizzled core-matrix layout the instruction reads: 16-byte units
 *     [k / 8][row], i.e. 8 rows x 16 B core matrices, 128 B apart along rows (SBO) and
 *     one [k/8] plane apart along K (LBO);
 *   - the activations (bf16 -> f16, exact in the normal range) go beside them as [k / 8][batch row];
 *   - one thread issues eight tcgen05.mma (M 128, N = padded batch, K 16, f16 x f16 -> f32 in
 *     TMEM) per slab and commits them to an mbarrier; two slabs are in flight, so the
 *     dequantisation of slab i+1 overlaps the MMAs of slab i;
 *   - epilogue: tcgen05.ld of the accumulator (lane = weight row, column = batch row), row
 *     scale, bf16, stores coalesced over weight rows.
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
constexpr int SK_MAX_SPLIT = 8;

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

/* 16-byte asynchronous copy into shared memory; `valid` false writes zeros without reading */
__device__ __forceinline__ void sk_cp16(void* dst, const void* src, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(valid ? 16 : 0) : "memory");
}
/* 4-, 8- or 16-byte copy of group scales (bytes is uniform over the launch) */
__device__ __forceinline__ void sk_cp_small(void* dst, const void* src, int bytes, bool valid) {
    const uint32_t d = smem_u32(dst);
    if (bytes == 4) asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(valid ? 4 : 0) : "memory");
    else if (bytes == 8) asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(d), "l"(src), "r"(valid ? 8 : 0) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(valid ? 16 : 0) : "memory");
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

template <int WK, int NT> struct SkGeom {
    static constexpr int KC = NT / 4;                                     /* K extent of a slab: one or two 16-byte units of codes per thread */
    static constexpr int UPR = (WK == WK_INT4_PACK) ? KC / 32 : KC / 16;  /* 16-byte units of packed codes per row and slab */
    static constexpr int PITCH = UPR * 16;
    static constexpr int SWZ_SHIFT = UPR == 2 ? 2 : (UPR == 4 ? 1 : 0);   /* 8 / UPR consecutive rows share a swizzle value */
    static constexpr int W_BYTES = SK_BM * PITCH;
    static constexpr int SC_ROW = 16;                                     /* room per row for the copied scales */
    static constexpr int SC_BYTES = (WK == WK_INT8_CH) ? 0 : SK_BM * SC_ROW;
    static constexpr int WPU = (WK == WK_INT4_PACK) ? 32 : 16;            /* weights per 16-byte unit */
    static constexpr int NLD = UPR * SK_BM / NT;                          /* units per thread and slab: 1 (INT4) or 2 (INT8) */
    static constexpr int A_BYTES = SK_BM * KC * 2;                        /* converted stage */
    static_assert(UPR == 2 || UPR == 4 || UPR == 8, "swizzle covers 2, 4 or 8 units per row");
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

template <int WK, int NT>
__global__ void __launch_bounds__(NT, 512 / NT) k_skinny_tc(const void* __restrict__ w, const void* __restrict__ scales, int N,
                                                            int K, int gshift, const __nv_bfloat16* __restrict__ x, int M,
                                                            int lgNB, int D, __nv_bfloat16* y, const __nv_bfloat16* resid,
                                                            float* __restrict__ partial, unsigned* __restrict__ arrivals) {
    /* resid (may alias y): y = bf16(f32(resid) + f32(bf16(product))), the residual add of the decode layers */
    /* gridDim.y > 1: the K range is split over gridDim.y CTAs per row tile; each leaves its f32 partial in
     * `partial`[split][batch row][weight row] and the last one to arrive adds them in split order */
    /* D: depth of the ring of raw slabs (packed codes, scales, activations) that asynchronous copies
     * fill D - 1 slabs ahead of the conversion: what keeps enough bytes in flight to stream from HBM */
    /* Everything a thread needs per slab (source pointers, offsets inside a ring slot and a stage) is
     * worked out once; the loop only advances pointers: the conversion is bound by instruction issue. */
    typedef SkGeom<WK, NT> G;
    constexpr int KC = G::KC;
    int* status = &g_sk_status;
    extern __shared__ __align__(1024) unsigned char smem[];
    const int NB = 1 << lgNB;
    const int b_bytes = NB * KC * 2;
    const int x_units = NB * (KC / 8);
    const int slot_bytes = G::W_BYTES + G::SC_BYTES + x_units * 16;
    const int ring_bytes = D * slot_bytes;
    unsigned char* ring = smem + 2 * (G::A_BYTES + b_bytes);
    uint64_t* done = reinterpret_cast<uint64_t*>(ring + ring_bytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 2);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * SK_BM;
    const size_t row_bytes = (WK == WK_INT4_PACK) ? (size_t)(K >> 1) : (size_t)K;
    int ncols = 32;
    while (ncols < NB) ncols <<= 1;

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        mbar_init(done, 1);
        mbar_init(done + 1, 1);
        mbar_init_fence();
    }

    const int nk_all = K / KC, KS = gridDim.y, ks = blockIdx.y;
    const int it_first = (int)((long long)nk_all * ks / KS), nk = (int)((long long)nk_all * (ks + 1) / KS) - it_first;
    /* scales travel as aligned pieces of at least 4 bytes: cpy elements starting at a multiple of cpy */
    const int nsc = KC >> gshift, cpy = nsc < 2 ? 2 : nsc;

    /* ---- copy side: UPR neighbouring threads read one row's run of codes; the unit index inside a slot is
     * XOR-swizzled so that 8 consecutive rows read back without bank conflicts */
    const unsigned char* wsrc[G::NLD];
    int wdst[G::NLD];
    bool wvalid[G::NLD];
#pragma unroll
    for (int i = 0; i < G::NLD; i++) {
        const int idx = tid + NT * i, row = idx / G::UPR, c = idx % G::UPR, grow = n0 + row;
        wvalid[i] = grow < N;
        wsrc[i] = static_cast<const unsigned char*>(w);
        if (wvalid[i]) wsrc[i] += (size_t)grow * row_bytes + (size_t)it_first * (WK == WK_INT4_PACK ? KC / 2 : KC) + c * 16;
        wdst[i] = row * G::PITCH + ((c ^ ((row >> G::SWZ_SHIFT) & (G::UPR - 1))) << 4);
    }
    const bool sc_copier = WK != WK_INT8_CH && tid < SK_BM;
    const bool sc_valid = sc_copier && n0 + tid < N;
    const __half* sc_row = static_cast<const __half*>(scales);
    if (sc_valid) sc_row += (size_t)(n0 + tid) * (K >> gshift);
    /* activations: unit c = [k / 8][batch row] sits in the slot where the B tile wants it; c = tid + NT u */
    const int xn = tid & (NB - 1);
    const bool x_valid = xn < M;
    const int x_mine = tid < x_units ? (x_units + NT - 1 - tid) / NT : 0; /* units of this thread */
    const int x_step = (NT >> lgNB) * 8;                                   /* elements between them (NB <= NT) */
    const __nv_bfloat16* xsrc = x;
    if (x_valid) xsrc += (size_t)xn * K + (size_t)it_first * KC + (tid >> lgNB) * 8;
    const int xdst = G::W_BYTES + G::SC_BYTES + tid * 16;

    int w_slot = 0, issued = 0; /* byte offset of the slot the next copy fills; slabs issued so far */
    auto issue = [&]() {
        unsigned char* slot = ring + w_slot;
#pragma unroll
        for (int i = 0; i < G::NLD; i++) {
            sk_cp16(slot + wdst[i], wsrc[i], wvalid[i]);
            if (wvalid[i]) wsrc[i] += (WK == WK_INT4_PACK ? KC / 2 : KC);
        }
        if (sc_copier) {
            const int e0 = (((it_first + issued) * KC) >> gshift) & ~(cpy - 1);
            sk_cp_small(slot + G::W_BYTES + tid * G::SC_ROW, sc_row + (sc_valid ? e0 : 0), cpy * 2, sc_valid);
        }
        for (int u = 0; u < x_mine; u++) sk_cp16(slot + xdst + u * (NT * 16), xsrc + (x_valid ? u * x_step : 0), x_valid);
        if (x_valid) xsrc += KC;
        issued++;
        w_slot += slot_bytes;
        if (w_slot == ring_bytes) w_slot = 0;
    };
    /* one copy group per slab, also when it is empty, so the group count tells which slabs have landed */
    for (int j = 0; j < D - 1; j++) {
        if (j < nk) issue();
        asm volatile("cp.async.commit_group;" ::: "memory");
    }

    /* ---- conversion side: thread -> (row, unit q) of the slab; constant offsets into a slot and a stage */
    int rd_off[G::NLD], a_off[G::NLD], q_of[G::NLD], sc_off;
#pragma unroll
    for (int i = 0; i < G::NLD; i++) {
        const int idx = tid + NT * i, row = idx & (SK_BM - 1), q = idx >> 7;
        rd_off[i] = row * G::PITCH + ((q ^ ((row >> G::SWZ_SHIFT) & (G::UPR - 1))) << 4);
        a_off[i] = (q * (G::WPU / 8) * SK_BM + row) * 16;
        q_of[i] = q;
    }
    sc_off = G::W_BYTES + (tid & (SK_BM - 1)) * G::SC_ROW;

    sk_cp_wait(D - 2); /* slab 0 */
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    /* instruction descriptor: D f32, A and B f16, both K-major, N = NB, M = 128 */
    const uint32_t idesc = (1u << 4) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(SK_BM >> 4) << 24);
    const uint64_t desc_a0 = sk_smem_desc(smem_u32(smem), SK_BM * 16, 128);
    const uint64_t desc_b0 = sk_smem_desc(smem_u32(smem + 2 * G::A_BYTES), (uint32_t)NB * 16, 128);

    bool ok = true;
    int r_slot = 0;
    for (int it = 0; it < nk && ok; it++) {
        const int s = it & 1;
        /* the slot the next copy fills was read by every thread before the barrier that ended the last round */
        if (issued < nk) issue();
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (it >= 2) ok = mbar_wait_bounded(done + s, ((unsigned)(it >> 1) - 1u) & 1u, status); /* the MMAs that read this stage */
        if (!ok) break;
        const unsigned char* slot = ring + r_slot;
        unsigned char* A = smem + s * G::A_BYTES;
        unsigned char* B = smem + 2 * G::A_BYTES + s * b_bytes;
        const int kg = ((it_first + it) * KC) >> gshift; /* first scale group of the slab */
        /* weights: A[k / 8][row] (rows beyond N: zero codes, zero scale) */
#pragma unroll
        for (int i = 0; i < G::NLD; i++) {
            const uint4 pk = *reinterpret_cast<const uint4*>(slot + rd_off[i]);
            __half2 sc2 = __float2half2_rn(1.f);
            if (WK != WK_INT8_CH) {
                const int e = kg + ((q_of[i] * G::WPU) >> gshift) - (kg & ~(cpy - 1));
                sc2 = __half2half2(reinterpret_cast<const __half*>(slot + sc_off)[e]);
            }
            uint4* Au = reinterpret_cast<uint4*>(A + a_off[i]);
            if (WK == WK_INT4_PACK) {
                const uint32_t ws[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
                for (int j = 0; j < 4; j++) Au[j * SK_BM] = sk_int4_chunk(ws[j], sc2);
            } else {
                Au[0] = sk_int8_chunk<WK == WK_INT8_GRP>(pk.x, pk.y, sc2);
                Au[SK_BM] = sk_int8_chunk<WK == WK_INT8_GRP>(pk.z, pk.w, sc2);
            }
        }
        /* activations: B[k / 8][batch row]; rows beyond the batch were zero-filled (bf16 zero = f16 zero) */
        for (int u = 0; u < x_mine; u++)
            *reinterpret_cast<uint4*>(B + (tid + u * NT) * 16) = sk_x_unit<WK>(*reinterpret_cast<const uint4*>(slot + xdst + u * (NT * 16)));
        r_slot += slot_bytes;
        if (r_slot == ring_bytes) r_slot = 0;
        sk_cp_wait(D - 2);        /* this thread's share of slab it + 1; the barrier makes everyone's visible */
        fence_proxy_async_smem(); /* these generic-proxy stores are read by the tensor core (async proxy) */
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            /* the start-address field counts 16-byte units: stage s and K step kk are plain additions */
            const uint64_t da0 = desc_a0 + (uint64_t)((s * G::A_BYTES) >> 4);
            const uint64_t db0 = desc_b0 + (uint64_t)((s * b_bytes) >> 4);
#pragma unroll
            for (int kk = 0; kk < KC / 16; kk++) {
                const uint64_t da = da0 + (uint64_t)(kk * 2 * SK_BM);
                const uint64_t db = db0 + (uint64_t)(kk * 2 * NB);
                const uint32_t accumulate = (it > 0 || kk > 0) ? 1u : 0u;
                asm volatile(
                    "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                    ::"r"(tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
            }
            /* arrives on the barrier once every MMA issued so far has completed */
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(done + s)) : "memory");
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory"); /* nothing of this CTA's is in flight past here */
    /* the last commit covers every MMA before it */
    if (ok) ok = mbar_wait_bounded(done + ((nk - 1) & 1), (unsigned)((nk - 1) >> 1) & 1u, status);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) { /* warp w reads TMEM lanes 32 (w % 4) .. + 31 = weight rows; the warps of a lane quarter share the columns */
        const int grow = n0 + (warp & 3) * 32 + lane;
        float rs = 1.f;
        if (WK == WK_INT8_CH && grow < N) rs = static_cast<const float*>(scales)[grow];
        for (int col0 = (warp >> 2) * 32; col0 < NB; col0 += (NT / 128) * 32) {
            uint32_t v[32];
            const uint32_t taddr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)col0;
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
            if (grow < N) {
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const int m = col0 + j;
                    if (m < M) {
                        if (KS == 1) {
                            __nv_bfloat16 o = f2bf(__fmul_rn(__uint_as_float(v[j]), rs));
                            if (resid) o = f2bf(__fadd_rn(bf2f(resid[(size_t)m * N + grow]), bf2f(o)));
                            y[(size_t)m * N + grow] = o;
                        }
                        else partial[((size_t)ks * M + m) * N + grow] = __uint_as_float(v[j]);
                    }
                }
            }
        }
    }
    if (KS > 1) {
        __shared__ int s_last;
        __threadfence();
        __syncthreads();
        if (tid == 0) s_last = ok && (atomicAdd(arrivals + blockIdx.x, 1u) == (unsigned)(KS - 1));
        __syncthreads();
        if (s_last) {
            __threadfence();
            /* four outputs per thread and round, the loads of all splits in flight together; the adds keep split order */
            for (int e0 = tid; e0 < SK_BM * M; e0 += NT * 4) {
                float v[4][SK_MAX_SPLIT];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int e = e0 + u * NT, m = e >> 7, grow = n0 + (e & (SK_BM - 1));
                    const bool live = e < SK_BM * M && grow < N;
#pragma unroll
                    for (int q = 0; q < SK_MAX_SPLIT; q++)
                        v[u][q] = (live && q < KS) ? __ldcg(partial + ((size_t)q * M + m) * N + grow) : 0.f;
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int e = e0 + u * NT, m = e >> 7, grow = n0 + (e & (SK_BM - 1));
                    if (e >= SK_BM * M || grow >= N) continue;
                    float acc = 0.f;
#pragma unroll
                    for (int q = 0; q < SK_MAX_SPLIT; q++)
                        if (q < KS) acc += v[u][q];
                    if (WK == WK_INT8_CH) acc = __fmul_rn(acc, static_cast<const float*>(scales)[grow]);
                    __nv_bfloat16 o = f2bf(acc);
                    if (resid) o = f2bf(__fadd_rn(bf2f(resid[(size_t)m * N + grow]), bf2f(o)));
                    y[(size_t)m * N + grow] = o;
                }
            }
            if (tid == 0) arrivals[blockIdx.x] = 0u;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(ncols) : "memory");
}

constexpr size_t SK_SMEM_ONE = 226 * 1024; /* one CTA per SM */
constexpr size_t SK_SMEM_TWO = 111 * 1024; /* two, each with its static kilobyte and the system's */
constexpr int SK_MAX_DEPTH = 8;

/* scratch for split-K launches: partials [SK_MAX_SPLIT][rows][SK_SPLIT_MAX_N] f32 and one arrival counter per row tile */
constexpr int SK_SPLIT_MAX_N = 6144;
static float* g_partial[64];
static unsigned* g_arrivals[64];
static int g_partial_rows[64];

/* once per device, outside stream capture: room for split-K launches with up to `max_rows` batch rows */
extern "C" cudaError_t skinny_setup(int max_rows) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || max_rows < 1) return cudaErrorInvalidValue;
    if (g_partial_rows[dev] >= max_rows) return cudaSuccess;
    if (g_partial[dev]) cudaFree(g_partial[dev]);
    g_partial[dev] = nullptr;
    g_partial_rows[dev] = 0;
    if ((e = cudaMalloc((void**)&g_partial[dev], (size_t)SK_MAX_SPLIT * max_rows * SK_SPLIT_MAX_N * sizeof(float))) != cudaSuccess) return e;
    if (!g_arrivals[dev]) {
        if ((e = cudaMalloc((void**)&g_arrivals[dev], 256 * sizeof(unsigned))) != cudaSuccess) return e;
        if ((e = cudaMemset(g_arrivals[dev], 0, 256 * sizeof(unsigned))) != cudaSuccess) return e;
    }
    g_partial_rows[dev] = max_rows;
    return cudaSuccess;
}

/* shared memory of a launch: two converted stages, D raw slabs, barriers */
template <int WK, int NT> static size_t sk_fixed_bytes(int NB) {
    return 2 * ((size_t)SkGeom<WK, NT>::A_BYTES + (size_t)NB * SkGeom<WK, NT>::KC * 2) + 64;
}
template <int WK, int NT> static size_t sk_slot_bytes(int NB) {
    return (size_t)SkGeom<WK, NT>::W_BYTES + SkGeom<WK, NT>::SC_BYTES + (size_t)NB * (SkGeom<WK, NT>::KC / 8) * 16;
}

template <int WK, int NT>
static cudaError_t sk_launch_nt(const LinRef* lin, const void* x, int M, int lgNB, int tiles, int split, void* y, const void* resid,
                                float* partial, unsigned* arrivals, cudaStream_t st) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(k_skinny_tc<WK, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SK_SMEM_ONE);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    /* ring depth: what the shared memory of the SM allows beside the stages (shared by two CTAs of 256 threads) */
    const int NB = 1 << lgNB;
    const size_t fixed = sk_fixed_bytes<WK, NT>(NB), slot = sk_slot_bytes<WK, NT>(NB);
    int D = 0;
    if (NT == 256 && fixed < SK_SMEM_TWO) D = (int)((SK_SMEM_TWO - fixed) / slot);
    if (D < 4) D = fixed < SK_SMEM_ONE ? (int)((SK_SMEM_ONE - fixed) / slot) : 0;
    if (D > SK_MAX_DEPTH) D = SK_MAX_DEPTH;
    if (D < 2) return cudaErrorInvalidValue;
    k_skinny_tc<WK, NT><<<dim3((unsigned)tiles, (unsigned)split), NT, fixed + (size_t)D * slot, st>>>(
        lin->w, lin->scales, lin->N, lin->K, lin->gshift, (const __nv_bfloat16*)x, M, lgNB, D, (__nv_bfloat16*)y,
        (const __nv_bfloat16*)resid, partial, arrivals);
    return cudaGetLastError();
}

template <int WK>
static cudaError_t sk_launch(const LinRef* lin, const void* x, int M, void* y, const void* resid, cudaStream_t st) {
    int lgNB = 4; /* the batch is padded to a power of two: the MMA's N */
    while ((1 << lgNB) < M) lgNB++;
    const int tiles = (lin->N + SK_BM - 1) / SK_BM;
    int dev = 0, split = 1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    /* few row tiles and a long K: split K over several CTAs so the whole GPU streams the matrix */
    if (dev >= 0 && dev < 64 && g_partial_rows[dev] >= M && lin->N <= SK_SPLIT_MAX_N && tiles <= 74 && tiles <= 256) {
        split = 148 / tiles;
        if (split > SK_MAX_SPLIT) split = SK_MAX_SPLIT;
        if (split > lin->K / 128) split = lin->K / 128;
        if (split < 1) split = 1;
    }
    float* partial = split > 1 ? g_partial[dev] : nullptr;
    unsigned* arrivals = split > 1 ? g_arrivals[dev] : nullptr;
    /* at most one CTA per SM: 512 threads each (16 warps hide the conversion's latencies); more CTAs than SMs:
     * 256 threads, two CTAs per SM */
    const size_t fixed512 = sk_fixed_bytes<WK, 512>(1 << lgNB), slot512 = sk_slot_bytes<WK, 512>(1 << lgNB);
    if (tiles * split <= 148 && lin->K % 128 == 0 && fixed512 + 4 * slot512 <= SK_SMEM_ONE) /* and a ring of 4 slabs or more */
        return sk_launch_nt<WK, 512>(lin, x, M, lgNB, tiles, split, y, resid, partial, arrivals, st);
    return sk_launch_nt<WK, 256>(lin, x, M, lgNB, tiles, split, y, resid, partial, arrivals, st);
}

/* y[M, N] (bf16) = x[M, K] (bf16) · W^T for 1 <= M <= 256, plus `resid` [M, N] when given (it may be y
 * itself).  K must be a multiple of 64, the group size of grouped kinds at least 32 (INT4) / 16 (INT8 codes). */
extern "C" cudaError_t skinny_gemm_tc(const LinRef* lin, const void* x, int M, void* y, const void* resid, cudaStream_t st) {
    if (!lin || !x || !y || M < 1 || M > 256 || lin->K % 64) return cudaErrorInvalidValue;
    if (((uintptr_t)x | (uintptr_t)lin->w) & 15) return cudaErrorInvalidValue;
    if (lin->kind != WK_INT8_CH) { /* the scales of a slab are copied as an aligned piece of 4 to 16 bytes */
        if (lin->gshift < 3 || ((uintptr_t)lin->scales & 15)) return cudaErrorInvalidValue;
        const int nsc = 128 >> lin->gshift, cpy = nsc < 2 ? 2 : nsc; /* the wider of the two slab sizes */
        if ((lin->K >> lin->gshift) % cpy) return cudaErrorInvalidValue;
    }
    switch (lin->kind) {
    case WK_INT8_CH: return sk_launch<WK_INT8_CH>(lin, x, M, y, resid, st);
    case WK_INT8_GRP: return lin->gshift >= 4 ? sk_launch<WK_INT8_GRP>(lin, x, M, y, resid, st) : cudaErrorInvalidValue;
    case WK_INT4_PACK: return lin->gshift >= 5 ? sk_launch<WK_INT4_PACK>(lin, x, M, y, resid, st) : cudaErrorInvalidValue;
    }
    return cudaErrorInvalidValue;
}

/* status word of the launches so far on the current device (0 = no wait ever gave up); synchronises */
extern "C" cudaError_t skinny_status(int* out) { return cudaMemcpyFromSymbol(out, g_sk_status, sizeof(int)); }

}  // namespace s2p
