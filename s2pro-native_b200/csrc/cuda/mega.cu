/* Persistent batch-1 decode tick: one cooperative kernel per frame.
 *
 * The frame (slow-AR layers, head + sampler, ten fast-AR passes; the stage
 * sequence of src/slowar/slowar.c:162-258, :481-560 and
 * src/fastar/fastar.cu:726-788) is about 400 dependent stages, each a few
 * microseconds of work for the whole GPU.  Launched separately, every stage
 * pays a launch, a cold start of its weight stream and a tail; here the CTAs
 * (one per SM, 512 threads) stay resident and walk a stage list, meeting at a
 * grid barrier between stages.
 *
 * Weights reach the SM through a ring of shared-memory slots filled by 1-D TMA
 * bulk copies (cp.async.bulk + mbarrier transaction counts).  Each CTA owns a
 * fixed row block of every matrix, cut into chunks of whole rows that fit a
 * slot; one thread issues the copies from a per-CTA command list the host built
 * at load time, three chunks ahead of the one being consumed.  The list runs
 * across stage boundaries, so while the CTA waits at a grid barrier (or does
 * attention) the ring already holds the next GEMV stage's first chunks: weight
 * addresses never depend on activations.
 * The bytes in flight per SM are bounded by the ring (4 x 32 KB), not by
 * registers, which is what keeps HBM busy at 16 warps per SM.
 *
 * Arithmetic is that of the per-stage kernels (gemv.cuh, attn_body.cuh,
 * sampler_body.cuh): same lane ownership, same fma chains, same trees, so the
 * frame is bit-identical to the unfused sequence.
 */
#include "attn_body.cuh"
#include "gemv.cuh"
#include "pipe.cuh"
#include "sampler_body.cuh"
#include "s2p_b200_abi.h"

namespace s2p {

constexpr int MEGA_WORKERS = 512;
constexpr int MEGA_THREADS = MEGA_WORKERS;
constexpr int MEGA_ISSUER = MEGA_WORKERS - 32;  /* lane 0 of the last warp issues the copies */
constexpr int MEGA_SLOTS = MEGA_RING_SLOTS;
constexpr int MEGA_PARTS = MEGA_PARTIAL_BUFFERS;
constexpr int MEGA_RED_BYTES = 3072;            /* 260 floats tree | 256 residuals | 252 row scales */
constexpr int MEGA_TAIL_BYTES = 1024;           /* mbarriers, the staged copy command, two stage descriptors */
static_assert(sizeof(MegaStage) % 16 == 0 && 2 * sizeof(MegaStage) + 256 <= MEGA_TAIL_BYTES, "descriptor staging");
constexpr int MEGA_SMEM_MAX = 225 * 1024; /* 227 KB per CTA less the kernel's static shared memory */
constexpr int MEGA_PART_BYTES_DEFAULT = 19456;  /* 152 (row, tile) units: 30 rows of 5 tiles, 19 of 8, 8 of 19 */
/* shared memory: ring slots | work area (x | partial buffers | red) | tail.  Attention and the
 * sampler overlay the work area. */
constexpr int MEGA_MIN_WORK = 19456 + MEGA_PARTS * MEGA_PART_BYTES_DEFAULT;
static_assert(sizeof(AttnSmem<false>) <= MEGA_MIN_WORK && sizeof(AttnSmem<true>) <= MEGA_MIN_WORK, "attention scratch must fit the work area");
static_assert(sizeof(SamplerSmem<MEGA_WORKERS>) <= MEGA_MIN_WORK, "sampler scratch must fit the work area");
static_assert(sizeof(MegaCopyCmd) == 64, "one copy command per 64-byte line");

__device__ __forceinline__ bool cta_sync_and(bool p) { return __syncthreads_and(p ? 1 : 0) != 0; }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

/* order-preserving arg-max key: larger value first, then lower index
 * (src/slowar/kernels.cu:1326-1357); -0 counts as +0 */
__device__ __forceinline__ unsigned long long argmax_key(__nv_bfloat16 yb, int n) {
    uint32_t uu = __float_as_uint(bf2f(yb));
    if (uu == 0x80000000u) uu = 0u;
    uu = (uu & 0x80000000u) ? ~uu : (uu | 0x80000000u);
    return ((unsigned long long)uu << 32) | (0xFFFFFFFFu - (uint32_t)n);
}

/* The tensor-parallel group as the kernel uses it: the OTHER ranks' arenas as byte offsets
 * from the own one (a pointer into the own arena plus delta[i] is the same cell in a peer's).
 * Kept in shared memory: indexing the kernel parameter array with a run-time index would cost
 * a local-memory copy of the parameters. */
struct TpPeers {
    long long delta[7];
    int n; /* tp_world - 1; 0 on a single GPU */
};
__shared__ TpPeers g_tp;

/* store a stage output into the own exchange arena and, tensor-parallel, into every peer's */
template <class T>
__device__ __forceinline__ void store_all(T* p, T v) {
    *p = v;
    for (int i = 0; i < g_tp.n; i++) *reinterpret_cast<T*>(reinterpret_cast<unsigned char*>(p) + g_tp.delta[i]) = v;
}

struct Ring {
    unsigned char* slots;
    uint64_t* full;    /* [MEGA_SLOTS] a chunk has landed */
    uint64_t* pfull;   /* [MEGA_PARTS] all warps have written their partials of a chunk */
    uint64_t* pdone;   /* [MEGA_PARTS] all warps have folded their rows of it (its slot and buffer are free) */
    int* status;
    int cta, n_cta;
    int slot_bytes, part_floats, x_bytes;
    unsigned seq_base; /* stage instances of earlier ticks */
    unsigned tag;      /* the tag this stage writes into its flagged outputs */
    unsigned consumed; /* chunks consumed so far (every thread keeps its own copy) */
    /* issuer thread only: this CTA's command list (built by the host with mega_stage_geom,
     * the function the consumers use), how many were issued, and the next one, loaded early */
    const MegaCopyCmd* cmds;
    unsigned n_cmds, issued;
    MegaCopyCmd* next; /* shared memory, filled by an asynchronous copy */
};

__device__ __forceinline__ void ring_load_next(Ring& r) {
    if (r.issued < r.n_cmds) {
        const char* src = reinterpret_cast<const char*>(r.cmds + r.issued);
        const uint32_t dst = smem_u32(r.next);
#pragma unroll
        for (int i = 0; i < 4; i++)
            asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst + 16u * i), "l"(src + 16 * i) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
}

/* Issuer thread: start the copies of every chunk with index < limit that has not been
 * started.  The caller guarantees their slots are free: chunk q reuses the slot of chunk
 * q - MEGA_SLOTS, so limit = q + 1 + MEGA_SLOTS once chunk q is known to be completely
 * consumed (and MEGA_SLOTS at kernel start). */
__device__ __forceinline__ void ring_issue_upto(Ring& r, unsigned limit) {
    while (r.issued < limit && r.issued < r.n_cmds) {
        const unsigned slot = r.issued % MEGA_SLOTS;
        unsigned char* dst = r.slots + (size_t)slot * r.slot_bytes;
        asm volatile("cp.async.wait_all;" ::: "memory");
        const MegaCopyCmd c = *r.next;
        fence_proxy_async_smem(); /* the slot's previous chunk was read through the generic proxy */
        mbar_expect_tx(r.full + slot, c.bytes[0] + c.bytes[1] + c.bytes[2] + c.bytes[3]);
#pragma unroll
        for (int k = 0; k < 4; k++)
            if (c.bytes[k])
                tma_load_1d(dst + c.dst_off[k], reinterpret_cast<const void*>(c.src[k]), c.bytes[k], r.full + slot);
        r.issued++;
        ring_load_next(r);
    }
}

/* One GEMV stage of this CTA, chunk by chunk out of the ring.  Returns false
 * (uniformly over the working warps) if a bounded wait gave up. */
template <int WK, int TT> /* TT: K / 512 known at compile time (loops unroll), or 0 */
__device__ bool gemv_chunks(const MegaStage& s, Ring& r, unsigned char* work, unsigned long long* trace) {
    typedef typename LaneTile<WK>::type tile_t;
    const MegaGeom ge = mega_stage_geom(s.lin.N, s.epi == EPI_SWIGLU, s.rows_per_chunk, r.cta, r.n_cta);
    if (ge.cnt <= 0) { /* uniform over the CTA; leave as a GEMV stage always does: copies landed, warps together */
        asm volatile("cp.async.wait_all;" ::: "memory");
        S2P_CTA_SYNC();
        return true;
    }
    const int K = s.lin.K, T = TT ? TT : (K >> 9), gshift = s.lin.gshift;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int SW = (s.epi == EPI_SWIGLU) ? 2 : 1;
    const int F = s.lin.N >> 1;
    const unsigned rb = (WK == WK_INT4_PACK) ? (unsigned)(K >> 1) : (unsigned)K;
    const unsigned sb = (WK == WK_INT8_CH) ? 0u : (unsigned)(K >> gshift) * 2u;

    bool ok = true;
    unsigned char* xs = work;
    float* part0 = reinterpret_cast<float*>(work + r.x_bytes);
    float* red = part0 + MEGA_PARTS * r.part_floats;
    float* resid_s = red + 260;  /* residual values of this CTA's rows */
    float* rscale_s = red + 516; /* per-channel row scales of this CTA's rows (gate rows, then up rows) */
    {
        /* what the epilogue needs from global memory, fetched while the activation is staged */
        if (s.epi == EPI_RESID && threadIdx.x < ge.cnt) {
            const __nv_bfloat16* resid = s.resid.base;
            if (s.resid.index) resid += (size_t)__ldcg(s.resid.index) * s.lin.N;
            else if (s.resid.key) resid += (size_t)key_index(__ldcg(s.resid.key)) * s.lin.N;
            /* a flagged residual needs no wait: this CTA has already read the whole vector as an input */
            resid_s[threadIdx.x] = (s.io_flags & MEGA_RESID_LL)
                                       ? flag_payload(__ldcg(reinterpret_cast<const uint32_t*>(resid) + ge.row0 + threadIdx.x))
                                       : ldcg_bf16(resid + ge.row0 + threadIdx.x);
        }
        if (WK == WK_INT8_CH && threadIdx.x < ge.cnt * SW) {
            const int l = threadIdx.x;
            const int grow = l < ge.cnt ? ge.row0 + l : F + ge.row0 + (l - ge.cnt);
            rscale_s[l] = static_cast<const float*>(s.lin.scales)[grow];
        }
        GemvStage g = {};
        g.K = K; g.x = s.x.base; g.x_index = s.x.index; g.x_key = s.x.key;
        g.norm_w = s.norm_w; g.eps = S2P_NORM_EPS; g.normed_out = s.normed_out;
        /* the input arrives as flagged words from the CTAs (of all ranks) of stage x_from - wait
         * for each word's tag instead of a grid barrier - or is a plain bf16 row that an earlier
         * grid barrier has published (x_from < 0) */
        const bool ll = s.x_from >= 0;
        const uint4* xsrc;
        {
            const __nv_bfloat16* x = s.x.base;
            if (s.x.index) x += (size_t)__ldcg(s.x.index) * K;
            else if (s.x.key) x += (size_t)key_index(__ldcg(s.x.key)) * K;
            xsrc = reinterpret_cast<const uint4*>(x);
        }
        const unsigned tag = (r.seq_base + (unsigned)s.x_from + 1u) & 0xFFFFu;
        int* status = r.status;
        auto load = [xsrc, ll, tag, status, &ok](int v) -> uint4 {
            if (!ll) return __ldcg(xsrc + v);
            uint4 a, b;
            if (!flag_wait4(xsrc + 2 * v, tag, status, a) || !flag_wait4(xsrc + 2 * v + 1, tag, status, b)) {
                ok = false;
                return make_uint4(0, 0, 0, 0);
            }
            return make_uint4((a.x & 0xFFFFu) | (a.y << 16), (a.z & 0xFFFFu) | (a.w << 16), (b.x & 0xFFFFu) | (b.y << 16),
                              (b.z & 0xFFFFu) | (b.w << 16));
        };
        if (s.pro == PRO_NORM) stage_activation_from<WK, PRO_NORM>(g, load, xs, red, MEGA_WORKERS);
        else stage_activation_from<WK, PRO_VEC>(g, load, xs, red, MEGA_WORKERS);
    }
    if (!cta_sync_and(ok)) return false;
    if (trace && threadIdx.x == 0) trace[1] = clock64();
    unsigned long long best = 0ull;
    const unsigned q0 = r.consumed;
    long long tacc[6] = {0, 0, 0, 0, 0, 0}; /* trace: cycles of thread 0 in stream wait, stream, fold wait, fold, fold chain, fold tree */
    const int pstride = T * 32;

    /* Every warp streams its share of each chunk's (row, tile) units into a partial buffer
     * and, one chunk later, folds one row (or one gate/up pair) of it.  Three buffers and
     * mbarriers instead of CTA barriers let the warps drift apart by a chunk; odd warps
     * fold before they stream and even warps after, so that at any time some warps run
     * the issue-bound unit loop while others sit in the latency-bound fold. */
    auto stream_chunk = [&](int j) -> bool {
        const unsigned q = q0 + (unsigned)j, slot = q % MEGA_SLOTS, b = q % MEGA_PARTS;
        const int cnt = min(ge.rc, ge.cnt - j * ge.rc);
        const int local_rows = cnt * SW;
        const unsigned char* wsl = r.slots + (size_t)slot * r.slot_bytes;
        float* part = part0 + b * r.part_floats;
        const long long c0 = trace ? clock64() : 0;
        if (!mbar_wait_bounded(r.full + slot, (q / MEGA_SLOTS) & 1u, r.status)) return false;
        /* the buffer's previous chunk (q - 3) must be folded by everyone; that also frees its slot */
        if (q >= MEGA_PARTS) {
            if (!mbar_wait_bounded(r.pdone + b, ((q / MEGA_PARTS) - 1u) & 1u, r.status)) return false;
            if (threadIdx.x == MEGA_ISSUER) ring_issue_upto(r, q - MEGA_PARTS + 1 + MEGA_SLOTS);
        }
        const long long c1 = trace ? clock64() : 0;
        /* tile-major units; this warp's contiguous range, walked one tile segment at a time:
         * the activations of the tile stay in registers while up to four rows, whose chains
         * are independent, run side by side */
        const int U = local_rows * T;
        int u = (int)((long long)U * warp / GEMV_WARPS);
        const int u_end = (int)((long long)U * (warp + 1) / GEMV_WARPS);
#pragma unroll 1
        while (u < u_end) {
            const int tile = u / local_rows, lr0 = u - tile * local_rows;
            const int n = min(local_rows - lr0, u_end - u);
            LaneX<WK> lx;
            lx.load(xs, tile, lane);
            const unsigned char* wp = wsl + (size_t)lr0 * rb + (size_t)(tile * 32 + lane) * sizeof(tile_t);
            float* pp = part + ((size_t)lr0 * T + tile) * 32 + lane;
            int rr = 0;
#pragma unroll 1
            for (; rr + 4 <= n; rr += 4) {
                const tile_t t0 = *reinterpret_cast<const tile_t*>(wp);
                const tile_t t1 = *reinterpret_cast<const tile_t*>(wp + rb);
                const tile_t t2 = *reinterpret_cast<const tile_t*>(wp + 2 * rb);
                const tile_t t3 = *reinterpret_cast<const tile_t*>(wp + 3 * rb);
                pp[0] = lx.unit(t0);
                pp[pstride] = lx.unit(t1);
                pp[2 * pstride] = lx.unit(t2);
                pp[3 * pstride] = lx.unit(t3);
                wp += 4 * rb;
                pp += 4 * pstride;
            }
            if (n - rr >= 2) {
                const tile_t t0 = *reinterpret_cast<const tile_t*>(wp);
                const tile_t t1 = *reinterpret_cast<const tile_t*>(wp + rb);
                pp[0] = lx.unit(t0);
                pp[pstride] = lx.unit(t1);
                wp += 2 * rb;
                pp += 2 * pstride;
                rr += 2;
            }
            if (rr < n) pp[0] = lx.unit(*reinterpret_cast<const tile_t*>(wp));
            u += n;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(r.pfull + b); /* release: the partials are visible to whoever waits */
        if (trace && threadIdx.x == 0) {
            const long long c2 = clock64();
            tacc[0] += c1 - c0; tacc[1] += c2 - c1;
        }
        return true;
    };

    /* output n of the stage: a bf16 cell, or a flagged word consumers wait on */
    const bool y_ll = (s.io_flags & MEGA_Y_LL) != 0;
    const unsigned my_tag = r.tag;
    auto put_y = [&](int n, __nv_bfloat16 v) {
        if (y_ll) store_all(reinterpret_cast<uint32_t*>(s.y) + n, flag_word(v, my_tag));
        else store_all(s.y + n, v);
    };

    /* fold the tiles of row `warp` (rows `warp` and `warp + cnt` of a SwiGLU pair, chains
     * interleaved) in ascending order, merge lanes, run the epilogue */
    auto fold_chunk = [&](int j) -> bool {
        const unsigned q = q0 + (unsigned)j, slot = q % MEGA_SLOTS, b = q % MEGA_PARTS;
        const int cnt = min(ge.rc, ge.cnt - j * ge.rc);
        const int l0 = j * ge.rc, r0 = ge.row0 + l0;
        const int local_rows = cnt * SW;
        const unsigned char* ssl = r.slots + (size_t)slot * r.slot_bytes + (size_t)local_rows * rb;
        const float* part = part0 + b * r.part_floats;
        const long long c0 = trace ? clock64() : 0;
        if (!mbar_wait_bounded(r.pfull + b, (q / MEGA_PARTS) & 1u, r.status)) return false;
        const long long c1 = trace ? clock64() : 0;
        if (warp < cnt) {
            /* second chain: the up row of the pair, or (plain rows) row warp + 16 of the chunk */
            const bool two = (SW == 2);
            const bool second = !two && warp + GEMV_WARPS < cnt;
            const int la = warp, lb = two ? warp + cnt : (second ? warp + GEMV_WARPS : warp);
            float accA = 0.f, accB = 0.f;
            const float* pa = part + (size_t)la * pstride + lane;
            const float* pb = part + (size_t)lb * pstride + lane;
            if (WK == WK_INT8_CH) {
#pragma unroll
                for (int i = 0; i < T; i++) { accA += pa[i * 32]; accB += pb[i * 32]; }
            } else {
                const __half* sa = reinterpret_cast<const __half*>(ssl + (size_t)la * sb);
                const __half* sbp = reinterpret_cast<const __half*>(ssl + (size_t)lb * sb);
                const int sl = (lane * 16) >> gshift, sstep = 512 >> gshift;
#pragma unroll
                for (int i = 0; i < T; i++) {
                    accA = __fmaf_rn(pa[i * 32], __half2float(sa[sl + i * sstep]), accA);
                    accB = __fmaf_rn(pb[i * 32], __half2float(sbp[sl + i * sstep]), accB);
                }
            }
            const long long f1 = trace ? clock64() : 0;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                accA += __shfl_xor_sync(S2P_FULL_MASK, accA, off);
                accB += __shfl_xor_sync(S2P_FULL_MASK, accB, off);
            }
            const long long f2 = trace ? clock64() : 0;
            if (trace && threadIdx.x == 0) { tacc[4] += f1 - c1; tacc[5] += f2 - f1; }
            if (WK == WK_INT8_CH) {
                accA = __fmul_rn(accA, rscale_s[l0 + la]);
                accB = __fmul_rn(accB, rscale_s[two ? ge.cnt + l0 + la : l0 + lb]);
            }
            if (lane == 0) {
                const int n = r0 + la;
                if (two) {
                    const float gate = bf16_round(accA), up = bf16_round(accB);
                    const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-gate)));
                    const float sil = bf16_round(__fmul_rn(gate, sig));
                    put_y(n, f2bf(__fmul_rn(sil, up)));
                } else {
                    const __nv_bfloat16 yb = f2bf(accA);
                    put_y(n, s.epi == EPI_RESID ? f2bf(__fadd_rn(resid_s[l0 + la], bf2f(yb))) : yb);
                    if (s.epi == EPI_ARGMAX) best = max(best, argmax_key(yb, n));
                    if (second) {
                        const int n2 = n + GEMV_WARPS;
                        const __nv_bfloat16 y2 = f2bf(accB);
                        put_y(n2, s.epi == EPI_RESID ? f2bf(__fadd_rn(resid_s[l0 + lb], bf2f(y2))) : y2);
                        if (s.epi == EPI_ARGMAX) best = max(best, argmax_key(y2, n2));
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(r.pdone + b); /* this warp is done with the chunk's scales and partials */
        if (trace && threadIdx.x == 0) {
            const long long c2 = clock64();
            tacc[2] += c1 - c0; tacc[3] += c2 - c1;
        }
        return true;
    };

    /* Odd warps alternate strictly (stream 0, fold 0, stream 1, fold 1, ...); even warps run one
     * chunk ahead with the streaming (stream 0, stream 1, fold 0, stream 2, fold 1, ..., fold n-1).
     * One loop over 2 n actions so that each body exists once in the kernel's code. */
    const bool fold_first = (warp & 1) != 0;
    const int n = ge.n_chunks;
#pragma unroll 1
    for (int t = 0; t < 2 * n && ok; t++) {
        bool do_stream;
        int idx;
        if (fold_first) { do_stream = !(t & 1); idx = t >> 1; }
        else if (t == 0) { do_stream = true; idx = 0; }
        else if (t & 1) { idx = (t + 1) >> 1; do_stream = idx < n; if (!do_stream) idx = n - 1; }
        else { do_stream = false; idx = (t >> 1) - 1; }
        ok = do_stream ? stream_chunk(idx) : fold_chunk(idx);
    }
    if (trace && threadIdx.x == 0) {
#pragma unroll
        for (int i = 0; i < 6; i++) trace[4 + i] = (unsigned long long)tacc[i]; /* plain stores: no round trip on the traced path */
    }
    if (s.epi == EPI_ARGMAX && lane == 0 && best) {
        atomicMax(s.key, best);
        for (int i = 0; i < g_tp.n; i++)
            atomicMax_system(reinterpret_cast<unsigned long long*>(reinterpret_cast<unsigned char*>(s.key) + g_tp.delta[i]), best);
    }
    r.consumed = q0 + (unsigned)ge.n_chunks;
    /* a warp that gave up skipped its remaining chunks: everyone leaves with the same verdict.  The
     * barrier also publishes the next stage's descriptor (staged by asynchronous copies). */
    asm volatile("cp.async.wait_all;" ::: "memory");
    if (!cta_sync_and(ok)) return false;
    /* every chunk so far is folded by every warp: all their slots are free */
    if (threadIdx.x == MEGA_ISSUER) ring_issue_upto(r, r.consumed + MEGA_SLOTS);
    return true;
}

template <int WK>
__device__ __forceinline__ bool gemv_dispatch_t(const MegaStage& s, Ring& r, unsigned char* work, unsigned long long* tr) {
    /* one body per weight kind (tile count at run time): the kernel's code has to stay within
     * reach of the instruction caches, every stage switches between these bodies */
    return gemv_chunks<WK, 0>(s, r, work, tr);
}
__device__ bool gemv_dispatch(const MegaStage& s, Ring& r, unsigned char* work, unsigned long long* tr) {
    switch (s.lin.kind) {
    case WK_INT8_CH: return gemv_dispatch_t<WK_INT8_CH>(s, r, work, tr);
    case WK_INT8_GRP: return gemv_dispatch_t<WK_INT8_GRP>(s, r, work, tr);
    default: return gemv_dispatch_t<WK_INT4_PACK>(s, r, work, tr);
    }
}

/* ---- fast-AR attention stage: head RoPE, cache append and single-tile causal
 * attention for one kv head (CTA = kv head, 512 threads = 4 q heads x 128).
 * Operation order of the unfused pair (q/k RoPE and append: src/slowar/
 * kernels.cu:114-139, 172-195; attention over at most 11 cached positions:
 * :234-309 with a single tile): scores as one 128-term fma chain per position
 * against the query scaled by rsqrtf((float)head_dim); tile max; p = expf(s - m);
 * the exp-sum tree over 128 slots reduces to the 16/8/4/2/1 tree of the first 32
 * (the other slots hold exact zeros); l = fma(0, 0, sum); acc = fma(p_j, v_j, acc)
 * from acc = 0 * 0; out = bf16(acc / l). */
struct FastAttnSmem {
    float sq[4][128];
    float kt[S2P_FAST_SEQ][128];
    float vt[S2P_FAST_SEQ][128];
    float sp[4][32];
};

__device__ void fast_attn_cta(const MegaStage& s, int kvh, float rope_base, int head_dim, unsigned in_tag, unsigned out_tag,
                              int* status, FastAttnSmem& sm) {
    auto qkv_at = [&](size_t idx) -> float { /* flagged words from the projection stage */
        uint32_t w;
        if (!flag_wait1(reinterpret_cast<const uint32_t*>(s.qkv) + idx, in_tag, status, w)) return 0.f;
        return flag_payload(w);
    };
    const int tid = threadIdx.x, g = tid >> 7, t = tid & 127;
    const int QH = S2P_SLOW_Q_HEADS, KVH = S2P_SLOW_KV_HEADS;
    const int pos = s.pos, len = pos + 1;
    __nv_bfloat16* kc = reinterpret_cast<__nv_bfloat16*>(kv_payload(s.kv, 0) + s.kv.k_off) + (size_t)kvh * S2P_FAST_SEQ * 128;
    __nv_bfloat16* vc = reinterpret_cast<__nv_bfloat16*>(kv_payload(s.kv, 0) + s.kv.v_off) + (size_t)kvh * S2P_FAST_SEQ * 128;
    float c, sn;
    rope_cs(t >> 1, pos, rope_base, c, sn);
    {   /* query of head kvh*4+g: RoPE, bf16, scale */
        float v = qkv_at((size_t)(kvh * 4 + g) * 128 + t);
        const float other = __shfl_xor_sync(S2P_FULL_MASK, v, 1);
        v = rope_elem(t, v, other, c, sn);
        sm.sq[g][t] = __fmul_rn(v, rsqrtf((float)head_dim));
    }
    if (g < 2) { /* g 0: new key (RoPE), g 1: new value; both appended at `pos` */
        float v = qkv_at((size_t)(QH + (g == 1 ? KVH : 0) + kvh) * 128 + t);
        if (g == 0) {
            const float other = __shfl_xor_sync(S2P_FULL_MASK, v, 1);
            v = rope_elem(t, v, other, c, sn);
        }
        const __nv_bfloat16 vb = f2bf(v);
        (g == 0 ? kc : vc)[(size_t)pos * 128 + t] = vb;
        (g == 0 ? sm.kt : sm.vt)[pos][t] = bf2f(vb);
    }
    /* earlier positions of this frame, written by this CTA in earlier passes */
    for (int i = tid; i < pos * 128; i += MEGA_WORKERS) {
        sm.kt[0][i] = ldcg_bf(kc + i);
        sm.vt[0][i] = ldcg_bf(vc + i);
    }
    __syncthreads();
    if (t < 32) { /* first warp of each head: one position per lane */
        float d = -INFINITY;
        if (t < len) {
            d = 0.f;
#pragma unroll 8
            for (int e = 0; e < 128; e++) d = __fmaf_rn(sm.sq[g][e], sm.kt[t][e], d);
        }
        const float m = warp_tree_max(d);
        const float p = (t < len) ? expf(d - m) : 0.f;
        sm.sp[g][t] = p;
        const float sum = warp_tree_sum(p);
        if (t == 0) sm.sp[g][31] = __fmaf_rn(0.f, 0.f, sum); /* len <= 11: slot 31 is free */
    }
    __syncthreads();
    {
        float acc = __fmul_rn(0.f, 0.f);
        for (int j = 0; j < len; j++) acc = __fmaf_rn(sm.sp[g][j], sm.vt[j][t], acc);
        store_all(reinterpret_cast<uint32_t*>(s.out) + (size_t)(kvh * 4 + g) * 128 + t, flag_word(f2bf(__fdiv_rn(acc, sm.sp[g][31])), out_tag));
    }
    __syncthreads();
}

/* frame start for the single decode row (k_tick_begin of tick.cu, row 0) */
__device__ void tick_begin_cta(const TickBeginArgs& a, unsigned tag) {
    const int64_t id = a.ids[0];
    const bool vq = a.mask[0] != 0;
    int idx[S2P_NUM_CODEBOOKS];
#pragma unroll
    for (int cb = 0; cb < S2P_NUM_CODEBOOKS; cb++) {
        int c = a.codes[cb];
        c = max(0, min(S2P_CB_SIZE - 1, c));
        idx[cb] = cb * S2P_CB_SIZE + c;
    }
    const float inv_sqrt11 = (float)(1.0 / 3.3166247903554);
    for (int d = threadIdx.x; d < S2P_DIM; d += MEGA_WORKERS) {
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
        reinterpret_cast<uint32_t*>(a.x)[d] = flag_word(f2bf(v), tag); /* own arena only: every rank runs the frame start */
    }
    if (a.keys && threadIdx.x < 9) a.keys[threadIdx.x] = 0ull;
}

__global__ void __launch_bounds__(MEGA_THREADS, 1) k_tick_mega(MegaParams P) {
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* work = smem + (size_t)MEGA_SLOTS * P.lay.slot_bytes;
    unsigned char* tail = work + P.lay.x_bytes + MEGA_PARTS * P.lay.part_bytes + MEGA_RED_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail);
    MegaCopyCmd* next_cmd = reinterpret_cast<MegaCopyCmd*>(tail + 128);
    static_assert(MEGA_SLOTS + 2 * MEGA_PARTS <= 16, "the barrier words precede the staged command");
    /* cta / n_cta: position in the grid of all ranks (they equal blockIdx.x / gridDim.x on one GPU) */
    const int n_local = gridDim.x, tid = threadIdx.x;
    const int cta = P.tp_rank * n_local + blockIdx.x, n_cta = P.tp_world * n_local;
    const bool cta0 = blockIdx.x == 0; /* the CTA of each rank that runs the frame start, the sampler and the frame end */

    if (tid == 0) { /* constant indices only: see TpPeers */
        int n = 0;
#pragma unroll
        for (int q = 0; q < 8; q++)
            if (q < P.tp_world && q != P.tp_rank) {
                long long d = 0;
#pragma unroll
                for (int me = 0; me < 8; me++)
                    if (me == P.tp_rank) d = (long long)(P.tp_base[q] - P.tp_base[me]);
                g_tp.delta[n++] = d;
            }
        g_tp.n = n;
    }
    Ring ring;
    ring.slots = smem; ring.full = bars; ring.pfull = bars + MEGA_SLOTS; ring.pdone = bars + MEGA_SLOTS + MEGA_PARTS;
    ring.status = P.status;
    ring.seq_base = P.seq_base; ring.tag = 0;
    ring.slot_bytes = P.lay.slot_bytes; ring.part_floats = P.lay.part_bytes / 4; ring.x_bytes = P.lay.x_bytes;
    ring.cta = cta; ring.n_cta = n_cta; ring.consumed = 0;
    ring.cmds = P.cmds + P.cmd_start[blockIdx.x];
    ring.n_cmds = (unsigned)(P.cmd_start[blockIdx.x + 1] - P.cmd_start[blockIdx.x]);
    ring.issued = 0; ring.next = next_cmd;
    if (tid == MEGA_ISSUER) {
        for (int i = 0; i < MEGA_SLOTS; i++) mbar_init(ring.full + i, 1);
        for (int i = 0; i < MEGA_PARTS; i++) {
            mbar_init(ring.pfull + i, GEMV_WARPS);
            mbar_init(ring.pdone + i, GEMV_WARPS);
        }
        mbar_init_fence();
        ring_load_next(ring);
        ring_issue_upto(ring, MEGA_SLOTS);
    }
    __syncthreads(); /* the barriers are initialised before anyone waits on them */

    /* Stage descriptors are staged one stage ahead in shared memory: read from global
     * memory at the start of a stage they would cost two dependent cache misses. */
    MegaStage* st_buf = reinterpret_cast<MegaStage*>(tail + 256);
    constexpr int ST_VECS = (int)(sizeof(MegaStage) / 16);
    auto stage_prefetch = [&](int si) {
        if (si < P.n_stages && tid < ST_VECS)
            asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(st_buf + (si & 1)) + 16u * tid),
                         "l"(reinterpret_cast<const char*>(P.stages + si) + 16 * tid) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage_prefetch(0);
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();

    unsigned n_bar = 0;
    bool ok = true;
    for (int si = 0; si < P.n_stages && ok; si++) {
        const MegaStage& s = st_buf[si & 1];
        /* what is needed after the stage's last barrier is read now: past that barrier a faster
         * thread may already be staging stage si + 2 over this descriptor */
        const int no_barrier = s.flags & MEGA_NO_BARRIER, stage_type = s.type;
        stage_prefetch(si + 1); /* the other buffer held stage si - 1, which every thread has left */
        unsigned long long* tr = (P.trace && cta0) ? P.trace + (size_t)si * 16 : nullptr;
        if (tr && tid == 0) { tr[0] = clock64(); }
        const unsigned my_tag = (P.seq_base + (unsigned)si + 1u) & 0xFFFFu;
        const unsigned in_tag = (P.seq_base + (unsigned)s.x_from + 1u) & 0xFFFFu;
        ring.tag = my_tag;
        switch (s.type) {
        case MEGA_BEGIN:
            if (cta0) tick_begin_cta(P.begin, my_tag);
            break;
        case MEGA_GEMV:
            ok = gemv_dispatch(s, ring, work, tr);
            break;
        case MEGA_ATTN_SLOW: {
            /* the workers of one kv head are consecutive CTAs of one rank (8 divides by tp_world);
             * its cache planes are only kept current on that rank */
            const int workers = n_cta / S2P_SLOW_KV_HEADS;
            if (cta < workers * S2P_SLOW_KV_HEADS) {
                AttnArgs a = {};
                a.out = s.out;
                a.q_heads = S2P_SLOW_Q_HEADS; a.kv_heads = S2P_SLOW_KV_HEADS; a.max_seq = P.ctx_len; a.kv8 = P.kv8;
                a.pos_arr = P.pos_arr; a.kv = s.kv; a.part = P.part; a.counters = P.counters;
                a.n_split_slots = P.n_split_slots; a.workers = workers; a.head_dim = P.head_dim;
                a.n_out_peers = g_tp.n; a.out_peer_delta = g_tp.delta;
                a.out_ll = 1; a.out_ll_tag = my_tag;
                const AttnPrep pz = {s.qkv, s.q_norm, s.k_norm, P.eps, P.rope_base,
                                     reinterpret_cast<const uint32_t*>(s.qkv), in_tag, P.status};
                if (P.kv8)
                    attn_decode_cta<true, true, 1>(a, pz, 0, cta / workers, cta % workers, workers,
                                                *reinterpret_cast<AttnSmem<true>*>(work));
                else
                    attn_decode_cta<false, true, 1>(a, pz, 0, cta / workers, cta % workers, workers,
                                                 *reinterpret_cast<AttnSmem<false>*>(work));
            }
            break;
        }
        case MEGA_ATTN_FAST:
            /* kv head h of the fast-AR lives on rank h / (8 / tp_world), always in the same CTA */
            if ((int)blockIdx.x < S2P_SLOW_KV_HEADS / P.tp_world)
                fast_attn_cta(s, P.tp_rank * (S2P_SLOW_KV_HEADS / P.tp_world) + blockIdx.x, P.rope_base, P.head_dim, in_tag,
                              my_tag, P.status, *reinterpret_cast<FastAttnSmem*>(work));
            break;
        case MEGA_SAMPLE:
            if (cta0) { /* every rank samples for itself: same logits, same state, same draw */
                /* the head stages wrote flagged words: wait for them and unflag into the scratch row */
                const uint32_t* lc = reinterpret_cast<const uint32_t*>(P.sem_logits);
                const unsigned tc = (P.seq_base + (unsigned)P.logc_from + 1u) & 0xFFFFu;
                const unsigned te = (P.seq_base + (unsigned)P.loge_from + 1u) & 0xFFFFu;
                for (int i = tid; i < 4097; i += MEGA_WORKERS) {
                    uint32_t w = 0;
                    if (i < 4096) flag_wait1(lc + i, tc, P.status, w);
                    else flag_wait1(reinterpret_cast<const uint32_t*>(P.eos_logit), te, P.status, w);
                    reinterpret_cast<unsigned short*>(P.logits_plain)[i] = (unsigned short)(w & 0xFFFFu);
                }
                __threadfence_block();
                S2P_CTA_SYNC();
                sampler_cta<MEGA_WORKERS>(P.logits_plain, P.logits_plain + 4096, P.states[0], P.out_tok, P.out_sem,
                                          P.out_codes, P.out_eos, *reinterpret_cast<SamplerSmem<MEGA_WORKERS>*>(work));
            }
            break;
        case MEGA_FINISH:
            if (cta0 && tid < 9) P.out_codes[tid + 1] = (int32_t)key_index(__ldcg(P.keys + tid));
            break;
        default: break;
        }
        if (tr && tid == 0) tr[2] = clock64();
        if (P.trace && tid == 0) { /* every CTA: when its own work of the stage was done, on the GPU-wide timer */
            unsigned long long gt;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
            P.trace[(size_t)P.n_stages * 16 + (size_t)si * n_local + blockIdx.x] = gt;
        }
        asm volatile("cp.async.wait_all;" ::: "memory"); /* the next descriptor; the barrier below publishes it */
        /* without a grid barrier the next stage still reuses the work area: wait for this
         * CTA's slowest warp */
        if (no_barrier && stage_type != MEGA_GEMV) S2P_CTA_SYNC(); /* a GEMV stage ends with its own barrier */
        if (ok && !no_barrier) {
            n_bar++;
            ok = grid_barrier_tp(P.barrier, g_tp.delta, g_tp.n, (P.bar_base + n_bar) * (unsigned)n_cta, P.status);
        }
        if (tr && tid == 0) tr[3] = clock64();
    }
    /* A wait gave up: the copies this CTA already started still land in its shared memory,
     * so it stays until they have (bounded), then leaves. */
    if (!ok && tid == MEGA_ISSUER) {
        for (unsigned q = ring.consumed; q < ring.issued; q++) {
            uint64_t* bar = bars + (q % MEGA_SLOTS);
            const unsigned parity = (q / MEGA_SLOTS) & 1u;
            for (unsigned i = 0; i < PIPE_MBAR_TRIES && !mbar_try_wait(bar, parity); i++) {}
        }
    }
}

extern "C" void mega_layout(int x_bytes, MegaLayout* out) {
    out->x_bytes = (x_bytes + 255) & ~255;
    out->part_bytes = MEGA_PART_BYTES_DEFAULT;
    const int fixed = out->x_bytes + MEGA_PARTS * out->part_bytes + MEGA_RED_BYTES + MEGA_TAIL_BYTES;
    out->slot_bytes = ((MEGA_SMEM_MAX - fixed) / MEGA_SLOTS) & ~255;
    out->total_bytes = MEGA_SLOTS * out->slot_bytes + fixed;
}
extern "C" int mega_max_local_rows(const MegaLayout* lay, int K) {
    const int fit = lay->part_bytes / ((K >> 9) * 128);
    return fit < 2 * GEMV_WARPS ? fit : 2 * GEMV_WARPS; /* the fold takes two rows per warp */
}

/* host-side probe of the row partition (tests) */
extern "C" void mega_geom_probe(int N, int swiglu, int rows_per_chunk, int cta, int n_cta, int out[4]) {
    const MegaGeom g = mega_stage_geom(N, swiglu, rows_per_chunk, cta, n_cta);
    out[0] = g.row0; out[1] = g.cnt; out[2] = g.rc; out[3] = g.n_chunks;
}

extern "C" cudaError_t mega_setup(int* n_cta_out) {
    cudaError_t e = cudaFuncSetAttribute(k_tick_mega, cudaFuncAttributeMaxDynamicSharedMemorySize, MEGA_SMEM_MAX);
    if (e != cudaSuccess) return e;
    int dev = 0, sms = 0, coop = 0, per_sm = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev)) != cudaSuccess) return e;
    if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_tick_mega, MEGA_THREADS, MEGA_SMEM_MAX)) !=
        cudaSuccess)
        return e;
    if (!coop || per_sm < 1 || sms < 2 * S2P_SLOW_KV_HEADS) return cudaErrorNotSupported;
    *n_cta_out = sms;
    return cudaSuccess;
}

extern "C" cudaError_t mega_launch(const MegaParams* p, int n_cta, cudaStream_t st) {
    MegaParams P = *p;
    void* args[] = {&P};
    if (P.lay.total_bytes <= 0 || P.lay.total_bytes > MEGA_SMEM_MAX) return cudaErrorInvalidValue;
    return cudaLaunchCooperativeKernel((const void*)k_tick_mega, dim3((unsigned)n_cta), dim3(MEGA_THREADS), args,
                                       (size_t)P.lay.total_bytes, st);
}

}  // namespace s2p
