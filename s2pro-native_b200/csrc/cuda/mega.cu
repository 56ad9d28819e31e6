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
constexpr int MEGA_TAIL_BYTES = 1536;           /* mbarriers, the staged copy command, two stage descriptors, the stage kinds */
constexpr int MEGA_MAX_STAGES = 512;
static_assert(sizeof(MegaStage) % 16 == 0 && 2 * sizeof(MegaStage) + 256 + MEGA_MAX_STAGES <= MEGA_TAIL_BYTES, "descriptor staging");
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

/* What every thread needs to know about the ring and the partial buffers.  One copy in shared
 * memory, written once at kernel start: the per-stage functions below are compiled out of line
 * (their registers are their own), and what they share travels through here rather than through
 * by-reference arguments, which would live in local memory. */
struct Ring {
    int* status;
    int cta, n_cta;
    int slot_bytes, part_floats, x_bytes;
    int tail_off;      /* the mbarriers' offset in dynamic shared memory */
    unsigned seq_base; /* stage instances of earlier ticks */
    /* issuer thread only: this CTA's command list (built by the host with mega_stage_geom,
     * the function the consumers use), how many were issued */
    const MegaCopyCmd* cmds;
    unsigned n_cmds, issued;
};
__shared__ Ring g_ring;
/* the kernel's parameters, for the functions compiled out of line (a kernel parameter has no address
 * they could take without a copy in local memory) */
__shared__ MegaParams g_P;
extern __shared__ __align__(1024) unsigned char g_smem[];

__device__ __forceinline__ unsigned char* ring_slot(unsigned slot) { return g_smem + (size_t)slot * g_ring.slot_bytes; }
__device__ __forceinline__ unsigned char* ring_work() { return g_smem + (size_t)MEGA_SLOTS * g_ring.slot_bytes; }
__device__ __forceinline__ uint64_t* ring_bars() { return reinterpret_cast<uint64_t*>(g_smem + g_ring.tail_off); }
__device__ __forceinline__ uint64_t* ring_full(unsigned slot) { return ring_bars() + slot; }                      /* a chunk has landed */
__device__ __forceinline__ uint64_t* ring_pfull(unsigned b) { return ring_bars() + MEGA_SLOTS + b; }              /* the streaming warps have written a buffer */
__device__ __forceinline__ uint64_t* ring_pdone(unsigned b) { return ring_bars() + MEGA_SLOTS + MEGA_PARTS + b; } /* the folding warps have finished it */
__device__ __forceinline__ MegaCopyCmd* ring_next_cmd() { return reinterpret_cast<MegaCopyCmd*>(g_smem + g_ring.tail_off + 128); }

__device__ __forceinline__ void ring_load_next() {
    if (g_ring.issued < g_ring.n_cmds) {
        const char* src = reinterpret_cast<const char*>(g_ring.cmds + g_ring.issued);
        const uint32_t dst = smem_u32(ring_next_cmd());
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
__device__ __forceinline__ void ring_issue_upto(unsigned limit) {
    while (g_ring.issued < limit && g_ring.issued < g_ring.n_cmds) {
        const unsigned slot = g_ring.issued % MEGA_SLOTS;
        unsigned char* dst = ring_slot(slot);
        asm volatile("cp.async.wait_all;" ::: "memory");
        const MegaCopyCmd c = *ring_next_cmd();
        fence_proxy_async_smem(); /* the slot's previous chunk was read through the generic proxy */
        mbar_expect_tx(ring_full(slot), c.bytes[0] + c.bytes[1] + c.bytes[2] + c.bytes[3]);
#pragma unroll
        for (int k = 0; k < 4; k++)
            if (c.bytes[k])
                tma_load_1d(dst + c.dst_off[k], reinterpret_cast<const void*>(c.src[k]), c.bytes[k], ring_full(slot));
        g_ring.issued++;
        ring_load_next();
    }
}

/* ---- a GEMV stage: two groups of eight warps -------------------------------------------
 * The streaming warps (0..7) stage the activation vector and turn every chunk of weights
 * into per-(row, K-tile) lane partials in one of the partial buffers; the folding warps
 * (8..15) turn a finished buffer into outputs: tiles folded in ascending order with the
 * group scales, the 16/8/4/2/1 lane tree, the epilogue, the store.  The groups meet only at
 * mbarriers (`pfull`: a buffer is written, `pdone`: it is folded), so the streaming warps,
 * which are bound by instruction issue, never sit in the latency-bound fold, and at a stage
 * boundary they already wait for and stage the next stage's input while the last chunk is
 * folded and published.  Eight warps keep the integer pipe as busy as sixteen did.
 * Named barriers 1 and 2 synchronise the two groups separately. */
constexpr int MEGA_STREAM_WARPS = 8;
constexpr int MEGA_FOLD_WARPS = 8;
constexpr int MEGA_GROUP_THREADS = 256;
constexpr int MEGA_FOLD_CHAINS = 4; /* rows of one chunk a folding warp takes (two pairs with the SwiGLU epilogue) */
constexpr int MEGA_NORM_ELEMS = 10; /* elements a streaming thread normalises itself: inputs up to 2560 wide */
static_assert(MEGA_STREAM_WARPS + MEGA_FOLD_WARPS == GEMV_WARPS && MEGA_ISSUER >= 32 * MEGA_STREAM_WARPS,
              "the copy issuer belongs to the folding group");

struct StreamSync {
    __device__ __forceinline__ void operator()() const { asm volatile("bar.sync 1, 256;" ::: "memory"); }
};
__device__ __forceinline__ bool stream_sync_and(bool p) {
    uint32_t r;
    asm volatile("{ .reg .pred a, b; setp.ne.u32 a, %1, 0; bar.red.and.pred b, 1, 256, a; selp.u32 %0, 1, 0, b; }"
                 : "=r"(r) : "r"((uint32_t)p) : "memory");
    return r != 0;
}

/* Stage the input vector of a GEMV stage (streaming group only): wait for it, normalise it if the
 * stage asks for that, lay it out in shared memory for the unit loop.  Returns false, uniformly over
 * the group, if a bounded wait gave up. */
template <int WK>
__device__ __noinline__ bool gemv_stage_input(const MegaStage* sp) {
    const MegaStage& s = *sp;
    const int K = s.lin.K;
    bool ok = true;
    unsigned char* xs = ring_work();
    float* red = reinterpret_cast<float*>(xs + g_ring.x_bytes) + MEGA_PARTS * g_ring.part_floats;
    if (mega_stage_geom(s.lin.N, s.epi == EPI_SWIGLU, s.rows_per_chunk, g_ring.cta, g_ring.n_cta).cnt <= 0) return true; /* no rows here */
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
    const unsigned tag = (g_ring.seq_base + (unsigned)s.x_from + 1u) & 0xFFFFu;
    int* status = g_ring.status;
    /* eight elements = two 16-byte groups of flagged words, fetched together, again and again until
     * both carry the tag (one L2 round trip once they are there, not two) */
    auto load = [xsrc, ll, tag, status, &ok](int v) -> uint4 {
        if (!ll) return __ldcg(xsrc + v);
        uint4 a, b;
        PipeDeadline dl;
        for (unsigned spin = 0;; spin++) {
            a = flag_ld4(xsrc + 2 * v);
            b = flag_ld4(xsrc + 2 * v + 1);
            if (flag_tags4(a, tag) & flag_tags4(b, tag)) break;
            if (flag_wait_over(spin, dl, status)) { ok = false; return make_uint4(0, 0, 0, 0); }
        }
        return make_uint4((a.x & 0xFFFFu) | (a.y << 16), (a.z & 0xFFFFu) | (a.w << 16), (b.x & 0xFFFFu) | (b.y << 16),
                          (b.z & 0xFFFFu) | (b.w << 16));
    };
    if (s.pro == PRO_NORM && ll && (K & 255) == 0 && K <= 256 * MEGA_NORM_ELEMS) {
        /* Normalised flagged input: thread t takes the elements t, t + 256, ... - the ones whose
         * squares it sums in the reference's order (src/slowar/kernels.cu:46-68) - as single words,
         * all in flight together, so the sum needs neither shared memory nor a barrier; the 256 sums
         * meet in the halving tree, and the thread normalises its own elements
         * (y = bf16(x * inv * w)) straight into the staged layout.  Gains are fetched before the wait. */
        const int tid = threadIdx.x;
        const uint32_t* wsrc32 = reinterpret_cast<const uint32_t*>(xsrc);
        const unsigned short* gain = reinterpret_cast<const unsigned short*>(s.norm_w);
        const int ne = K >> 8;
        unsigned short gw[MEGA_NORM_ELEMS];
        uint32_t xw[MEGA_NORM_ELEMS];
#pragma unroll
        for (int m = 0; m < MEGA_NORM_ELEMS; m++) gw[m] = m < ne ? __ldg(gain + tid + 256 * m) : (unsigned short)0;
        PipeDeadline dl;
        for (unsigned spin = 0;; spin++) {
            bool here = true;
#pragma unroll
            for (int m = 0; m < MEGA_NORM_ELEMS; m++) xw[m] = m < ne ? flag_ld1(wsrc32 + tid + 256 * m) : (tag << 16);
#pragma unroll
            for (int m = 0; m < MEGA_NORM_ELEMS; m++) here &= (xw[m] >> 16) == tag;
            if (here) break;
            if (flag_wait_over(spin, dl, status)) { ok = false; break; }
        }
        float ss = 0.f;
#pragma unroll
        for (int m = 0; m < MEGA_NORM_ELEMS; m++)
            if (m < ne) {
                const float v = flag_payload(xw[m]);
                ss = __fmaf_rn(v, v, ss);
            }
        const float tot = tree256_sum(ss, red, StreamSync());
        const float inv = rsqrtf(__fdiv_rn(tot, (float)K) + S2P_NORM_EPS);
        const bool emit = s.normed_out != nullptr && blockIdx.x == 0;
#pragma unroll
        for (int m = 0; m < MEGA_NORM_ELEMS; m++)
            if (m < ne) {
                const int k = tid + 256 * m;
                const __nv_bfloat16 y = f2bf(__fmul_rn(__fmul_rn(flag_payload(xw[m]), inv), bf_bits_to_f32(gw[m])));
                xs_store<WK>(xs, k, y);
                if (emit) s.normed_out[k] = y;
            }
    } else if (s.pro == PRO_NORM) {
        stage_activation_from<WK, PRO_NORM>(g, load, xs, red, MEGA_GROUP_THREADS, StreamSync());
    } else {
        stage_activation_from<WK, PRO_VEC>(g, load, xs, red, MEGA_GROUP_THREADS, StreamSync());
    }
    return stream_sync_and(ok); /* uniform over the group; the staged vector is complete */
}

/* The streaming group's part of a GEMV stage after its input is staged; `q0`: chunks this CTA consumed before the stage.
 * Returns the stage's chunk count times two, plus one if no bounded wait gave up (uniform over
 * the group up to the end of the staging, per warp after it). */
template <int WK>
__device__ __noinline__ int gemv_stream(const MegaStage* sp, unsigned q0, unsigned long long* trace) {
    typedef typename LaneTile<WK>::type tile_t;
    const MegaStage& s = *sp;
    const int cta = g_ring.cta, n_cta = g_ring.n_cta;
    const MegaGeom ge = mega_stage_geom(s.lin.N, s.epi == EPI_SWIGLU, s.rows_per_chunk, cta, n_cta);
    if (ge.cnt <= 0) return 1; /* uniform over the CTA */
    unsigned char* work = ring_work();
    int* const status = g_ring.status;
    const int part_floats = g_ring.part_floats;
    const int K = s.lin.K, T = K >> 9;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int SW = (s.epi == EPI_SWIGLU) ? 2 : 1;
    const unsigned rb = (WK == WK_INT4_PACK) ? (unsigned)(K >> 1) : (unsigned)K;

    unsigned char* xs = work;
    float* part0 = reinterpret_cast<float*>(work + g_ring.x_bytes);
    long long tacc[2] = {0, 0}; /* trace: cycles of thread 0 waiting for a chunk / a buffer, and streaming */
    const int pstride = T * 32;

#pragma unroll 1
    for (int j = 0; j < ge.n_chunks; j++) {
        const unsigned q = q0 + (unsigned)j, slot = q % MEGA_SLOTS, b = q % MEGA_PARTS;
        const int cnt = min(ge.rc, ge.cnt - j * ge.rc);
        const int local_rows = cnt * SW;
        const unsigned char* wsl = ring_slot(slot);
        float* part = part0 + b * part_floats;
        const long long c0 = trace ? clock64() : 0;
        if (!mbar_wait_bounded(ring_full(slot), (q / MEGA_SLOTS) & 1u, status)) return 0;
        /* the buffer's previous chunk (q - MEGA_PARTS) must be folded */
        if (q >= MEGA_PARTS && !mbar_wait_bounded(ring_pdone(b), ((q / MEGA_PARTS) - 1u) & 1u, status)) return 0;
        const long long c1 = trace ? clock64() : 0;
        /* tile-major units; this warp's contiguous range, walked one tile segment at a time:
         * the activations of the tile stay in registers while up to four rows, whose chains
         * are independent, run side by side */
        const int U = local_rows * T;
        int u = (int)((long long)U * warp / MEGA_STREAM_WARPS);
        const int u_end = (int)((long long)U * (warp + 1) / MEGA_STREAM_WARPS);
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
        if (lane == 0) mbar_arrive(ring_pfull(b)); /* release: the partials are visible to whoever waits */
        if (trace && threadIdx.x == 0) {
            const long long c2 = clock64();
            tacc[0] += c1 - c0; tacc[1] += c2 - c1;
        }
    }
    if (trace && threadIdx.x == 0) { trace[4] = (unsigned long long)tacc[0]; trace[5] = (unsigned long long)tacc[1]; }
    if (trace && lane == 0) trace[8 + warp] = clock64(); /* when each streaming warp was through */
    return 2 * ge.n_chunks + 1;
}

/* What the folding group needs of a stage descriptor, read from global memory (the staged
 * copy in shared memory belongs to the streaming group, which may be a stage ahead). */
struct FoldDesc {
    int N, K, gshift, epi, rows_per_chunk, io_flags;
    const void* scales;
    __nv_bfloat16* y;
    VecRef resid;
    unsigned long long* key;
};
__device__ __forceinline__ FoldDesc fold_desc_load(const MegaStage* g) {
    FoldDesc d;
    d.N = __ldg(&g->lin.N); d.K = __ldg(&g->lin.K); d.gshift = __ldg(&g->lin.gshift);
    d.epi = __ldg(&g->epi); d.rows_per_chunk = __ldg(&g->rows_per_chunk); d.io_flags = __ldg(&g->io_flags);
    d.scales = reinterpret_cast<const void*>(__ldg(reinterpret_cast<const unsigned long long*>(&g->lin.scales)));
    d.y = reinterpret_cast<__nv_bfloat16*>(__ldg(reinterpret_cast<const unsigned long long*>(&g->y)));
    d.resid.base = reinterpret_cast<const __nv_bfloat16*>(__ldg(reinterpret_cast<const unsigned long long*>(&g->resid.base)));
    d.resid.index = reinterpret_cast<const int32_t*>(__ldg(reinterpret_cast<const unsigned long long*>(&g->resid.index)));
    d.resid.key = reinterpret_cast<const unsigned long long*>(__ldg(reinterpret_cast<const unsigned long long*>(&g->resid.key)));
    d.key = reinterpret_cast<unsigned long long*>(__ldg(reinterpret_cast<const unsigned long long*>(&g->key)));
    return d;
}

/* Fold up to four rows of a chunk (chains c < nch; row c's partials at pp[c], its group scales
 * at ss[c]): per lane the tiles in ascending order, acc = fma(partial, group scale, acc) (INT4,
 * grouped INT8) or acc += partial (per-channel INT8), then the 16/8/4/2/1 lane tree.  TT > 0:
 * the tile count at compile time, so that all loads of the chains are in flight together. */
template <int WK, int TT, int C0, int C1>
__device__ __forceinline__ void fold_chain_pass(int T, int nch, const float* const* pp, const __half* const* ss, int sstep, float* acc) {
    if (TT) {
#pragma unroll
        for (int i = 0; i < (TT ? TT : 1); i++) {
#pragma unroll
            for (int c = C0; c < C1; c++)
                if (c < nch) {
                    if (WK == WK_INT8_CH) acc[c] += pp[c][i * 32];
                    else acc[c] = __fmaf_rn(pp[c][i * 32], __half2float(ss[c][i * sstep]), acc[c]);
                }
        }
    } else {
#pragma unroll 2
        for (int i = 0; i < T; i++) {
#pragma unroll
            for (int c = C0; c < C1; c++)
                if (c < nch) {
                    if (WK == WK_INT8_CH) acc[c] += pp[c][i * 32];
                    else acc[c] = __fmaf_rn(pp[c][i * 32], __half2float(ss[c][i * sstep]), acc[c]);
                }
        }
    }
}
/* PASS2: the chains run as two passes of two (fewer loads in flight: wide rows), else all four together */
template <int WK, int TT, bool PASS2>
__device__ __forceinline__ void fold_chains(int T, int nch, const float* const* pp, const __half* const* ss, int sstep, float* acc) {
#pragma unroll
    for (int c = 0; c < MEGA_FOLD_CHAINS; c++) acc[c] = 0.f;
    if (PASS2) {
        fold_chain_pass<WK, TT, 0, 2>(T, nch, pp, ss, sstep, acc);
        if (nch > 2) fold_chain_pass<WK, TT, 2, 4>(T, nch, pp, ss, sstep, acc);
    } else {
        fold_chain_pass<WK, TT, 0, 4>(T, nch, pp, ss, sstep, acc);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
        for (int c = 0; c < MEGA_FOLD_CHAINS; c++) acc[c] += __shfl_xor_sync(S2P_FULL_MASK, acc[c], off);
    }
}

/* The folding group's part of a GEMV stage (`gs`: the descriptor in global memory, `my_tag`: the tag
 * of the stage's flagged outputs).  Returns like gemv_stream, per warp. */
template <int WK>
__device__ __noinline__ int gemv_fold(const MegaStage* gs, unsigned q0, unsigned my_tag, unsigned long long* trace) {
    const FoldDesc d = fold_desc_load(gs);
    const bool two = d.epi == EPI_SWIGLU;
    const MegaGeom ge = mega_stage_geom(d.N, two, d.rows_per_chunk, g_ring.cta, g_ring.n_cta);
    if (ge.cnt <= 0) return 1;
    unsigned char* work = ring_work();
    int* const status = g_ring.status;
    const int part_floats = g_ring.part_floats;
    const int K = d.K, T = K >> 9, gshift = d.gshift;
    const int lane = threadIdx.x & 31, fw = (threadIdx.x >> 5) - MEGA_STREAM_WARPS;
    const int SW = two ? 2 : 1;
    const int F = d.N >> 1;
    const unsigned rb = (WK == WK_INT4_PACK) ? (unsigned)(K >> 1) : (unsigned)K;
    const unsigned sb = (WK == WK_INT8_CH) ? 0u : (unsigned)(K >> gshift) * 2u;
    const float* part0 = reinterpret_cast<const float*>(work + g_ring.x_bytes);
    const int pstride = T * 32;
    const int sl = (lane * 16) >> gshift, sstep = 512 >> gshift;
    const bool y_ll = (d.io_flags & MEGA_Y_LL) != 0;
    unsigned long long best = 0ull;
    bool ok = true;
    long long tacc[2] = {0, 0};
    /* the residual row (EPI_RESID): the vector itself, or a row of a table picked on the device */
    const __nv_bfloat16* resid = d.resid.base;
    if (d.epi == EPI_RESID) {
        if (d.resid.index) resid += (size_t)__ldcg(d.resid.index) * d.N;
        else if (d.resid.key) resid += (size_t)key_index(__ldcg(d.resid.key)) * d.N;
    }

#pragma unroll 1
    for (int j = 0; j < ge.n_chunks; j++) {
        const unsigned q = q0 + (unsigned)j, slot = q % MEGA_SLOTS, b = q % MEGA_PARTS;
        const int cnt = min(ge.rc, ge.cnt - j * ge.rc);
        const int l0 = j * ge.rc, r0 = ge.row0 + l0;
        const int local_rows = cnt * SW;
        const unsigned char* ssl = ring_slot(slot) + (size_t)local_rows * rb;
        const float* part = part0 + b * part_floats;
        /* chains of this warp: plain rows fw, fw+8, fw+16, fw+24 of the chunk; with SwiGLU the
         * gate rows of pairs fw, fw+8 (chains 0, 1) and their up rows (chains 2, 3) */
        int lr[MEGA_FOLD_CHAINS], nch;
        if (two) {
            lr[0] = fw; lr[1] = fw + MEGA_FOLD_WARPS; lr[2] = fw + cnt; lr[3] = fw + MEGA_FOLD_WARPS + cnt;
            nch = fw + MEGA_FOLD_WARPS < cnt ? 4 : (fw < cnt ? 3 : 0); /* a lone pair uses chains 0 and 2 */
        } else {
#pragma unroll
            for (int c = 0; c < MEGA_FOLD_CHAINS; c++) lr[c] = fw + c * MEGA_FOLD_WARPS;
            nch = fw >= cnt ? 0 : min(MEGA_FOLD_CHAINS, (cnt - fw + MEGA_FOLD_WARPS - 1) / MEGA_FOLD_WARPS);
        }
        const float* pp[MEGA_FOLD_CHAINS];
        const __half* ss[MEGA_FOLD_CHAINS];
#pragma unroll
        for (int c = 0; c < MEGA_FOLD_CHAINS; c++) {
            const int l = lr[c] < local_rows ? lr[c] : 0; /* unused chains point at valid memory */
            pp[c] = part + (size_t)l * pstride + lane;
            ss[c] = reinterpret_cast<const __half*>(ssl + (size_t)l * sb) + sl;
        }
        /* what the epilogue of lane c needs from global memory, fetched before the wait: the
         * residual value and the per-channel row scale(s) of row r0 + fw + 8 c */
        const int my_l = fw + lane * MEGA_FOLD_WARPS;             /* row (pair) of the chunk this lane finishes */
        const bool mine = lane < (two ? 2 : MEGA_FOLD_CHAINS) && my_l < cnt;
        const int my_n = r0 + my_l;
        float res_v = 0.f, rs_a = 1.f, rs_b = 1.f;
        if (mine) {
            if (d.epi == EPI_RESID)
                res_v = (d.io_flags & MEGA_RESID_LL) ? flag_payload(__ldcg(reinterpret_cast<const uint32_t*>(resid) + my_n))
                                                     : ldcg_bf16(resid + my_n);
            if (WK == WK_INT8_CH) {
                rs_a = __ldg(static_cast<const float*>(d.scales) + my_n);
                if (two) rs_b = __ldg(static_cast<const float*>(d.scales) + F + my_n);
            }
        }
        const long long c0 = trace ? clock64() : 0;
        if (!mbar_wait_bounded(ring_pfull(b), (q / MEGA_PARTS) & 1u, status)) return 0;
        const long long c1 = trace ? clock64() : 0;
        if (nch > 0) {
            float acc[MEGA_FOLD_CHAINS];
            switch (T) {
            /* the model's widths with the tile count at compile time */
            case 5: fold_chains<WK, 5, false>(T, nch, pp, ss, sstep, acc); break;
            case 8: fold_chains<WK, 8, true>(T, nch, pp, ss, sstep, acc); break;
            case 19: fold_chains<WK, 19, true>(T, nch, pp, ss, sstep, acc); break;
            default: fold_chains<WK, 0, false>(T, nch, pp, ss, sstep, acc); break;
            }
            if (mine) {
                if (two) {
                    float gate = lane == 0 ? acc[0] : acc[1], up = lane == 0 ? acc[2] : acc[3];
                    if (WK == WK_INT8_CH) { gate = __fmul_rn(gate, rs_a); up = __fmul_rn(up, rs_b); }
                    gate = bf16_round(gate); up = bf16_round(up);
                    const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-gate)));
                    const float sil = bf16_round(__fmul_rn(gate, sig));
                    const __nv_bfloat16 v = f2bf(__fmul_rn(sil, up));
                    if (y_ll) store_all(reinterpret_cast<uint32_t*>(d.y) + my_n, flag_word(v, my_tag));
                    else store_all(d.y + my_n, v);
                } else {
                    float a = lane == 0 ? acc[0] : (lane == 1 ? acc[1] : (lane == 2 ? acc[2] : acc[3]));
                    if (WK == WK_INT8_CH) a = __fmul_rn(a, rs_a);
                    const __nv_bfloat16 yb = f2bf(a);
                    const __nv_bfloat16 v = d.epi == EPI_RESID ? f2bf(__fadd_rn(res_v, bf2f(yb))) : yb;
                    if (y_ll) store_all(reinterpret_cast<uint32_t*>(d.y) + my_n, flag_word(v, my_tag));
                    else store_all(d.y + my_n, v);
                    if (d.epi == EPI_ARGMAX) best = max(best, argmax_key(yb, my_n));
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(ring_pdone(b)); /* this warp is done with the chunk's scales and partials */
        if (threadIdx.x == MEGA_ISSUER) {
            /* once every folding warp has left the chunk its slot takes the chunk MEGA_SLOTS further on */
            if (mbar_wait_bounded(ring_pdone(b), (q / MEGA_PARTS) & 1u, status)) ring_issue_upto(q + 1 + MEGA_SLOTS);
            else ok = false;
        }
        __syncwarp();
        if (trace && fw == 0 && lane == 0) {
            const long long c2 = clock64();
            tacc[0] += c1 - c0; tacc[1] += c2 - c1;
        }
    }
    if (trace && fw == 0 && lane == 0) { trace[6] = (unsigned long long)tacc[0]; trace[7] = (unsigned long long)tacc[1]; }
    if (d.epi == EPI_ARGMAX && best) {
        atomicMax(d.key, best);
        for (int i = 0; i < g_tp.n; i++)
            atomicMax_system(reinterpret_cast<unsigned long long*>(reinterpret_cast<unsigned char*>(d.key) + g_tp.delta[i]), best);
    }
    return 2 * ge.n_chunks + (ok ? 1 : 0);
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

/* The stages that take the whole CTA: frame start, attention of both stacks, sampler, frame end.
 * Each out of line with registers of its own, so that the stage loop of the kernel stays small and
 * holds few registers across its calls. */
__device__ __noinline__ void cta_stage_attn_slow(const MegaStage* sp, unsigned my_tag) {
    const MegaStage& s = *sp;
    const int n_local = gridDim.x;
    const int cta = g_P.tp_rank * n_local + blockIdx.x, n_cta = g_P.tp_world * n_local;
    const unsigned in_tag = (g_P.seq_base + (unsigned)s.x_from + 1u) & 0xFFFFu;
    /* the workers of one kv head are consecutive CTAs of one rank (8 divides by tp_world);
     * its cache planes are only kept current on that rank */
    const int workers = n_cta / S2P_SLOW_KV_HEADS;
    if (cta >= workers * S2P_SLOW_KV_HEADS) return;
    AttnArgs a = {};
    a.out = s.out;
    a.q_heads = S2P_SLOW_Q_HEADS; a.kv_heads = S2P_SLOW_KV_HEADS; a.max_seq = g_P.ctx_len; a.kv8 = g_P.kv8;
    a.pos_arr = g_P.pos_arr; a.kv = s.kv; a.part = g_P.part; a.counters = g_P.counters;
    a.n_split_slots = g_P.n_split_slots; a.workers = workers; a.head_dim = g_P.head_dim;
    a.n_out_peers = g_tp.n; a.out_peer_delta = g_tp.delta;
    a.out_ll = 1; a.out_ll_tag = my_tag;
    const AttnPrep pz = {s.qkv, s.q_norm, s.k_norm, g_P.eps, g_P.rope_base,
                         reinterpret_cast<const uint32_t*>(s.qkv), in_tag, g_P.status};
    if (g_P.kv8)
        attn_decode_cta<true, true, 1>(a, pz, 0, cta / workers, cta % workers, workers, *reinterpret_cast<AttnSmem<true>*>(ring_work()));
    else
        attn_decode_cta<false, true, 1>(a, pz, 0, cta / workers, cta % workers, workers, *reinterpret_cast<AttnSmem<false>*>(ring_work()));
}

__device__ __noinline__ void cta_stage_other(const MegaStage* sp, int stage_type, unsigned my_tag) {
    const MegaStage& s = *sp;
    const int tid = threadIdx.x;
    const bool cta0 = blockIdx.x == 0;
    unsigned char* work = ring_work();
    const unsigned in_tag = (g_P.seq_base + (unsigned)s.x_from + 1u) & 0xFFFFu;
    switch (stage_type) {
    case MEGA_BEGIN:
        if (cta0) tick_begin_cta(g_P.begin, my_tag);
        break;
    case MEGA_ATTN_FAST:
        /* kv head h of the fast-AR lives on rank h / (8 / tp_world), always in the same CTA */
        if ((int)blockIdx.x < S2P_SLOW_KV_HEADS / g_P.tp_world)
            fast_attn_cta(s, g_P.tp_rank * (S2P_SLOW_KV_HEADS / g_P.tp_world) + blockIdx.x, g_P.rope_base, g_P.head_dim, in_tag,
                          my_tag, g_P.status, *reinterpret_cast<FastAttnSmem*>(work));
        break;
    case MEGA_SAMPLE:
        if (cta0) { /* every rank samples for itself: same logits, same state, same draw */
            /* the head stages wrote flagged words: wait for them and unflag into the scratch row */
            const uint32_t* lc = reinterpret_cast<const uint32_t*>(g_P.sem_logits);
            const unsigned tc = (g_P.seq_base + (unsigned)g_P.logc_from + 1u) & 0xFFFFu;
            const unsigned te = (g_P.seq_base + (unsigned)g_P.loge_from + 1u) & 0xFFFFu;
            for (int i = tid; i < 4097; i += MEGA_WORKERS) {
                uint32_t w = 0;
                if (i < 4096) flag_wait1(lc + i, tc, g_P.status, w);
                else flag_wait1(reinterpret_cast<const uint32_t*>(g_P.eos_logit), te, g_P.status, w);
                reinterpret_cast<unsigned short*>(g_P.logits_plain)[i] = (unsigned short)(w & 0xFFFFu);
            }
            __threadfence_block();
            S2P_CTA_SYNC();
            sampler_cta<MEGA_WORKERS>(g_P.logits_plain, g_P.logits_plain + 4096, g_P.states[0], g_P.out_tok, g_P.out_sem,
                                      g_P.out_codes, g_P.out_eos, *reinterpret_cast<SamplerSmem<MEGA_WORKERS>*>(work));
        }
        break;
    case MEGA_FINISH:
        if (cta0 && tid < 9) g_P.out_codes[tid + 1] = (int32_t)key_index(__ldcg(g_P.keys + tid));
        break;
    default: break;
    }
}

__global__ void __launch_bounds__(MEGA_THREADS, 1) k_tick_mega(MegaParams P) {
    unsigned char* const smem = g_smem;
    unsigned char* work = smem + (size_t)MEGA_SLOTS * P.lay.slot_bytes;
    unsigned char* tail = work + P.lay.x_bytes + MEGA_PARTS * P.lay.part_bytes + MEGA_RED_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail);
    static_assert(MEGA_SLOTS + 2 * MEGA_PARTS + 1 <= 16, "the barrier words precede the staged command");
    /* cta / n_cta: position in the grid of all ranks (they equal blockIdx.x / gridDim.x on one GPU) */
    const int n_local = gridDim.x, tid = threadIdx.x;
    const int cta = P.tp_rank * n_local + blockIdx.x, n_cta = P.tp_world * n_local;

    if (tid == 32) g_P = P;
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
    uint64_t* join = bars + MEGA_SLOTS + 2 * MEGA_PARTS; /* where the two groups meet before a stage that needs the whole CTA */
    if (tid == MEGA_ISSUER) {
        g_ring.status = P.status;
        g_ring.seq_base = P.seq_base;
        g_ring.slot_bytes = P.lay.slot_bytes; g_ring.part_floats = P.lay.part_bytes / 4; g_ring.x_bytes = P.lay.x_bytes;
        g_ring.tail_off = (int)(tail - smem);
        g_ring.cta = cta; g_ring.n_cta = n_cta;
        g_ring.cmds = P.cmds + P.cmd_start[blockIdx.x];
        g_ring.n_cmds = (unsigned)(P.cmd_start[blockIdx.x + 1] - P.cmd_start[blockIdx.x]);
        g_ring.issued = 0;
        for (int i = 0; i < MEGA_SLOTS; i++) mbar_init(ring_full(i), 1);
        for (int i = 0; i < MEGA_PARTS; i++) {
            mbar_init(ring_pfull(i), MEGA_STREAM_WARPS);
            mbar_init(ring_pdone(i), MEGA_FOLD_WARPS);
        }
        mbar_init(join, GEMV_WARPS);
        mbar_init_fence();
        ring_load_next();
        ring_issue_upto(MEGA_SLOTS);
    }
    /* kind and flags of every stage, for both groups: one byte each (kind | flags << 4) */
    unsigned char* kinds = tail + 256 + 2 * sizeof(MegaStage);
#define MEGA_KINDS() (g_smem + g_ring.tail_off + 256 + 2 * sizeof(MegaStage))
#define MEGA_STBUF() reinterpret_cast<MegaStage*>(g_smem + g_ring.tail_off + 256)
#define MEGA_JOIN() (reinterpret_cast<uint64_t*>(g_smem + g_ring.tail_off) + MEGA_SLOTS + 2 * MEGA_PARTS)
#define MEGA_TR() ((P.trace && blockIdx.x == 0) ? P.trace + (size_t)si * 16 : nullptr)
    for (int i = tid; i < P.n_stages; i += MEGA_THREADS)
        kinds[i] = (unsigned char)(__ldg(&P.stages[i].type) | (__ldg(&P.stages[i].flags) << 4));

    /* Stage descriptors are staged one stage ahead in shared memory by the streaming group: read
     * from global memory at the start of a stage they would cost two dependent cache misses. */
    constexpr int ST_VECS = (int)(sizeof(MegaStage) / 16);
    static_assert(ST_VECS <= MEGA_GROUP_THREADS, "one thread per 16 bytes of a descriptor");
    auto stage_prefetch = [&](int si) {
        if (si < P.n_stages && threadIdx.x < ST_VECS)
            asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(MEGA_STBUF() + (si & 1)) + 16u * threadIdx.x),
                         "l"(reinterpret_cast<const char*>(P.stages + si) + 16 * threadIdx.x) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage_prefetch(0);
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads(); /* barriers initialised, first descriptor and the kinds table in place */

    /* `ok` turns false when a bounded wait of this thread gave up (the status word is set then, and
     * every other wait gives up soon after).  A thread that sees it leaves the stage loop; nobody
     * may be left behind at a barrier, so the verdict is made uniform where a barrier follows: over
     * the streaming group at its barrier on entering a GEMV stage, over the CTA at the join
     * (an mbarrier with a bounded wait). */
    unsigned n_bar = 0, n_join = 0, consumed = 0; /* consumed: chunks of the ring this CTA is through (every thread counts) */
    bool ok = true;
    for (int si = 0; si < P.n_stages; si++) {
        const int stage_type = MEGA_KINDS()[si] & 15, no_barrier = (MEGA_KINDS()[si] >> 4) & MEGA_NO_BARRIER;
        const unsigned my_tag = (P.seq_base + (unsigned)si + 1u) & 0xFFFFu;
        if (stage_type == MEGA_GEMV) {
            if (threadIdx.x < MEGA_GROUP_THREADS) {
                /* the descriptor was staged while the previous stage ran; the group barrier inside
                 * gemv_stream (or the join below) publishes it to the group */
                asm volatile("cp.async.wait_all;" ::: "memory");
                if (!stream_sync_and(ok)) { ok = false; break; }
                const MegaStage& s = MEGA_STBUF()[si & 1];
                stage_prefetch(si + 1); /* the other buffer held stage si - 1, which the group has left */
                if (MEGA_TR() && threadIdx.x == 0) MEGA_TR()[0] = clock64();
                /* (the group barrier above: every streaming warp has left the previous stage's activation) */
                int rc = 0;
                bool staged;
                switch (s.lin.kind) {
                case WK_INT8_CH: staged = gemv_stage_input<WK_INT8_CH>(&s); break;
                case WK_INT8_GRP: staged = gemv_stage_input<WK_INT8_GRP>(&s); break;
                default: staged = gemv_stage_input<WK_INT4_PACK>(&s); break;
                }
                if (MEGA_TR() && threadIdx.x == 0) MEGA_TR()[1] = clock64();
                if (P.trace && threadIdx.x == 0) { /* every CTA: when its input was staged, on the GPU-wide timer */
                    unsigned long long gt;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
                    P.trace[(size_t)P.n_stages * (16 + (int)gridDim.x) + (size_t)si * (int)gridDim.x + blockIdx.x] = gt;
                }
                if (staged) switch (s.lin.kind) {
                case WK_INT8_CH: rc = gemv_stream<WK_INT8_CH>(&s, consumed, MEGA_TR()); break;
                case WK_INT8_GRP: rc = gemv_stream<WK_INT8_GRP>(&s, consumed, MEGA_TR()); break;
                default: rc = gemv_stream<WK_INT4_PACK>(&s, consumed, MEGA_TR()); break;
                }
                ok = rc & 1; consumed += (unsigned)(rc >> 1);
                if (MEGA_TR() && threadIdx.x == 0) MEGA_TR()[2] = clock64();
            } else {
                if (!ok) break; /* the folding warps share no barrier: each leaves on its own */
                const MegaStage* gs = P.stages + si;
                int rc;
                switch (__ldg(&gs->lin.kind)) {
                case WK_INT8_CH: rc = gemv_fold<WK_INT8_CH>(gs, consumed, my_tag, MEGA_TR()); break;
                case WK_INT8_GRP: rc = gemv_fold<WK_INT8_GRP>(gs, consumed, my_tag, MEGA_TR()); break;
                default: rc = gemv_fold<WK_INT4_PACK>(gs, consumed, my_tag, MEGA_TR()); break;
                }
                ok = rc & 1; consumed += (unsigned)(rc >> 1);
                if (MEGA_TR() && threadIdx.x == MEGA_GROUP_THREADS) MEGA_TR()[3] = clock64();
                if (P.trace && threadIdx.x == MEGA_GROUP_THREADS) { /* every CTA: when its outputs of the stage were out, on the GPU-wide timer */
                    unsigned long long gt;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
                    P.trace[(size_t)P.n_stages * 16 + (size_t)si * (int)gridDim.x + blockIdx.x] = gt;
                }
            }
            if (no_barrier) continue; /* the groups go on separately; the next stage's waits order them */
        }
        /* A stage of the whole CTA (or a grid barrier) follows: the groups meet.  One arrival per
         * warp; the wait is bounded like every other, so a group that gave up cannot strand the other. */
        if (!ok) break; /* without arriving: the others' wait at the join runs out */
        __syncwarp();
        if ((threadIdx.x & 31) == 0) mbar_arrive(MEGA_JOIN());
        if (!mbar_wait_bounded(MEGA_JOIN(), n_join & 1u, P.status)) { ok = false; break; }
        n_join++;
        /* all sixteen warps arrived, so all of them are fine and take the CTA barriers below */
        if (stage_type != MEGA_GEMV) {
            if (threadIdx.x < MEGA_GROUP_THREADS) asm volatile("cp.async.wait_all;" ::: "memory");
            __syncthreads();
            if (MEGA_TR() && threadIdx.x == 0) MEGA_TR()[0] = clock64();
            if (stage_type == MEGA_ATTN_SLOW) cta_stage_attn_slow(MEGA_STBUF() + (si & 1), my_tag);
            else cta_stage_other(MEGA_STBUF() + (si & 1), stage_type, my_tag);
            if (MEGA_TR() && threadIdx.x == 0) MEGA_TR()[2] = clock64();
            if (P.trace && threadIdx.x == 0) {
                unsigned long long gt;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
                P.trace[(size_t)P.n_stages * 16 + (size_t)si * (int)gridDim.x + blockIdx.x] = gt;
            }
            __syncthreads(); /* the work area and the descriptor buffer are free again */
            if (threadIdx.x < MEGA_GROUP_THREADS) stage_prefetch(si + 1);
        }
        if (!no_barrier) {
            n_bar++;
            if (!grid_barrier_tp(P.barrier, g_tp.delta, g_tp.n, (P.bar_base + n_bar) * (unsigned)n_cta, P.status)) {
                ok = false; /* uniform over the CTA */
                break;
            }
        }
        if (MEGA_TR() && threadIdx.x == 0 && stage_type != MEGA_GEMV) MEGA_TR()[3] = clock64();
    }
    /* A wait gave up: the copies this CTA already started still land in its shared memory,
     * so it stays until they have (bounded), then leaves. */
    if (!ok && threadIdx.x == MEGA_ISSUER) {
        for (unsigned q = consumed; q < g_ring.issued; q++) {
            uint64_t* bar = ring_full(q % MEGA_SLOTS);
            const unsigned parity = (q / MEGA_SLOTS) & 1u;
            PipeDeadline dl; /* these copies do land (nothing but memory is waited for): a fixed, generous limit, whatever
                              * deadline the other waits were given */
            for (unsigned i = 0; i < PIPE_MBAR_TRIES && !mbar_try_wait(bar, parity); i++)
                if ((i & 63u) == 63u && dl.expired(2000000000ull)) break;
        }
    }
}

#undef MEGA_KINDS
#undef MEGA_STBUF
#undef MEGA_JOIN
#undef MEGA_TR

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

/* Test hooks for the bounded waits.  mega_set_wait_ns: the deadline of every wait of the persistent
 * tick on the current device (default two seconds).  pipe_wait_probe: one small CTA waits on an mbarrier
 * (which = 0) or a flagged word (which = 1) that nobody will ever signal, with a deadline of limit_ns;
 * the wait gives up, the kernel ends normally, and the status code and the time the wait took come back.
 * Nothing hangs or faults: this is how the give-up path is exercised. */
extern "C" cudaError_t mega_set_wait_ns(unsigned long long ns) {
    return cudaMemcpyToSymbol(c_pipe_wait_ns, &ns, sizeof(ns));
}
__global__ void k_wait_probe(int which, uint32_t* word, int* status, unsigned long long* elapsed) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_init_fence(); }
    __syncthreads();
    const unsigned long long t0 = pipe_now();
    bool got;
    if (which == 0) got = mbar_wait_bounded(&bar, 0u, status);
    else { uint32_t w; got = flag_wait1(word, 0x1234u, status, w); }
    if (threadIdx.x == 0) { elapsed[0] = pipe_now() - t0; elapsed[1] = got ? 1ull : 0ull; }
}
extern "C" cudaError_t pipe_wait_probe(int which, unsigned long long limit_ns, int* status_out, unsigned long long* elapsed_ns_out,
                                       int* got_out) {
    unsigned long long saved = 0, h[2] = {0, 0};
    unsigned char* d = nullptr;
    cudaError_t e = cudaMemcpyFromSymbol(&saved, c_pipe_wait_ns, sizeof(saved));
    if (e == cudaSuccess) e = cudaMalloc((void**)&d, 64);
    if (e == cudaSuccess) e = cudaMemset(d, 0, 64);
    if (e == cudaSuccess) e = mega_set_wait_ns(limit_ns);
    if (e == cudaSuccess) {
        k_wait_probe<<<1, 32>>>(which, reinterpret_cast<uint32_t*>(d), reinterpret_cast<int*>(d + 16),
                                reinterpret_cast<unsigned long long*>(d + 32));
        e = cudaDeviceSynchronize();
    }
    if (e == cudaSuccess) e = cudaMemcpy(status_out, d + 16, sizeof(int), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(h, d + 32, sizeof(h), cudaMemcpyDeviceToHost);
    *elapsed_ns_out = h[0];
    *got_out = (int)h[1];
    const cudaError_t r = mega_set_wait_ns(saved ? saved : 2000000000ull);
    if (d) cudaFree(d);
    return e != cudaSuccess ? e : r;
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
