/* Primitives of the persistent decode-tick kernel: mbarrier + TMA bulk copies
 * into a shared-memory ring, and a grid-wide barrier.  Every wait is bounded by
 * a deadline on the GPU-wide timer: past it a wait records an error code in a
 * global status word and returns false; all other waits see the word and give
 * up too, so the kernel always runs to its normal exit and the host reads the
 * status.
 */
#pragma once
#include <stdint.h>
#include <cuda_runtime.h>

namespace s2p {

enum PipeError { PIPE_OK = 0, PIPE_ERR_TMA_WAIT = 1, PIPE_ERR_GRID_BARRIER = 2, PIPE_ERR_FLAG_WAIT = 3 };

/* How long a wait may last before it gives up, in nanoseconds of the GPU-wide timer (read every 64
 * polls).  Two seconds: far beyond anything a healthy run shows, short enough that a lost peer costs
 * the GPU's other users nothing.  One copy per translation unit; a test lowers it to make a wait run
 * out on purpose (nothing hangs or faults: the wait returns false and the kernel ends normally). */
static __constant__ unsigned long long c_pipe_wait_ns = 2000000000ull;
constexpr unsigned PIPE_MBAR_TRIES = 1u << 26;   /* backstops in polls, should the timer ever stand still */
constexpr unsigned PIPE_GRID_SPINS = 1u << 26;

__device__ __forceinline__ unsigned long long pipe_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
/* started at its first check, so that a wait that succeeds at once never reads the timer */
struct PipeDeadline {
    unsigned long long t0 = 0;
    __device__ __forceinline__ bool expired(unsigned long long limit_ns) {
        const unsigned long long now = pipe_now();
        if (!t0) { t0 = now; return false; }
        return now - t0 > limit_ns;
    }
    __device__ __forceinline__ bool expired() { return expired(c_pipe_wait_ns); }
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
/* 1-D bulk copy global -> this CTA's shared memory, completion counted on `bar`.
 * Both addresses 16-byte aligned, size a multiple of 16.  No multicast. */
__device__ __forceinline__ void tma_load_1d(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

/* orders this thread's earlier generic-proxy accesses to shared memory (and those it
 * has synchronised with) before its later async-proxy (bulk copy) writes */
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ int status_peek(const int* status) { return *reinterpret_cast<const volatile int*>(status); }

/* Wait for phase `parity` of an mbarrier; false (and status set) on time-out or when
 * another wait already failed. */
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, unsigned parity, int* status) {
    PipeDeadline dl;
    const unsigned every = c_pipe_wait_ns < 1000ull ? 0u : 63u; /* a sub-microsecond deadline (tests) is looked at on every poll */
    for (unsigned i = 0; i < PIPE_MBAR_TRIES; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & every) == every) {
            if (status_peek(status) != PIPE_OK) return false;
            if (dl.expired()) break;
        }
    }
    atomicCAS(status, PIPE_OK, PIPE_ERR_TMA_WAIT);
    return false;
}

/* ---- flagged words -------------------------------------------------------------
 * A value handed from one CTA (or GPU) to another without a barrier: a 32-bit word
 * carrying a bf16 payload in its low half and a 16-bit tag in its high half.  The
 * producer writes the word with one store; a consumer that reads the expected tag has
 * the payload of the same store (a 32-bit store is single-copy atomic), so no fence
 * and no separate flag are involved.  Tags count stage instances modulo 65536; every
 * cell is rewritten at least once per frame (a few hundred stage instances), so a
 * stale word can never carry the expected tag. */
constexpr unsigned PIPE_FLAG_SPINS = 1u << 26; /* backstop in polls; the limit is the deadline above */

__device__ __forceinline__ uint32_t flag_word(__nv_bfloat16 v, unsigned tag) {
    return (uint32_t)__bfloat16_as_ushort(v) | (tag << 16);
}
__device__ __forceinline__ uint32_t flag_ld1(const uint32_t* p) {
    uint32_t w;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(w) : "l"(p) : "memory");
    return w;
}
__device__ __forceinline__ uint4 flag_ld4(const uint4* p) {
    uint4 q;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w) : "l"(p) : "memory");
    return q;
}
/* wait for one word / four consecutive words to carry `tag`; false (status set) on time-out */
/* one poll of a flag wait that did not find its words: true when the wait has to give up (status set) */
__device__ __forceinline__ bool flag_wait_over(unsigned i, PipeDeadline& dl, int* status) {
    if ((i & 63u) != 63u) return false;
    if (status_peek(status) != PIPE_OK) return true;
    if (i > PIPE_FLAG_SPINS || dl.expired()) { atomicCAS(status, PIPE_OK, PIPE_ERR_FLAG_WAIT); return true; }
    return false;
}
__device__ __forceinline__ bool flag_wait1(const uint32_t* p, unsigned tag, int* status, uint32_t& w) {
    PipeDeadline dl;
    for (unsigned i = 0;; i++) {
        w = flag_ld1(p);
        if ((w >> 16) == tag) return true;
        if (flag_wait_over(i, dl, status)) return false;
    }
}
__device__ __forceinline__ bool flag_wait4(const uint4* p, unsigned tag, int* status, uint4& q) {
    PipeDeadline dl;
    for (unsigned i = 0;; i++) {
        q = flag_ld4(p);
        if (((q.x >> 16) == tag) & ((q.y >> 16) == tag) & ((q.z >> 16) == tag) & ((q.w >> 16) == tag)) return true;
        if (flag_wait_over(i, dl, status)) return false;
    }
}
__device__ __forceinline__ bool flag_tags4(const uint4& q, unsigned tag) {
    return ((q.x >> 16) == tag) & ((q.y >> 16) == tag) & ((q.z >> 16) == tag) & ((q.w >> 16) == tag);
}
/* the payload of a flagged word as f32 */
__device__ __forceinline__ float flag_payload(uint32_t w) { return __uint_as_float(w << 16); }

/* Grid-wide barrier of a persistent kernel whose CTAs are all resident (cooperative launch),
 * also across the persistent kernels of several GPUs: thread 0 of every CTA
 * publishes its CTA's stores system-wide and adds one to the counter in the own exchange arena
 * and in every peer's (the same cell, peer_delta[i] bytes away), then polls the own counter.
 * The counters are never reset: `target` is the running total (barriers so far, this one
 * included) x CTAs of all ranks, compared wrap-safely.  n_peers == 0: one GPU. */
__device__ __forceinline__ bool grid_barrier_tp(unsigned* counter, const long long* peer_delta, int n_peers, unsigned target,
                                                int* status) {
    __shared__ int ok_tp;
    S2P_CTA_SYNC();
    if (threadIdx.x == 0) {
        int ok = 1;
        if (n_peers > 0) {
            asm volatile("fence.acq_rel.sys;" ::: "memory");
            asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
            for (int i = 0; i < n_peers; i++)
                asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;"
                             ::"l"(reinterpret_cast<unsigned char*>(counter) + peer_delta[i]) : "memory");
        } else {
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
        }
        unsigned spins = 0, seen;
        PipeDeadline dl;
        for (;;) {
            if (n_peers > 0) asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
            else asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
            if ((int)(seen - target) >= 0) break;
            if ((++spins & 63u) == 0u) {
                if (status_peek(status) != PIPE_OK) { ok = 0; break; }
                if (spins > PIPE_GRID_SPINS || dl.expired()) { atomicCAS(status, PIPE_OK, PIPE_ERR_GRID_BARRIER); ok = 0; break; }
            }
        }
        ok_tp = ok && status_peek(status) == PIPE_OK;
    }
    S2P_CTA_SYNC();
    return ok_tp != 0;
}

}  // namespace s2p
