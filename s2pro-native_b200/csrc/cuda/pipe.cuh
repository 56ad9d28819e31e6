/* Primitives of the persistent decode-tick kernel: mbarrier + TMA bulk copies
 * into a shared-memory ring, and a grid-wide barrier.  Every wait is bounded:
 * after its iteration limit a wait records an error code in a global status
 * word and returns false; all other waits see the word and give up too, so the
 * kernel always runs to its normal exit and the host reads the status.
 */
#pragma once
#include <stdint.h>
#include <cuda_runtime.h>

namespace s2p {

enum PipeError { PIPE_OK = 0, PIPE_ERR_TMA_WAIT = 1, PIPE_ERR_GRID_BARRIER = 2 };

constexpr unsigned PIPE_MBAR_TRIES = 1u << 20;   /* each try_wait already blocks for a hardware time slice */
constexpr unsigned PIPE_GRID_SPINS = 1u << 22;   /* a few seconds of polling an L2 word */

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
    for (unsigned i = 0; i < PIPE_MBAR_TRIES; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u && status_peek(status) != PIPE_OK) return false;
    }
    atomicCAS(status, PIPE_OK, PIPE_ERR_TMA_WAIT);
    return false;
}

/* Grid-wide barrier for a kernel whose CTAs are all resident (cooperative launch).
 * `counter` starts at 0 for the launch; the k-th barrier (k = 1, 2, ...) completes
 * when it reaches k * n_cta.  Called by every thread of the CTA. */
__device__ __forceinline__ bool grid_barrier(unsigned* counter, unsigned target, int* status) {
    __shared__ int ok_s;
    S2P_CTA_SYNC();
    if (threadIdx.x == 0) {
        int ok = 1;
        /* release: publishes this CTA's stores (ordered before it by the CTA barrier above) */
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
        unsigned spins = 0, seen;
        for (;;) {
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
            if (seen >= target) break;
            if (++spins > PIPE_GRID_SPINS) { atomicCAS(status, PIPE_OK, PIPE_ERR_GRID_BARRIER); ok = 0; break; }
            if ((spins & 255u) == 0u && status_peek(status) != PIPE_OK) { ok = 0; break; }
        }
        ok_s = ok && status_peek(status) == PIPE_OK;
    }
    S2P_CTA_SYNC();
    return ok_s != 0;
}

/* The same barrier across the persistent kernels of several GPUs: thread 0 of every CTA
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
        for (;;) {
            if (n_peers > 0) asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
            else asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
            if ((int)(seen - target) >= 0) break;
            if (++spins > PIPE_GRID_SPINS) { atomicCAS(status, PIPE_OK, PIPE_ERR_GRID_BARRIER); ok = 0; break; }
            if ((spins & 255u) == 0u && status_peek(status) != PIPE_OK) { ok = 0; break; }
        }
        ok_tp = ok && status_peek(status) == PIPE_OK;
    }
    S2P_CTA_SYNC();
    return ok_tp != 0;
}

}  // namespace s2p
