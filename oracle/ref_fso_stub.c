/* Test infrastructure (not product code).
 *
 * The reference's linear-layer file calls an FP8 shim whose sources are not
 * part of the reference tree (an external CUTLASS project cloned at build
 * time).  The rebuilt reference library used as the parity checker never
 * selects the FP8 mode, so this file answers "FP8 unavailable" for the nine
 * entry points that src/fso/fso.h:28-56 of the reference declares, which is
 * enough to link src/sched/gemm.c unchanged. */
#include <stddef.h>
#include <cuda_runtime.h>
#include "s2pro/status.h"

int s2p_fso_arch_ok(void) { return 0; }
size_t s2p_fso_weight_fp8_bytes(int N, int K) { (void)N; (void)K; return 0; }
size_t s2p_fso_sfb_bytes(int N, int K) { (void)N; (void)K; return 0; }
size_t s2p_fso_weight_scratch_bytes(int N, int K) { (void)N; (void)K; return 0; }
size_t s2p_fso_act_fp8_bytes(int M, int K) { (void)M; (void)K; return 0; }
size_t s2p_fso_sa_bytes(int M, int K) { (void)M; (void)K; return 0; }
s2p_status s2p_fso_quant_weight_128x128(void* a, void* b, void* c, const void* d,
                                        int N, int K, cudaStream_t s) {
    (void)a; (void)b; (void)c; (void)d; (void)N; (void)K; (void)s;
    return S2P_ERR_UNSUPPORTED;
}
s2p_status s2p_fso_quant_act_1x128_packed(void* a, void* b, const void* c, int M,
                                          int K, cudaStream_t s) {
    (void)a; (void)b; (void)c; (void)M; (void)K; (void)s;
    return S2P_ERR_UNSUPPORTED;
}
s2p_status s2p_fso_gemm_fp8(void* y, const void* a, const void* b, const void* c,
                            const void* d, int M, int N, int K, cudaStream_t s) {
    (void)y; (void)a; (void)b; (void)c; (void)d; (void)M; (void)N; (void)K; (void)s;
    return S2P_ERR_UNSUPPORTED;
}
