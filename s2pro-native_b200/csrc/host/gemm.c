/* Linear layers of the C ABI: lifecycle, the INT8 / INT4 conversion policy and
 * the forward dispatch (reference contract include/s2pro/gemm.h:37-82;
 * behaviour of src/sched/gemm.c:57-515).
 *
 * Decode-sized calls (M <= 16) go to this library's weight-streaming GEMV
 * kernels.  Larger M (prefill) dequantises the layer into a shared bf16 scratch
 * and calls cuBLAS with exactly the reference's GemmEx arguments, so prefill
 * results track the reference's as closely as a closed library allows.  FP8 is
 * not served (its kernels live outside the reference tree): such requests stay
 * BF16 with a log line, as the reference does on hardware without FP8 support.
 */
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <cublas_v2.h>
#include "internal.h"

static struct {
    int inited;
    cublasHandle_t handle;
    pthread_mutex_t mu;
    void* deq;
    size_t deq_bytes;
} G = {0, NULL, PTHREAD_MUTEX_INITIALIZER, NULL, 0};

s2p_status s2p_gemm_init(int max_m) {
    (void)max_m; /* sizing hint of the reference's FP8 scratch; nothing to size here */
    pthread_mutex_lock(&G.mu);
    s2p_status rc = S2P_OK;
    if (!G.inited) {
        const cublasStatus_t cs = cublasCreate(&G.handle);
        if (cs != CUBLAS_STATUS_SUCCESS) {
            fprintf(stderr, "[s2pro] cublasCreate failed: status %d\n", (int)cs);
            rc = S2P_ERR_CUDA;
        } else {
            G.inited = 1;
        }
    }
    pthread_mutex_unlock(&G.mu);
    return rc;
}

void s2p_gemm_shutdown(void) {
    pthread_mutex_lock(&G.mu);
    if (G.inited) {
        if (G.deq) cudaFree(G.deq);
        G.deq = NULL;
        G.deq_bytes = 0;
        cublasDestroy(G.handle);
        G.handle = NULL;
        G.inited = 0;
    }
    pthread_mutex_unlock(&G.mu);
}

int s2p_env_is_one(const char* name) {
    const char* v = getenv(name);
    return v && v[0] == '1' && v[1] == '\0';
}

static int env_default(const char* name, int def) {
    const char* v = getenv(name);
    return (v && v[0]) ? (v[0] == '1' && v[1] == '\0') : def;
}

s2p_gemm_mode s2p_gemm_mode_from_env(void) {
    if (s2p_env_is_one("S2P_INT8")) return S2P_GEMM_INT8;
    if (s2p_env_is_one("S2P_FP8"))
        fprintf(stderr, "[s2pro] S2P_FP8=1 but FP8 path unavailable — using BF16\n");
    return S2P_GEMM_BF16;
}

int s2p_fso_available(void) { return 0; }

/* y[M,N] = x[M,K] w[N,K]^T through cuBLAS: column-major view, op(T) on w
 * (src/sched/gemm.c:114-129).  Caller holds G.mu. */
static s2p_status cublas_xwT(const void* x, const void* w, void* y, int M, int N, int K, cudaStream_t stream) {
    const float alpha = 1.0f, beta = 0.0f;
    cublasStatus_t cs = cublasSetStream(G.handle, stream);
    if (cs == CUBLAS_STATUS_SUCCESS)
        cs = cublasGemmEx(G.handle, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha, w, CUDA_R_16BF, K, x, CUDA_R_16BF, K,
                          &beta, y, CUDA_R_16BF, N, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    if (cs != CUBLAS_STATUS_SUCCESS) {
        fprintf(stderr, "[s2pro] cublasGemmEx(M=%d,N=%d,K=%d) failed: %d\n", M, N, K, (int)cs);
        return S2P_ERR_CUDA;
    }
    return S2P_OK;
}

s2p_status s2p_gemm_bf16(const void* x, const void* w, void* y, int M, int N, int K, cudaStream_t stream) {
    if (!x || !w || !y || M <= 0 || N <= 0 || K <= 0) return S2P_ERR_INVALID;
    if (!G.inited) return S2P_ERR_STATE;
    pthread_mutex_lock(&G.mu);
    const s2p_status rc = cublas_xwT(x, w, y, M, N, K, stream);
    pthread_mutex_unlock(&G.mu);
    return rc;
}

s2p_status s2p_linear_from_st(s2p_linear* lin, s2p_st* st, const char* name, int in_features, int out_features,
                              cudaStream_t stream) {
    if (!lin || !st || !name || in_features <= 0 || out_features <= 0) return S2P_ERR_INVALID;
    memset(lin, 0, sizeof(*lin));
    lin->in_features = in_features;
    lin->out_features = out_features;
    const int64_t shape[2] = {out_features, in_features};
    return s2p_st_load_device(st, name, S2P_DT_BF16, 2, shape, &lin->w_bf16, stream);
}

s2p_status s2p_linear_prepare_fp8(s2p_linear* lin, cudaStream_t stream) {
    (void)stream;
    if (!lin || !lin->w_bf16.data) return S2P_ERR_INVALID;
    fprintf(stderr, "[s2pro] fp8 prepare [%d,%d]: FP8 path unavailable, layer stays BF16\n", lin->out_features,
            lin->in_features);
    return S2P_OK;
}

/* INT4 policy of src/sched/gemm.c:228-265: S2P_INT4=1 moves backbone linears to
 * group-wise 4-bit; the fast-AR follows only under S2P_INT4_ALL=1. */
static int int4_group(void) {
    const char* v = getenv("S2P_INT4_GROUP");
    int g = v ? atoi(v) : 32;
    if (g < 16 || g > 512 || (g & (g - 1))) {
        fprintf(stderr, "[s2pro] S2P_INT4_GROUP=%s invalid, using 32\n", v ? v : "");
        g = 32;
    }
    return g;
}
static int int4_for_site(s2p_qsite site) {
    if (!s2p_env_is_one("S2P_INT4")) return 0;
    return site == S2P_QSITE_FASTAR ? s2p_env_is_one("S2P_INT4_ALL") : 1;
}

static s2p_status sync_stream(cudaStream_t stream, const char* what) {
    const cudaError_t ce = cudaStreamSynchronize(stream);
    if (ce == cudaSuccess) return S2P_OK;
    fprintf(stderr, "[s2pro] %s sync: %s\n", what, cudaGetErrorString(ce));
    return S2P_ERR_CUDA;
}

s2p_status s2p_linear_prepare_int8(s2p_linear* lin, cudaStream_t stream) {
    if (!lin) return S2P_ERR_INVALID;
    if (lin->int8_ready) return S2P_OK;
    if (!lin->w_bf16.data) return S2P_ERR_INVALID;
    const int N = lin->out_features, K = lin->in_features;
    if (K % 512 != 0) {
        fprintf(stderr, "[s2pro] int8 prepare [%d,%d]: K %% 512 != 0, layer stays BF16\n", N, K);
        return S2P_OK;
    }
    const int64_t qshape[2] = {N, K}, sshape[1] = {N};
    S2P_TRY(s2p_tensor_device_alloc(&lin->w_int8, S2P_DT_I8, 2, qshape));
    s2p_status rc = s2p_tensor_device_alloc(&lin->w_iscale, S2P_DT_F32, 1, sshape);
    if (rc == S2P_OK) rc = s2p_int8_quant(lin->w_int8.data, (float*)lin->w_iscale.data, lin->w_bf16.data, N, K, stream);
    if (rc == S2P_OK) rc = sync_stream(stream, "int8 prepare"); /* the bf16 source is released next */
    if (rc != S2P_OK) {
        s2p_tensor_free(&lin->w_int8);
        s2p_tensor_free(&lin->w_iscale);
        return rc;
    }
    lin->int8_ready = 1;
    if (!s2p_env_is_one("S2P_INT8_KEEP_BF16")) s2p_tensor_free(&lin->w_bf16);
    return S2P_OK;
}

static s2p_status prepare_int4(s2p_linear* lin, cudaStream_t stream) {
    if (!lin) return S2P_ERR_INVALID;
    if (lin->int8_ready) return S2P_OK;
    if (!lin->w_bf16.data) return S2P_ERR_INVALID;
    const int N = lin->out_features, K = lin->in_features, Gq = int4_group();
    if (K % 512 != 0 || K % Gq != 0) {
        fprintf(stderr, "[s2pro] int4 prepare [%d,%d]: shape not servable (K %% 512 or K %% %d), layer stays BF16\n", N,
                K, Gq);
        return S2P_OK;
    }
    const int64_t qshape[2] = {N, K}, sshape[1] = {(int64_t)N * (K / Gq)};
    S2P_TRY(s2p_tensor_device_alloc(&lin->w_int8, S2P_DT_I8, 2, qshape));
    s2p_status rc = s2p_tensor_device_alloc(&lin->w_iscale, S2P_DT_F16, 1, sshape);
    if (rc == S2P_OK)
        rc = s2p_intq_quant(lin->w_int8.data, lin->w_iscale.data, lin->w_bf16.data, N, K, Gq, 7,
                            env_default("S2P_INT4_MSE", 1), stream);
    if (rc == S2P_OK && env_default("S2P_INT4_PACKED", 1)) {
        const int64_t pshape[2] = {N, K / 2};
        rc = s2p_tensor_device_alloc(&lin->w_pack, S2P_DT_I8, 2, pshape);
        if (rc == S2P_OK) rc = s2p_int4_pack(lin->w_pack.data, lin->w_int8.data, N, K, stream);
        if (rc == S2P_OK) rc = sync_stream(stream, "int4 pack");
        if (rc == S2P_OK) {
            s2p_tensor_free(&lin->w_int8); /* the nibbles replace the container */
            lin->q_packed = 1;
        }
    }
    if (rc == S2P_OK) rc = sync_stream(stream, "int4 prepare");
    if (rc != S2P_OK) {
        s2p_tensor_free(&lin->w_int8);
        s2p_tensor_free(&lin->w_iscale);
        s2p_tensor_free(&lin->w_pack);
        lin->q_packed = 0;
        return rc;
    }
    lin->int8_ready = 1;
    lin->q_group = Gq;
    if (!s2p_env_is_one("S2P_INT8_KEEP_BF16")) s2p_tensor_free(&lin->w_bf16);
    return S2P_OK;
}

s2p_status s2p_linear_prepare_int8_site(s2p_linear* lin, s2p_qsite site, cudaStream_t stream) {
    static int banner = 0;
    if (int4_for_site(site)) {
        if (!banner) {
            banner = 1;
            fprintf(stderr, "[s2pro] S2P_INT4=1: group-wise 4-bit weights (g=%d, mse=%d, fastar=%s, %s)\n", int4_group(),
                    env_default("S2P_INT4_MSE", 1), s2p_env_is_one("S2P_INT4_ALL") ? "int4" : "int8",
                    env_default("S2P_INT4_PACKED", 1) ? "packed" : "int8 container");
        }
        return prepare_int4(lin, stream);
    }
    return s2p_linear_prepare_int8(lin, stream);
}

/* GEMV for decode-sized M of any count: rows are independent products, so M > 16
 * is served in slices of 16 with results identical to one-row calls. */
/* the tensor-core kernel copies the group scales of 256 k at a time, as 4 to 32 aligned bytes */
static int tc_scales_ok(const s2p_linear* lin) {
    const int g = lin->q_group;
    if (!g) return 1;
    return g >= (lin->q_packed ? 32 : 16) && g <= 128 && !(g & (g - 1));
}

/* set once a launch of the tensor-core kernel gave up on a wait: batched linears take the exact-order
 * kernel from then on, as with S2P_NO_TC=1 */
static int g_tc_disabled = 0;
void s2p_linear_tc_disable(void) { g_tc_disabled = 1; }

/* 1 when M decode rows of this linear go to the tensor-core kernel */
int s2p_linear_rows_on_tc(const s2p_linear* lin, int M) {
    if (g_tc_disabled) return 0;
    const int K = lin->in_features;
    static int tc_min_rows = 0;
    if (!tc_min_rows) {
        const char* e = getenv("S2P_TC_MIN_ROWS");
        const int v = e ? atoi(e) : 0;
        tc_min_rows = (v >= 2 && v <= S2P_INT8_GEMV_MAX_M) ? v : S2P_INT8_GEMV_MAX_M + 1;
    }
    return M >= tc_min_rows && M <= 256 && K % 256 == 0 && !s2p_env_is_one("S2P_NO_TC") &&
           tc_scales_ok(lin);
}

/* y += x · Wᵀ in one launch (the residual add of a decode layer fused into the batched linear); only
 * where s2p_linear_rows_on_tc says so */
s2p_status s2p_linear_tc_add(const s2p_linear* lin, const void* x_bf16, void* y_inout_bf16, int M, cudaStream_t stream) {
    LinRef lr;
    s2p_lin_ref(lin, &lr);
    const cudaError_t ce = skinny_gemm_tc(&lr, x_bf16, M, y_inout_bf16, y_inout_bf16, stream);
    if (ce != cudaSuccess) {
        fprintf(stderr, "[s2pro] batched tensor-core linear (M=%d,N=%d,K=%d): %s\n", M, lin->out_features, lin->in_features,
                cudaGetErrorString(ce));
        return S2P_ERR_CUDA;
    }
    return S2P_OK;
}

/* h = silu(x · Wgᵀ) * (x · Wuᵀ) for a stacked [gate | up] linear in one launch; only where
 * s2p_linear_rows_on_tc says so */
s2p_status s2p_linear_tc_swiglu(const s2p_linear* lin, const void* x_bf16, void* h_bf16, int M, cudaStream_t stream) {
    LinRef lr;
    s2p_lin_ref(lin, &lr);
    const cudaError_t ce = skinny_gemm_tc_swiglu(&lr, x_bf16, M, h_bf16, stream);
    if (ce != cudaSuccess) {
        fprintf(stderr, "[s2pro] batched tensor-core linear + SwiGLU (M=%d,N=%d,K=%d): %s\n", M, lin->out_features,
                lin->in_features, cudaGetErrorString(ce));
        return S2P_ERR_CUDA;
    }
    return S2P_OK;
}

s2p_status s2p_linear_gemv_rows(const s2p_linear* lin, const void* x_bf16, void* y_bf16, int M, cudaStream_t stream) {
    const int N = lin->out_features, K = lin->in_features;
    /* beyond the reference's 16-row GEMV the batch goes to the tensor cores in one launch
     * (S2P_NO_TC=1 keeps the exact-order kernel, 16 rows at a time; S2P_TC_MIN_ROWS=n, 2 <= n <= 16,
     * sends batches of n rows and more there too, giving up bit-equality with the reference's
     * batched GEMV for them) */
    if (s2p_linear_rows_on_tc(lin, M)) {
        LinRef lr;
        s2p_lin_ref(lin, &lr);
        const cudaError_t ce = skinny_gemm_tc(&lr, x_bf16, M, y_bf16, NULL, stream);
        if (ce != cudaSuccess) {
            fprintf(stderr, "[s2pro] batched tensor-core linear (M=%d,N=%d,K=%d): %s\n", M, N, K, cudaGetErrorString(ce));
            return S2P_ERR_CUDA;
        }
        return S2P_OK;
    }
    for (int m0 = 0; m0 < M; m0 += S2P_INT8_GEMV_MAX_M) {
        const int mm = M - m0 < S2P_INT8_GEMV_MAX_M ? M - m0 : S2P_INT8_GEMV_MAX_M;
        const char* xs = (const char*)x_bf16 + (size_t)m0 * K * 2;
        char* ys = (char*)y_bf16 + (size_t)m0 * N * 2;
        s2p_status rc;
        if (lin->q_packed) rc = s2p_int4p_gemv(ys, xs, lin->w_pack.data, lin->w_iscale.data, mm, N, K, lin->q_group, stream);
        else if (lin->q_group > 0) rc = s2p_intq_gemv(ys, xs, lin->w_int8.data, lin->w_iscale.data, mm, N, K, lin->q_group, stream);
        else rc = s2p_int8_gemv(ys, xs, lin->w_int8.data, (const float*)lin->w_iscale.data, mm, N, K, stream);
        if (rc != S2P_OK) return rc;
    }
    return S2P_OK;
}

s2p_status s2p_linear_forward(const s2p_linear* lin, const void* x_bf16, void* y_bf16, int M, s2p_gemm_mode mode,
                              cudaStream_t stream) {
    if (!lin || !x_bf16 || !y_bf16 || M <= 0) return S2P_ERR_INVALID;
    if (!G.inited) return S2P_ERR_STATE;
    const int N = lin->out_features, K = lin->in_features;
    if (mode == S2P_GEMM_INT8 && lin->int8_ready) {
        if (M <= S2P_INT8_GEMV_MAX_M) return s2p_linear_gemv_rows(lin, x_bf16, y_bf16, M, stream);
        /* S2P_PREFILL_TC=1 (the reference's switch, src/sched/gemm.c:458-466, off by default there and here
         * because the summation order differs from cuBLAS): prompt slices of any length go to the tensor
         * cores straight from the quantised weights, no bf16 copy of the layer is written or read. */
        if (s2p_env_is_one("S2P_PREFILL_TC") && !g_tc_disabled && K % 256 == 0 && tc_scales_ok(lin)) {
            LinRef lr;
            s2p_lin_ref(lin, &lr);
            const cudaError_t ce = skinny_prefill_tc(&lr, x_bf16, M, y_bf16, stream);
            if (ce != cudaSuccess) {
                fprintf(stderr, "[s2pro] tensor-core prefill linear (M=%d,N=%d,K=%d): %s\n", M, N, K, cudaGetErrorString(ce));
                return S2P_ERR_CUDA;
            }
            return S2P_OK;
        }
        /* prefill-sized M: dequantise the whole layer, then the library GEMM; the lock
         * spans both so a concurrent caller cannot resize the scratch underneath */
        pthread_mutex_lock(&G.mu);
        s2p_status rc = S2P_OK;
        const size_t need = (size_t)N * K * 2;
        if (need > G.deq_bytes) {
            if (cudaStreamSynchronize(stream) != cudaSuccess) rc = S2P_ERR_CUDA;
            if (G.deq) cudaFree(G.deq);
            G.deq = NULL;
            G.deq_bytes = 0;
            if (rc == S2P_OK && cudaMalloc(&G.deq, need) != cudaSuccess) rc = S2P_ERR_OOM;
            if (rc == S2P_OK) G.deq_bytes = need;
        }
        if (rc == S2P_OK) {
            if (lin->q_packed) rc = s2p_int4p_dequant(G.deq, lin->w_pack.data, lin->w_iscale.data, N, K, lin->q_group, stream);
            else if (lin->q_group > 0) rc = s2p_intq_dequant(G.deq, lin->w_int8.data, lin->w_iscale.data, N, K, lin->q_group, stream);
            else rc = s2p_int8_dequant(G.deq, lin->w_int8.data, (const float*)lin->w_iscale.data, N, K, stream);
        }
        if (rc == S2P_OK) rc = cublas_xwT(x_bf16, G.deq, y_bf16, M, N, K, stream);
        pthread_mutex_unlock(&G.mu);
        return rc;
    }
    if (!lin->w_bf16.data) {
        fprintf(stderr, "[s2pro] forward without a BF16 copy [N=%d,K=%d] M=%d mode=%d ready=%d\n", N, K, M, (int)mode,
                lin->int8_ready);
        return S2P_ERR_STATE;
    }
    return s2p_gemm_bf16(x_bf16, lin->w_bf16.data, y_bf16, M, N, K, stream);
}

void s2p_linear_free(s2p_linear* lin) {
    if (!lin) return;
    s2p_tensor_free(&lin->w_bf16);
    s2p_tensor_free(&lin->w_fp8);
    s2p_tensor_free(&lin->w_scales);
    s2p_tensor_free(&lin->w_int8);
    s2p_tensor_free(&lin->w_iscale);
    s2p_tensor_free(&lin->w_pack);
    lin->fp8_ready = lin->int8_ready = lin->q_group = lin->q_packed = 0;
}
