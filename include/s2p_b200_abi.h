/* s2pro-b200 — C ABI of the B200-native token loop.
 *
 * This header declares every entry point the shared library exports for the
 * language-model token loop of s2pro-native (slow-AR backbone tick + fast-AR
 * residual loop + sampler + the linear / quantisation / weight-loading calls
 * beneath them).  Names, argument order, struct layouts and status values are
 * binary-compatible with the reference's module contracts, so an object file
 * compiled against the reference's own headers links against this library
 * unchanged.  Each group cites the reference declaration it stands in for
 * (paths relative to the reference project root).
 *
 * Host code is C11; all pointers named *_dev / "device" are CUDA device
 * pointers of the current device; nothing here is thread-safe — exactly one
 * host thread issues GPU work after load, as in the reference.
 */
#ifndef S2P_B200_ABI_H
#define S2P_B200_ABI_H

#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif
/* the library is built with hidden visibility; only what is declared here is exported */
#pragma GCC visibility push(default)

/* ===== status codes — replaces include/s2pro/status.h:10-41 ================ */
typedef enum {
    S2P_OK = 0,
    S2P_ERR_INVALID = -1,     /* argument or precondition */
    S2P_ERR_CUDA = -2,        /* CUDA runtime error */
    S2P_ERR_IO = -3,          /* file I/O */
    S2P_ERR_OOM = -4,         /* host or device allocation */
    S2P_ERR_FORMAT = -5,      /* malformed checkpoint / header */
    S2P_ERR_STATE = -6,       /* lifecycle misuse */
    S2P_ERR_UNSUPPORTED = -7, /* dtype / feature not served */
    S2P_ERR_INTERNAL = -8,    /* invariant broken (incl. a bounded device wait that gave up) */
    S2P_ERR_FULL = -9         /* session capacity exhausted */
} s2p_status;

const char* s2p_status_str(s2p_status s);

#define S2P_TRY(expr)                         \
    do {                                      \
        s2p_status s2p_try_rc_ = (expr);      \
        if (s2p_try_rc_ != S2P_OK) return s2p_try_rc_; \
    } while (0)

#define S2P_CUDA_TRY(expr)                                                        \
    do {                                                                          \
        cudaError_t s2p_try_ce_ = (expr);                                         \
        if (s2p_try_ce_ != cudaSuccess) {                                         \
            fprintf(stderr, "[s2pro] CUDA error %s:%d: %s\n", __FILE__, __LINE__, \
                    cudaGetErrorString(s2p_try_ce_));                             \
            return S2P_ERR_CUDA;                                                  \
        }                                                                         \
    } while (0)

/* ===== model constants — replaces include/s2pro/config.h:16-53 ============= */
#define S2P_SLOW_LAYERS 36 /* layer count of the full model; the loader accepts
                            * checkpoints with fewer backbone layers (see
                            * s2p_b200_ext.h) */
#define S2P_DIM 2560
#define S2P_SLOW_Q_HEADS 32
#define S2P_SLOW_KV_HEADS 8
#define S2P_HEAD_DIM 128
#define S2P_Q_WIDTH 4096
#define S2P_KV_WIDTH 1024
#define S2P_QKV_WIDTH 6144
#define S2P_FFN_DIM 9728
#define S2P_TEXT_VOCAB 155776
#define S2P_ROPE_BASE 1000000.0f
#define S2P_NORM_EPS 1e-6f
#define S2P_MAX_SEQ 32768
#define S2P_CTX_LEN_DEFAULT 4096
#define S2P_FAST_LAYERS 4
#define S2P_CB_SIZE 4096
#define S2P_NUM_CODEBOOKS 10
#define S2P_FAST_SEQ 11
#define S2P_TOK_EOS 151645
#define S2P_TOK_SEMANTIC_START 151678
#define S2P_TOK_SEMANTIC_END 155773
#define S2P_MAX_SESSIONS 16 /* default session capacity when opts give 0 */

/* ===== tensors — replaces include/s2pro/tensor.h:12-43 ===================== */
typedef enum {
    S2P_DT_BF16 = 0, S2P_DT_F32 = 1, S2P_DT_F16 = 2, S2P_DT_I8 = 3,
    S2P_DT_I32 = 4, S2P_DT_I64 = 5, S2P_DT_U8 = 6
} s2p_dtype;

typedef struct {
    void* data;       /* device pointer, or pinned host pointer */
    s2p_dtype dtype;
    int ndim;         /* 1..4 */
    int64_t shape[4];
    size_t bytes;
    int on_device;    /* 1 = device memory */
} s2p_tensor;

size_t s2p_dtype_size(s2p_dtype dt);
int64_t s2p_tensor_numel(const s2p_tensor* t);
s2p_status s2p_tensor_device_alloc(s2p_tensor* t, s2p_dtype dt, int ndim, const int64_t* shape);
s2p_status s2p_tensor_host_alloc(s2p_tensor* t, s2p_dtype dt, int ndim, const int64_t* shape);
s2p_status s2p_tensor_upload(s2p_tensor* dev_dst, const void* host_src, size_t bytes, cudaStream_t stream);
s2p_status s2p_tensor_download(void* host_dst, const s2p_tensor* dev_src, size_t bytes, cudaStream_t stream);
void s2p_tensor_free(s2p_tensor* t);

/* ===== weight loader — replaces include/s2pro/safetensors.h:17-38 ==========
 * A directory holds model.safetensors, or shards named by
 * model.safetensors.index.json.  Views stay valid until close. */
typedef struct s2p_st s2p_st;
typedef struct {
    const char* name;
    s2p_dtype dtype;
    int ndim;
    int64_t shape[4];
    const void* data; /* host pointer into the mapped file */
    size_t nbytes;
} s2p_st_view;

s2p_status s2p_st_open_dir(const char* model_dir, s2p_st** out);
s2p_status s2p_st_find(s2p_st* st, const char* name, s2p_st_view* out);
int s2p_st_count(const s2p_st* st);
s2p_status s2p_st_at(const s2p_st* st, int index, s2p_st_view* out);
void s2p_st_close(s2p_st* st);
/* find + check dtype/shape (-1 = any) + upload into a fresh device tensor */
s2p_status s2p_st_load_device(s2p_st* st, const char* name, s2p_dtype expect_dt, int ndim,
                              const int64_t* expect_shape, s2p_tensor* out_dev, cudaStream_t stream);

/* ===== linear layers and quantisation — replaces include/s2pro/gemm.h:21-140
 * Row-major x [M,in], w [out,in], y [M,out] = x w^T; bf16 activations, f32
 * accumulation. */
typedef enum {
    S2P_GEMM_BF16 = 0,
    S2P_GEMM_FP8 = 1, /* not served: the FP8 shim is outside the reference tree; requests fall back to BF16 */
    S2P_GEMM_INT8 = 2 /* weight-only INT8 per channel, or group-wise INT4 under S2P_INT4 */
} s2p_gemm_mode;

#define S2P_INT8_GEMV_MAX_M 16

s2p_status s2p_gemm_init(int max_m);
void s2p_gemm_shutdown(void);
s2p_gemm_mode s2p_gemm_mode_from_env(void); /* S2P_INT8=1 -> INT8, else BF16 */
int s2p_fso_available(void);                /* always 0 here */

typedef struct {
    int in_features;
    int out_features;
    s2p_tensor w_bf16;   /* [out,in] bf16; released by prepare_int8 unless S2P_INT8_KEEP_BF16=1 */
    s2p_tensor w_fp8;    /* unused (FP8 not served) */
    s2p_tensor w_scales; /* unused */
    int fp8_ready;
    s2p_tensor w_int8;   /* [out,in] int8 (absent when q_packed) */
    s2p_tensor w_iscale; /* q_group==0: f32 [out]; else f16 [out, in/q_group] */
    s2p_tensor w_pack;   /* [out,in/2] nibbles, low nibble = even column */
    int int8_ready;
    int q_group;
    int q_packed;
} s2p_linear;

typedef enum { S2P_QSITE_BACKBONE = 0, S2P_QSITE_FASTAR = 1 } s2p_qsite;

s2p_status s2p_linear_from_st(s2p_linear* lin, s2p_st* st, const char* name, int in_features,
                              int out_features, cudaStream_t stream);
s2p_status s2p_linear_prepare_fp8(s2p_linear* lin, cudaStream_t stream); /* logs, leaves the layer BF16 */
s2p_status s2p_linear_prepare_int8(s2p_linear* lin, cudaStream_t stream);
s2p_status s2p_linear_prepare_int8_site(s2p_linear* lin, s2p_qsite site, cudaStream_t stream);
s2p_status s2p_linear_forward(const s2p_linear* lin, const void* x_bf16, void* y_bf16, int M,
                              s2p_gemm_mode mode, cudaStream_t stream);
void s2p_linear_free(s2p_linear* lin);
s2p_status s2p_gemm_bf16(const void* x, const void* w, void* y, int M, int N, int K, cudaStream_t stream);

/* raw per-channel INT8 (gemm.h:84-103) */
s2p_status s2p_int8_quant(void* w_i8, float* scales, const void* w_bf16, int N, int K, cudaStream_t stream);
s2p_status s2p_int8_gemv(void* y_bf16, const void* x_bf16, const void* w_i8, const float* scales,
                         int M, int N, int K, cudaStream_t stream);
s2p_status s2p_int8_dequant(void* w_bf16, const void* w_i8, const float* scales, int N, int K, cudaStream_t stream);
/* raw group-wise low-bit on an int8 container (gemm.h:105-121); scales are f16 */
s2p_status s2p_intq_quant(void* w_i8, void* scales_f16, const void* w_bf16, int N, int K, int G,
                          int levels, int mse, cudaStream_t stream);
s2p_status s2p_intq_gemv(void* y_bf16, const void* x_bf16, const void* w_i8, const void* scales_f16,
                         int M, int N, int K, int G, cudaStream_t stream);
s2p_status s2p_intq_dequant(void* w_bf16, const void* w_i8, const void* scales_f16, int N, int K, int G,
                            cudaStream_t stream);
/* packed 4-bit storage (gemm.h:123-140) */
s2p_status s2p_int4_pack(void* w_pack, const void* w_i8, int N, int K, cudaStream_t stream);
s2p_status s2p_int4p_gemv(void* y_bf16, const void* x_bf16, const void* w_pack, const void* scales_f16,
                          int M, int N, int K, int G, cudaStream_t stream);
s2p_status s2p_int4p_dequant(void* w_bf16, const void* w_pack, const void* scales_f16, int N, int K, int G,
                             cudaStream_t stream);

/* ===== prequantised-weight sidecar — replaces include/s2pro/qcache.h:34-54 == */
typedef struct s2p_qcache s2p_qcache;
s2p_status s2p_qcache_open(const char* model_dir, s2p_gemm_mode mode, s2p_qcache** out);
int s2p_qcache_reading(const s2p_qcache* qc);
int s2p_qcache_try_load(s2p_qcache* qc, const char* name, int in_features, int out_features,
                        s2p_linear* lin, cudaStream_t stream);
s2p_status s2p_qcache_put_linear(s2p_qcache* qc, const char* name, const s2p_linear* lin, cudaStream_t stream);
s2p_status s2p_qcache_finish(s2p_qcache* qc, cudaStream_t stream);
void s2p_qcache_free(s2p_qcache* qc);

/* ===== primitive launchers — replaces include/s2pro/kernels.h:20-70 ========
 * bf16 pointers are passed as uint16_t* here (the reference names
 * __nv_bfloat16, a 2-byte POD: identical ABI).  Each returns the launch's
 * cudaError_t. */
typedef uint16_t s2p_bf16;
cudaError_t s2pk_rms_norm(const s2p_bf16* x, const s2p_bf16* w, s2p_bf16* y, int rows, int width,
                          float eps, cudaStream_t st);
cudaError_t s2pk_qk_norm(s2p_bf16* qk, const s2p_bf16* w, int rows, int heads, int head_dim, float eps,
                         cudaStream_t st);
cudaError_t s2pk_rope(s2p_bf16* q, s2p_bf16* k, int rows, int q_heads, int kv_heads, int head_dim,
                      int pos, float rope_base, cudaStream_t st);
cudaError_t s2pk_kv_append(const s2p_bf16* k, const s2p_bf16* v, s2p_bf16* k_cache, s2p_bf16* v_cache,
                           int rows, int kv_heads, int head_dim, int pos, int max_seq, cudaStream_t st);
cudaError_t s2pk_attention(const s2p_bf16* q, const s2p_bf16* k_cache, const s2p_bf16* v_cache,
                           s2p_bf16* out, int rows, int q_heads, int kv_heads, int head_dim, int pos,
                           int max_seq, cudaStream_t st);
cudaError_t s2pk_silu_mul(const s2p_bf16* gu, s2p_bf16* h, int rows, int ffn, cudaStream_t st);
cudaError_t s2pk_add(s2p_bf16* y, const s2p_bf16* x, int64_t n, cudaStream_t st);
cudaError_t s2pk_embed(const s2p_bf16* table, const int64_t* ids, s2p_bf16* out, int rows, int dim,
                       cudaStream_t st);
cudaError_t s2pk_sample_prepare(const s2p_bf16* logits, float* scratch, int vocab, cudaStream_t st);
cudaError_t s2pk_argmax(const s2p_bf16* logits, int32_t* ids, int rows, int vocab, cudaStream_t st);

/* ===== model and sessions — replaces include/s2pro/model.h:28-76 =========== */
typedef struct s2p_model s2p_model;
typedef struct s2p_session s2p_session;

typedef struct {
    s2p_gemm_mode gemm_mode;
    int ctx_len;      /* 0 -> S2P_CTX_LEN_DEFAULT */
    int max_sessions; /* 0 -> S2P_MAX_SESSIONS */
} s2p_model_opts;

typedef struct {
    float temperature; /* 0 -> greedy */
    float top_p;
    float repetition_penalty;
    int repetition_window;
    uint64_t seed; /* 0 -> unseeded */
} s2p_sampling_cfg;

/* One reference clip for VQ injection, codebook-major codes[cb*T + t]
 * (include/s2pro/tokenizer.h:24-28). */
typedef struct {
    const int32_t* codes;
    int T;
} s2p_vq_part;

s2p_sampling_cfg s2p_sampling_defaults(void);

s2p_status s2p_model_load(const char* model_dir, const s2p_model_opts* opts, s2p_model** out);
void s2p_model_free(s2p_model* m);

s2p_status s2p_session_create(s2p_model* m, const s2p_sampling_cfg* cfg, s2p_session** out);
s2p_status s2p_session_prefill(s2p_session* s, const int64_t* ids, const uint8_t* vq_mask, int n_ids,
                               const s2p_vq_part* parts, int n_parts);
size_t s2p_session_kv_bytes(const s2p_model* m, int n_tokens);
s2p_status s2p_session_kv_save(s2p_session* s, int n_tokens, void* blob_dev);
s2p_status s2p_session_kv_load(s2p_session* s, const void* blob_dev, int n_tokens);
s2p_status s2p_session_next_frame(s2p_session* s, int32_t out_codes[S2P_NUM_CODEBOOKS], int* is_eos);
void s2p_session_destroy(s2p_session* s);
s2p_status s2p_model_batch_next_frame(s2p_model* m, s2p_session** sess, int n, int32_t* out_codes, int* eos);

#pragma GCC visibility pop
#ifdef __cplusplus
}
#endif
#endif /* S2P_B200_ABI_H */
