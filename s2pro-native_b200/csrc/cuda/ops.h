/* Internal launch interface between the CUDA translation units and the C11
 * host code.  Everything here is extern "C" with plain pointers so model.c /
 * session.c can call it; none of it is exported from the shared library. */
#ifndef S2P_OPS_H
#define S2P_OPS_H

#include <stdint.h>
#include <cuda_runtime.h>

#ifdef __cplusplus
#include <cuda_bf16.h>
namespace s2p {
extern "C" {
typedef __nv_bfloat16 s2p_dev_bf16;
#else
typedef uint16_t s2p_dev_bf16;
#endif

/* Where the KV planes of row r live.  Payload base of row r is
 * (bases ? bases[r] : base0 + r * row_stride); the K plane [kv_heads, max_seq,
 * 128] starts k_off bytes in, the V plane v_off bytes in.  With an INT8 cache
 * the f16 scale planes [kv_heads, max_seq, 4] are addressed the same way from
 * sbases / sbase0 with ks_off / vs_off. */
typedef struct {
    void* base0; void* const* bases; size_t row_stride, k_off, v_off;
    void* sbase0; void* const* sbases; size_t srow_stride, ks_off, vs_off;
} KvRef;

/* qkv post-processing (see k_qkv_post): per-row cache pointers (decode) or one
 * base pointer + consecutive positions (prefill). */
typedef struct {
    const s2p_dev_bf16* qkv; /* [rows, (q_heads + 2 kv_heads) * 128] */
    s2p_dev_bf16* q;         /* [rows, q_heads * 128] */
    const s2p_dev_bf16* q_norm; /* [128] or NULL (fast-AR) */
    const s2p_dev_bf16* k_norm;
    float eps, rope_base;
    int q_heads, kv_heads, max_seq, kv8;
    int pos0, pos_row_step;
    const int32_t* pos_arr; /* per-row positions, or NULL -> pos0 + row * pos_row_step */
    KvRef kv;
} QkvPostArgs;

typedef struct {
    const s2p_dev_bf16* q; /* [rows, q_heads*128], post norm/rope */
    s2p_dev_bf16* out;
    int q_heads, kv_heads, max_seq, kv8;
    int pos0, pos_row_step;
    const int32_t* pos_arr;
    KvRef kv;
    /* split-K decode only */
    float* part;            /* [rows][q_heads][n_split_slots][130] */
    unsigned int* counters; /* [rows][kv_heads], zero between launches */
    int n_split_slots;      /* ceil(ctx_len / 64) */
    int workers;            /* CTAs per (row, kv head) */
    /* tensor-parallel ticks: the merged output is also stored into the peers' buffers, the same
     * cell out_peer_delta[i] bytes away (i < n_out_peers) */
    int n_out_peers;
    const long long* out_peer_delta;
    /* persistent tick only: when non-zero the merged output is written as flagged 32-bit words
     * (bf16 | out_ll_tag << 16) into `out` taken as a uint32 array */
    int out_ll;
    unsigned out_ll_tag;
    /* Always 128, but passed at run time: the single-pass kernel derives its query
     * scale as rsqrtf((float)head_dim) on the device, as the reference's does
     * (src/slowar/kernels.cu:258); a compile-time 128 would be folded to the
     * correctly rounded constant, which differs from the device result in the last bit. */
    int head_dim;
} AttnArgs;

/* device-resident sampler state; layout of the reference's s2ps_dev_state
 * (src/slowar/slowar_kernels.h:134-142) */
typedef struct {
    int64_t prev[64];
    uint64_t count;
    uint64_t rng[4];
    float temperature, top_p, rep_penalty;
    int32_t window, seeded;
    uint32_t seed31;
    uint32_t pad_;
} SamplerState;

/* A quantised linear as the fused stage kernels see it. */
typedef struct {
    int kind;           /* 0 per-channel INT8, 1 group scale on int8 codes, 2 packed INT4 */
    const void* w;      /* int8 [N,K] or nibbles [N,K/2] */
    const void* scales; /* f32 [N] or f16 [N, K/G] */
    int N, K, gshift;
} LinRef;

/* Where a [K] activation (or residual) vector comes from: a plain vector, or a
 * row of a table selected on the device by an int32 index or by the low word
 * of a packed arg-max key (index = 0xFFFFFFFF - low32). */
typedef struct {
    const s2p_dev_bf16* base;
    const int32_t* index;
    const unsigned long long* key;
} VecRef;

/* fused batch-1 decode stages (tick.cu) */
cudaError_t stage_norm_gemv(const LinRef* lin, const VecRef* x, const s2p_dev_bf16* norm_w, float eps,
                            s2p_dev_bf16* y, cudaStream_t st);
cudaError_t stage_gemv_resid(const LinRef* lin, const s2p_dev_bf16* x, const VecRef* resid, s2p_dev_bf16* dst,
                             cudaStream_t st);
cudaError_t stage_norm_swiglu(const LinRef* lin, const VecRef* x, const s2p_dev_bf16* norm_w, float eps,
                              s2p_dev_bf16* h, cudaStream_t st);
cudaError_t stage_norm_argmax(const LinRef* lin, const s2p_dev_bf16* x, const s2p_dev_bf16* norm_w, float eps,
                              s2p_dev_bf16* logits, unsigned long long* key, cudaStream_t st);
/* decode attention that also does q/k norm, RoPE and the KV append from raw qkv */
cudaError_t stage_attn_decode_prep(const AttnArgs* a, const s2p_dev_bf16* qkv, const s2p_dev_bf16* q_norm,
                                   const s2p_dev_bf16* k_norm, float eps, float rope_base, int rows,
                                   cudaStream_t st);

/* Frame start for `rows` decode rows: x[r] = embedding of the fed-back token
 * (bf16 table, or INT8 sidecar with row scales) plus, where mask[r], the sum of
 * the 10 codebook embeddings of the previous frame's codes, times f32(1/sqrt 11);
 * also clears the 9 arg-max keys of every row. */
typedef struct {
    const s2p_dev_bf16* embed;  /* bf16 table or NULL */
    const int8_t* embed_i8; const float* embed_scale;
    const s2p_dev_bf16* cb_emb; /* [10*4096, 2560] */
    const int64_t* ids; const int32_t* codes /* [rows][10] */; const uint8_t* mask;
    s2p_dev_bf16* x;
    unsigned long long* keys;   /* [rows][9] or NULL */
} TickBeginArgs;
cudaError_t tick_begin(const TickBeginArgs* a, int rows, cudaStream_t st);
/* Frame end: codes[r][1..9] from the arg-max keys (fused path) */
cudaError_t tick_finish_keys(const unsigned long long* keys, int rows, int32_t* codes, cudaStream_t st);

cudaError_t gemv_setup_all(void); /* once per device, before any stream capture */

/* batched decode linear on the tensor cores (skinny.cu): y[M, N] = x[M, K] · W^T, 1 <= M <= 256 */
cudaError_t skinny_gemm_tc(const LinRef* lin, const void* x, int M, void* y, const void* resid, cudaStream_t st);
/* h[M, N / 2] = silu(x · Wg^T) * (x · Wu^T) for W = [Wg | Wu] stacked along N (gate/up linear + SwiGLU in one launch) */
cudaError_t skinny_gemm_tc_swiglu(const LinRef* lin, const void* x, int M, void* h, cudaStream_t st);
/* any M >= 1: prompt slices in blocks of 256 rows, activations pre-tiled (not under stream capture) */
cudaError_t skinny_prefill_tc(const LinRef* lin, const void* x, int M, void* y, cudaStream_t st);
cudaError_t skinny_status(int* out);
cudaError_t skinny_reset(cudaStream_t st);            /* clears the status code and the arrival counters */
cudaError_t skinny_set_wait_ns(unsigned long long ns); /* test hook: deadline of the kernel's bounded waits */
cudaError_t skinny_setup(int max_rows); /* once per device, outside stream capture: scratch for split-K launches */
/* the launch plan for a shape as 10 ints (padding, tiles, split tiles, pieces, threads, slab, ring depths, grid,
 * shared memory), 0 if the shape cannot be served; no CUDA call (CPU tests) */
int skinny_plan_probe(int kind, int N, int K, int M, int scratch_rows, int out[10]);
/* measurement aid: CTAs the split aims at, kernel shape (0: 256 threads / 64-k slabs, 1: 512 / 128, 2: 256 / 128) */
void skinny_tune(int target_ctas, int shape);

/* ---- persistent batch-1 decode tick (mega.cu) --------------------------------
 * The whole frame is one cooperative kernel that walks a list of stages; a grid
 * barrier separates stages unless MEGA_NO_BARRIER is set on the earlier one. */
enum { MEGA_BEGIN = 0, MEGA_GEMV = 1, MEGA_ATTN_SLOW = 2, MEGA_ATTN_FAST = 3, MEGA_SAMPLE = 4, MEGA_FINISH = 5 };
#define MEGA_NO_BARRIER 1
typedef struct {
    int type, flags;
    /* MEGA_GEMV: y = epilogue(W * prologue(x)) */
    LinRef lin;
    int pro, epi;                 /* Prologue / Epilogue of gemv.cuh */
    VecRef x;
    const s2p_dev_bf16* norm_w;
    s2p_dev_bf16* y;
    VecRef resid;
    unsigned long long* key;
    s2p_dev_bf16* normed_out;
    int rows_per_chunk;           /* rows (row pairs with the SwiGLU epilogue) one ring slot holds */
    /* MEGA_ATTN_*: raw qkv in, attention output out */
    const s2p_dev_bf16* qkv;
    const s2p_dev_bf16* q_norm;
    const s2p_dev_bf16* k_norm;
    s2p_dev_bf16* out;
    KvRef kv;
    int pos;                      /* MEGA_ATTN_FAST: position in the fast-AR cache (= pass index) */
    /* Flagged exchange (see mega.cu): the index of the stage that produces this stage's input
     * vector (x for a GEMV, qkv for attention) as flagged words, or -1 when the input is plain
     * bf16 that an earlier grid barrier has published; and what else is flagged. */
    int x_from;
    int io_flags;                 /* MEGA_Y_LL: the output is written as flagged words; MEGA_RESID_LL: the residual is read from them */
    int pad_;                     /* the kernel stages descriptors with 16-byte copies */
} MegaStage;
#define MEGA_Y_LL 1
#define MEGA_RESID_LL 2

/* Ring geometry shared by the kernel and the host code that builds the copy commands. */
#define MEGA_RING_SLOTS 4
#define MEGA_PARTIAL_BUFFERS 2
/* How one CTA's shared memory is cut up; chosen by the host per model (an all-INT4 model
 * stages bf16 activations and has room for larger ring slots than one with INT8 layers). */
typedef struct {
    int x_bytes;     /* staged activation vector */
    int slot_bytes;  /* one ring slot */
    int part_bytes;  /* one buffer of per-tile lane partials */
    int total_bytes; /* dynamic shared memory of the launch */
} MegaLayout;

/* One chunk of weights for the ring: up to four 1-D bulk copies (weight rows and group
 * scales, each for the gate and the up half of a SwiGLU stage) into one slot. */
typedef struct {
    unsigned long long src[4];
    unsigned int bytes[4];    /* 0 = unused; multiples of 16 */
    unsigned int dst_off[4];  /* byte offset inside the slot; multiples of 16 */
} MegaCopyCmd;

/* Rows [row0, row0 + cnt) of a stage's N rows (row pairs with the SwiGLU epilogue) belong
 * to CTA `cta` of `n_cta`; they are cut into n_chunks chunks of rc rows (the last may be
 * shorter), rc <= rows_per_chunk. */
typedef struct { int row0, cnt, rc, n_chunks; } MegaGeom;
#ifdef __CUDACC__
__host__ __device__
#endif
static inline MegaGeom mega_stage_geom(int N, int swiglu, int rows_per_chunk, int cta, int n_cta) {
    MegaGeom g;
    const int units = swiglu ? (N >> 1) : N;
    if ((long long)units * (long long)n_cta <= 0x7fffffffLL) {
        /* the products fit 32 bits for every matrix of the model: unsigned 32-bit divisions, a fraction of the
         * instructions of the 64-bit ones, and this runs at the head of every stage on both warp groups */
        g.row0 = (int)((unsigned)units * (unsigned)cta / (unsigned)n_cta);
        g.cnt = (int)((unsigned)units * (unsigned)(cta + 1) / (unsigned)n_cta) - g.row0;
    } else {
        g.row0 = (int)((long long)units * cta / n_cta);
        g.cnt = (int)((long long)units * (cta + 1) / n_cta) - g.row0;
    }
    g.n_chunks = g.cnt > 0 ? (g.cnt + rows_per_chunk - 1) / rows_per_chunk : 0;
    g.rc = g.n_chunks ? (g.cnt + g.n_chunks - 1) / g.n_chunks : 0;
    return g;
}

typedef struct {
    const MegaStage* stages;      /* device memory */
    int n_stages;
    MegaLayout lay;
    const MegaCopyCmd* cmds;      /* device memory: every CTA's copy commands in program order */
    const int* cmd_start;         /* [n_cta + 1] first command of each CTA */
    /* Tensor parallelism over `tp_world` GPUs (1 = single GPU): the CTAs of all ranks form one
     * grid of tp_world * gridDim.x CTAs for the row partition of every matrix; every output of a
     * stage is stored into the exchange arena of every rank (tp_base[r] is rank r's arena as
     * mapped into this process, tp_base[tp_rank] its own), and the stage barrier counts the CTAs
     * of all ranks.  Every pointer of a stage descriptor that is written points into the own arena. */
    int tp_rank, tp_world;
    unsigned char* tp_base[8];
    unsigned int bar_base;        /* barriers completed by earlier ticks (the counters are never reset) */
    unsigned int seq_base;        /* stages run by earlier ticks: stage i of this tick flags its words with (seq_base + i + 1) & 0xFFFF */
    int logc_from, loge_from;     /* stages that produce the sampler's flagged logits */
    s2p_dev_bf16* logits_plain;   /* [4097] scratch: the sampler's logits unflagged (own CTA only) */
    unsigned int* barrier;        /* arena word counting barrier arrivals of all ranks' CTAs */
    int* status;                  /* device word, zero at launch; non-zero afterwards = a bounded wait gave up */
    TickBeginArgs begin;
    /* slow-AR attention */
    int ctx_len, kv8, n_split_slots;
    const int32_t* pos_arr;
    float* part;
    unsigned int* counters;
    float eps, rope_base;
    int head_dim;
    /* sampler */
    const s2p_dev_bf16* sem_logits; const s2p_dev_bf16* eos_logit;
    SamplerState* const* states;
    int64_t* out_tok; int32_t* out_sem; int32_t* out_codes; uint8_t* out_eos;
    const unsigned long long* keys; /* [9] arg-max keys of the fast-AR steps */
    /* optional per-stage SM-clock stamps of CTA 0: [n_stages][4] = stage entered, activation
     * staged (GEMV), work done, barrier passed */
    unsigned long long* trace;
} MegaParams;

/* bytes of one ring slot; a stage's rows_per_chunk must satisfy
 * rows * regions * (row bytes + scale bytes per row) <= this */
/* layout for a model whose widest staged activation needs x_bytes */
void mega_layout(int x_bytes, MegaLayout* out);
int mega_max_local_rows(const MegaLayout* lay, int K); /* rows of one chunk the fold and the partial buffer can take */
void mega_geom_probe(int N, int swiglu, int rows_per_chunk, int cta, int n_cta, int out[4]);
cudaError_t mega_setup(int* n_cta_out);   /* once per device: attribute + occupancy check; grid size */
/* test hooks: the deadline of the persistent tick's bounded waits on the current device, and a one-CTA kernel
 * that lets a wait nobody will satisfy run out (which: 0 mbarrier, 1 flagged word) */
cudaError_t mega_set_wait_ns(unsigned long long ns);
cudaError_t pipe_wait_probe(int which, unsigned long long limit_ns, int* status_out, unsigned long long* elapsed_ns_out, int* got_out);
cudaError_t mega_launch(const MegaParams* p, int n_cta, cudaStream_t st);

cudaError_t qkv_post(const QkvPostArgs* a, int rows, cudaStream_t st);
cudaError_t attn_single(const AttnArgs* a, int rows, cudaStream_t st);
cudaError_t attn_decode(const AttnArgs* a, int rows, cudaStream_t st);

cudaError_t rms_norm(const void* x, const void* w, void* y, int rows, int width, float eps, cudaStream_t st);
cudaError_t silu_mul(const void* gu, void* h, int rows, int ffn, cudaStream_t st);
cudaError_t add_inplace(void* y, const void* x, int64_t n, cudaStream_t st);
cudaError_t embed_rows(const void* table, const int64_t* ids, void* out, int rows, int dim, cudaStream_t st);
cudaError_t embed_rows_i8(const void* table, const float* scales, const int64_t* ids, void* out, int rows, int dim,
                          cudaStream_t st);
cudaError_t vq_embed_add(const void* cb_table, const int32_t* codes_dev, int T, void* rows, cudaStream_t st);
cudaError_t scale_div(void* x, int64_t n, float divisor, cudaStream_t st);
cudaError_t scale_rows_masked(void* x, const uint8_t* mask, int rows, int dim, float scale, cudaStream_t st);
cudaError_t embed_codes(const void* table, const int32_t* codes, void* out, int rows, cudaStream_t st);
cudaError_t argmax_rows(const void* logits, int32_t* ids, int rows, int vocab, cudaStream_t st);
cudaError_t pack_frame(const int32_t* stage, int rows, int32_t* codes, cudaStream_t st);

/* sampler: semantic logits sem_logits[r*stride + i] (i < 4096) and the EOS logit
 * eos_logits[r*eos_stride]; writes tok/sem/codes[r*10]/eos and updates the states. */
cudaError_t sample_rows(const void* sem_logits, int64_t stride, const void* eos_logits, int64_t eos_stride,
                        SamplerState* const* states, int rows, int64_t* out_tok, int32_t* out_sem,
                        int32_t* out_codes, uint8_t* out_eos, cudaStream_t st);

#ifdef __cplusplus
}  /* extern "C" */
}  /* namespace s2p */
#endif
#endif
