/* Private structures of the host side (model, sessions, tick staging). */
#ifndef S2P_INTERNAL_H
#define S2P_INTERNAL_H

#include <stdint.h>
#include "s2p_b200_abi.h"
#include "s2p_b200_ext.h"
#include "../cuda/ops.h"

#define S2P_TP_ARENA_BYTES (256 * 1024)
#define S2P_MAX_BATCH 256 /* cap on lockstep rows / concurrent sessions */
#define S2P_KV_PLANES_PER_LAYER (2 * S2P_SLOW_KV_HEADS)

int s2p_env_is_one(const char* name);
s2p_status s2p_linear_gemv_rows(const s2p_linear* lin, const void* x_bf16, void* y_bf16, int M, cudaStream_t stream);
int s2p_linear_rows_on_tc(const s2p_linear* lin, int M);
void s2p_linear_tc_disable(void);
/* what a tensor-parallel model may do (session.c) */
s2p_status s2p_tp_guard_tick(int tp_world, int decoding_rows, int persistent_path);
s2p_status s2p_tp_guard_kv_save(int tp_world);
s2p_status s2p_linear_tc_add(const s2p_linear* lin, const void* x_bf16, void* y_inout_bf16, int M, cudaStream_t stream);
s2p_status s2p_linear_tc_swiglu(const s2p_linear* lin, const void* x_bf16, void* h_bf16, int M, cudaStream_t stream);

typedef struct {
    s2p_linear wqkv, wo, gate_up, w2;
    s2p_tensor attn_norm, ffn_norm, q_norm, k_norm; /* q/k_norm empty in the fast-AR */
} s2p_layer;

/* host sampler parameters and history mirror (reference: src/slowar/slowar_internal.h:40-55) */
typedef struct {
    float temperature, top_p, rep_penalty;
    int window, seeded;
    uint32_t seed31;
    int64_t prev[64];
    uint64_t count;
    uint64_t rng[4];
} s2p_sampler;
void s2p_sampler_init(s2p_sampler* sp, const s2p_sampling_cfg* cfg, uint64_t entropy);

typedef enum { SESS_NEW = 0, SESS_PREFILLED, SESS_DECODING, SESS_FINISHED } sess_state;

struct s2p_model {
    s2p_gemm_mode mode;
    int kv8, embed_i8_only, head_full;
    int ctx_len, max_sessions, n_sessions;
    int n_slow;        /* backbone layers found in the checkpoint (<= S2P_SLOW_LAYERS) */
    int scratch_rows;  /* prefill row capacity */
    int fused_b1;      /* batch-1 fused stages enabled */
    /* persistent batch-1 tick: stage program in device memory, sync words, grid size */
    int mega_ok, mega_ctas, mega_n_stages, mega_built;
    int mega_barriers;          /* grid barriers of one tick */
    int mega_logc_from, mega_loge_from; /* stages producing the sampler's logits */
    unsigned int mega_ticks;    /* persistent ticks issued so far */
    /* exchange arena (all buffers the persistent tick writes) and its mappings on the ranks of a
     * tensor-parallel group; tp_base[tp_rank] == tp_arena */
    void* tp_arena;
    void* tp_base[8];
    int tp_rank, tp_world;
    MegaLayout mega_lay;
    MegaStage* d_mega_stages;
    MegaCopyCmd* d_mega_cmds;   /* every CTA's weight-copy commands */
    int* d_mega_cmd_start;
    unsigned int* d_mega_sync;  /* [0] grid-barrier counter, [1] status */
    int* h_mega_status;         /* pinned copy of the status word */
    unsigned long long* d_mega_trace; /* [stages][4] clock stamps, when S2P_TICK_TRACE=1 */
    int32_t* mega_types;        /* host copy of the stage kinds */
    cudaStream_t stream;

    /* weights */
    s2p_tensor embed, embed_i8, embed_scale;
    s2p_layer slow[S2P_SLOW_LAYERS];
    s2p_tensor final_norm;
    s2p_layer fast[S2P_FAST_LAYERS];
    s2p_tensor fast_norm, cb_emb, fast_emb;
    s2p_linear fast_out;

    /* activation scratch: rows = max(scratch_rows, max_sessions) */
    s2p_tensor sx, snorm, sqkv, sq, sattn, sproj, sgu, sffn;
    s2p_tensor shidden, slogc, sloge, slogits;
    s2p_tensor sids, svq;
    /* split-K decode attention */
    s2p_tensor attn_part;
    unsigned int* attn_ctr;
    int n_split_slots, attn_workers;
    /* fast-AR workspace */
    s2p_tensor fx, ft, fqkv, fq, fattn, fproj, fgu, fhff, flogits, fkv;
    int32_t* fstage;                /* [9][max_sessions] */
    int32_t* fcodes;                /* [max_sessions] clamped step inputs */
    unsigned long long* fkeys;      /* [max_sessions][9] arg-max keys (fused path) */
    /* per-tick staging */
    size_t up_bytes, off_kvb, off_kvsb, off_samp, off_ids, off_codes, off_pos, off_mask;
    void *d_up, *h_up;
    size_t out_bytes, off_sem, off_ocodes, off_eos;
    void *d_out, *h_out;
    /* one executable graph per steady batch size */
    cudaGraphExec_t gexec[S2P_MAX_BATCH + 1];
    unsigned char gready[S2P_MAX_BATCH + 1];
    uint64_t frames_decoded;
    /* measurement */
    cudaEvent_t ev0, ev1;
    int tick_kernels;                 /* counted while a tick is enqueued or captured */
    int graph_kernels[S2P_MAX_BATCH + 1];
    int last_rows, last_fused, last_graph, last_kernels, last_mega;
    float last_device_ms;
};

struct s2p_session {
    s2p_model* m;
    sess_state state;
    int kv_len;
    s2p_tensor kv;  /* [n_slow][16][ctx][128] bf16 or i8 */
    s2p_tensor kvs; /* kv8: [n_slow][16][ctx][4] f16 */
    s2p_tensor pending_hidden;
    int64_t prev_token;
    int32_t prev_codes[S2P_NUM_CODEBOOKS];
    void* dsamp; /* device SamplerState */
    s2p_sampler sampler;
};

/* model.c helpers used by session.c */
size_t s2p_kv_vec_bytes(const s2p_model* m);
size_t s2p_kv_plane_bytes(const s2p_model* m);  /* one [ctx] plane of payload */
size_t s2p_kvs_plane_bytes(const s2p_model* m); /* one [ctx] plane of scales */
void s2p_lin_ref(const s2p_linear* lin, LinRef* out);

/* S2P_CUDA_TRY for a kernel launch of the tick, counted for the statistics */
#define S2P_LAUNCH(m, expr) do { (m)->tick_kernels++; S2P_CUDA_TRY(expr); } while (0)

#endif
