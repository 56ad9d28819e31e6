/* s2pro-b200 — additive entry points that have no counterpart in the
 * reference's headers.  Everything the reference's callers use is in
 * s2p_b200_abi.h; a drop-in build never needs this file. */
#ifndef S2P_B200_EXT_H
#define S2P_B200_EXT_H

#include "s2p_b200_abi.h"

#ifdef __cplusplus
extern "C" {
#endif
/* the library is built with hidden visibility; only what is declared here is exported */
#pragma GCC visibility push(default)

/* Library identification: "s2pro-b200 <version> sm_100a". */
const char* s2p_b200_version(void);

/* Measurement hooks (no counterpart in the reference). */
typedef struct {
    uint64_t frames_decoded;        /* session-frames produced since load */
    int n_slow_layers;              /* backbone depth found in the checkpoint */
    int last_tick_rows;             /* rows of the most recent tick */
    int last_tick_fused;            /* 1 = batch-1 fused stages, 0 = general sequence */
    int last_tick_graph;            /* 1 = replayed from a captured CUDA graph */
    int last_tick_kernels;          /* kernel launches of the most recent tick */
    float last_tick_device_ms;      /* device time of the most recent tick (events on the model stream) */
    size_t upload_bytes;            /* host->device bytes per tick */
    size_t download_bytes;          /* device->host bytes per tick */
    double weight_bytes_per_frame;  /* quantised weight + scale bytes one batch-1 frame streams */
    double kv_bytes_per_token;      /* KV bytes one session reads per cached token per frame */
    int last_tick_persistent;       /* 1 = the whole tick ran as one persistent cooperative kernel */
} s2p_b200_stats;

s2p_status s2p_b200_model_stats(const s2p_model* m, s2p_b200_stats* out);

/* Stage trace of the persistent tick kernel (no counterpart in the reference).  With
 * S2P_TICK_TRACE=1 in the environment at model load, CTA 0 of every persistent tick
 * records sixteen 64-bit words per stage; this call copies those of the most recent tick:
 * out[16 * stage + w].  Words 0..3 are SM-clock stamps: stage entered, activation staged
 * (GEMV stages; 0 otherwise), own work done, grid barrier passed (or stage left where
 * the stage ends without one).  Words 4..7 are SM-clock sums of thread 0's streaming
 * role (waiting for weight chunks, multiplying) and of fold warp 0 (waiting for
 * partial sums, folding); words 8..15 are the SM clock at which each of the eight
 * streaming warps was through.  types[stage] = stage kind (0 frame start, 1 GEMV,
 * 2 backbone attention, 3 fast-AR attention, 4 sampler, 5 frame end).  *n_stages
 * receives the stage count; at most max_stages stages are written.  S2P_ERR_STATE if
 * tracing is off or no persistent tick has run. */
s2p_status s2p_b200_model_tick_trace(s2p_model* m, uint64_t* out, int32_t* types, int max_stages, int* n_stages);
/* Per-CTA stamps of the same tick, in nanoseconds of the GPU's global timer:
 * fold_done_ns[stage * n_ctas + cta] = the CTA's last output of the stage was published
 * (for stages without a GEMV: the stage body returned), staged_ns[...] = its
 * activation vector of a GEMV stage was staged in shared memory (0 elsewhere).  The
 * difference between the latest fold_done of stage s and a CTA's staged stamp of stage
 * s+1 is the hand-off latency between two GEMV stages.  Both arrays must hold
 * n_stages * n_ctas words (S2P_ERR_INVALID with the two counts filled in otherwise). */
s2p_status s2p_b200_model_tick_trace_ctas(s2p_model* m, uint64_t* fold_done_ns, uint64_t* staged_ns, int max_stages, int max_ctas,
                                          int* n_stages, int* n_ctas);
/* The stream every tick of this model is issued on (for external event timing). */
cudaStream_t s2p_b200_model_stream(s2p_model* m);

/* Tensor-parallel batch-1 decode over 2, 4 or 8 GPUs of one node (no counterpart in the
 * reference, which runs one GPU per process and has no sharded path).  One process per GPU
 * loads the same checkpoint, exports a handle to its exchange arena, receives the handles of
 * all ranks (any transport: the caller exchanges 64-byte blobs), and attaches before creating
 * sessions.  From then on every rank must issue the same API calls with the same arguments in
 * the same order; the persistent tick kernels of the ranks split the rows of every matrix
 * between them, store each stage's outputs into every rank's arena over NVLink and meet at a
 * barrier that spans the ranks.  Every row is still computed by one thread block with the
 * single-GPU arithmetic, so the frames are bit-identical to a single-GPU run.  Each kv head's
 * cache is kept current only on the rank that attends over it.  Consequences, enforced with
 * S2P_ERR_UNSUPPORTED and a message rather than left to produce wrong frames:
 *  - s2p_session_kv_save is refused for a tensor-parallel session (the blob would be incomplete);
 *  - a tick with decoding rows that cannot run as the persistent kernel is refused: more than one
 *    session, or any tick after the persistent kernel was disabled because one of its bounded waits
 *    gave up (that tick returned S2P_ERR_INTERNAL).  The single-GPU fallbacks of an unsharded model
 *    do not exist here.
 * Prefill is replicated on every rank. */
#define S2P_B200_TP_HANDLE_BYTES 64
s2p_status s2p_b200_model_tp_export(s2p_model* m, void* handle_out);
s2p_status s2p_b200_model_tp_attach(s2p_model* m, int rank, int world, const void* handles);

/* Decode attention that never asks the driver for memory.  (No counterpart in the
 * reference: its split-K attention takes a caller-allocated scratch pointer.)
 *
 * Some hosts of this library may not allocate device memory while they run: a
 * real-time audio worker whose tick must never wait on cudaMalloc / cudaFree (both
 * serialise against every stream of the device, the vocoder's included), or an
 * embedding application that gives a plug-in no memory pool of its own.  For them
 * this entry point computes the split-K GQA decode attention of ONE query row —
 * 32 query heads over 8 kv heads of width 128, bf16 cache planes
 * [kv_heads, max_seq, 128], attending positions 0..pos — with its scratch (split
 * partials and arrival counters) in a fixed ~2.1 MB array built into the library.
 * The result equals the library's regular split-K decode attention bit for bit.
 *
 * Limits and rules:
 *  - pos + 1 <= 8192 cached positions; anything larger is refused with S2P_ERR_INVALID
 *    and a message (use the regular path, whose scratch is sized at model load);
 *  - the first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress); make that first call before starting any stream capture;
 *  - all calls share the one array: calls that can overlap on the GPU (different
 *    streams, or two host threads) race — issue them on one stream;
 *  - no cudaMalloc, cudaFree or allocating library routine is called, ever. */
s2p_status s2p_b200_attention_decode_noalloc(const s2p_bf16* q, const s2p_bf16* k_cache, const s2p_bf16* v_cache,
                                             s2p_bf16* out, int q_heads, int kv_heads, int head_dim, int pos,
                                             int max_seq, cudaStream_t stream);

#pragma GCC visibility pop
#ifdef __cplusplus
}
#endif
#endif
