/* Sessions, prefill, KV-prefix blobs and the lockstep decode tick of the model
 * contract (include/s2pro/model.h:46-76 of the reference; semantics of
 * src/slowar/slowar.c:40-117 sessions, :264-379 prefill, :399-449 KV blobs,
 * :463-606 the device sequence of one tick, :609-826 staging / graph / harvest,
 * and src/fastar/fastar.cu:726-788 the fast-AR frame).
 *
 * Two device sequences produce one frame, with bit-identical results:
 *   - the general one (any number of rows): one launch per operation group,
 *     GEMVs in slices of <= 16 rows;
 *   - the batch-1 one: fused stages (norm -> GEMV, GEMV -> residual,
 *     norm -> GEMV -> SwiGLU, attention with its prologue, head -> arg-max).
 * Either is captured once per batch size into a CUDA graph and replayed; all
 * per-frame variation travels through the pinned upload block.
 */
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include "internal.h"

#define BF(t) ((s2p_dev_bf16*)(t).data)
#define FA_KVSZ (S2P_SLOW_KV_HEADS * S2P_FAST_SEQ * S2P_HEAD_DIM)

static const double SQRT11 = 3.3166247903554; /* sqrt(num_codebooks + 1) */

static int is_semantic(int64_t tok) { return tok >= S2P_TOK_SEMANTIC_START && tok <= S2P_TOK_SEMANTIC_END; }

/* ---- parity dump hooks: S2P_DUMP_DIR/<name>.f32, raw little-endian f32
 * (src/slowar/debug_dump.c:15-61) ------------------------------------------ */
static const char* dump_dir(void) {
    static int init = 0;
    static const char* dir = NULL;
    if (!init) {
        dir = getenv("S2P_DUMP_DIR");
        if (dir && !dir[0]) dir = NULL;
        init = 1;
    }
    return dir;
}

static void dump_bf16(const char* name, const void* dev, int64_t n, cudaStream_t st) {
    const char* dir = dump_dir();
    if (!dir) return;
    uint16_t* h = (uint16_t*)malloc((size_t)n * 2);
    float* f = (float*)malloc((size_t)n * 4);
    if (h && f && cudaStreamSynchronize(st) == cudaSuccess &&
        cudaMemcpy(h, dev, (size_t)n * 2, cudaMemcpyDeviceToHost) == cudaSuccess) {
        for (int64_t i = 0; i < n; i++) {
            const uint32_t u = (uint32_t)h[i] << 16;
            memcpy(&f[i], &u, 4);
        }
        char path[1200];
        snprintf(path, sizeof(path), "%s/%s.f32", dir, name);
        FILE* fp = fopen(path, "wb");
        if (fp) {
            fwrite(f, 4, (size_t)n, fp);
            fclose(fp);
        } else {
            fprintf(stderr, "[s2pro] dump: cannot open %s\n", path);
        }
    }
    free(h);
    free(f);
}

/* ---- sessions ---------------------------------------------------------------- */
s2p_status s2p_session_create(s2p_model* m, const s2p_sampling_cfg* cfg, s2p_session** out) {
    if (!m || !out) return S2P_ERR_INVALID;
    *out = NULL;
    if (m->n_sessions >= m->max_sessions) return S2P_ERR_FULL;
    s2p_session* s = (s2p_session*)calloc(1, sizeof(*s));
    if (!s) return S2P_ERR_OOM;
    s->m = m;
    s->state = SESS_NEW;
    const int64_t kv_shape[4] = {m->n_slow, S2P_KV_PLANES_PER_LAYER, m->ctx_len, S2P_HEAD_DIM};
    s2p_status rc = s2p_tensor_device_alloc(&s->kv, m->kv8 ? S2P_DT_I8 : S2P_DT_BF16, 4, kv_shape);
    if (rc == S2P_OK && m->kv8) {
        const int64_t sc_shape[4] = {m->n_slow, S2P_KV_PLANES_PER_LAYER, m->ctx_len, S2P_HEAD_DIM / 32};
        rc = s2p_tensor_device_alloc(&s->kvs, S2P_DT_F16, 4, sc_shape);
    }
    if (rc == S2P_OK) {
        const int64_t h_shape[1] = {S2P_DIM};
        rc = s2p_tensor_device_alloc(&s->pending_hidden, S2P_DT_BF16, 1, h_shape);
    }
    if (rc == S2P_OK) {
        struct timespec ts;
        clock_gettime(CLOCK_MONOTONIC, &ts);
        const uint64_t entropy = ((uint64_t)ts.tv_sec * 1000000000ULL + (uint64_t)ts.tv_nsec) ^ (uint64_t)(uintptr_t)s;
        s2p_sampler_init(&s->sampler, cfg, entropy);
        SamplerState hst;
        memset(&hst, 0, sizeof(hst));
        memcpy(hst.rng, s->sampler.rng, sizeof(hst.rng));
        hst.temperature = s->sampler.temperature;
        hst.top_p = s->sampler.top_p;
        hst.rep_penalty = s->sampler.rep_penalty;
        hst.window = s->sampler.window;
        hst.seeded = s->sampler.seeded;
        hst.seed31 = s->sampler.seed31;
        if (cudaMalloc(&s->dsamp, sizeof(hst)) != cudaSuccess ||
            cudaMemcpy(s->dsamp, &hst, sizeof(hst), cudaMemcpyHostToDevice) != cudaSuccess)
            rc = S2P_ERR_CUDA;
    }
    if (rc != S2P_OK) {
        if (s->dsamp) cudaFree(s->dsamp);
        s2p_tensor_free(&s->kv);
        s2p_tensor_free(&s->kvs);
        s2p_tensor_free(&s->pending_hidden);
        free(s);
        return rc;
    }
    m->n_sessions++;
    *out = s;
    return S2P_OK;
}

void s2p_session_destroy(s2p_session* s) {
    if (!s) return;
    if (s->m) {
        cudaStreamSynchronize(s->m->stream);
        s->m->n_sessions--;
    }
    s2p_tensor_free(&s->kv);
    s2p_tensor_free(&s->kvs);
    s2p_tensor_free(&s->pending_hidden);
    if (s->dsamp) cudaFree(s->dsamp);
    free(s);
}

/* ---- one layer, general sequence ---------------------------------------------- */
typedef struct {
    int rows;
    KvRef kv;       /* k_off/v_off/ks_off/vs_off filled per layer by the caller */
    int max_seq, kv8;
    int pos0, pos_row_step;
    const int32_t* pos_arr;
    int split_k;    /* decode: split-K attention; else the single-pass kernel */
    int decode;     /* decode-sized rows: GEMV in slices instead of the prefill GEMM */
} layer_ctx;

static s2p_status lin_apply(s2p_model* m, const s2p_linear* lin, const void* x, void* y, int rows, int decode) {
    m->tick_kernels += !decode ? 2 : (m->mode == S2P_GEMM_INT8 && lin->int8_ready && s2p_linear_rows_on_tc(lin, rows))
                                         ? 1 : (rows + S2P_INT8_GEMV_MAX_M - 1) / S2P_INT8_GEMV_MAX_M;
    if (decode && m->mode == S2P_GEMM_INT8 && lin->int8_ready) return s2p_linear_gemv_rows(lin, x, y, rows, m->stream);
    return s2p_linear_forward(lin, x, y, rows, m->mode, m->stream);
}

/* CTAs per (row, kv head) of the split-K decode attention: enough CTAs in total (about 2048) that a
 * long context is walked by several workers even when the batch alone would fill the GPU */
/* x += in · Wᵀ: one launch where the batch runs on the tensor cores, else linear into `proj` and the add kernel */
static s2p_status lin_add(s2p_model* m, const s2p_linear* lin, const void* in, void* x, void* proj, int rows, int decode) {
    if (decode && m->mode == S2P_GEMM_INT8 && lin->int8_ready && s2p_linear_rows_on_tc(lin, rows)) {
        m->tick_kernels += 1;
        return s2p_linear_tc_add(lin, in, x, rows, m->stream);
    }
    S2P_TRY(lin_apply(m, lin, in, proj, rows, decode));
    S2P_LAUNCH(m, add_inplace(x, proj, (int64_t)rows * lin->out_features, m->stream));
    return S2P_OK;
}

static int attn_workers_for(int rows) {
    static int forced = -1; /* S2P_ATTN_WORKERS=n (1..16) overrides the choice */
    if (forced < 0) {
        const char* e = getenv("S2P_ATTN_WORKERS");
        const int v = e ? atoi(e) : 0;
        forced = (v >= 1 && v <= 16) ? v : 0;
    }
    if (forced) return forced;
    int w = 2048 / (rows * S2P_SLOW_KV_HEADS);
    return w < 1 ? 1 : (w > 16 ? 16 : w);
}

/* x: residual stream [rows, 2560]; scratch tensors: norm/qkv/q/attn/proj/gu/hff */
static s2p_status layer_general(s2p_model* m, const s2p_layer* L, const layer_ctx* c, s2p_dev_bf16* x,
                                s2p_dev_bf16* norm, s2p_dev_bf16* qkv, s2p_dev_bf16* q, s2p_dev_bf16* attn,
                                s2p_dev_bf16* proj, s2p_dev_bf16* gu, s2p_dev_bf16* hff) {
    cudaStream_t st = m->stream;
    const int rows = c->rows;
    S2P_LAUNCH(m, rms_norm(x, L->attn_norm.data, norm, rows, S2P_DIM, S2P_NORM_EPS, st));
    S2P_TRY(lin_apply(m, &L->wqkv, norm, qkv, rows, c->decode));
    QkvPostArgs qa;
    memset(&qa, 0, sizeof(qa));
    qa.qkv = qkv; qa.q = q;
    qa.q_norm = (const s2p_dev_bf16*)L->q_norm.data; qa.k_norm = (const s2p_dev_bf16*)L->k_norm.data;
    qa.eps = S2P_NORM_EPS; qa.rope_base = S2P_ROPE_BASE;
    qa.q_heads = S2P_SLOW_Q_HEADS; qa.kv_heads = S2P_SLOW_KV_HEADS; qa.max_seq = c->max_seq; qa.kv8 = c->kv8;
    qa.pos0 = c->pos0; qa.pos_row_step = c->pos_row_step; qa.pos_arr = c->pos_arr; qa.kv = c->kv;
    S2P_LAUNCH(m, qkv_post(&qa, rows, st));
    AttnArgs aa;
    memset(&aa, 0, sizeof(aa));
    aa.q = q; aa.out = attn;
    aa.q_heads = S2P_SLOW_Q_HEADS; aa.kv_heads = S2P_SLOW_KV_HEADS; aa.max_seq = c->max_seq; aa.kv8 = c->kv8;
    aa.pos0 = c->pos0; aa.pos_row_step = c->pos_row_step; aa.pos_arr = c->pos_arr; aa.kv = c->kv;
    aa.head_dim = S2P_HEAD_DIM;
    if (c->split_k) {
        aa.part = (float*)m->attn_part.data; aa.counters = m->attn_ctr;
        aa.n_split_slots = m->n_split_slots; aa.workers = attn_workers_for(rows);
        S2P_LAUNCH(m, attn_decode(&aa, rows, st));
    } else {
        S2P_LAUNCH(m, attn_single(&aa, rows, st));
    }
    S2P_TRY(lin_add(m, &L->wo, attn, x, proj, rows, c->decode));
    S2P_LAUNCH(m, rms_norm(x, L->ffn_norm.data, norm, rows, S2P_DIM, S2P_NORM_EPS, st));
    if (c->decode && m->mode == S2P_GEMM_INT8 && L->gate_up.int8_ready && s2p_linear_rows_on_tc(&L->gate_up, rows) &&
        L->gate_up.out_features == 2 * S2P_FFN_DIM) {
        m->tick_kernels += 1; /* gate/up linear and SwiGLU in one launch */
        S2P_TRY(s2p_linear_tc_swiglu(&L->gate_up, norm, hff, rows, st));
    } else {
        S2P_TRY(lin_apply(m, &L->gate_up, norm, gu, rows, c->decode));
        S2P_LAUNCH(m, silu_mul(gu, hff, rows, S2P_FFN_DIM, st));
    }
    S2P_TRY(lin_add(m, &L->w2, hff, x, proj, rows, c->decode));
    return S2P_OK;
}

static void slow_kv_offsets(const s2p_model* m, int layer, KvRef* kv) {
    const size_t plane = s2p_kv_plane_bytes(m), splane = s2p_kvs_plane_bytes(m);
    kv->k_off = (size_t)layer * S2P_KV_PLANES_PER_LAYER * plane;
    kv->v_off = kv->k_off + (size_t)S2P_SLOW_KV_HEADS * plane;
    kv->ks_off = (size_t)layer * S2P_KV_PLANES_PER_LAYER * splane;
    kv->vs_off = kv->ks_off + (size_t)S2P_SLOW_KV_HEADS * splane;
}

static void fast_kv_ref(const s2p_model* m, int layer, KvRef* kv) {
    memset(kv, 0, sizeof(*kv));
    kv->base0 = (char*)m->fkv.data + (size_t)layer * m->max_sessions * 2 * FA_KVSZ * 2;
    kv->row_stride = (size_t)2 * FA_KVSZ * 2;
    kv->k_off = 0;
    kv->v_off = (size_t)FA_KVSZ * 2;
}

/* ---- prefill ------------------------------------------------------------------ */
s2p_status s2p_session_prefill(s2p_session* s, const int64_t* ids, const uint8_t* vq_mask, int n_ids,
                               const s2p_vq_part* parts, int n_parts) {
    if (!s || !ids || n_ids <= 0) return S2P_ERR_INVALID;
    if (n_parts > 0 && (!parts || !vq_mask)) return S2P_ERR_INVALID;
    s2p_model* m = s->m;
    /* NEW, or PREFILLED again: a chunked prompt extends the cache at kv_len and
     * refreshes the pending hidden state (src/slowar/slowar.c:271-278) */
    if (s->state != SESS_NEW && s->state != SESS_PREFILLED) return S2P_ERR_STATE;
    const int pos0 = s->kv_len;
    if (pos0 + n_ids > m->ctx_len - 1) return S2P_ERR_INVALID; /* at least one decode slot must remain */
    if (n_ids > m->scratch_rows) {
        fprintf(stderr, "[s2pro] prefill of %d ids exceeds scratch capacity %d (raise S2P_SCRATCH_ROWS)\n", n_ids,
                m->scratch_rows);
        return S2P_ERR_INVALID;
    }
    for (int i = 0; i < n_ids; i++)
        if (ids[i] < 0 || ids[i] >= S2P_TEXT_VOCAB) return S2P_ERR_INVALID;
    int64_t total_mask = 0, total_t = 0;
    if (vq_mask)
        for (int i = 0; i < n_ids; i++) total_mask += vq_mask[i] ? 1 : 0;
    if (n_parts > 64) return S2P_ERR_INVALID;
    for (int p = 0; p < n_parts; p++) {
        if (!parts[p].codes || parts[p].T <= 0) return S2P_ERR_INVALID;
        for (int64_t j = 0; j < (int64_t)S2P_NUM_CODEBOOKS * parts[p].T; j++)
            if (parts[p].codes[j] < 0 || parts[p].codes[j] >= S2P_CB_SIZE) return S2P_ERR_INVALID;
        total_t += parts[p].T;
    }
    if (total_mask != total_t) return S2P_ERR_INVALID;

    cudaStream_t st = m->stream;
    /* caller buffers are pageable: synchronous copies */
    S2P_CUDA_TRY(cudaMemcpy(m->sids.data, ids, (size_t)n_ids * sizeof(int64_t), cudaMemcpyHostToDevice));
    int part_start[64];
    size_t part_off[64];
    {
        int cur = 0;
        size_t off = 0;
        for (int p = 0; p < n_parts; p++) {
            while (cur < n_ids && !vq_mask[cur]) cur++;
            const int T = parts[p].T;
            if (cur + T > n_ids) return S2P_ERR_INVALID;
            for (int t = 0; t < T; t++)
                if (!vq_mask[cur + t]) return S2P_ERR_INVALID; /* a part must cover one unbroken masked run */
            part_start[p] = cur;
            part_off[p] = off;
            S2P_CUDA_TRY(cudaMemcpy((int32_t*)m->svq.data + off, parts[p].codes,
                                    (size_t)S2P_NUM_CODEBOOKS * T * sizeof(int32_t), cudaMemcpyHostToDevice));
            off += (size_t)S2P_NUM_CODEBOOKS * T;
            cur += T;
        }
    }
    if (m->embed_i8_only)
        S2P_LAUNCH(m, embed_rows_i8(m->embed_i8.data, (const float*)m->embed_scale.data, (const int64_t*)m->sids.data,
                                   m->sx.data, n_ids, S2P_DIM, st));
    else
        S2P_LAUNCH(m, embed_rows(m->embed.data, (const int64_t*)m->sids.data, m->sx.data, n_ids, S2P_DIM, st));
    for (int p = 0; p < n_parts; p++) {
        const int T = parts[p].T;
        s2p_dev_bf16* rows0 = BF(m->sx) + (size_t)part_start[p] * S2P_DIM;
        S2P_LAUNCH(m, vq_embed_add(m->cb_emb.data, (const int32_t*)m->svq.data + part_off[p], T, rows0, st));
        /* prefill DIVIDES by sqrt(11); decode multiplies by the reciprocal (slowar.c:350-353) */
        S2P_LAUNCH(m, scale_div(rows0, (int64_t)T * S2P_DIM, (float)SQRT11, st));
    }

    layer_ctx c;
    memset(&c, 0, sizeof(c));
    c.rows = n_ids;
    c.kv.base0 = s->kv.data;
    c.kv.sbase0 = s->kvs.data;
    c.max_seq = m->ctx_len;
    c.kv8 = m->kv8;
    c.pos0 = pos0;
    c.pos_row_step = 1;
    for (int l = 0; l < m->n_slow; l++) {
        slow_kv_offsets(m, l, &c.kv);
        S2P_TRY(layer_general(m, &m->slow[l], &c, BF(m->sx), BF(m->snorm), BF(m->sqkv), BF(m->sq), BF(m->sattn),
                              BF(m->sproj), BF(m->sgu), BF(m->sffn)));
        if (dump_dir()) {
            char nm[32];
            snprintf(nm, sizeof(nm), "backbone_layer%02d", l);
            dump_bf16(nm, BF(m->sx) + (size_t)(n_ids - 1) * S2P_DIM, S2P_DIM, st);
        }
    }
    /* the final-normed LAST hidden is what frame 0 samples from and what primes the fast-AR */
    S2P_LAUNCH(m, rms_norm(BF(m->sx) + (size_t)(n_ids - 1) * S2P_DIM, m->final_norm.data, s->pending_hidden.data, 1,
                          S2P_DIM, S2P_NORM_EPS, st));
    dump_bf16("backbone_final_norm", s->pending_hidden.data, S2P_DIM, st);
    S2P_CUDA_TRY(cudaStreamSynchronize(st));
    if (n_ids > S2P_INT8_GEMV_MAX_M && m->mode == S2P_GEMM_INT8 && s2p_env_is_one("S2P_PREFILL_TC")) {
        /* the slice's linears ran on the tensor-core kernel: a bounded wait that gave up inside it left a code */
        int sk = 0;
        S2P_CUDA_TRY(skinny_status(&sk));
        if (sk != 0) {
            fprintf(stderr, "[s2pro] tensor-core prefill linear gave up on a bounded wait (code %d); the slice is lost and later "
                            "linears use the other kernels\n", sk);
            S2P_CUDA_TRY(skinny_reset(st));
            s2p_linear_tc_disable();
            return S2P_ERR_INTERNAL;
        }
    }
    s->kv_len = pos0 + n_ids;
    s->state = SESS_PREFILLED;
    return S2P_OK;
}

/* ---- KV prefix blobs: the session's plane order at n_tokens depth, payload
 * planes first, then (INT8 KV) the scale planes -------------------------------- */
size_t s2p_session_kv_bytes(const s2p_model* m, int n_tokens) {
    if (!m || n_tokens <= 0) return 0;
    const size_t planes = (size_t)m->n_slow * S2P_KV_PLANES_PER_LAYER;
    return planes * n_tokens * s2p_kv_vec_bytes(m) + (m->kv8 ? planes * n_tokens * (S2P_HEAD_DIM / 32) * 2 : 0);
}

static s2p_status kv_blob_copy(s2p_session* s, void* blob, int n_tokens, int save) {
    s2p_model* m = s->m;
    const size_t planes = (size_t)m->n_slow * S2P_KV_PLANES_PER_LAYER;
    const size_t width = (size_t)n_tokens * s2p_kv_vec_bytes(m), pitch = s2p_kv_plane_bytes(m);
    if (save)
        S2P_CUDA_TRY(cudaMemcpy2DAsync(blob, width, s->kv.data, pitch, width, planes, cudaMemcpyDeviceToDevice, m->stream));
    else
        S2P_CUDA_TRY(cudaMemcpy2DAsync(s->kv.data, pitch, blob, width, width, planes, cudaMemcpyDeviceToDevice, m->stream));
    if (m->kv8) {
        char* sblob = (char*)blob + planes * width;
        const size_t swidth = (size_t)n_tokens * (S2P_HEAD_DIM / 32) * 2, spitch = s2p_kvs_plane_bytes(m);
        if (save)
            S2P_CUDA_TRY(cudaMemcpy2DAsync(sblob, swidth, s->kvs.data, spitch, swidth, planes, cudaMemcpyDeviceToDevice,
                                           m->stream));
        else
            S2P_CUDA_TRY(cudaMemcpy2DAsync(s->kvs.data, spitch, sblob, swidth, swidth, planes, cudaMemcpyDeviceToDevice,
                                           m->stream));
    }
    S2P_CUDA_TRY(cudaStreamSynchronize(m->stream));
    return S2P_OK;
}

/* What a tensor-parallel model may do.  Each kv head's cache is current only on the rank that attends
 * over it, so a tick with decoding rows is served by the persistent kernel or not at all (the
 * single-GPU paths would attend over heads this rank never wrote), and a cache blob saved here would
 * be incomplete.  Returns S2P_OK or the status the caller hands back. */
s2p_status s2p_tp_guard_tick(int tp_world, int decoding_rows, int persistent_path) {
    if (tp_world > 1 && decoding_rows >= 1 && !persistent_path) return S2P_ERR_UNSUPPORTED;
    return S2P_OK;
}
s2p_status s2p_tp_guard_kv_save(int tp_world) { return tp_world > 1 ? S2P_ERR_UNSUPPORTED : S2P_OK; }

s2p_status s2p_session_kv_save(s2p_session* s, int n_tokens, void* blob_dev) {
    if (!s || !blob_dev || n_tokens <= 0 || n_tokens > s->kv_len) return S2P_ERR_INVALID;
    if (s2p_tp_guard_kv_save(s->m->tp_world) != S2P_OK) {
        fprintf(stderr, "[s2pro] kv_save: a tensor-parallel session's cache is spread over the ranks; not saved\n");
        return S2P_ERR_UNSUPPORTED;
    }
    return kv_blob_copy(s, blob_dev, n_tokens, 1);
}

s2p_status s2p_session_kv_load(s2p_session* s, const void* blob_dev, int n_tokens) {
    if (!s || !blob_dev || n_tokens <= 0) return S2P_ERR_INVALID;
    if (s->state != SESS_NEW || s->kv_len != 0) return S2P_ERR_STATE;
    if (n_tokens > s->m->ctx_len - 1) return S2P_ERR_INVALID;
    S2P_TRY(kv_blob_copy(s, (void*)blob_dev, n_tokens, 0));
    s->kv_len = n_tokens;
    return S2P_OK;
}

/* ---- the decode tick ------------------------------------------------------------ */
typedef struct {
    const int64_t* ids; const int32_t* codes; const int32_t* pos; const uint8_t* mask;
    void* const* kv_bases; void* const* kvs_bases; SamplerState* const* samp;
    int64_t* tok; int32_t* sem; int32_t* ocodes; uint8_t* eos;
} tick_dev;

static void tick_views(const s2p_model* m, tick_dev* d) {
    char* u = (char*)m->d_up;
    d->kv_bases = (void* const*)(u + m->off_kvb);
    d->kvs_bases = (void* const*)(u + m->off_kvsb);
    d->samp = (SamplerState* const*)(u + m->off_samp);
    d->ids = (const int64_t*)(u + m->off_ids);
    d->codes = (const int32_t*)(u + m->off_codes);
    d->pos = (const int32_t*)(u + m->off_pos);
    d->mask = (const uint8_t*)(u + m->off_mask);
    char* o = (char*)m->d_out;
    d->tok = (int64_t*)o;
    d->sem = (int32_t*)(o + m->off_sem);
    d->ocodes = (int32_t*)(o + m->off_ocodes);
    d->eos = (uint8_t*)(o + m->off_eos);
}

static s2p_status tick_begin_rows(s2p_model* m, const tick_dev* d, int bd) {
    TickBeginArgs a;
    memset(&a, 0, sizeof(a));
    if (!m->embed_i8_only) a.embed = (const s2p_dev_bf16*)m->embed.data;
    a.embed_i8 = (const int8_t*)m->embed_i8.data;
    a.embed_scale = (const float*)m->embed_scale.data;
    a.cb_emb = (const s2p_dev_bf16*)m->cb_emb.data;
    a.ids = d->ids; a.codes = d->codes; a.mask = d->mask;
    a.x = BF(m->sx);
    a.keys = m->fkeys;
    S2P_LAUNCH(m, tick_begin(&a, bd, m->stream));
    return S2P_OK;
}

/* tied head + sampler on `nact` final-normed rows of shidden */
static s2p_status head_and_sample(s2p_model* m, const tick_dev* d, int nact, int dump_ok) {
    cudaStream_t st = m->stream;
    const int full = m->head_full;
    if (!full) {
        /* only the 4096 semantic rows and the EOS row of the sidecar can be sampled
         * (src/slowar/slowar.c:519-541) */
        const int8_t* q = (const int8_t*)m->embed_i8.data;
        const float* sc = (const float*)m->embed_scale.data;
        for (int m0 = 0; m0 < nact; m0 += S2P_INT8_GEMV_MAX_M) {
            const int mm = nact - m0 < S2P_INT8_GEMV_MAX_M ? nact - m0 : S2P_INT8_GEMV_MAX_M;
            const char* hh = (const char*)m->shidden.data + (size_t)m0 * S2P_DIM * 2;
            m->tick_kernels += 2;
            S2P_TRY(s2p_int8_gemv((char*)m->slogc.data + (size_t)m0 * 4096 * 2, hh,
                                  q + (size_t)S2P_TOK_SEMANTIC_START * S2P_DIM, sc + S2P_TOK_SEMANTIC_START, mm, 4096,
                                  S2P_DIM, st));
            S2P_TRY(s2p_int8_gemv((char*)m->sloge.data + (size_t)m0 * 2, hh, q + (size_t)S2P_TOK_EOS * S2P_DIM,
                                  sc + S2P_TOK_EOS, mm, 1, S2P_DIM, st));
        }
        S2P_LAUNCH(m, sample_rows(m->slogc.data, 4096, m->sloge.data, 1, d->samp, nact, d->tok, d->sem, d->ocodes,
                                 d->eos, st));
        return S2P_OK;
    }
    if (m->mode == S2P_GEMM_INT8 && m->embed_i8.data) {
        for (int m0 = 0; m0 < nact; m0 += S2P_INT8_GEMV_MAX_M) {
            const int mm = nact - m0 < S2P_INT8_GEMV_MAX_M ? nact - m0 : S2P_INT8_GEMV_MAX_M;
            S2P_TRY(s2p_int8_gemv((char*)m->slogits.data + (size_t)m0 * S2P_TEXT_VOCAB * 2,
                                  (const char*)m->shidden.data + (size_t)m0 * S2P_DIM * 2, m->embed_i8.data,
                                  (const float*)m->embed_scale.data, mm, S2P_TEXT_VOCAB, S2P_DIM, st));
        }
    } else {
        S2P_TRY(s2p_gemm_bf16(m->shidden.data, m->embed.data, m->slogits.data, nact, S2P_TEXT_VOCAB, S2P_DIM, st));
    }
    if (dump_ok && dump_dir() && nact == 1) {
        static int dump_step = 0;
        if (dump_step < 2) dump_bf16(dump_step == 0 ? "prefill_logits" : "step1_logits", m->slogits.data, S2P_TEXT_VOCAB, st);
        dump_step++;
    }
    S2P_LAUNCH(m, sample_rows((const uint16_t*)m->slogits.data + S2P_TOK_SEMANTIC_START, S2P_TEXT_VOCAB,
                             (const uint16_t*)m->slogits.data + S2P_TOK_EOS, S2P_TEXT_VOCAB, d->samp, nact, d->tok,
                             d->sem, d->ocodes, d->eos, st));
    return S2P_OK;
}

/* fast-AR frame, general sequence (src/fastar/fastar.cu:726-788) */
static s2p_status fast_frame_general(s2p_model* m, const tick_dev* d, int nact, int dump_ok) {
    cudaStream_t st = m->stream;
    layer_ctx c;
    memset(&c, 0, sizeof(c));
    c.rows = nact; c.max_seq = S2P_FAST_SEQ; c.kv8 = 0; c.pos_row_step = 0; c.decode = 1; c.split_k = 0;
    S2P_CUDA_TRY(cudaMemcpyAsync(m->fx.data, m->shidden.data, (size_t)nact * S2P_DIM * 2, cudaMemcpyDeviceToDevice, st));
    for (int cb = 0; cb < S2P_NUM_CODEBOOKS; cb++) {
        c.pos0 = cb;
        for (int l = 0; l < S2P_FAST_LAYERS; l++) {
            fast_kv_ref(m, l, &c.kv);
            S2P_TRY(layer_general(m, &m->fast[l], &c, BF(m->fx), BF(m->ft), BF(m->fqkv), BF(m->fq), BF(m->fattn),
                                  BF(m->fproj), BF(m->fgu), BF(m->fhff)));
        }
        const int32_t* next_codes;
        if (cb == 0) {
            next_codes = d->sem; /* the prime pass produces no logits; step 1 is fed embeddings[sem] */
        } else {
            S2P_LAUNCH(m, rms_norm(m->fx.data, m->fast_norm.data, m->ft.data, nact, S2P_DIM, S2P_NORM_EPS, st));
            S2P_TRY(lin_apply(m, &m->fast_out, m->ft.data, m->flogits.data, nact, 1));
            if (dump_ok && dump_dir() && nact == 1) {
                static int dump_frame = 0;
                if (cb == 1) dump_frame++;
                if (dump_frame == 1) {
                    char nm[48];
                    snprintf(nm, sizeof(nm), "fast_ar_step0_cb%d", cb);
                    dump_bf16(nm, m->flogits.data, S2P_CB_SIZE, st);
                }
            }
            int32_t* dst = m->fstage + (size_t)(cb - 1) * nact;
            S2P_LAUNCH(m, argmax_rows(m->flogits.data, dst, nact, S2P_CB_SIZE, st));
            next_codes = dst;
        }
        if (cb < S2P_NUM_CODEBOOKS - 1) S2P_LAUNCH(m, embed_codes(m->fast_emb.data, next_codes, m->fx.data, nact, st));
    }
    S2P_LAUNCH(m, pack_frame(m->fstage, nact, d->ocodes, st));
    return S2P_OK;
}

/* general tick: bd decode rows (rows [0,bd) of the upload block), nact >= bd rows to sample */
static s2p_status tick_general(s2p_model* m, s2p_session* const* act, int bd, int nact) {
    cudaStream_t st = m->stream;
    tick_dev d;
    tick_views(m, &d);
    S2P_CUDA_TRY(cudaMemcpyAsync(m->d_up, m->h_up, m->up_bytes, cudaMemcpyHostToDevice, st));
    if (bd > 0) {
        S2P_TRY(tick_begin_rows(m, &d, bd));
        layer_ctx c;
        memset(&c, 0, sizeof(c));
        c.rows = bd; c.kv.bases = d.kv_bases; c.kv.sbases = d.kvs_bases;
        c.max_seq = m->ctx_len; c.kv8 = m->kv8; c.pos_arr = d.pos; c.split_k = 1; c.decode = 1;
        for (int l = 0; l < m->n_slow; l++) {
            slow_kv_offsets(m, l, &c.kv);
            S2P_TRY(layer_general(m, &m->slow[l], &c, BF(m->sx), BF(m->snorm), BF(m->sqkv), BF(m->sq), BF(m->sattn),
                                  BF(m->sproj), BF(m->sgu), BF(m->sffn)));
        }
        S2P_LAUNCH(m, rms_norm(m->sx.data, m->final_norm.data, m->shidden.data, bd, S2P_DIM, S2P_NORM_EPS, st));
    }
    for (int b = bd; b < nact; b++) /* freshly prefilled rows sample from their stashed hidden (eager only) */
        S2P_CUDA_TRY(cudaMemcpyAsync(BF(m->shidden) + (size_t)b * S2P_DIM, act[b]->pending_hidden.data,
                                     (size_t)S2P_DIM * 2, cudaMemcpyDeviceToDevice, st));
    S2P_TRY(head_and_sample(m, &d, nact, 1));
    S2P_TRY(fast_frame_general(m, &d, nact, 1));
    S2P_CUDA_TRY(cudaMemcpyAsync(m->h_out, m->d_out, m->out_bytes, cudaMemcpyDeviceToHost, st));
    return S2P_OK;
}

/* batch-1 tick out of fused stages; `decode` = 0 when the row is freshly prefilled */
static s2p_status tick_fused_b1(s2p_model* m, s2p_session* const* act, int decode) {
    cudaStream_t st = m->stream;
    tick_dev d;
    tick_views(m, &d);
    S2P_CUDA_TRY(cudaMemcpyAsync(m->d_up, m->h_up, m->up_bytes, cudaMemcpyHostToDevice, st));
    LinRef lr;
    VecRef xr;
    if (decode) {
        S2P_TRY(tick_begin_rows(m, &d, 1));
        AttnArgs aa;
        memset(&aa, 0, sizeof(aa));
        aa.out = BF(m->sattn);
        aa.q_heads = S2P_SLOW_Q_HEADS; aa.kv_heads = S2P_SLOW_KV_HEADS; aa.max_seq = m->ctx_len; aa.kv8 = m->kv8;
        aa.pos_arr = d.pos; aa.kv.bases = d.kv_bases; aa.kv.sbases = d.kvs_bases;
        aa.part = (float*)m->attn_part.data; aa.counters = m->attn_ctr;
        aa.n_split_slots = m->n_split_slots; aa.workers = attn_workers_for(1); aa.head_dim = S2P_HEAD_DIM;
        memset(&xr, 0, sizeof(xr));
        xr.base = BF(m->sx);
        for (int l = 0; l < m->n_slow; l++) {
            const s2p_layer* L = &m->slow[l];
            s2p_lin_ref(&L->wqkv, &lr);
            S2P_LAUNCH(m, stage_norm_gemv(&lr, &xr, L->attn_norm.data, S2P_NORM_EPS, BF(m->sqkv), st));
            slow_kv_offsets(m, l, &aa.kv);
            S2P_LAUNCH(m, stage_attn_decode_prep(&aa, BF(m->sqkv), L->q_norm.data, L->k_norm.data, S2P_NORM_EPS,
                                                S2P_ROPE_BASE, 1, st));
            s2p_lin_ref(&L->wo, &lr);
            S2P_LAUNCH(m, stage_gemv_resid(&lr, BF(m->sattn), &xr, BF(m->sx), st));
            s2p_lin_ref(&L->gate_up, &lr);
            S2P_LAUNCH(m, stage_norm_swiglu(&lr, &xr, L->ffn_norm.data, S2P_NORM_EPS, BF(m->sffn), st));
            s2p_lin_ref(&L->w2, &lr);
            S2P_LAUNCH(m, stage_gemv_resid(&lr, BF(m->sffn), &xr, BF(m->sx), st));
        }
        S2P_LAUNCH(m, rms_norm(m->sx.data, m->final_norm.data, m->shidden.data, 1, S2P_DIM, S2P_NORM_EPS, st));
    } else {
        S2P_CUDA_TRY(cudaMemcpyAsync(m->shidden.data, act[0]->pending_hidden.data, (size_t)S2P_DIM * 2,
                                     cudaMemcpyDeviceToDevice, st));
        S2P_CUDA_TRY(cudaMemsetAsync(m->fkeys, 0, 9 * sizeof(unsigned long long), st));
    }
    S2P_TRY(head_and_sample(m, &d, 1, 0));

    /* fast-AR: the input of a pass is a row selected on the device — the slow hidden
     * (prime), embeddings[sem] (step 1) or embeddings[arg-max of the previous step] */
    QkvPostArgs qa;
    memset(&qa, 0, sizeof(qa));
    qa.qkv = BF(m->fqkv); qa.q = BF(m->fq);
    qa.eps = S2P_NORM_EPS; qa.rope_base = S2P_ROPE_BASE;
    qa.q_heads = S2P_SLOW_Q_HEADS; qa.kv_heads = S2P_SLOW_KV_HEADS; qa.max_seq = S2P_FAST_SEQ;
    AttnArgs fa;
    memset(&fa, 0, sizeof(fa));
    fa.q = BF(m->fq); fa.out = BF(m->fattn);
    fa.q_heads = S2P_SLOW_Q_HEADS; fa.kv_heads = S2P_SLOW_KV_HEADS; fa.max_seq = S2P_FAST_SEQ;
    fa.head_dim = S2P_HEAD_DIM;
    for (int cb = 0; cb < S2P_NUM_CODEBOOKS; cb++) {
        VecRef in; /* input of layer 0 of this pass */
        memset(&in, 0, sizeof(in));
        if (cb == 0) in.base = BF(m->shidden);
        else {
            in.base = BF(m->fast_emb);
            if (cb == 1) in.index = d.sem;
            else in.key = m->fkeys + (cb - 2);
        }
        VecRef fx;
        memset(&fx, 0, sizeof(fx));
        fx.base = BF(m->fx);
        qa.pos0 = cb; fa.pos0 = cb;
        for (int l = 0; l < S2P_FAST_LAYERS; l++) {
            const s2p_layer* L = &m->fast[l];
            const VecRef* src = l == 0 ? &in : &fx;
            s2p_lin_ref(&L->wqkv, &lr);
            S2P_LAUNCH(m, stage_norm_gemv(&lr, src, L->attn_norm.data, S2P_NORM_EPS, BF(m->fqkv), st));
            fast_kv_ref(m, l, &qa.kv);
            fa.kv = qa.kv;
            S2P_LAUNCH(m, qkv_post(&qa, 1, st));
            S2P_LAUNCH(m, attn_single(&fa, 1, st));
            s2p_lin_ref(&L->wo, &lr);
            S2P_LAUNCH(m, stage_gemv_resid(&lr, BF(m->fattn), src, BF(m->fx), st));
            s2p_lin_ref(&L->gate_up, &lr);
            S2P_LAUNCH(m, stage_norm_swiglu(&lr, &fx, L->ffn_norm.data, S2P_NORM_EPS, BF(m->fhff), st));
            s2p_lin_ref(&L->w2, &lr);
            S2P_LAUNCH(m, stage_gemv_resid(&lr, BF(m->fhff), &fx, BF(m->fx), st));
        }
        if (cb > 0) {
            s2p_lin_ref(&m->fast_out, &lr);
            S2P_LAUNCH(m, stage_norm_argmax(&lr, BF(m->fx), m->fast_norm.data, S2P_NORM_EPS, BF(m->flogits),
                                           m->fkeys + (cb - 1), st));
        }
    }
    S2P_LAUNCH(m, tick_finish_keys(m->fkeys, 1, d.ocodes, st));
    S2P_CUDA_TRY(cudaMemcpyAsync(m->h_out, m->d_out, m->out_bytes, cudaMemcpyDeviceToHost, st));
    return S2P_OK;
}

/* ---- persistent batch-1 tick ------------------------------------------------------
 * The stage list mirrors tick_fused_b1 for a decoding row (it is built once per
 * model: every per-frame quantity is read on the device from the upload block). */
static int mega_gemv(const MegaLayout* lay, MegaStage* st, const s2p_linear* lin, int pro, int epi) {
    memset(st, 0, sizeof(*st));
    st->type = MEGA_GEMV;
    s2p_lin_ref(lin, &st->lin);
    st->pro = pro; st->epi = epi;
    const int regions = epi == 2 ? 2 : 1;
    const size_t rb = st->lin.kind == 2 ? (size_t)st->lin.K / 2 : (size_t)st->lin.K;
    const size_t sb = st->lin.kind == 0 ? 0 : (size_t)(st->lin.K >> st->lin.gshift) * 2;
    if (st->lin.K % 512 || rb % 16 || sb % 16 || ((uintptr_t)st->lin.w & 15) || ((uintptr_t)st->lin.scales & 15)) return 0;
    int rpc = (int)((size_t)lay->slot_bytes / ((size_t)regions * (rb + sb)));
    const int cap = mega_max_local_rows(lay, st->lin.K) / regions;
    if (rpc > cap) rpc = cap;
    st->rows_per_chunk = rpc;
    return rpc >= 1;
}

/* The buffers the persistent tick writes live in one allocation, the exchange arena, so that
 * tensor-parallel peers can address them at the same offsets in their mapping of it. */
typedef struct {
    s2p_dev_bf16 *x, *qkv, *attn, *ffn, *hidden, *logc, *loge, *fx, *fqkv, *fattn, *fhff, *flogits, *logits_plain;
    unsigned long long* keys;
    unsigned int* barrier;
} mega_arena;

static void arena_views(const s2p_model* m, mega_arena* a) {
    char* p = (char*)m->tp_arena;
    size_t off = 0;
#define ARENA_TAKE(field, type, count) a->field = (type*)(p + off); off += (((size_t)(count) * sizeof(type)) + 255) & ~(size_t)255
    ARENA_TAKE(barrier, unsigned int, 1);
    ARENA_TAKE(keys, unsigned long long, 16);
    /* flagged vectors: one 32-bit word (bf16 | tag << 16) per element */
    ARENA_TAKE(x, s2p_dev_bf16, 2 * S2P_DIM);
    ARENA_TAKE(qkv, s2p_dev_bf16, 2 * S2P_QKV_WIDTH);
    ARENA_TAKE(attn, s2p_dev_bf16, 2 * S2P_SLOW_Q_HEADS * S2P_HEAD_DIM);
    ARENA_TAKE(ffn, s2p_dev_bf16, 2 * S2P_FFN_DIM);
    ARENA_TAKE(logc, s2p_dev_bf16, 2 * 4096);
    ARENA_TAKE(loge, s2p_dev_bf16, 2 * 8);
    ARENA_TAKE(fx, s2p_dev_bf16, 2 * S2P_DIM);
    ARENA_TAKE(fqkv, s2p_dev_bf16, 2 * S2P_QKV_WIDTH);
    ARENA_TAKE(fattn, s2p_dev_bf16, 2 * S2P_SLOW_Q_HEADS * S2P_HEAD_DIM);
    ARENA_TAKE(fhff, s2p_dev_bf16, 2 * S2P_FFN_DIM);
    /* plain bf16 */
    ARENA_TAKE(hidden, s2p_dev_bf16, S2P_DIM);
    ARENA_TAKE(flogits, s2p_dev_bf16, S2P_CB_SIZE);
    ARENA_TAKE(logits_plain, s2p_dev_bf16, 4104);
#undef ARENA_TAKE
    (void)off; /* < S2P_TP_ARENA_BYTES */
}

static s2p_status mega_build(s2p_model* m) {
    const int cap = m->n_slow * 5 + 4 + S2P_NUM_CODEBOOKS * (S2P_FAST_LAYERS * 5 + 1) + 2;
    MegaStage* prog = (MegaStage*)calloc((size_t)cap, sizeof(MegaStage));
    if (!prog) return S2P_ERR_OOM;
    tick_dev d;
    tick_views(m, &d);
    mega_arena A;
    arena_views(m, &A);
    int n = 0, ok = 1;
    MegaStage* st;
    {   /* widest staged activation: bf16 for packed INT4 weights, f32 for int8 codes */
        int xb = S2P_DIM * 4; /* the tied head is per-channel INT8 on the model width */
        for (int l = 0; l < m->n_slow + S2P_FAST_LAYERS; l++) {
            const s2p_layer* L = l < m->n_slow ? &m->slow[l] : &m->fast[l - m->n_slow];
            const s2p_linear* lins[4] = {&L->wqkv, &L->wo, &L->gate_up, &L->w2};
            for (int i = 0; i < 4; i++) {
                LinRef lr;
                s2p_lin_ref(lins[i], &lr);
                const int b = lr.K * (lr.kind == 2 ? 2 : 4);
                if (b > xb) xb = b;
            }
        }
        mega_layout(xb, &m->mega_lay);
    }
    /* Stage outputs travel as flagged words (x_from = the producing stage); a grid barrier is
     * kept only where plain memory is handed over: after the sampler (its token index) and after
     * every arg-max stage (the packed keys). */
    prog[n].type = MEGA_BEGIN; prog[n].flags = MEGA_NO_BARRIER; prog[n].x_from = -1; n++;
    int last_x = 0, from;
    for (int l = 0; l < m->n_slow && ok; l++) {
        const s2p_layer* L = &m->slow[l];
        st = &prog[n++]; ok &= mega_gemv(&m->mega_lay, st, &L->wqkv, 1, 0);
        st->x.base = A.x; st->norm_w = L->attn_norm.data; st->y = A.qkv;
        st->x_from = last_x; st->io_flags = MEGA_Y_LL; st->flags = MEGA_NO_BARRIER;
        from = n - 1;
        st = &prog[n++]; memset(st, 0, sizeof(*st));
        st->type = MEGA_ATTN_SLOW; st->qkv = A.qkv; st->q_norm = L->q_norm.data; st->k_norm = L->k_norm.data;
        st->out = A.attn; st->kv.bases = d.kv_bases; st->kv.sbases = d.kvs_bases;
        st->x_from = from; st->flags = MEGA_NO_BARRIER;
        slow_kv_offsets(m, l, &st->kv);
        from = n - 1;
        st = &prog[n++]; ok &= mega_gemv(&m->mega_lay, st, &L->wo, 0, 1);
        st->x.base = A.attn; st->resid.base = A.x; st->y = A.x;
        st->x_from = from; st->io_flags = MEGA_Y_LL | MEGA_RESID_LL; st->flags = MEGA_NO_BARRIER;
        last_x = n - 1;
        st = &prog[n++]; ok &= mega_gemv(&m->mega_lay, st, &L->gate_up, 1, 2);
        st->x.base = A.x; st->norm_w = L->ffn_norm.data; st->y = A.ffn;
        st->x_from = last_x; st->io_flags = MEGA_Y_LL; st->flags = MEGA_NO_BARRIER;
        from = n - 1;
        st = &prog[n++]; ok &= mega_gemv(&m->mega_lay, st, &L->w2, 0, 1);
        st->x.base = A.ffn; st->resid.base = A.x; st->y = A.x;
        st->x_from = from; st->io_flags = MEGA_Y_LL | MEGA_RESID_LL; st->flags = MEGA_NO_BARRIER;
        last_x = n - 1;
    }
    /* tied head on the INT8 sidecar: the 4096 semantic rows, then the EOS row; the first of
     * the two also leaves the final-normed hidden state for the fast-AR */
    for (int part = 0; part < 2 && ok; part++) {
        st = &prog[n++]; memset(st, 0, sizeof(*st));
        st->type = MEGA_GEMV; st->pro = 1; st->epi = 0;
        st->lin.kind = 0; st->lin.K = S2P_DIM; st->lin.gshift = 0;
        const int row = part == 0 ? S2P_TOK_SEMANTIC_START : S2P_TOK_EOS;
        st->lin.N = part == 0 ? 4096 : 1;
        st->lin.w = (const int8_t*)m->embed_i8.data + (size_t)row * S2P_DIM;
        st->lin.scales = (const float*)m->embed_scale.data + row;
        st->rows_per_chunk = m->mega_lay.slot_bytes / S2P_DIM;
        if (st->rows_per_chunk > mega_max_local_rows(&m->mega_lay, S2P_DIM))
            st->rows_per_chunk = mega_max_local_rows(&m->mega_lay, S2P_DIM);
        if (((uintptr_t)st->lin.w & 15) || !m->embed_i8.data) ok = 0;
        st->x.base = A.x; st->norm_w = m->final_norm.data;
        st->y = part == 0 ? A.logc : A.loge;
        st->x_from = last_x; st->io_flags = MEGA_Y_LL; st->flags = MEGA_NO_BARRIER; /* the sampler waits on the words */
        if (part == 0) { st->normed_out = A.hidden; m->mega_logc_from = n - 1; }
        else m->mega_loge_from = n - 1;
    }
    st = &prog[n++]; memset(st, 0, sizeof(*st)); st->type = MEGA_SAMPLE; st->x_from = -1;
    for (int cb = 0; cb < S2P_NUM_CODEBOOKS && ok; cb++) {
        VecRef in;
        memset(&in, 0, sizeof(in));
        if (cb == 0) in.base = A.hidden;
        else {
            in.base = BF(m->fast_emb);
            if (cb == 1) in.index = d.sem;
            else in.key = A.keys + (cb - 2);
        }
        VecRef fx;
        memset(&fx, 0, sizeof(fx));
        fx.base = A.fx;
        int last_fx = -1; /* layer 0 of a pass reads a plain row (published by a barrier) */
        for (int l = 0; l < S2P_FAST_LAYERS && ok; l++) {
            const s2p_layer* L = &m->fast[l];
            const VecRef* src = l == 0 ? &in : &fx;
            st = &prog[n++]; ok &= mega_gemv(&m->mega_lay, st, &L->wqkv, 1, 0);
            st->x = *src; st->norm_w = L->attn_norm.data; st->y = A.fqkv;
            st->x_from = last_fx; st->io_flags = MEGA_Y_LL; st->flags = MEGA_NO_BARRIER;
            from = n - 1;
            st = &prog[n++]; memset(st, 0, sizeof(*st));
            st->type = MEGA_ATTN_FAST; st->qkv = A.fqkv; st->out = A.fattn; st->pos = cb;
            st->x_from = from; st->flags = MEGA_NO_BARRIER;
            fast_kv_ref(m, l, &st->kv);
            from = n - 1;
            st = &prog[n++]; ok &= mega_gemv(&m->mega_lay, st, &L->wo, 0, 1);
            st->x.base = A.fattn; st->resid = *src; st->y = A.fx;
            st->x_from = from; st->io_flags = MEGA_Y_LL | (l == 0 ? 0 : MEGA_RESID_LL); st->flags = MEGA_NO_BARRIER;
            last_fx = n - 1;
            st = &prog[n++]; ok &= mega_gemv(&m->mega_lay, st, &L->gate_up, 1, 2);
            st->x = fx; st->norm_w = L->ffn_norm.data; st->y = A.fhff;
            st->x_from = last_fx; st->io_flags = MEGA_Y_LL; st->flags = MEGA_NO_BARRIER;
            from = n - 1;
            st = &prog[n++]; ok &= mega_gemv(&m->mega_lay, st, &L->w2, 0, 1);
            st->x.base = A.fhff; st->resid = fx; st->y = A.fx;
            st->x_from = from; st->io_flags = MEGA_Y_LL | MEGA_RESID_LL; st->flags = MEGA_NO_BARRIER;
            last_fx = n - 1;
        }
        if (cb > 0 && ok) {
            st = &prog[n++]; ok &= mega_gemv(&m->mega_lay, st, &m->fast_out, 1, 3);
            st->x = fx; st->norm_w = m->fast_norm.data; st->y = A.flogits; st->key = A.keys + (cb - 1);
            st->x_from = last_fx; /* plain logits and packed keys out: the grid barrier stays */
        }
    }
    st = &prog[n++]; memset(st, 0, sizeof(*st)); st->type = MEGA_FINISH; st->flags = MEGA_NO_BARRIER; st->x_from = -1;
    m->mega_built = 1;
    m->mega_barriers = 0;
    for (int i = 0; i < n; i++) m->mega_barriers += !(prog[i].flags & MEGA_NO_BARRIER);
    /* every CTA's copy commands, in the order its working warps consume the chunks */
    const int n_cta = m->mega_ctas;
    int* cmd_start = (int*)calloc((size_t)n_cta + 1, sizeof(int));
    MegaCopyCmd* cmds = NULL;
    size_t n_cmds = 0;
    if (!cmd_start) { free(prog); return S2P_ERR_OOM; }
    for (int pass = 0; pass < 2 && ok; pass++) {
        size_t at = 0;
        for (int c = 0; c < n_cta; c++) {
            if (pass) cmd_start[c] = (int)at;
            for (int i = 0; i < n; i++) {
                const MegaStage* g = &prog[i];
                if (g->type != MEGA_GEMV) continue;
                const int regions = g->epi == 2 ? 2 : 1;
                const MegaGeom ge = mega_stage_geom(g->lin.N, regions == 2, g->rows_per_chunk, m->tp_rank * n_cta + c,
                                                    m->tp_world * n_cta);
                if (!pass) { at += (size_t)ge.n_chunks; continue; }
                const size_t rb = g->lin.kind == 2 ? (size_t)g->lin.K / 2 : (size_t)g->lin.K;
                const size_t sb = g->lin.kind == 0 ? 0 : (size_t)(g->lin.K >> g->lin.gshift) * 2;
                for (int j = 0; j < ge.n_chunks; j++) {
                    MegaCopyCmd* cc = &cmds[at++];
                    memset(cc, 0, sizeof(*cc));
                    const int rows = ge.rc < ge.cnt - j * ge.rc ? ge.rc : ge.cnt - j * ge.rc;
                    const size_t first = (size_t)ge.row0 + (size_t)j * ge.rc;
                    const size_t wbytes = (size_t)rows * rb, sbytes = (size_t)rows * sb;
                    int k = 0;
                    for (int reg = 0; reg < regions; reg++) {
                        const size_t grow = first + (reg ? (size_t)(g->lin.N >> 1) : 0);
                        cc->src[k] = (unsigned long long)(uintptr_t)((const char*)g->lin.w + grow * rb);
                        cc->bytes[k] = (unsigned int)wbytes;
                        cc->dst_off[k] = (unsigned int)((size_t)reg * wbytes);
                        k++;
                        if (sbytes) {
                            cc->src[k] = (unsigned long long)(uintptr_t)((const char*)g->lin.scales + grow * sb);
                            cc->bytes[k] = (unsigned int)sbytes;
                            cc->dst_off[k] = (unsigned int)((size_t)regions * wbytes + (size_t)reg * sbytes);
                            k++;
                        }
                    }
                    if ((size_t)regions * (wbytes + sbytes) > (size_t)m->mega_lay.slot_bytes) ok = 0;
                }
            }
        }
        if (!pass) {
            n_cmds = at;
            cmds = (MegaCopyCmd*)malloc((n_cmds ? n_cmds : 1) * sizeof(MegaCopyCmd));
            if (!cmds) { free(prog); free(cmd_start); return S2P_ERR_OOM; }
        } else {
            cmd_start[n_cta] = (int)at;
        }
    }
    if (!ok || n > cap) {
        free(cmds); free(cmd_start);
        free(prog);
        m->mega_ok = 0;
        fprintf(stderr, "[s2pro] persistent tick kernel: a weight layout does not fit its copy engine rules; "
                        "using per-stage launches\n");
        return S2P_OK;
    }
    cudaError_t e = cudaMalloc((void**)&m->d_mega_stages, (size_t)n * sizeof(MegaStage));
    if (e == cudaSuccess) e = cudaMalloc((void**)&m->d_mega_sync, 2 * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMallocHost((void**)&m->h_mega_status, sizeof(int));
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(m->d_mega_stages, prog, (size_t)n * sizeof(MegaStage), cudaMemcpyHostToDevice, m->stream);
    if (e == cudaSuccess) e = cudaMalloc((void**)&m->d_mega_cmds, (n_cmds ? n_cmds : 1) * sizeof(MegaCopyCmd));
    if (e == cudaSuccess) e = cudaMalloc((void**)&m->d_mega_cmd_start, ((size_t)n_cta + 1) * sizeof(int));
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(m->d_mega_cmds, cmds, n_cmds * sizeof(MegaCopyCmd), cudaMemcpyHostToDevice, m->stream);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(m->d_mega_cmd_start, cmd_start, ((size_t)n_cta + 1) * sizeof(int), cudaMemcpyHostToDevice,
                            m->stream);
    if (e == cudaSuccess && s2p_env_is_one("S2P_TICK_TRACE")) {
        const size_t tb = (size_t)n * (16 + 2 * (size_t)n_cta) * sizeof(unsigned long long);
        e = cudaMalloc((void**)&m->d_mega_trace, tb);
        if (e == cudaSuccess) e = cudaMemsetAsync(m->d_mega_trace, 0, tb, m->stream);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(m->stream);
    m->mega_types = (int32_t*)malloc((size_t)n * sizeof(int32_t));
    if (m->mega_types)
        for (int i = 0; i < n; i++) m->mega_types[i] = prog[i].type;
    free(prog);
    free(cmds);
    free(cmd_start);
    if (e != cudaSuccess) {
        fprintf(stderr, "[s2pro] CUDA error %s at %s:%d\n", cudaGetErrorString(e), __FILE__, __LINE__);
        return S2P_ERR_CUDA;
    }
    m->mega_n_stages = n;
    return S2P_OK;
}

static s2p_status tick_mega(s2p_model* m) {
    cudaStream_t st = m->stream;
    tick_dev d;
    tick_views(m, &d);
    S2P_CUDA_TRY(cudaMemcpyAsync(m->d_up, m->h_up, m->up_bytes, cudaMemcpyHostToDevice, st));
    S2P_CUDA_TRY(cudaMemsetAsync(m->d_mega_sync, 0, 2 * sizeof(unsigned int), st)); /* [1]: the status word */
    mega_arena A;
    arena_views(m, &A);
    MegaParams P;
    memset(&P, 0, sizeof(P));
    P.stages = m->d_mega_stages; P.n_stages = m->mega_n_stages;
    P.cmds = m->d_mega_cmds; P.cmd_start = m->d_mega_cmd_start; P.lay = m->mega_lay;
    P.barrier = A.barrier; P.status = (int*)(m->d_mega_sync + 1);
    P.tp_rank = m->tp_rank; P.tp_world = m->tp_world;
    for (int r = 0; r < m->tp_world; r++) P.tp_base[r] = (unsigned char*)m->tp_base[r];
    P.bar_base = m->mega_ticks * (unsigned int)m->mega_barriers; /* wraps with the device counters */
    P.seq_base = m->mega_ticks * (unsigned int)m->mega_n_stages;
    P.logc_from = m->mega_logc_from; P.loge_from = m->mega_loge_from; P.logits_plain = A.logits_plain;
    m->mega_ticks++;
    if (!m->embed_i8_only) P.begin.embed = (const s2p_dev_bf16*)m->embed.data;
    P.begin.embed_i8 = (const int8_t*)m->embed_i8.data;
    P.begin.embed_scale = (const float*)m->embed_scale.data;
    P.begin.cb_emb = (const s2p_dev_bf16*)m->cb_emb.data;
    P.begin.ids = d.ids; P.begin.codes = d.codes; P.begin.mask = d.mask;
    P.begin.x = A.x; P.begin.keys = A.keys;
    P.ctx_len = m->ctx_len; P.kv8 = m->kv8; P.n_split_slots = m->n_split_slots;
    P.pos_arr = d.pos; P.part = (float*)m->attn_part.data; P.counters = m->attn_ctr;
    P.eps = S2P_NORM_EPS; P.rope_base = S2P_ROPE_BASE; P.head_dim = S2P_HEAD_DIM;
    P.sem_logits = A.logc; P.eos_logit = A.loge;
    P.states = d.samp; P.out_tok = d.tok; P.out_sem = d.sem; P.out_codes = d.ocodes; P.out_eos = d.eos;
    P.keys = A.keys;
    P.trace = m->d_mega_trace;
    S2P_LAUNCH(m, mega_launch(&P, m->mega_ctas, st));
    S2P_CUDA_TRY(cudaMemcpyAsync(m->h_out, m->d_out, m->out_bytes, cudaMemcpyDeviceToHost, st));
    S2P_CUDA_TRY(cudaMemcpyAsync(m->h_mega_status, m->d_mega_sync + 1, sizeof(int), cudaMemcpyDeviceToHost, st));
    return S2P_OK;
}

s2p_status s2p_model_batch_next_frame(s2p_model* m, s2p_session** sess, int n, int32_t* out_codes, int* eos) {
    if (!m || !sess || !out_codes || !eos || n < 0 || n > m->max_sessions) return S2P_ERR_INVALID;
    for (int i = 0; i < n; i++) {
        if (!sess[i] || sess[i]->m != m) return S2P_ERR_INVALID;
        if (sess[i]->state == SESS_NEW) return S2P_ERR_STATE;
    }
    cudaStream_t st = m->stream;
    memset(out_codes, 0, (size_t)n * S2P_NUM_CODEBOOKS * sizeof(int32_t));

    /* decode rows first (their final norm lands in shidden[0..bd)), then freshly prefilled ones */
    s2p_session* act[S2P_MAX_BATCH];
    int act_ix[S2P_MAX_BATCH];
    int nact = 0;
    for (int i = 0; i < n; i++) {
        s2p_session* s = sess[i];
        eos[i] = s->state == SESS_FINISHED;
        if (s->state == SESS_DECODING) {
            if (s->kv_len >= m->ctx_len) { /* context exhausted: forced stop */
                s->state = SESS_FINISHED;
                eos[i] = 1;
                continue;
            }
            act[nact] = s;
            act_ix[nact++] = i;
        }
    }
    const int bd = nact;
    for (int i = 0; i < n; i++)
        if (sess[i]->state == SESS_PREFILLED) {
            act[nact] = sess[i];
            act_ix[nact++] = i;
        }
    if (nact == 0) return S2P_OK;

    /* host staging */
    {
        char* h = (char*)m->h_up;
        void** kvb = (void**)(h + m->off_kvb);
        void** kvsb = (void**)(h + m->off_kvsb);
        void** samp = (void**)(h + m->off_samp);
        int64_t* ids = (int64_t*)(h + m->off_ids);
        int32_t* codes = (int32_t*)(h + m->off_codes);
        int32_t* pos = (int32_t*)(h + m->off_pos);
        uint8_t* mask = (uint8_t*)(h + m->off_mask);
        for (int b = 0; b < nact; b++) {
            s2p_session* s = act[b];
            samp[b] = s->dsamp;
            kvb[b] = s->kv.data;
            kvsb[b] = s->kvs.data;
            if (b < bd) {
                ids[b] = s->prev_token;
                pos[b] = s->kv_len;
                mask[b] = (uint8_t)is_semantic(s->prev_token);
                memcpy(codes + (size_t)b * S2P_NUM_CODEBOOKS, s->prev_codes, sizeof(s->prev_codes));
            }
        }
    }

    /* the library GEMM of the BF16 mode is kept out of stream capture */
    const int graphs = !s2p_env_is_one("S2P_NO_GRAPHS") && dump_dir() == NULL && m->mode == S2P_GEMM_INT8;
    const int fused = m->fused_b1 && nact == 1 && !m->head_full;
    s2p_status rc = S2P_OK;
    if (fused && bd == 1 && m->mega_ok && !m->mega_built && dump_dir() == NULL) S2P_TRY(mega_build(m));
    const int mega = fused && bd == 1 && m->mega_ok && m->mega_built && dump_dir() == NULL;
    const int steady = bd == nact && graphs && !mega; /* every row decoding: the launch sequence is frame-invariant */
    if (s2p_tp_guard_tick(m->tp_world, bd, mega) != S2P_OK) {
        fprintf(stderr, "[s2pro] tensor-parallel model: this tick (%d decoding rows%s) cannot run as the persistent kernel, and no "
                        "other path sees the whole KV cache; not served\n", bd, m->mega_ok ? "" : ", persistent path disabled");
        return S2P_ERR_UNSUPPORTED;
    }
    m->tick_kernels = 0;
    if (mega) {
        S2P_CUDA_TRY(cudaEventRecord(m->ev0, st));
        S2P_TRY(tick_mega(m));
    } else if (steady) {
        if (!m->gready[bd]) {
            S2P_CUDA_TRY(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
            rc = fused ? tick_fused_b1(m, act, 1) : tick_general(m, act, bd, nact);
            m->graph_kernels[bd] = m->tick_kernels;
            cudaGraph_t g = NULL;
            const cudaError_t ce = cudaStreamEndCapture(st, &g);
            if (rc != S2P_OK) {
                if (g) cudaGraphDestroy(g);
                return rc;
            }
            if (ce != cudaSuccess) {
                fprintf(stderr, "[s2pro] graph capture failed: %s\n", cudaGetErrorString(ce));
                return S2P_ERR_CUDA;
            }
            const cudaError_t ci = cudaGraphInstantiate(&m->gexec[bd], g, 0);
            cudaGraphDestroy(g);
            if (ci != cudaSuccess) {
                fprintf(stderr, "[s2pro] graph instantiate failed: %s\n", cudaGetErrorString(ci));
                return S2P_ERR_CUDA;
            }
            m->gready[bd] = 1;
        }
        S2P_CUDA_TRY(cudaEventRecord(m->ev0, st));
        S2P_CUDA_TRY(cudaGraphLaunch(m->gexec[bd], st));
        m->tick_kernels = m->graph_kernels[bd];
    } else {
        S2P_CUDA_TRY(cudaEventRecord(m->ev0, st));
        rc = fused ? tick_fused_b1(m, act, bd == 1) : tick_general(m, act, bd, nact);
        if (rc != S2P_OK) return rc;
    }
    S2P_CUDA_TRY(cudaEventRecord(m->ev1, st));
    S2P_CUDA_TRY(cudaStreamSynchronize(st));
    if (mega && *m->h_mega_status != 0) {
        fprintf(stderr, "[s2pro] persistent tick kernel gave up on a bounded wait (code %d); the frame is lost and later "
                        "ticks %s\n", *m->h_mega_status,
                m->tp_world > 1 ? "of this tensor-parallel model are refused" : "use per-stage launches");
        m->mega_ok = 0; /* its barrier counters and tags are no longer in step */
        /* CTAs that left the kernel early did not take part in the arrival counting of its last attention
         * stage: the per-stage kernels that take over expect the counters at zero */
        if (m->attn_ctr)
            S2P_CUDA_TRY(cudaMemsetAsync(m->attn_ctr, 0, (size_t)m->max_sessions * S2P_SLOW_KV_HEADS * sizeof(unsigned int), st));
        return S2P_ERR_INTERNAL;
    }
    if (!mega && m->n_slow > 0 && m->mode == S2P_GEMM_INT8 && m->slow[0].wqkv.int8_ready &&
        s2p_linear_rows_on_tc(&m->slow[0].wqkv, nact)) {
        /* the batched linears ran on the tensor-core kernel: a bounded wait that gave up inside it left a code */
        int sk = 0;
        S2P_CUDA_TRY(skinny_status(&sk));
        if (sk != 0) {
            fprintf(stderr, "[s2pro] batched tensor-core linear gave up on a bounded wait (code %d); the frame is lost and later "
                            "batched ticks use the exact-order kernel\n", sk);
            S2P_CUDA_TRY(skinny_reset(st));
            s2p_linear_tc_disable();
            for (int b = 0; b <= S2P_MAX_BATCH; b++) /* captured ticks hold launches of the kernel that is now off */
                if (m->gready[b]) {
                    cudaGraphExecDestroy(m->gexec[b]);
                    m->gexec[b] = NULL;
                    m->gready[b] = 0;
                }
            return S2P_ERR_INTERNAL;
        }
    }
    m->last_rows = nact; m->last_fused = fused; m->last_graph = steady; m->last_kernels = m->tick_kernels;
    m->last_mega = mega;
    if (cudaEventElapsedTime(&m->last_device_ms, m->ev0, m->ev1) != cudaSuccess) m->last_device_ms = 0.f;
    for (int b = 0; b < bd; b++) act[b]->kv_len++;
    m->frames_decoded += (uint64_t)nact;

    const int64_t* toks = (const int64_t*)m->h_out;
    const int32_t* codes = (const int32_t*)((char*)m->h_out + m->off_ocodes);
    const uint8_t* eflag = (const uint8_t*)((char*)m->h_out + m->off_eos);
    for (int b = 0; b < nact; b++) {
        s2p_session* s = act[b];
        const int i = act_ix[b];
        if (eflag[b]) { /* the EOS frame carries no codes */
            s->state = SESS_FINISHED;
            eos[i] = 1;
            continue;
        }
        const int32_t* frame = codes + (size_t)b * S2P_NUM_CODEBOOKS;
        memcpy(out_codes + (size_t)i * S2P_NUM_CODEBOOKS, frame, S2P_NUM_CODEBOOKS * sizeof(int32_t));
        s->prev_token = toks[b];
        memcpy(s->prev_codes, frame, sizeof(s->prev_codes));
        s->state = SESS_DECODING;
        eos[i] = 0;
    }
    return S2P_OK;
}

/* ---- tensor-parallel attach (include/s2p_b200_ext.h) ------------------------------- */
s2p_status s2p_b200_model_tp_export(s2p_model* m, void* handle_out) {
    if (!m || !handle_out) return S2P_ERR_INVALID;
    if (!m->mega_ok || !m->tp_arena) return S2P_ERR_UNSUPPORTED;
    cudaIpcMemHandle_t h;
    S2P_CUDA_TRY(cudaIpcGetMemHandle(&h, m->tp_arena));
    memcpy(handle_out, &h, sizeof(h));
    return S2P_OK;
}

s2p_status s2p_b200_model_tp_attach(s2p_model* m, int rank, int world, const void* handles) {
    if (!m || !handles || rank < 0 || rank >= world) return S2P_ERR_INVALID;
    if (world != 1 && world != 2 && world != 4 && world != 8) return S2P_ERR_INVALID;
    if (!m->mega_ok || !m->tp_arena) return S2P_ERR_UNSUPPORTED;
    if (m->tp_world != 1 || m->mega_ticks != 0 || m->n_sessions != 0) return S2P_ERR_STATE; /* attach once, before any session */
    for (int r = 0; r < world; r++) {
        if (r == rank) { m->tp_base[r] = m->tp_arena; continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char*)handles + (size_t)r * sizeof(h), sizeof(h));
        void* p = NULL;
        S2P_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        m->tp_base[r] = p;
    }
    m->tp_rank = rank; m->tp_world = world;
    m->mega_built = 0; /* the row partition depends on the world size */
    return S2P_OK;
}

s2p_status s2p_b200_model_tick_trace(s2p_model* m, uint64_t* out, int32_t* types, int max_stages, int* n_stages) {
    if (!m || !out || !n_stages || max_stages < 0) return S2P_ERR_INVALID;
    if (!m->d_mega_trace || !m->last_mega) return S2P_ERR_STATE;
    const int n = m->mega_n_stages < max_stages ? m->mega_n_stages : max_stages;
    *n_stages = m->mega_n_stages;
    S2P_CUDA_TRY(cudaMemcpy(out, m->d_mega_trace, (size_t)n * 16 * sizeof(uint64_t), cudaMemcpyDeviceToHost));
    if (types && m->mega_types) memcpy(types, m->mega_types, (size_t)n * sizeof(int32_t));
    return S2P_OK;
}

s2p_status s2p_b200_model_tick_trace_ctas(s2p_model* m, uint64_t* fold_done_ns, uint64_t* staged_ns, int max_stages, int max_ctas,
                                          int* n_stages, int* n_ctas) {
    if (!m || !fold_done_ns || !staged_ns || !n_stages || !n_ctas || max_stages < 0 || max_ctas < 0) return S2P_ERR_INVALID;
    if (!m->d_mega_trace || !m->last_mega) return S2P_ERR_STATE;
    *n_stages = m->mega_n_stages;
    *n_ctas = m->mega_ctas;
    if (max_stages < m->mega_n_stages || max_ctas < m->mega_ctas) return S2P_ERR_INVALID;
    const size_t words = (size_t)m->mega_n_stages * m->mega_ctas;
    const uint64_t* base = (const uint64_t*)m->d_mega_trace + (size_t)m->mega_n_stages * 16;
    S2P_CUDA_TRY(cudaMemcpy(fold_done_ns, base, words * sizeof(uint64_t), cudaMemcpyDeviceToHost));
    S2P_CUDA_TRY(cudaMemcpy(staged_ns, base + words, words * sizeof(uint64_t), cudaMemcpyDeviceToHost));
    return S2P_OK;
}

s2p_status s2p_session_next_frame(s2p_session* s, int32_t out_codes[S2P_NUM_CODEBOOKS], int* is_eos) {
    if (!s || !out_codes || !is_eos) return S2P_ERR_INVALID;
    return s2p_model_batch_next_frame(s->m, &s, 1, out_codes, is_eos);
}
