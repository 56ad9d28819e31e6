/* Model load / free of the model contract (include/s2pro/model.h:42-44 of the
 * reference; load order and modes follow src/slowar/model.c:178-339 and
 * src/fastar/fastar.cu:206-395).
 *
 * Differences that stay behind the contract: the backbone depth is taken from
 * the checkpoint (1..36 layers), the session cap is 256 instead of 64, the
 * fast-AR is a second layer stack of the same engine rather than a separate
 * module, the device is chosen with S2P_DEVICE, and one activation scratch
 * serves prefill and decode.
 */
#include <stdlib.h>
#include <string.h>
#include "internal.h"

#define GU_ROWS (2 * S2P_FFN_DIM)
#define FA_KVSZ (S2P_SLOW_KV_HEADS * S2P_FAST_SEQ * S2P_HEAD_DIM) /* elements of one fast-AR cache plane set */

size_t s2p_kv_vec_bytes(const s2p_model* m) { return m->kv8 ? S2P_HEAD_DIM : S2P_HEAD_DIM * 2; }
size_t s2p_kv_plane_bytes(const s2p_model* m) { return (size_t)m->ctx_len * s2p_kv_vec_bytes(m); }
size_t s2p_kvs_plane_bytes(const s2p_model* m) { return m->kv8 ? (size_t)m->ctx_len * (S2P_HEAD_DIM / 32) * 2 : 0; }

void s2p_lin_ref(const s2p_linear* lin, LinRef* out) {
    memset(out, 0, sizeof(*out));
    out->N = lin->out_features;
    out->K = lin->in_features;
    if (lin->q_packed) {
        out->kind = 2; out->w = lin->w_pack.data;
    } else {
        out->kind = lin->q_group > 0 ? 1 : 0; out->w = lin->w_int8.data;
    }
    out->scales = lin->w_iscale.data;
    int gs = 0;
    while (lin->q_group > 0 && (1 << gs) < lin->q_group) gs++;
    out->gshift = gs;
}

static s2p_status load_vec(s2p_st* st, const char* fmt, int layer, int width, s2p_tensor* out, cudaStream_t stream) {
    char name[192];
    snprintf(name, sizeof(name), fmt, layer);
    const int64_t shape[1] = {width};
    return s2p_st_load_device(st, name, S2P_DT_BF16, 1, shape, out, stream);
}

static s2p_status finish_linear(s2p_model* m, s2p_qcache* qc, const char* cache_name, s2p_linear* lin, s2p_qsite site) {
    if (m->mode == S2P_GEMM_INT8) S2P_TRY(s2p_linear_prepare_int8_site(lin, site, m->stream));
    return s2p_qcache_put_linear(qc, cache_name, lin, m->stream);
}

static s2p_status load_linear(s2p_model* m, s2p_st* st, s2p_qcache* qc, const char* fmt, int layer, int in_f,
                              int out_f, s2p_qsite site, s2p_linear* lin) {
    char name[192];
    snprintf(name, sizeof(name), fmt, layer);
    if (s2p_qcache_try_load(qc, name, in_f, out_f, lin, m->stream)) return S2P_OK;
    S2P_TRY(s2p_linear_from_st(lin, st, name, in_f, out_f, m->stream));
    return finish_linear(m, qc, name, lin, site);
}

/* gate (w1) rows then up (w3) rows in one [19456, 2560] linear, so that one
 * product feeds the SwiGLU (src/slowar/model.c:55-92; fastar.cu:177-197). */
static s2p_status load_gate_up(s2p_model* m, s2p_st* st, s2p_qcache* qc, const char* prefix, int layer,
                               const char* fused_suffix, s2p_qsite site, s2p_linear* lin) {
    char fused[192], n1[192], n3[192];
    snprintf(fused, sizeof(fused), "%s.%d.feed_forward.%s", prefix, layer, fused_suffix);
    if (s2p_qcache_try_load(qc, fused, S2P_DIM, GU_ROWS, lin, m->stream)) return S2P_OK;
    snprintf(n1, sizeof(n1), "%s.%d.feed_forward.w1.weight", prefix, layer);
    snprintf(n3, sizeof(n3), "%s.%d.feed_forward.w3.weight", prefix, layer);
    s2p_st_view w1, w3;
    S2P_TRY(s2p_st_find(st, n1, &w1));
    S2P_TRY(s2p_st_find(st, n3, &w3));
    const s2p_st_view* v[2] = {&w1, &w3};
    for (int i = 0; i < 2; i++)
        if (v[i]->dtype != S2P_DT_BF16 || v[i]->ndim != 2 || v[i]->shape[0] != S2P_FFN_DIM || v[i]->shape[1] != S2P_DIM)
            return S2P_ERR_FORMAT;
    memset(lin, 0, sizeof(*lin));
    lin->in_features = S2P_DIM;
    lin->out_features = GU_ROWS;
    const int64_t shape[2] = {GU_ROWS, S2P_DIM};
    S2P_TRY(s2p_tensor_device_alloc(&lin->w_bf16, S2P_DT_BF16, 2, shape));
    const size_t half = (size_t)S2P_FFN_DIM * S2P_DIM * 2;
    S2P_CUDA_TRY(cudaMemcpyAsync(lin->w_bf16.data, w1.data, half, cudaMemcpyHostToDevice, m->stream));
    S2P_CUDA_TRY(cudaMemcpyAsync((char*)lin->w_bf16.data + half, w3.data, half, cudaMemcpyHostToDevice, m->stream));
    return finish_linear(m, qc, fused, lin, site);
}

static s2p_status load_stack(s2p_model* m, s2p_st* st, s2p_qcache* qc, s2p_layer* layers, int n, const char* prefix,
                             int qk_norm, const char* fused_suffix, s2p_qsite site) {
    char fmt[192];
    for (int l = 0; l < n; l++) {
        s2p_layer* L = &layers[l];
        snprintf(fmt, sizeof(fmt), "%s.%%d.attention.wqkv.weight", prefix);
        S2P_TRY(load_linear(m, st, qc, fmt, l, S2P_DIM, S2P_QKV_WIDTH, site, &L->wqkv));
        snprintf(fmt, sizeof(fmt), "%s.%%d.attention.wo.weight", prefix);
        S2P_TRY(load_linear(m, st, qc, fmt, l, S2P_Q_WIDTH, S2P_DIM, site, &L->wo));
        S2P_TRY(load_gate_up(m, st, qc, prefix, l, fused_suffix, site, &L->gate_up));
        snprintf(fmt, sizeof(fmt), "%s.%%d.feed_forward.w2.weight", prefix);
        S2P_TRY(load_linear(m, st, qc, fmt, l, S2P_FFN_DIM, S2P_DIM, site, &L->w2));
        snprintf(fmt, sizeof(fmt), "%s.%%d.attention_norm.weight", prefix);
        S2P_TRY(load_vec(st, fmt, l, S2P_DIM, &L->attn_norm, m->stream));
        snprintf(fmt, sizeof(fmt), "%s.%%d.ffn_norm.weight", prefix);
        S2P_TRY(load_vec(st, fmt, l, S2P_DIM, &L->ffn_norm, m->stream));
        if (qk_norm) {
            snprintf(fmt, sizeof(fmt), "%s.%%d.attention.q_norm.weight", prefix);
            S2P_TRY(load_vec(st, fmt, l, S2P_HEAD_DIM, &L->q_norm, m->stream));
            snprintf(fmt, sizeof(fmt), "%s.%%d.attention.k_norm.weight", prefix);
            S2P_TRY(load_vec(st, fmt, l, S2P_HEAD_DIM, &L->k_norm, m->stream));
        }
    }
    return S2P_OK;
}

static s2p_status alloc2(s2p_tensor* t, int64_t r, int64_t c, s2p_dtype dt) {
    const int64_t shape[2] = {r, c};
    return s2p_tensor_device_alloc(t, dt, 2, shape);
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) & ~(a - 1); }

static s2p_status alloc_workspace(s2p_model* m) {
    const int64_t ctx = m->ctx_len, B = m->max_sessions;
    int64_t pr = 2048; /* longest single prefill pass (src/slowar/model.c:99-112) */
    const char* e = getenv("S2P_SCRATCH_ROWS");
    if (e && atoi(e) > 0) pr = atoi(e);
    if (pr > ctx) pr = ctx;
    m->scratch_rows = (int)pr;
    const int64_t rows = pr > B ? pr : B;
    S2P_TRY(alloc2(&m->sx, rows, S2P_DIM, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->snorm, rows, S2P_DIM, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->sqkv, rows, S2P_QKV_WIDTH, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->sq, rows, S2P_Q_WIDTH, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->sattn, rows, S2P_Q_WIDTH, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->sproj, rows, S2P_DIM, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->sgu, rows, GU_ROWS, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->sffn, rows, S2P_FFN_DIM, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->shidden, B, S2P_DIM, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->slogc, B, 4096, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->sloge, B, 1, S2P_DT_BF16));
    m->head_full = s2p_env_is_one("S2P_HEAD_FULL") || m->mode != S2P_GEMM_INT8 || getenv("S2P_DUMP_DIR") != NULL;
    if (m->head_full) S2P_TRY(alloc2(&m->slogits, B, S2P_TEXT_VOCAB, S2P_DT_BF16));
    {
        const int64_t n1[1] = {ctx};
        S2P_TRY(s2p_tensor_device_alloc(&m->sids, S2P_DT_I64, 1, n1));
        const int64_t n2[1] = {(int64_t)S2P_NUM_CODEBOOKS * ctx};
        S2P_TRY(s2p_tensor_device_alloc(&m->svq, S2P_DT_I32, 1, n2));
    }
    /* split-K partials [B][32][ctx/64][130] f32 and the per-(row, kv head) arrival counters */
    m->n_split_slots = (int)((ctx + 63) / 64);
    {
        const int64_t n[1] = {B * S2P_SLOW_Q_HEADS * (int64_t)m->n_split_slots * (S2P_HEAD_DIM + 2)};
        S2P_TRY(s2p_tensor_device_alloc(&m->attn_part, S2P_DT_F32, 1, n));
        S2P_CUDA_TRY(cudaMalloc((void**)&m->attn_ctr, (size_t)B * S2P_SLOW_KV_HEADS * sizeof(unsigned int)));
        S2P_CUDA_TRY(cudaMemset(m->attn_ctr, 0, (size_t)B * S2P_SLOW_KV_HEADS * sizeof(unsigned int)));
    }
    /* fast-AR */
    S2P_TRY(alloc2(&m->fx, B, S2P_DIM, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->ft, B, S2P_DIM, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->fqkv, B, S2P_QKV_WIDTH, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->fq, B, S2P_Q_WIDTH, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->fattn, B, S2P_Q_WIDTH, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->fproj, B, S2P_DIM, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->fgu, B, GU_ROWS, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->fhff, B, S2P_FFN_DIM, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->flogits, B, S2P_CB_SIZE, S2P_DT_BF16));
    S2P_TRY(alloc2(&m->fkv, (int64_t)S2P_FAST_LAYERS * B, 2 * FA_KVSZ, S2P_DT_BF16));
    S2P_CUDA_TRY(cudaMemset(m->fkv.data, 0, m->fkv.bytes));
    S2P_CUDA_TRY(cudaMalloc((void**)&m->fstage, (size_t)9 * B * sizeof(int32_t)));
    S2P_CUDA_TRY(cudaMalloc((void**)&m->fcodes, (size_t)B * sizeof(int32_t)));
    S2P_CUDA_TRY(cudaMalloc((void**)&m->fkeys, (size_t)9 * B * sizeof(unsigned long long)));
    S2P_CUDA_TRY(cudaMemset(m->fkeys, 0, (size_t)9 * B * sizeof(unsigned long long)));

    /* per-tick upload block: pointer tables first (natural alignment), then ids, codes, pos, mask */
    size_t off = 0;
    m->off_kvb = off;  off += (size_t)B * sizeof(void*);
    m->off_kvsb = off; off += (size_t)B * sizeof(void*);
    m->off_samp = off; off += (size_t)B * sizeof(void*);
    m->off_ids = off;  off += (size_t)B * sizeof(int64_t);
    m->off_codes = off; off += (size_t)B * S2P_NUM_CODEBOOKS * sizeof(int32_t);
    m->off_pos = off;  off += (size_t)B * sizeof(int32_t);
    m->off_mask = off; off += (size_t)B;
    m->up_bytes = align_up(off, 16);
    S2P_CUDA_TRY(cudaMalloc(&m->d_up, m->up_bytes));
    S2P_CUDA_TRY(cudaMallocHost(&m->h_up, m->up_bytes));
    memset(m->h_up, 0, m->up_bytes);
    /* result block: i64 tok[B] | i32 sem[B] | i32 codes[10B] | u8 eos[B] */
    m->off_sem = (size_t)B * sizeof(int64_t);
    m->off_ocodes = m->off_sem + (size_t)B * sizeof(int32_t);
    m->off_eos = m->off_ocodes + (size_t)B * S2P_NUM_CODEBOOKS * sizeof(int32_t);
    m->out_bytes = align_up(m->off_eos + (size_t)B, 16);
    S2P_CUDA_TRY(cudaMalloc(&m->d_out, m->out_bytes));
    S2P_CUDA_TRY(cudaMallocHost(&m->h_out, m->out_bytes));
    return S2P_OK;
}

static int count_backbone_layers(s2p_st* st) {
    int n = 0;
    for (; n < S2P_SLOW_LAYERS; n++) {
        char name[160];
        s2p_st_view v;
        snprintf(name, sizeof(name), "text_model.model.layers.%d.attention.wqkv.weight", n);
        if (s2p_st_find(st, name, &v) != S2P_OK) break;
    }
    return n;
}

s2p_status s2p_model_load(const char* model_dir, const s2p_model_opts* opts, s2p_model** out) {
    if (!model_dir || !out) return S2P_ERR_INVALID;
    *out = NULL;
    {
        const char* dv = getenv("S2P_DEVICE");
        if (dv && dv[0]) S2P_CUDA_TRY(cudaSetDevice(atoi(dv)));
    }
    s2p_model* m = (s2p_model*)calloc(1, sizeof(*m));
    if (!m) return S2P_ERR_OOM;
    m->mode = opts ? opts->gemm_mode : S2P_GEMM_BF16;
    m->ctx_len = (opts && opts->ctx_len > 0) ? opts->ctx_len : S2P_CTX_LEN_DEFAULT;
    m->max_sessions = (opts && opts->max_sessions > 0) ? opts->max_sessions : S2P_MAX_SESSIONS;
    if (m->max_sessions > S2P_MAX_BATCH) m->max_sessions = S2P_MAX_BATCH;
    if (m->ctx_len > S2P_MAX_SEQ) { free(m); return S2P_ERR_INVALID; }
    if (m->mode == S2P_GEMM_FP8) {
        fprintf(stderr, "[s2pro] FP8 gemm requested but unavailable; falling back to BF16\n");
        m->mode = S2P_GEMM_BF16;
    }
    {   /* INT8 KV cache: on by default in the quantised mode (src/slowar/model.c:201-215) */
        const char* e = getenv("S2P_KV8");
        m->kv8 = (e && e[0]) ? (e[0] == '1' && e[1] == '\0') : (m->mode == S2P_GEMM_INT8);
        if (s2p_env_is_one("S2P_KV4"))
            fprintf(stderr, "[s2pro] S2P_KV4 is not served (measured out upstream); using INT8 KV\n");
        if (m->kv8) fprintf(stderr, "[s2pro] S2P_KV8: INT8 KV cache (g32 per head vector, f16 scales)\n");
    }
    m->tp_world = 1;
    m->fused_b1 = (m->mode == S2P_GEMM_INT8) && !s2p_env_is_one("S2P_NO_FUSED");

    s2p_status rc;
    s2p_st* st = NULL;
    s2p_qcache* qc = NULL;
    if ((rc = s2p_gemm_init(m->ctx_len)) != S2P_OK) goto fail;
    if (gemv_setup_all() != cudaSuccess) { rc = S2P_ERR_CUDA; goto fail; }
    if (m->max_sessions > 1 && skinny_setup(m->max_sessions) != cudaSuccess) { rc = S2P_ERR_OOM; goto fail; }
    if (m->fused_b1 && !s2p_env_is_one("S2P_NO_MEGA")) {
        if (mega_setup(&m->mega_ctas) == cudaSuccess && cudaMalloc(&m->tp_arena, S2P_TP_ARENA_BYTES) == cudaSuccess &&
            cudaMemset(m->tp_arena, 0, S2P_TP_ARENA_BYTES) == cudaSuccess) {
            m->mega_ok = 1;
            m->tp_base[0] = m->tp_arena;
        }
        else {
            (void)cudaGetLastError();
            fprintf(stderr, "[s2pro] persistent tick kernel unavailable on this device; using per-stage launches\n");
        }
    }
    if ((rc = s2p_qcache_open(model_dir, m->mode, &qc)) != S2P_OK) goto fail;
    if (cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking) != cudaSuccess) { rc = S2P_ERR_CUDA; goto fail; }
    if ((rc = s2p_st_open_dir(model_dir, &st)) != S2P_OK) goto fail;

    {
        const int64_t eshape[2] = {S2P_TEXT_VOCAB, S2P_DIM};
        rc = s2p_st_load_device(st, "text_model.model.embeddings.weight", S2P_DT_BF16, 2, eshape, &m->embed, m->stream);
        if (rc != S2P_OK) goto fail;
    }
    if (m->mode == S2P_GEMM_INT8) {
        /* per-row INT8 sidecar of the tied head; it also serves the embedding lookups
         * unless S2P_EMBED_BF16=1 keeps the bf16 table (src/slowar/model.c:243-271) */
        const int64_t qshape[2] = {S2P_TEXT_VOCAB, S2P_DIM}, sshape[1] = {S2P_TEXT_VOCAB};
        rc = s2p_tensor_device_alloc(&m->embed_i8, S2P_DT_I8, 2, qshape);
        if (rc == S2P_OK) rc = s2p_tensor_device_alloc(&m->embed_scale, S2P_DT_F32, 1, sshape);
        if (rc == S2P_OK)
            rc = s2p_int8_quant(m->embed_i8.data, (float*)m->embed_scale.data, m->embed.data, S2P_TEXT_VOCAB, S2P_DIM,
                                m->stream);
        if (rc != S2P_OK) goto fail;
        if (!s2p_env_is_one("S2P_EMBED_BF16")) {
            if (cudaStreamSynchronize(m->stream) != cudaSuccess) { rc = S2P_ERR_CUDA; goto fail; }
            s2p_tensor_free(&m->embed);
            m->embed_i8_only = 1;
            fprintf(stderr, "[s2pro] embed: bf16 table dropped, int8 sidecar serves lookups\n");
        }
    }
    m->n_slow = count_backbone_layers(st);
    if (m->n_slow < 1) { rc = S2P_ERR_FORMAT; goto fail; }
    if (m->n_slow != S2P_SLOW_LAYERS)
        fprintf(stderr, "[s2pro] checkpoint holds %d backbone layers (full model: %d)\n", m->n_slow, S2P_SLOW_LAYERS);
    rc = load_stack(m, st, qc, m->slow, m->n_slow, "text_model.model.layers", 1, "gate_up.fused", S2P_QSITE_BACKBONE);
    if (rc != S2P_OK) goto fail;
    {
        const int64_t nshape[1] = {S2P_DIM};
        rc = s2p_st_load_device(st, "text_model.model.norm.weight", S2P_DT_BF16, 1, nshape, &m->final_norm, m->stream);
        if (rc != S2P_OK) goto fail;
    }
    rc = load_stack(m, st, qc, m->fast, S2P_FAST_LAYERS, "audio_decoder.layers", 0, "w13.fused", S2P_QSITE_FASTAR);
    if (rc != S2P_OK) goto fail;
    {
        const int64_t nshape[1] = {S2P_DIM};
        rc = s2p_st_load_device(st, "audio_decoder.norm.weight", S2P_DT_BF16, 1, nshape, &m->fast_norm, m->stream);
        if (rc != S2P_OK) goto fail;
        const char* oname = "audio_decoder.output.weight";
        if (!s2p_qcache_try_load(qc, oname, S2P_DIM, S2P_CB_SIZE, &m->fast_out, m->stream)) {
            rc = s2p_linear_from_st(&m->fast_out, st, oname, S2P_DIM, S2P_CB_SIZE, m->stream);
            if (rc == S2P_OK) rc = finish_linear(m, qc, oname, &m->fast_out, S2P_QSITE_FASTAR);
            if (rc != S2P_OK) goto fail;
        }
        const int64_t cshape[2] = {(int64_t)S2P_NUM_CODEBOOKS * S2P_CB_SIZE, S2P_DIM};
        rc = s2p_st_load_device(st, "audio_decoder.codebook_embeddings.weight", S2P_DT_BF16, 2, cshape, &m->cb_emb,
                                m->stream);
        if (rc != S2P_OK) goto fail;
        const int64_t fshape[2] = {S2P_CB_SIZE, S2P_DIM};
        rc = s2p_st_load_device(st, "audio_decoder.embeddings.weight", S2P_DT_BF16, 2, fshape, &m->fast_emb, m->stream);
        if (rc != S2P_OK) goto fail;
    }
    if ((rc = alloc_workspace(m)) != S2P_OK) goto fail;
    if (cudaEventCreate(&m->ev0) != cudaSuccess || cudaEventCreate(&m->ev1) != cudaSuccess) { rc = S2P_ERR_CUDA; goto fail; }
    if (cudaStreamSynchronize(m->stream) != cudaSuccess) { rc = S2P_ERR_CUDA; goto fail; }
    s2p_st_close(st);
    st = NULL;
    rc = s2p_qcache_finish(qc, m->stream);
    s2p_qcache_free(qc);
    qc = NULL;
    if (rc != S2P_OK) goto fail;
    *out = m;
    return S2P_OK;

fail:
    if (st) {
        if (m->stream) cudaStreamSynchronize(m->stream);
        s2p_st_close(st);
    }
    s2p_qcache_free(qc);
    s2p_model_free(m);
    return rc;
}

static void free_layer(s2p_layer* L) {
    s2p_linear_free(&L->wqkv); s2p_linear_free(&L->wo); s2p_linear_free(&L->gate_up); s2p_linear_free(&L->w2);
    s2p_tensor_free(&L->attn_norm); s2p_tensor_free(&L->ffn_norm);
    s2p_tensor_free(&L->q_norm); s2p_tensor_free(&L->k_norm);
}

void s2p_model_free(s2p_model* m) {
    if (!m) return;
    if (m->stream) cudaStreamSynchronize(m->stream);
    for (int b = 0; b <= S2P_MAX_BATCH; b++)
        if (m->gready[b]) cudaGraphExecDestroy(m->gexec[b]);
    for (int l = 0; l < S2P_SLOW_LAYERS; l++) free_layer(&m->slow[l]);
    for (int l = 0; l < S2P_FAST_LAYERS; l++) free_layer(&m->fast[l]);
    s2p_tensor* ts[] = {&m->embed, &m->embed_i8, &m->embed_scale, &m->final_norm, &m->fast_norm, &m->cb_emb,
                        &m->fast_emb, &m->sx, &m->snorm, &m->sqkv, &m->sq, &m->sattn, &m->sproj, &m->sgu, &m->sffn,
                        &m->shidden, &m->slogc, &m->sloge, &m->slogits, &m->sids, &m->svq, &m->attn_part, &m->fx,
                        &m->ft, &m->fqkv, &m->fq, &m->fattn, &m->fproj, &m->fgu, &m->fhff, &m->flogits, &m->fkv};
    for (size_t i = 0; i < sizeof(ts) / sizeof(ts[0]); i++) s2p_tensor_free(ts[i]);
    s2p_linear_free(&m->fast_out);
    if (m->attn_ctr) cudaFree(m->attn_ctr);
    if (m->d_mega_stages) cudaFree(m->d_mega_stages);
    if (m->d_mega_sync) cudaFree(m->d_mega_sync);
    for (int r = 0; r < m->tp_world; r++)
        if (r != m->tp_rank && m->tp_base[r]) cudaIpcCloseMemHandle(m->tp_base[r]);
    if (m->tp_arena) cudaFree(m->tp_arena);
    if (m->d_mega_cmds) cudaFree(m->d_mega_cmds);
    if (m->d_mega_cmd_start) cudaFree(m->d_mega_cmd_start);
    if (m->h_mega_status) cudaFreeHost(m->h_mega_status);
    if (m->d_mega_trace) cudaFree(m->d_mega_trace);
    free(m->mega_types);
    if (m->fstage) cudaFree(m->fstage);
    if (m->fcodes) cudaFree(m->fcodes);
    if (m->fkeys) cudaFree(m->fkeys);
    if (m->d_up) cudaFree(m->d_up);
    if (m->h_up) cudaFreeHost(m->h_up);
    if (m->d_out) cudaFree(m->d_out);
    if (m->h_out) cudaFreeHost(m->h_out);
    if (m->ev0) cudaEventDestroy(m->ev0);
    if (m->ev1) cudaEventDestroy(m->ev1);
    if (m->stream) cudaStreamDestroy(m->stream);
    free(m);
}

/* ---- measurement hooks (include/s2p_b200_ext.h) ------------------------------ */
static double linear_bytes(const s2p_linear* lin) {
    return (double)lin->w_int8.bytes + (double)lin->w_pack.bytes + (double)lin->w_iscale.bytes +
           (lin->int8_ready ? 0.0 : (double)lin->w_bf16.bytes);
}
static double layer_bytes(const s2p_layer* L) {
    return linear_bytes(&L->wqkv) + linear_bytes(&L->wo) + linear_bytes(&L->gate_up) + linear_bytes(&L->w2);
}

s2p_status s2p_b200_model_stats(const s2p_model* m, s2p_b200_stats* out) {
    if (!m || !out) return S2P_ERR_INVALID;
    memset(out, 0, sizeof(*out));
    out->frames_decoded = m->frames_decoded;
    out->n_slow_layers = m->n_slow;
    out->last_tick_rows = m->last_rows;
    out->last_tick_fused = m->last_fused;
    out->last_tick_graph = m->last_graph;
    out->last_tick_kernels = m->last_kernels;
    out->last_tick_persistent = m->last_mega;
    out->last_tick_device_ms = m->last_device_ms;
    out->upload_bytes = m->up_bytes;
    out->download_bytes = m->out_bytes;
    /* one frame reads: every backbone linear once, every fast-AR linear ten times (prime + 9 steps),
     * the fast head nine times, and the 4096 + 1 sampled rows of the tied head */
    double w = 0.0;
    for (int l = 0; l < m->n_slow; l++) w += layer_bytes(&m->slow[l]);
    for (int l = 0; l < S2P_FAST_LAYERS; l++) w += 10.0 * layer_bytes(&m->fast[l]);
    w += 9.0 * linear_bytes(&m->fast_out);
    if (m->mode == S2P_GEMM_INT8 && !m->head_full) w += 4097.0 * (S2P_DIM + 4);
    else w += (double)S2P_TEXT_VOCAB * S2P_DIM * (m->mode == S2P_GEMM_INT8 ? 1.0 : 2.0);
    out->weight_bytes_per_frame = w;
    out->kv_bytes_per_token = (double)m->n_slow * S2P_KV_PLANES_PER_LAYER *
                              (m->kv8 ? S2P_HEAD_DIM + (S2P_HEAD_DIM / 32) * 2 : S2P_HEAD_DIM * 2);
    return S2P_OK;
}

cudaStream_t s2p_b200_model_stream(s2p_model* m) { return m ? m->stream : NULL; }
