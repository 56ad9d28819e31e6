/* Test infrastructure: stand-ins for the parts of the reference that its scheduler
 * (src/sched/scheduler.c of the reference) calls besides the model API - the prompt builder, the
 * vocoder's streaming interface, the voice registry and the float -> S16 helper.  They are
 * deterministic functions of their inputs and touch no GPU, so a scheduler binary linked with
 * either model library produces the same audio callbacks exactly when the model API returned the
 * same frame codes.
 *
 * Prompt stand-in: with reference clips the prompt opens with a "system block"
 *   [3 fixed ids] + per clip: T ids S2P_SEMANTIC_ID(codes[0][t]) with vq_mask = 1 + [2 fixed ids]
 * (n_sys_ids = its length, the key of the scheduler's KV-prefix cache); then one id per byte of the
 * transcript and of the text.  Vocoder stand-in: a pushed frame becomes a 2048-sample chunk whose
 * first ten samples encode the frame's ten codes exactly (code / 8192 is exact in float and in S16
 * after the x32767 rounding for codes < 4096, see s2p_f32_to_s16 below).
 */
#include <math.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "s2pro/status.h"
#include "s2pro/config.h"
#include "s2pro/dac.h"
#include "s2pro/tokenizer.h"
#include "s2pro/voices.h"
#include "s2pro/wav.h"

/* ---- admission gate ------------------------------------------------------------------------
 * The scheduler admits a request as soon as its worker sees it, so how many sessions share the
 * first ticks would depend on thread timing.  The caller closes this gate, submits a group of
 * requests and opens it: the worker blocks in the prompt builder of the first one until the whole
 * group is queued, which makes the composition of every lockstep batch reproducible. */
static pthread_mutex_t g_gate_mu = PTHREAD_MUTEX_INITIALIZER;
static pthread_cond_t  g_gate_cv = PTHREAD_COND_INITIALIZER;
static int             g_gate_closed;

void dropin_gate(int closed) {
    pthread_mutex_lock(&g_gate_mu);
    g_gate_closed = closed;
    pthread_cond_broadcast(&g_gate_cv);
    pthread_mutex_unlock(&g_gate_mu);
}
static void gate_pass(void) {
    pthread_mutex_lock(&g_gate_mu);
    while (g_gate_closed) pthread_cond_wait(&g_gate_cv, &g_gate_mu);
    pthread_mutex_unlock(&g_gate_mu);
}

/* ---- prompt ------------------------------------------------------------------------------ */

s2p_status s2p_prompt_build(s2p_tok* t, const s2p_config* cfg, const s2p_request_text* req, int64_t** ids, uint8_t** vq_mask,
                            int* n_ids, s2p_vq_part** parts, int* n_parts, int* n_sys_ids) {
    (void)t; (void)cfg;
    gate_pass();
    if (!req || !req->text || !ids || !vq_mask || !n_ids || !parts || !n_parts) return S2P_ERR_INVALID;
    size_t n = 0, n_sys = 0;
    if (req->n_refs > 0) {
        n_sys = 3;
        for (int i = 0; i < req->n_refs; i++) n_sys += (size_t)req->refs[i].T + 2;
    }
    const size_t n_ref_text = req->ref_text ? strlen(req->ref_text) : 0, n_text = strlen(req->text);
    n = n_sys + n_ref_text + n_text + 2;
    int64_t* id = (int64_t*)malloc(n * sizeof(int64_t));
    uint8_t* mk = (uint8_t*)calloc(n, 1);
    s2p_vq_part* pt = req->n_refs > 0 ? (s2p_vq_part*)malloc((size_t)req->n_refs * sizeof(s2p_vq_part)) : NULL;
    if (!id || !mk || (req->n_refs > 0 && !pt)) {
        free(id); free(mk); free(pt);
        return S2P_ERR_OOM;
    }
    size_t p = 0;
    if (req->n_refs > 0) {
        id[p++] = 11; id[p++] = 12; id[p++] = 13;
        for (int i = 0; i < req->n_refs; i++) {
            pt[i] = req->refs[i]; /* the codes stay the request's */
            for (int f = 0; f < req->refs[i].T; f++) {
                mk[p] = 1;
                id[p++] = S2P_SEMANTIC_ID(req->refs[i].codes[f] & (S2P_CB_SIZE - 1));
            }
            id[p++] = 14; id[p++] = 15;
        }
    }
    for (size_t i = 0; i < n_ref_text; i++) id[p++] = 2000 + (unsigned char)req->ref_text[i];
    id[p++] = 16;
    for (size_t i = 0; i < n_text; i++) id[p++] = 1000 + (unsigned char)req->text[i];
    id[p++] = 17;
    *ids = id; *vq_mask = mk; *n_ids = (int)p;
    *parts = pt; *n_parts = req->n_refs;
    if (n_sys_ids) *n_sys_ids = (int)n_sys;
    return S2P_OK;
}

/* ---- vocoder streams ------------------------------------------------------------------------ */

struct s2p_dac_stream {
    int     pending;
    int32_t codes[S2P_NUM_CODEBOOKS];
    long    pushed;
};

s2p_status s2p_dac_stream_create(s2p_dac* d, s2p_dac_stream** out) {
    (void)d;
    if (!out) return S2P_ERR_INVALID;
    *out = (s2p_dac_stream*)calloc(1, sizeof(s2p_dac_stream));
    return *out ? S2P_OK : S2P_ERR_OOM;
}

s2p_status s2p_dac_stream_push_async(s2p_dac_stream* s, const int32_t frame_codes[S2P_NUM_CODEBOOKS], cudaStream_t stream) {
    (void)stream;
    if (!s || !frame_codes) return S2P_ERR_INVALID;
    if (s->pending) return S2P_ERR_STATE; /* one frame in flight per stream */
    memcpy(s->codes, frame_codes, sizeof(s->codes));
    s->pending = 1;
    s->pushed++;
    return S2P_OK;
}

s2p_status s2p_dac_stream_push_batch(s2p_dac_stream* const* strs, int nb, const int32_t* frame_codes, cudaStream_t stream) {
    for (int i = 0; i < nb; i++) {
        const s2p_status rc = s2p_dac_stream_push_async(strs[i], frame_codes + (size_t)i * S2P_NUM_CODEBOOKS, stream);
        if (rc != S2P_OK) return rc;
    }
    return S2P_OK;
}

s2p_status s2p_dac_stream_collect(s2p_dac_stream* s, float** pcm_chunk, int64_t* n_out, cudaStream_t stream) {
    (void)stream;
    if (!s || !pcm_chunk || !n_out) return S2P_ERR_INVALID;
    *pcm_chunk = NULL;
    *n_out = 0;
    if (!s->pending) return S2P_OK;
    float* pcm = (float*)malloc(S2P_FRAME_SAMPLES * sizeof(float));
    if (!pcm) return S2P_ERR_OOM;
    for (int i = 0; i < S2P_FRAME_SAMPLES; i++) pcm[i] = 0.0f;
    for (int c = 0; c < S2P_NUM_CODEBOOKS; c++) pcm[c] = (float)s->codes[c] / 8192.0f;
    pcm[S2P_NUM_CODEBOOKS] = (float)(s->pushed & 1023) / 8192.0f;
    s->pending = 0;
    *pcm_chunk = pcm;
    *n_out = S2P_FRAME_SAMPLES;
    return S2P_OK;
}

s2p_status s2p_dac_stream_push(s2p_dac_stream* s, const int32_t frame_codes[S2P_NUM_CODEBOOKS], float** pcm_chunk, int64_t* n_out,
                               cudaStream_t stream) {
    const s2p_status rc = s2p_dac_stream_push_async(s, frame_codes, stream);
    return rc != S2P_OK ? rc : s2p_dac_stream_collect(s, pcm_chunk, n_out, stream);
}

s2p_status s2p_dac_stream_finish(s2p_dac_stream* s, float** pcm_chunk, int64_t* n_out, cudaStream_t stream) {
    (void)stream;
    if (!s || !pcm_chunk || !n_out) return S2P_ERR_INVALID;
    *pcm_chunk = NULL; /* the incremental engine has no tail */
    *n_out = 0;
    return S2P_OK;
}

void s2p_dac_stream_destroy(s2p_dac_stream* s) { free(s); }

/* Clone encode stand-in: one frame per 2048 samples, every code a function of the frame's first sample. */
s2p_status s2p_dac_encode(s2p_dac* d, const float* pcm, int64_t n_samples, int32_t** codes_out, int* T_out, cudaStream_t stream) {
    (void)d; (void)stream;
    if (!pcm || n_samples < S2P_FRAME_SAMPLES || !codes_out || !T_out) return S2P_ERR_INVALID;
    const int T = (int)(n_samples / S2P_FRAME_SAMPLES);
    int32_t* codes = (int32_t*)malloc((size_t)S2P_NUM_CODEBOOKS * T * sizeof(int32_t));
    if (!codes) return S2P_ERR_OOM;
    for (int c = 0; c < S2P_NUM_CODEBOOKS; c++)
        for (int f = 0; f < T; f++) {
            const int v = (int)lrintf(fabsf(pcm[(size_t)f * S2P_FRAME_SAMPLES]) * 4095.0f);
            codes[(size_t)c * T + f] = (v * 31 + c * 397 + f * 7) & (S2P_CB_SIZE - 1);
        }
    *codes_out = codes;
    *T_out = T;
    return S2P_OK;
}

/* ---- voice registry: the caller fills this table before s2p_sched_warm_voices ------------- */

struct s2p_voices {
    int       n;
    s2p_voice v[8];
};
static struct s2p_voices g_voices;

struct s2p_voices* dropin_voices(void) { return &g_voices; }
int dropin_voices_add(const char* name, const char* transcript, const int32_t* codes, int T) {
    if (g_voices.n >= 8) return -1;
    s2p_voice* v = &g_voices.v[g_voices.n++];
    v->name = name; v->transcript = transcript;
    v->part.codes = codes; v->part.T = T;
    v->duration_s = (double)T * S2P_FRAME_SAMPLES / S2P_SAMPLE_RATE;
    return 0;
}
int s2p_voices_count(const s2p_voices* v) { return v ? v->n : 0; }
const s2p_voice* s2p_voices_at(const s2p_voices* v, int i) { return (v && i >= 0 && i < v->n) ? &v->v[i] : NULL; }

/* ---- float -> S16 (include/s2pro/wav.h:29 of the reference: NaN -> 0, clip to [-1, 1], scale by 32767, round halves away from zero) ---- */

void s2p_f32_to_s16(const float* in, int16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; i++) {
        float v = in[i];
        if (isnan(v)) v = 0.0f;
        v = fminf(1.0f, fmaxf(-1.0f, v));
        out[i] = (int16_t)lroundf(v * 32767.0f); /* halves away from zero */
    }
}
