/* Test infrastructure: drives the reference's own request scheduler (src/sched/scheduler.c of the
 * reference, compiled unchanged from where it lies) on top of a model library - this repository's
 * or the reference's - with the vocoder, prompt builder and voice registry replaced by the
 * deterministic stand-ins of sched_stubs.c.  Both binaries must print the same lines.
 *
 *   sched_caller <checkpoint dir> <frames per request>
 *
 * Group 1 (admitted together): a text-only greedy request; a request for a pre-warmed registry
 * voice (KV prefix loaded from the scheduler's cache); a request with its own 120-frame reference
 * clip (VQ rows in a chunked prefill); an on-the-fly clone from PCM with a cache key.
 * Group 2: the same clone key again (cache hit on the entry group 1 inserted) and a second text-only
 * request, sampled.  Every request ends by the callback reporting "client gone" after <frames>
 * chunks unless its stream ends earlier.
 */
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include "s2pro/status.h"
#include "s2pro/config.h"
#include "s2pro/model.h"
#include "s2pro/scheduler.h"
#include "s2pro/voices.h"

/* from sched_stubs.c */
void dropin_gate(int closed);
struct s2p_voices* dropin_voices(void);
int dropin_voices_add(const char* name, const char* transcript, const int32_t* codes, int T);

#define MAX_FRAMES 64
typedef struct {
    const char* tag;
    int         want;
    int         n_chunks, n_final, bad;
    int         codes[MAX_FRAMES][S2P_NUM_CODEBOOKS];
    int         serial[MAX_FRAMES];
} Sink;

static pthread_mutex_t g_mu = PTHREAD_MUTEX_INITIALIZER;
static pthread_cond_t  g_cv = PTHREAD_COND_INITIALIZER;

static int on_audio(void* user, const int16_t* pcm, int64_t n, int final) {
    Sink* k = (Sink*)user;
    int gone = 0;
    pthread_mutex_lock(&g_mu);
    if (n > 0 && pcm) {
        if (n != S2P_FRAME_SAMPLES || k->n_chunks >= MAX_FRAMES) k->bad++;
        else {
            for (int c = 0; c < S2P_NUM_CODEBOOKS; c++) k->codes[k->n_chunks][c] = pcm[c] / 4; /* the stand-in vocoder's encoding */
            k->serial[k->n_chunks] = pcm[S2P_NUM_CODEBOOKS] / 4;
            k->n_chunks++;
        }
    }
    if (final) k->n_final++;
    else if (k->n_chunks >= k->want) gone = 1; /* "client gone": the scheduler retires the session, no final call follows */
    if (final || gone) pthread_cond_broadcast(&g_cv);
    pthread_mutex_unlock(&g_mu);
    return gone;
}

static void wait_done(Sink* k) {
    pthread_mutex_lock(&g_mu);
    while (!k->n_final && k->n_chunks < k->want) pthread_cond_wait(&g_cv, &g_mu);
    pthread_mutex_unlock(&g_mu);
}

static void report(const Sink* k) {
    printf("%s: %d chunks, %d final, %d malformed\n", k->tag, k->n_chunks, k->n_final, k->bad);
    for (int f = 0; f < k->n_chunks; f++) {
        printf("  %s frame %d (push %d): [", k->tag, f, k->serial[f]);
        for (int c = 0; c < S2P_NUM_CODEBOOKS; c++) printf(c ? ",%d" : "%d", k->codes[f][c]);
        printf("]\n");
    }
}

#define TRY(call)                                                                            \
    do {                                                                                     \
        const s2p_status rc_ = (call);                                                       \
        if (rc_ != S2P_OK) {                                                                 \
            fprintf(stderr, "%s -> %d (%s)\n", #call, (int)rc_, s2p_status_str(rc_));       \
            return 2;                                                                        \
        }                                                                                    \
    } while (0)

static void fill_codes(int32_t* codes, int T, unsigned seed) {
    unsigned st = seed * 2654435761u + 12345u;
    for (int i = 0; i < S2P_NUM_CODEBOOKS * T; i++) {
        st = st * 1664525u + 1013904223u;
        codes[i] = (int32_t)((st >> 10) & (S2P_CB_SIZE - 1));
    }
}

static void wait_idle(s2p_sched* sched) { /* retirement follows the last callback by a moment */
    for (;;) {
        s2p_sched_stats st;
        s2p_sched_get_stats(sched, &st);
        if (st.active_sessions == 0 && st.queued == 0) return;
        struct timespec ts = {0, 2000000};
        nanosleep(&ts, NULL);
    }
}

int main(int argc, char** argv) {
    if (argc < 3) {
        fprintf(stderr, "usage: %s <checkpoint dir> <frames per request>\n", argv[0]);
        return 1;
    }
    const int want = atoi(argv[2]);
    if (want < 1 || want > MAX_FRAMES) return 1;

    s2p_model_opts opts;
    memset(&opts, 0, sizeof(opts));
    opts.gemm_mode = S2P_GEMM_INT8;
    opts.ctx_len = 1024;
    opts.max_sessions = 8;
    s2p_model* model = NULL;
    TRY(s2p_model_load(argv[1], &opts, &model));

    static int dummy_dac, dummy_tok; /* opaque to the scheduler; the stand-ins never look inside */
    s2p_sched_opts so = {8, 16};
    s2p_sched* sched = NULL;
    TRY(s2p_sched_create(model, (s2p_dac*)&dummy_dac, (s2p_tok*)&dummy_tok, NULL, &so, &sched));

    static int32_t voice_codes[S2P_NUM_CODEBOOKS * 40], clip_codes[S2P_NUM_CODEBOOKS * 120];
    fill_codes(voice_codes, 40, 1);
    fill_codes(clip_codes, 120, 2);
    if (dropin_voices_add("narrator", "a registry voice transcript", voice_codes, 40)) return 3;
    TRY(s2p_sched_warm_voices(sched, dropin_voices()));
    TRY(s2p_sched_start(sched));

    static float clone_pcm[S2P_FRAME_SAMPLES * 30];
    for (int i = 0; i < S2P_FRAME_SAMPLES * 30; i++) clone_pcm[i] = (float)((i * 37) % 2001 - 1000) / 1000.0f;

    static const char* const tags[6] = {"text-greedy", "registry-voice", "own-clip", "clone-first", "clone-again", "text-sampled"};
    static Sink sink[6];
    for (int i = 0; i < 6; i++) {
        sink[i].tag = tags[i];
        sink[i].want = want;
    }
    s2p_request_text rq[6];
    s2p_sampling_cfg sc[6];
    memset(rq, 0, sizeof(rq));
    for (int i = 0; i < 6; i++) {
        sc[i] = s2p_sampling_defaults();
        sc[i].seed = 500 + (uint64_t)i;
    }
    sc[0].temperature = 0.0f;
    rq[0].text = "The first request has no reference audio at all.";
    const s2p_vq_part voice_part = {voice_codes, 40}, clip_part = {clip_codes, 120};
    rq[1].text = "A registry voice speaks this sentence.";
    rq[1].ref_text = "a registry voice transcript";
    rq[1].refs = &voice_part; rq[1].n_refs = 1; rq[1].cache_key = "narrator";
    rq[2].text = "This one brings its own clip, longer than one prefill chunk.";
    rq[2].ref_text = "the clip's transcript";
    rq[2].refs = &clip_part; rq[2].n_refs = 1;
    s2p_vq_part memo = {NULL, 0};
    rq[3].text = "Cloned on the fly from raw samples.";
    rq[3].ref_text = "what the samples say";
    rq[3].ref_pcm = clone_pcm; rq[3].ref_pcm_n = S2P_FRAME_SAMPLES * 30; rq[3].cache_key = "clone-1";
    rq[3].clone_codes_out = &memo;

    dropin_gate(1);
    for (int i = 0; i < 4; i++) TRY(s2p_sched_submit(sched, &rq[i], &sc[i], on_audio, &sink[i], NULL));
    dropin_gate(0);
    for (int i = 0; i < 4; i++) wait_done(&sink[i]);
    wait_idle(sched);

    if (!memo.codes || memo.T != 30) {
        fprintf(stderr, "the scheduler did not hand back the clone's codes\n");
        return 4;
    }
    rq[4].text = "The same cloned voice again, now from the prefix cache.";
    rq[4].ref_text = "what the samples say";
    rq[4].refs = &memo; rq[4].n_refs = 1; rq[4].cache_key = "clone-1";
    rq[5].text = "And a second request without a reference.";
    dropin_gate(1);
    for (int i = 4; i < 6; i++) TRY(s2p_sched_submit(sched, &rq[i], &sc[i], on_audio, &sink[i], NULL));
    dropin_gate(0);
    for (int i = 4; i < 6; i++) wait_done(&sink[i]);
    wait_idle(sched);

    s2p_sched_stats st;
    s2p_sched_get_stats(sched, &st);
    TRY(s2p_sched_stop(sched));
    s2p_sched_destroy(sched);
    s2p_model_free(model);
    for (int i = 0; i < 6; i++) report(&sink[i]);
    printf("frames decoded %llu, requests completed %llu\n", (unsigned long long)st.frames_decoded, (unsigned long long)st.requests_done);
    free((void*)memo.codes);
    printf("done\n");
    return 0;
}
