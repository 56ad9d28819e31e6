/* Test infrastructure: a C caller written only against the reference's public headers
 * (include/s2pro/model.h of the reference).  The same object file is linked once with this
 * repository's library and once with the reference's own sources built as a library; run on
 * the same checkpoint, both binaries must print the same lines.
 *
 *   model_caller <checkpoint dir> <prompt tokens> <frames> <sessions>
 *
 * Per session: a seeded pseudo-random text-only prompt is prefilled, then <frames> lockstep
 * ticks of s2p_model_batch_next_frame over all sessions.  Output: one line per tick,
 * "tick t: [codes of session 0] eos | [codes of session 1] eos ...".
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "s2pro/status.h"
#include "s2pro/config.h"
#include "s2pro/model.h"

#define TRY(call)                                                                            \
    do {                                                                                     \
        const s2p_status rc_ = (call);                                                       \
        if (rc_ != S2P_OK) {                                                                 \
            fprintf(stderr, "%s -> %d (%s)\n", #call, (int)rc_, s2p_status_str(rc_));       \
            return 2;                                                                        \
        }                                                                                    \
    } while (0)

static uint64_t lcg(uint64_t* st) {
    *st = *st * 6364136223846793005ull + 1442695040888963407ull;
    return *st >> 33;
}

int main(int argc, char** argv) {
    if (argc < 5) {
        fprintf(stderr, "usage: %s <checkpoint dir> <prompt tokens> <frames> <sessions>\n", argv[0]);
        return 1;
    }
    const char* dir = argv[1];
    const int n_prompt = atoi(argv[2]), n_frames = atoi(argv[3]), n_sess = atoi(argv[4]);
    if (n_prompt < 1 || n_frames < 1 || n_sess < 1 || n_sess > S2P_MAX_SESSIONS) return 1;

    s2p_model_opts opts;
    memset(&opts, 0, sizeof(opts));
    opts.gemm_mode = S2P_GEMM_INT8;
    opts.ctx_len = 1024;
    opts.max_sessions = n_sess;
    s2p_model* model = NULL;
    TRY(s2p_model_load(dir, &opts, &model));

    s2p_session* sess[S2P_MAX_SESSIONS];
    for (int i = 0; i < n_sess; i++) {
        s2p_sampling_cfg cfg = s2p_sampling_defaults();
        cfg.temperature = i == 0 ? 0.0f : 0.8f; /* session 0 greedy, the others sampled */
        cfg.seed = 1000 + (uint64_t)i;
        TRY(s2p_session_create(model, &cfg, &sess[i]));
        const int n = n_prompt + 7 * i; /* ragged prompts */
        int64_t* ids = (int64_t*)malloc((size_t)n * sizeof(int64_t));
        if (!ids) return 3;
        uint64_t st = 77 + (uint64_t)i;
        for (int t = 0; t < n; t++) ids[t] = (int64_t)(lcg(&st) % 150000u); /* below the special ids */
        TRY(s2p_session_prefill(sess[i], ids, NULL, n, NULL, 0));
        free(ids);
    }

    int32_t codes[S2P_MAX_SESSIONS * S2P_NUM_CODEBOOKS];
    int eos[S2P_MAX_SESSIONS];
    for (int t = 0; t < n_frames; t++) {
        TRY(s2p_model_batch_next_frame(model, sess, n_sess, codes, eos));
        printf("tick %d:", t);
        for (int i = 0; i < n_sess; i++) {
            printf(" [");
            for (int c = 0; c < S2P_NUM_CODEBOOKS; c++) printf(c ? ",%d" : "%d", (int)codes[i * S2P_NUM_CODEBOOKS + c]);
            printf("] %d%s", eos[i], i + 1 < n_sess ? " |" : "");
        }
        printf("\n");
        for (int i = 0; i < n_sess; i++)
            if (eos[i]) { /* an ended session may not be stepped again: stop the whole run here */
                printf("stopped: session %d reached the end of its stream\n", i);
                t = n_frames;
                break;
            }
    }
    for (int i = 0; i < n_sess; i++) s2p_session_destroy(sess[i]);
    s2p_model_free(model);
    printf("done\n");
    return 0;
}
