/* Sampling defaults and sampler-state initialisation of the model contract
 * (include/s2pro/model.h:40 of the reference; values and clamping follow
 * src/slowar/sampling.c:83-112).  The draw itself runs on the device
 * (cuda/sampler.cu); the host keeps only the parameters it mirrors there. */
#include <string.h>
#include "internal.h"

s2p_sampling_cfg s2p_sampling_defaults(void) {
    s2p_sampling_cfg c;
    c.temperature = 0.8f;
    c.top_p = 0.8f;
    c.repetition_penalty = 1.1f;
    c.repetition_window = 16;
    c.seed = 0; /* unseeded */
    return c;
}

static uint64_t splitmix64(uint64_t* s) {
    uint64_t z = (*s += 0x9E3779B97F4A7C15ULL);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

void s2p_sampler_init(s2p_sampler* sp, const s2p_sampling_cfg* cfg, uint64_t entropy) {
    const s2p_sampling_cfg def = s2p_sampling_defaults();
    if (!cfg) cfg = &def;
    memset(sp, 0, sizeof(*sp));
    sp->temperature = cfg->temperature < 0.f ? 0.f : cfg->temperature;
    sp->top_p = (cfg->top_p <= 0.f || cfg->top_p > 1.f) ? 1.f : cfg->top_p;
    sp->rep_penalty = cfg->repetition_penalty > 0.f ? cfg->repetition_penalty : 1.f;
    sp->window = cfg->repetition_window > 0 ? cfg->repetition_window : 16;
    if (sp->window > 64) sp->window = 64;
    sp->seeded = cfg->seed != 0;
    sp->seed31 = (uint32_t)(cfg->seed & 0x7FFFFFFFULL);
    uint64_t sm = entropy ^ 0xD1B54A32D192ED03ULL;
    for (int i = 0; i < 4; i++) sp->rng[i] = splitmix64(&sm);
}
