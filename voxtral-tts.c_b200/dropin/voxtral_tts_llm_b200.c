/*
 * voxtral_tts_llm_b200.c - replaces the reference's voxtral_tts_llm.c when the
 * engine is built against libvoxtral_b200.so.
 *
 * Same four entry points, same signatures and side effects on tts_ctx_t
 * (voxtral_tts.h:360-363), so voxtral_tts.c links and runs unchanged:
 *   tts_llm_load            tensor names as voxtral_tts_llm.c:50-95
 *   tts_llm_kv_cache_alloc  sets kv_cache_len / kv_cache_max (voxtral_tts_llm.c:115-137);
 *                           the cache itself lives in HBM, no host copy is made
 *   tts_llm_prefill         all prompt rows on the GPU (the reference prefills on
 *                           the CPU and uploads 1.7 GB, voxtral_tts_llm.c:283-385)
 *   tts_llm_forward         one decoder step; the acoustic frame that the
 *                           orchestrator asks for next (voxtral_tts.c:302-305) is
 *                           computed in the same launch and handed over by
 *                           voxtral_tts_acoustic_b200.c
 *
 * Compile with the reference directory on the include path (-I<reference>) and
 * -DUSE_CUDA, together with the reference's other sources. There is no CPU
 * path in this file: without an initialised GPU context the calls report an
 * error and leave their outputs untouched.
 */
#include "voxtral_tts.h"
#include "voxtral_tts_kernels.h"
#include "voxtral_tts_safetensors.h"
#include "voxtral_b200_ext.h"
#include "voxtral_b200_dropin.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

vb200_pending_frame_t vb200_pending;

static uint16_t *bf16_tensor(safetensors_file_t *sf, const char *name) {
    const safetensor_t *t = safetensors_find(sf, name);
    if (!t) { fprintf(stderr, "llm: weight not found: %s\n", name); return NULL; }
    return safetensors_get_bf16_direct(sf, t);
}

static float *f32_tensor(safetensors_file_t *sf, const char *name) {
    const safetensor_t *t = safetensors_find(sf, name);
    if (!t) { fprintf(stderr, "llm: weight not found: %s\n", name); return NULL; }
    return safetensors_get_f32(sf, t);
}

int tts_llm_load(tts_decoder_t *dec, void *sf_ptr) {
    safetensors_file_t *sf = (safetensors_file_t *)sf_ptr;
    static const char *const mats[7] = {"attention.wq", "attention.wk", "attention.wv", "attention.wo",
                                        "feed_forward.w1", "feed_forward.w2", "feed_forward.w3"};
    char name[256];
    dec->tok_embeddings_bf16 = bf16_tensor(sf, "mm_audio_embeddings.tok_embeddings.weight");
    if (!dec->tok_embeddings_bf16) return -1;
    for (int i = 0; i < TTS_DEC_LAYERS; i++) {
        tts_dec_layer_t *l = &dec->layers[i];
        uint16_t **slots[7] = {&l->wq_bf16, &l->wk_bf16, &l->wv_bf16, &l->wo_bf16,
                               &l->w1_bf16, &l->w2_bf16, &l->w3_bf16};
        for (int k = 0; k < 7; k++) {
            snprintf(name, sizeof name, "layers.%d.%s.weight", i, mats[k]);
            *slots[k] = bf16_tensor(sf, name);
            if (!*slots[k]) return -1;
        }
        snprintf(name, sizeof name, "layers.%d.attention_norm.weight", i);
        l->attention_norm = f32_tensor(sf, name);
        snprintf(name, sizeof name, "layers.%d.ffn_norm.weight", i);
        l->ffn_norm = f32_tensor(sf, name);
        if (!l->attention_norm || !l->ffn_norm) return -1;
    }
    dec->norm = f32_tensor(sf, "norm.weight");
    return dec->norm ? 0 : -1;
}

int tts_llm_kv_cache_alloc(tts_ctx_t *ctx, int max_seq) {
    if (max_seq <= 0) return -1;
    ctx->kv_cache_k = NULL; /* tts_free() frees these; NULL is fine */
    ctx->kv_cache_v = NULL;
    ctx->kv_cache_len = 0;
    ctx->kv_cache_max = max_seq; /* passed on to tts_cuda_init (voxtral_tts.c:96) */
    return 0;
}

void tts_llm_prefill(tts_ctx_t *ctx, const float *embeds, int seq_len) {
    if (!tts_cuda_available()) {
        fprintf(stderr, "llm: no GPU context; this build has no CPU decoder\n");
        return;
    }
    vb200_pending.valid = 0;
    tts_cuda_llm_prefill(embeds, seq_len, ctx->kv_cache_len);
    ctx->kv_cache_len += seq_len;
}

void tts_llm_forward(tts_ctx_t *ctx, const float *input_embed, float *out_hidden) {
    if (!tts_cuda_available()) {
        fprintf(stderr, "llm: no GPU context; this build has no CPU decoder\n");
        return;
    }
    /* Draw this frame's noise from a copy of the caller's RNG; the copy becomes the
     * caller's state only if the acoustic stage turns out to need it (an END frame
     * draws nothing, voxtral_tts_acoustic.c:312-320). */
    vb200_pending_frame_t *p = &vb200_pending;
    uint64_t rng = ctx->rng_state;
    float noise[TTS_ACOUSTIC_DIM];
    tts_randn_fill(&rng, noise, TTS_ACOUSTIC_DIM);
    p->valid = 0;
    if (vb200_frame(input_embed, noise, ctx->kv_cache_len, out_hidden, p->codes) == 0) {
        memcpy(p->hidden, out_hidden, sizeof p->hidden);
        p->rng_before = ctx->rng_state;
        p->rng_after = rng;
        p->valid = 1;
    } else {
        fprintf(stderr, "llm: decoder step at position %d failed\n", ctx->kv_cache_len);
    }
    ctx->kv_cache_len++;
}
