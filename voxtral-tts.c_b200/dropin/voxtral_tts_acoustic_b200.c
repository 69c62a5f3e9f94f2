/*
 * voxtral_tts_acoustic_b200.c - replaces the reference's voxtral_tts_acoustic.c
 * when the engine is built against libvoxtral_b200.so.
 *
 *   tts_acoustic_load     tensor names, optional bias and the computed inverse
 *                         frequencies as voxtral_tts_acoustic.c:40-126
 *   tts_acoustic_forward  37 codes for one hidden state (voxtral_tts_acoustic.c:268-373):
 *                         the whole frame (semantic argmax, 7 Euler steps with both
 *                         guidance branches batched, FSQ) is one GPU launch instead of
 *                         14 predict_velocity calls; the RNG in ctx advances by 36 draws
 *                         unless the frame is END, exactly as the reference's does.
 *
 * Compile with -I<reference> -DUSE_CUDA. No CPU path.
 */
#include "voxtral_tts.h"
#include "voxtral_tts_kernels.h"
#include "voxtral_tts_safetensors.h"
#include "voxtral_b200_ext.h"
#include "voxtral_b200_dropin.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static uint16_t *bf16_tensor(safetensors_file_t *sf, const char *name) {
    const safetensor_t *t = safetensors_find(sf, name);
    if (!t) { fprintf(stderr, "acoustic: weight not found: %s\n", name); return NULL; }
    return safetensors_get_bf16_direct(sf, t);
}

static float *f32_tensor(safetensors_file_t *sf, const char *name, int required) {
    const safetensor_t *t = safetensors_find(sf, name);
    if (!t) {
        if (required) fprintf(stderr, "acoustic: weight not found: %s\n", name);
        return NULL;
    }
    return safetensors_get_f32(sf, t);
}

int tts_acoustic_load(tts_acoustic_t *ac, void *sf_ptr) {
    safetensors_file_t *sf = (safetensors_file_t *)sf_ptr;
    const char *P = "acoustic_transformer";
    char name[256];

    snprintf(name, sizeof name, "%s.time_embedding.inv_freq", P);
    ac->time_inv_freq = f32_tensor(sf, name, 0);
    if (!ac->time_inv_freq) {
        const int half = TTS_AC_DIM / 2;
        ac->time_inv_freq = (float *)malloc(sizeof(float) * half);
        if (!ac->time_inv_freq) return -1;
        for (int i = 0; i < half; i++) ac->time_inv_freq[i] = expf(-logf(10000.0f) * (float)i / (float)half);
    }
    snprintf(name, sizeof name, "%s.input_projection.weight", P);
    ac->input_proj_bf16 = bf16_tensor(sf, name);
    snprintf(name, sizeof name, "%s.time_projection.weight", P);
    ac->time_proj_bf16 = bf16_tensor(sf, name);
    snprintf(name, sizeof name, "%s.llm_projection.weight", P);
    ac->llm_proj_bf16 = bf16_tensor(sf, name);
    snprintf(name, sizeof name, "%s.semantic_codebook_output.weight", P);
    ac->semantic_out_bf16 = bf16_tensor(sf, name);
    snprintf(name, sizeof name, "%s.semantic_codebook_output.bias", P);
    ac->semantic_out_bias = f32_tensor(sf, name, 0);
    snprintf(name, sizeof name, "%s.acoustic_codebook_output.weight", P);
    ac->acoustic_out_bf16 = bf16_tensor(sf, name);
    snprintf(name, sizeof name, "%s.norm.weight", P);
    ac->norm = f32_tensor(sf, name, 1);
    if (!ac->input_proj_bf16 || !ac->time_proj_bf16 || !ac->llm_proj_bf16 || !ac->semantic_out_bf16 ||
        !ac->acoustic_out_bf16 || !ac->norm)
        return -1;

    static const char *const mats[7] = {"attention.wq", "attention.wk", "attention.wv", "attention.wo",
                                        "feed_forward.w1", "feed_forward.w2", "feed_forward.w3"};
    for (int i = 0; i < TTS_AC_LAYERS; i++) {
        tts_ac_layer_t *l = &ac->layers[i];
        uint16_t **slots[7] = {&l->wq_bf16, &l->wk_bf16, &l->wv_bf16, &l->wo_bf16,
                               &l->w1_bf16, &l->w2_bf16, &l->w3_bf16};
        for (int k = 0; k < 7; k++) {
            snprintf(name, sizeof name, "%s.layers.%d.%s.weight", P, i, mats[k]);
            *slots[k] = bf16_tensor(sf, name);
            if (!*slots[k]) return -1;
        }
        snprintf(name, sizeof name, "%s.layers.%d.attention_norm.weight", P, i);
        l->attention_norm = f32_tensor(sf, name, 1);
        snprintf(name, sizeof name, "%s.layers.%d.ffn_norm.weight", P, i);
        l->ffn_norm = f32_tensor(sf, name, 1);
        if (!l->attention_norm || !l->ffn_norm) return -1;
    }
    return 0;
}

void tts_acoustic_forward(tts_ctx_t *ctx, const float *llm_hidden, int *out_codes) {
    if (!tts_cuda_available()) {
        fprintf(stderr, "acoustic: no GPU context; this build has no CPU acoustic transformer\n");
        return;
    }
    vb200_pending_frame_t *p = &vb200_pending;
    uint64_t rng_after;
    if (p->valid && p->rng_before == ctx->rng_state &&
        memcmp(p->hidden, llm_hidden, sizeof p->hidden) == 0) {
        /* the decoder step's launch already produced this frame */
        memcpy(out_codes, p->codes, sizeof p->codes);
        rng_after = p->rng_after;
    } else {
        uint64_t rng = ctx->rng_state;
        float noise[TTS_ACOUSTIC_DIM];
        tts_randn_fill(&rng, noise, TTS_ACOUSTIC_DIM);
        if (vb200_acoustic_frame(llm_hidden, noise, out_codes, NULL) != 0) {
            fprintf(stderr, "acoustic: frame failed\n");
            return;
        }
        rng_after = rng;
    }
    p->valid = 0;
    if (out_codes[0] != TTS_AUDIO_SPECIAL_END) ctx->rng_state = rng_after;
}
