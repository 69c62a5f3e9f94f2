/*
 * ref_harness.c - drives the reference's own, unmodified CPU sources.
 *
 * TEST INFRASTRUCTURE ONLY. Compiled by oracle/build_oracle.py together with
 * the reference's voxtral_tts_kernels.c, voxtral_tts_llm.c, voxtral_tts_voice.c
 * and voxtral_tts_safetensors.c, taken by path from the reference checkout
 * (never copied); the output goes to oracle/_ref/. This file pulls in the
 * reference's voxtral_tts_acoustic.c through the include path so that its
 * file-static predict_velocity() can be called directly.
 *
 * The harness does what the orchestrator's frame loop does
 * (voxtral_tts.c:279-318) on a tts_ctx_t whose weight pointers are supplied by
 * the caller, so no model files are needed. tts_load is bypassed because it
 * insists on a tokenizer file and the codec tensors (voxtral_tts.c:47-91).
 *
 * The reference's voxtral_tts_llm.c is compiled with
 * -Dtts_add_inplace=oracle_tap_add_inplace; the tap below forwards to the real
 * tts_add_inplace and records the residual stream after every residual add
 * (voxtral_tts_llm.c:245,263 for decode; :354,366 for prefill).
 */
#include "voxtral_tts_acoustic.c" /* reference source, found through -I */

#include <stdint.h>

int tts_verbose = 0; /* defined in voxtral_tts.c, which is not linked here */

/* ---- residual tap ---- */
static float *g_tap_buf = NULL;
static size_t g_tap_cap = 0;    /* floats */
static size_t g_tap_used = 0;
static int g_tap_calls = 0;

void oracle_tap_add_inplace(float *a, const float *b, int n) {
    tts_add_inplace(a, b, n);
    g_tap_calls++;
    if (g_tap_buf && g_tap_used + (size_t)n <= g_tap_cap) {
        memcpy(g_tap_buf + g_tap_used, a, sizeof(float) * (size_t)n);
        g_tap_used += (size_t)n;
    }
}

void refh_tap_set(float *buf, size_t cap_floats) {
    g_tap_buf = buf;
    g_tap_cap = cap_floats;
    g_tap_used = 0;
    g_tap_calls = 0;
}
size_t refh_tap_used(void) { return g_tap_used; }
int refh_tap_calls(void) { return g_tap_calls; }

/* ---- context ---- */
void *refh_create(void) { return calloc(1, sizeof(tts_ctx_t)); }

/* Frees what the harness and the reference allocated lazily; weight pointers
 * belong to the caller. */
void refh_destroy(void *p) {
    tts_ctx_t *c = (tts_ctx_t *)p;
    if (!c) return;
    free(c->kv_cache_k); free(c->kv_cache_v);
    free(c->dec_x); free(c->dec_x_norm); free(c->dec_q); free(c->dec_k); free(c->dec_v);
    free(c->dec_attn_out); free(c->dec_proj_out); free(c->dec_gate); free(c->dec_up);
    free(c->dec_ffn_out);
    free(c->ac_tokens); free(c->ac_tokens_norm); free(c->ac_q); free(c->ac_k); free(c->ac_v);
    free(c->ac_attn_out); free(c->ac_proj_out); free(c->ac_gate); free(c->ac_up);
    free(c->ac_ffn_out); free(c->ac_time_emb); free(c->ac_velocity); free(c->ac_noise);
    free(c);
}

size_t refh_sizeof_ctx(void) { return sizeof(tts_ctx_t); }
size_t refh_sizeof_decoder(void) { return sizeof(tts_decoder_t); }
size_t refh_sizeof_acoustic(void) { return sizeof(tts_acoustic_t); }
size_t refh_sizeof_codec(void) { return sizeof(tts_codec_t); }
void *refh_decoder_ptr(void *p) { return &((tts_ctx_t *)p)->decoder; }
void *refh_acoustic_ptr(void *p) { return &((tts_ctx_t *)p)->acoustic; }

void refh_set_dec_layer(void *p, int i, uint16_t *wq, uint16_t *wk, uint16_t *wv, uint16_t *wo,
                        uint16_t *w1, uint16_t *w2, uint16_t *w3, float *an, float *fn) {
    tts_dec_layer_t *l = &((tts_ctx_t *)p)->decoder.layers[i];
    l->wq_bf16 = wq; l->wk_bf16 = wk; l->wv_bf16 = wv; l->wo_bf16 = wo;
    l->w1_bf16 = w1; l->w2_bf16 = w2; l->w3_bf16 = w3;
    l->attention_norm = an; l->ffn_norm = fn;
}

void refh_set_dec_misc(void *p, uint16_t *tok_embeddings, float *norm) {
    tts_ctx_t *c = (tts_ctx_t *)p;
    c->decoder.tok_embeddings_bf16 = tok_embeddings;
    c->decoder.norm = norm;
}

void refh_set_ac_layer(void *p, int i, uint16_t *wq, uint16_t *wk, uint16_t *wv, uint16_t *wo,
                       uint16_t *w1, uint16_t *w2, uint16_t *w3, float *an, float *fn) {
    tts_ac_layer_t *l = &((tts_ctx_t *)p)->acoustic.layers[i];
    l->wq_bf16 = wq; l->wk_bf16 = wk; l->wv_bf16 = wv; l->wo_bf16 = wo;
    l->w1_bf16 = w1; l->w2_bf16 = w2; l->w3_bf16 = w3;
    l->attention_norm = an; l->ffn_norm = fn;
}

void refh_set_ac_misc(void *p, float *inv_freq, uint16_t *input_proj, uint16_t *time_proj,
                      uint16_t *llm_proj, uint16_t *sem_out, float *sem_bias,
                      uint16_t *ac_out, float *norm) {
    tts_acoustic_t *a = &((tts_ctx_t *)p)->acoustic;
    a->time_inv_freq = inv_freq;
    a->input_proj_bf16 = input_proj; a->time_proj_bf16 = time_proj; a->llm_proj_bf16 = llm_proj;
    a->semantic_out_bf16 = sem_out; a->semantic_out_bias = sem_bias;
    a->acoustic_out_bf16 = ac_out; a->norm = norm;
}

/* Same table layout tts_audio_embed_load derives (voxtral_tts_voice.c:275-283),
 * but with the table pointer given by the caller instead of a safetensors file. */
void refh_set_audio_embed(void *p, uint16_t *table) {
    tts_audio_embed_t *ae = &((tts_ctx_t *)p)->audio_embed;
    ae->embeddings_bf16 = table;
    ae->embed_dim = TTS_DEC_DIM;
    ae->offsets[0] = 0;
    ae->offsets[1] = TTS_SEMANTIC_CB_SIZE + TTS_AUDIO_SPECIAL_COUNT;
    for (int i = 2; i <= TTS_NUM_CODEBOOKS; i++)
        ae->offsets[i] = ae->offsets[i - 1] + TTS_FSQ_LEVELS + TTS_AUDIO_SPECIAL_COUNT;
    ae->total_size = ae->offsets[TTS_NUM_CODEBOOKS];
}

/* Loads through the reference's own loaders from a safetensors file. */
int refh_load_file(void *p, const char *path) {
    tts_ctx_t *c = (tts_ctx_t *)p;
    safetensors_file_t *sf = safetensors_open(path);
    if (!sf) return -1;
    c->safetensors = sf;
    if (tts_llm_load(&c->decoder, sf) != 0) return -2;
    if (tts_acoustic_load(&c->acoustic, sf) != 0) return -3;
    if (tts_audio_embed_load(&c->audio_embed, sf) != 0) return -4;
    return 0;
}

int refh_kv_alloc(void *p, int max_seq) { return tts_llm_kv_cache_alloc((tts_ctx_t *)p, max_seq); }
float *refh_kv_k(void *p) { return ((tts_ctx_t *)p)->kv_cache_k; }
float *refh_kv_v(void *p) { return ((tts_ctx_t *)p)->kv_cache_v; }
int refh_kv_len(void *p) { return ((tts_ctx_t *)p)->kv_cache_len; }
void refh_set_kv_len(void *p, int n) { ((tts_ctx_t *)p)->kv_cache_len = n; }

void refh_seed(void *p, uint64_t seed) { tts_rng_seed(&((tts_ctx_t *)p)->rng_state, seed); }
uint64_t refh_rng_state(void *p) { return ((tts_ctx_t *)p)->rng_state; }
void refh_set_rng_state(void *p, uint64_t s) { ((tts_ctx_t *)p)->rng_state = s; }

void refh_llm_forward(void *p, const float *in, float *out) { tts_llm_forward((tts_ctx_t *)p, in, out); }
void refh_llm_prefill(void *p, const float *embeds, int n) { tts_llm_prefill((tts_ctx_t *)p, embeds, n); }
void refh_acoustic_forward(void *p, const float *hidden, int *codes) {
    tts_acoustic_forward((tts_ctx_t *)p, hidden, codes);
}
void refh_audio_embed(void *p, const int *codes, float *out) {
    tts_audio_embed_forward((tts_ctx_t *)p, codes, out);
}

/* predict_velocity is file-static in the reference; reachable here because the
 * reference TU is part of this one. Needs the acoustic buffers, which the
 * reference allocates on the first tts_acoustic_forward call. */
int refh_predict_velocity(void *p, const float *x_t, const float *hidden, float t, float *out_v) {
    tts_ctx_t *c = (tts_ctx_t *)p;
    if (!c->ac_tokens && alloc_acoustic_buffers(c) != 0) return -1;
    predict_velocity(c, x_t, hidden, t, out_v);
    return 0;
}

/* Model constants as compiled into the reference (voxtral_tts.h:19-79). */
void refh_constants(int *out) {
    out[0] = TTS_DEC_DIM; out[1] = TTS_DEC_LAYERS; out[2] = TTS_DEC_HEADS; out[3] = TTS_DEC_KV_HEADS;
    out[4] = TTS_DEC_HEAD_DIM; out[5] = TTS_DEC_HIDDEN; out[6] = TTS_AC_LAYERS;
    out[7] = TTS_ACOUSTIC_DIM; out[8] = TTS_SEMANTIC_CB_PADDED; out[9] = TTS_FLOW_STEPS;
    out[10] = TTS_FSQ_LEVELS; out[11] = TTS_CODES_PER_FRAME; out[12] = TTS_SEMANTIC_CB_SIZE;
    out[13] = TTS_VOCAB_SIZE;
}

/* ---- codec decoder (voxtral_tts_codec.c, compiled unchanged beside this file) ----
 * `weights` is a tts_codec_t filled by the caller (pointers into the caller's arrays). Runs
 * tts_codec_decode (voxtral_tts_codec.c:389-510) and copies the waveform out. Returns the number
 * of samples, or -1. */
int refh_codec_decode(void *p, const void *weights, const int *codes, int n_frames, float *out, int max_samples) {
    tts_ctx_t *c = (tts_ctx_t *)p;
    if (!c || !weights) return -1;
    memcpy(&c->codec, weights, sizeof(tts_codec_t));
    float *samples = NULL;
    int n = 0;
    tts_codec_decode(c, codes, n_frames, &samples, &n);
    memset(&c->codec, 0, sizeof(tts_codec_t));       /* the arrays are the caller's */
    if (!samples || n <= 0 || n > max_samples) { free(samples); return -1; }
    memcpy(out, samples, sizeof(float) * (size_t)n);
    free(samples);
    return n;
}
