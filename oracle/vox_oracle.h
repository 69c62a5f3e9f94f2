/*
 * vox_oracle.h - CPU restatement of the voxtral-tts.c per-frame hot path.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing shipped links or calls this; it is the
 * checker the CUDA path is compared with, and the "port" CPU baseline.
 *
 * Every function restates, in independent code, the arithmetic of the
 * reference's CPU path (file:line given per function in vox_oracle.c).
 * Dimensions are run-time so that small shapes can be tested quickly; the
 * reference fixes them at compile time (voxtral_tts.h:19-44).
 *
 * Parity status: PINNED. tests/test_oracle_pin.py compares this port with
 * the reference's own C sources compiled unmodified (oracle/_ref, built by
 * oracle/build_oracle.py) and with the fixtures in tests/golden/ that were
 * produced by that build.
 */
#ifndef VOX_ORACLE_H
#define VOX_ORACLE_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    int dim;          /* model width (3072) */
    int n_layers;     /* 26 decoder / 3 acoustic */
    int n_heads;      /* 32 */
    int n_kv_heads;   /* 8 */
    int head_dim;     /* 128 */
    int hidden;       /* FFN width 9216 */
    float eps;        /* RMSNorm epsilon 1e-5 */
    float rope_theta; /* 1e6 (decoder only) */
} vox_dims_t;

/* One transformer layer's weights: BF16 row-major [out,in], fp32 gains. */
typedef struct {
    const uint16_t *wq, *wk, *wv, *wo;
    const uint16_t *w1, *w2, *w3;      /* gate, down, up */
    const float *attn_norm, *ffn_norm;
} vox_layer_t;

typedef struct {
    vox_dims_t d;
    const vox_layer_t *layers;
    const float *final_norm;
} vox_decoder_t;

typedef struct {
    vox_dims_t d;
    const vox_layer_t *layers;
    const float *final_norm;
    const float *time_inv_freq;        /* [dim/2] */
    const uint16_t *input_proj;        /* [dim, n_acoustic] */
    const uint16_t *time_proj;         /* [dim, dim] */
    const uint16_t *llm_proj;          /* [dim, dim] */
    const uint16_t *semantic_out;      /* [sem_padded, dim] */
    const float *semantic_bias;        /* [sem_padded] or NULL */
    const uint16_t *acoustic_out;      /* [n_acoustic, dim] */
    int n_acoustic;                    /* 36 */
    int sem_padded;                    /* 8320 */
    int sem_valid_end;                 /* 8194: first masked padding index */
    int flow_steps;                    /* 8 timesteps -> 7 Euler intervals */
    int fsq_levels;                    /* 21 */
    float cfg_alpha;                   /* 1.2 */
    float noise_scale;                 /* 1.0 */
} vox_acoustic_t;

/* ---- primitives ---- */
void vox_linear_bf16(float *y, const float *x, const uint16_t *W, const float *bias,
                     int M, int K, int N);
void vox_rms_norm(float *out, const float *x, const float *gain, int rows, int dim, float eps);
void vox_rope_table(float *cs, const int *pos, int n_pos, int head_dim, float theta);
void vox_rope_apply(float *x, const float *cs, int rows, int heads, int head_dim);
void vox_silu_mul(float *gate, const float *up, int n);
void vox_attention_causal(float *out, const float *Q, const float *K, const float *V,
                          int seq_q, int seq_k, int n_heads, int n_kv_heads, int head_dim,
                          float scale, int q_offset);
void vox_attention_full(float *out, const float *Q, const float *K, const float *V,
                        int seq, int n_heads, int n_kv_heads, int head_dim, float scale);
void vox_time_embedding(float *out, const float *inv_freq, float t, int dim);
void vox_time_inv_freq(float *inv_freq, int dim);

/* ---- random numbers ---- */
void vox_rng_seed(uint64_t *state, uint64_t seed);
float vox_randn(uint64_t *state);
void vox_randn_fill(uint64_t *state, float *buf, int n);

/* ---- decoder ---- */
/* One decode step at cache position `pos`. kv_k/kv_v are [n_layers, kv_max, kv_dim].
 * tap (optional) receives the residual stream after attention and after the FFN
 * of every layer: [n_layers, 2, dim]. */
void vox_llm_forward(const vox_decoder_t *dec, float *kv_k, float *kv_v, int kv_max,
                     int pos, const float *input_embed, float *out_hidden, float *tap);
/* Prefill of seq_len rows starting at cache position start_pos.
 * tap (optional): [n_layers, 2, seq_len, dim]. */
void vox_llm_prefill(const vox_decoder_t *dec, float *kv_k, float *kv_v, int kv_max,
                     int start_pos, const float *embeds, int seq_len, float *tap);

/* ---- acoustic ---- */
void vox_predict_velocity(const vox_acoustic_t *ac, const float *x_t,
                          const float *llm_hidden, float t, float *out_v);
/* Full frame: semantic argmax, noise from *rng, Euler+CFG, FSQ.
 * logits_out (optional) receives the masked semantic logits [sem_padded];
 * x_final (optional) receives the final latent before quantisation. */
void vox_acoustic_forward(const vox_acoustic_t *ac, uint64_t *rng, const float *llm_hidden,
                          int *out_codes, float *logits_out, float *x_final);

/* ---- audio-code re-embedding ---- */
void vox_audio_embed(const uint16_t *table, int dim, const int *codes, int n_codebooks,
                     int semantic_rows, int acoustic_rows, float *out);
void vox_embed_row_bf16(float *out, const uint16_t *table, int row, int dim);

#ifdef __cplusplus
}
#endif
#endif
