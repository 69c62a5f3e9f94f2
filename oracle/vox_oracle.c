/*
 * vox_oracle.c - CPU restatement of the voxtral-tts.c per-frame hot path.
 *
 * TEST INFRASTRUCTURE ONLY (see vox_oracle.h). Independent code; each function
 * names the reference lines whose arithmetic it restates. Operation order is
 * kept identical to the reference's portable (non-BLAS) build so that the two
 * agree bit for bit; OpenMP only spreads independent output elements over
 * threads and never changes the order of a sum.
 */
#include "vox_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

static inline float bf16_as_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, sizeof f);
    return f;
}

/* y[M,N] = x[M,K] . W[N,K]^T (+ bias).
 * Restates bf16_matvec_fused (voxtral_tts_kernels.c:152-185, scalar tail loop
 * :177-182) for M == 1 and the portable branch of tts_linear
 * (voxtral_tts_kernels.c:127-138) reached through tts_linear_bf16
 * (:200-211) for M > 1: the accumulator starts at the bias (or 0) and adds
 * w*x for k = 0..K-1 in order. BF16 -> fp32 is the exact 16-bit shift
 * (voxtral_tts_kernels.c:49-53). */
void vox_linear_bf16(float *y, const float *x, const uint16_t *W, const float *bias,
                     int M, int K, int N) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        const uint16_t *wr = W + (size_t)n * K;
        for (int m = 0; m < M; m++) {
            const float *xr = x + (size_t)m * K;
            float acc = bias ? bias[n] : 0.0f;
            for (int k = 0; k < K; k++) acc += bf16_as_f32(wr[k]) * xr[k];
            y[(size_t)m * N + n] = acc;
        }
    }
}

/* tts_rms_norm, voxtral_tts_kernels.c:333-349. */
void vox_rms_norm(float *out, const float *x, const float *gain, int rows, int dim, float eps) {
    for (int r = 0; r < rows; r++) {
        const float *xr = x + (size_t)r * dim;
        float *orow = out + (size_t)r * dim;
        float ss = 0.0f;
        for (int i = 0; i < dim; i++) ss += xr[i] * xr[i];
        float inv = 1.0f / sqrtf(ss / dim + eps);
        for (int i = 0; i < dim; i++) orow[i] = xr[i] * inv * gain[i];
    }
}

/* tts_compute_rope_freqs, voxtral_tts_kernels.c:602-614: per position a table of
 * (cos, sin) pairs for d = 0..head_dim/2-1 with freq = 1/theta^(2d/head_dim). */
void vox_rope_table(float *cs, const int *pos, int n_pos, int head_dim, float theta) {
    int half = head_dim / 2;
    for (int s = 0; s < n_pos; s++) {
        float p = (float)pos[s];
        for (int d = 0; d < half; d++) {
            float freq = 1.0f / powf(theta, (float)(2 * d) / (float)head_dim);
            float ang = p * freq;
            cs[((size_t)s * half + d) * 2 + 0] = cosf(ang);
            cs[((size_t)s * half + d) * 2 + 1] = sinf(ang);
        }
    }
}

/* tts_apply_rope, voxtral_tts_kernels.c:616-634: rotate interleaved pairs (2d, 2d+1). */
void vox_rope_apply(float *x, const float *cs, int rows, int heads, int head_dim) {
    int half = head_dim / 2;
    for (int s = 0; s < rows; s++)
        for (int h = 0; h < heads; h++) {
            float *v = x + ((size_t)s * heads + h) * head_dim;
            for (int d = 0; d < half; d++) {
                float c = cs[((size_t)s * half + d) * 2 + 0];
                float sn = cs[((size_t)s * half + d) * 2 + 1];
                float a = v[2 * d], b = v[2 * d + 1];
                v[2 * d] = a * c - b * sn;
                v[2 * d + 1] = a * sn + b * c;
            }
        }
}

/* tts_silu then tts_mul_inplace, voxtral_tts_kernels.c:361-366 and :29-31. */
void vox_silu_mul(float *gate, const float *up, int n) {
    for (int i = 0; i < n; i++) {
        float g = gate[i];
        g = g / (1.0f + expf(-g));
        gate[i] = g * up[i];
    }
}

/* One (head, query) row of the streaming-softmax attention shared by
 * tts_causal_attention (voxtral_tts_kernels.c:426-462) and
 * tts_bidirectional_attention (:487-522): keys j0..j1-1 visited in order,
 * running maximum starts at -1e30, the score is scaled after the dot product,
 * a strictly larger score rescales the accumulator. */
static void attn_row(float *o, const float *q, const float *K, const float *V,
                     int j0, int j1, int kv_stride, int head_dim, float scale) {
    float run_max = -1e30f, denom = 0.0f;
    for (int d = 0; d < head_dim; d++) o[d] = 0.0f;
    for (int j = j0; j < j1; j++) {
        const float *kr = K + (size_t)j * kv_stride;
        const float *vr = V + (size_t)j * kv_stride;
        float s = 0.0f;
        for (int d = 0; d < head_dim; d++) s += q[d] * kr[d];
        s *= scale;
        if (s > run_max) {
            float corr = expf(run_max - s);
            denom = denom * corr + 1.0f;
            for (int d = 0; d < head_dim; d++) o[d] = o[d] * corr + vr[d];
            run_max = s;
        } else {
            float w = expf(s - run_max);
            denom += w;
            for (int d = 0; d < head_dim; d++) o[d] += w * vr[d];
        }
    }
    if (denom > 0.0f) {
        float inv = 1.0f / denom;
        for (int d = 0; d < head_dim; d++) o[d] *= inv;
    }
}

/* tts_causal_attention with window_size == 0, voxtral_tts_kernels.c:403-465:
 * query i sees keys 0..min(q_offset+i+1, seq_k)-1; query head h reads KV head
 * h / (n_heads/n_kv_heads). */
void vox_attention_causal(float *out, const float *Q, const float *K, const float *V,
                          int seq_q, int seq_k, int n_heads, int n_kv_heads, int head_dim,
                          float scale, int q_offset) {
    int group = n_heads / n_kv_heads;
    int qw = n_heads * head_dim, kw = n_kv_heads * head_dim;
#pragma omp parallel for collapse(2) schedule(static)
    for (int h = 0; h < n_heads; h++)
        for (int i = 0; i < seq_q; i++) {
            int kvh = h / group;
            int end = q_offset + i + 1;
            if (end > seq_k) end = seq_k;
            attn_row(out + (size_t)i * qw + h * head_dim, Q + (size_t)i * qw + h * head_dim,
                     K + kvh * head_dim, V + kvh * head_dim, 0, end, kw, head_dim, scale);
        }
}

/* tts_bidirectional_attention, voxtral_tts_kernels.c:467-525. */
void vox_attention_full(float *out, const float *Q, const float *K, const float *V,
                        int seq, int n_heads, int n_kv_heads, int head_dim, float scale) {
    int group = n_heads / n_kv_heads;
    int qw = n_heads * head_dim, kw = n_kv_heads * head_dim;
    for (int h = 0; h < n_heads; h++)
        for (int i = 0; i < seq; i++) {
            int kvh = h / group;
            attn_row(out + (size_t)i * qw + h * head_dim, Q + (size_t)i * qw + h * head_dim,
                     K + kvh * head_dim, V + kvh * head_dim, 0, seq, kw, head_dim, scale);
        }
}

/* compute_time_embedding, voxtral_tts_acoustic.c:166-176: cos block then sin block. */
void vox_time_embedding(float *out, const float *inv_freq, float t, int dim) {
    int half = dim / 2;
    for (int i = 0; i < half; i++) {
        float ang = t * inv_freq[i];
        out[i] = cosf(ang);
        out[half + i] = sinf(ang);
    }
}

/* Fallback inverse frequencies when the checkpoint has none,
 * voxtral_tts_acoustic.c:49-57: exp(-ln(10000) * i / (dim/2)). */
void vox_time_inv_freq(float *inv_freq, int dim) {
    int half = dim / 2;
    float theta = 10000.0f;
    for (int i = 0; i < half; i++)
        inv_freq[i] = expf(-logf(theta) * (float)i / (float)half);
}

/* ---- RNG: tts_rng_seed / xorshift64 / uniform01 / tts_randn,
 * voxtral_tts_kernels.c:640-669. Shifts 13, 7, 17; uniform = top 53 bits as
 * float times 2^-53; Box-Muller cosine branch, u1 redrawn while < 1e-30. ---- */
void vox_rng_seed(uint64_t *state, uint64_t seed) {
    *state = seed ? seed : 0x12345678ABCDEF01ULL;
}

static uint64_t rng_next(uint64_t *state) {
    uint64_t v = *state;
    v ^= v << 13;
    v ^= v >> 7;
    v ^= v << 17;
    *state = v;
    return v;
}

static float rng_unit(uint64_t *state) {
    return (float)(rng_next(state) >> 11) * (1.0f / 9007199254740992.0f);
}

float vox_randn(uint64_t *state) {
    float u1, u2;
    do { u1 = rng_unit(state); } while (u1 < 1e-30f);
    u2 = rng_unit(state);
    return sqrtf(-2.0f * logf(u1)) * cosf(6.2831853071795864f * u2);
}

void vox_randn_fill(uint64_t *state, float *buf, int n) {
    for (int i = 0; i < n; i++) buf[i] = vox_randn(state);
}

/* ---- decoder ---- */

typedef struct {
    float *x, *xn, *q, *k, *v, *attn, *proj, *gate, *up, *ffn;
} work_t;

static int work_alloc(work_t *w, const vox_dims_t *d, int rows) {
    size_t qd = (size_t)d->n_heads * d->head_dim, kd = (size_t)d->n_kv_heads * d->head_dim;
    w->x = malloc(sizeof(float) * rows * d->dim);
    w->xn = malloc(sizeof(float) * rows * d->dim);
    w->q = malloc(sizeof(float) * rows * qd);
    w->k = malloc(sizeof(float) * rows * kd);
    w->v = malloc(sizeof(float) * rows * kd);
    w->attn = malloc(sizeof(float) * rows * qd);
    w->proj = malloc(sizeof(float) * rows * d->dim);
    w->gate = malloc(sizeof(float) * rows * d->hidden);
    w->up = malloc(sizeof(float) * rows * d->hidden);
    w->ffn = malloc(sizeof(float) * rows * d->dim);
    return (w->x && w->xn && w->q && w->k && w->v && w->attn && w->proj && w->gate && w->up &&
            w->ffn) ? 0 : -1;
}

static void work_free(work_t *w) {
    free(w->x); free(w->xn); free(w->q); free(w->k); free(w->v);
    free(w->attn); free(w->proj); free(w->gate); free(w->up); free(w->ffn);
}

static void add_rows(float *a, const float *b, size_t n) {
    for (size_t i = 0; i < n; i++) a[i] += b[i];
}

/* Shared layer body of tts_llm_forward (voxtral_tts_llm.c:205-264, M = 1) and
 * tts_llm_prefill (voxtral_tts_llm.c:319-366, M = seq_len): norm, Q/K/V, RoPE,
 * cache write at rows start..start+M-1, causal attention over the whole cache
 * prefix, O + residual, norm, SwiGLU FFN + residual. */
static void decoder_layers(const vox_decoder_t *dec, float *kv_k, float *kv_v, int kv_max,
                           int start, int M, work_t *w, float *tap) {
    const vox_dims_t *d = &dec->d;
    int dim = d->dim, qd = d->n_heads * d->head_dim, kd = d->n_kv_heads * d->head_dim;
    float scale = 1.0f / sqrtf((float)d->head_dim);

    int *pos = malloc(sizeof(int) * M);
    float *cs = malloc(sizeof(float) * (size_t)M * d->head_dim);
    for (int i = 0; i < M; i++) pos[i] = start + i;
    vox_rope_table(cs, pos, M, d->head_dim, d->rope_theta);

    for (int l = 0; l < d->n_layers; l++) {
        const vox_layer_t *L = &dec->layers[l];
        float *ck = kv_k + (size_t)l * kv_max * kd;
        float *cv = kv_v + (size_t)l * kv_max * kd;

        vox_rms_norm(w->xn, w->x, L->attn_norm, M, dim, d->eps);
        vox_linear_bf16(w->q, w->xn, L->wq, NULL, M, dim, qd);
        vox_linear_bf16(w->k, w->xn, L->wk, NULL, M, dim, kd);
        vox_linear_bf16(w->v, w->xn, L->wv, NULL, M, dim, kd);
        vox_rope_apply(w->q, cs, M, d->n_heads, d->head_dim);
        vox_rope_apply(w->k, cs, M, d->n_kv_heads, d->head_dim);
        memcpy(ck + (size_t)start * kd, w->k, sizeof(float) * (size_t)M * kd);
        memcpy(cv + (size_t)start * kd, w->v, sizeof(float) * (size_t)M * kd);
        vox_attention_causal(w->attn, w->q, ck, cv, M, start + M, d->n_heads, d->n_kv_heads,
                             d->head_dim, scale, start);
        vox_linear_bf16(w->proj, w->attn, L->wo, NULL, M, qd, dim);
        add_rows(w->x, w->proj, (size_t)M * dim);
        if (tap) memcpy(tap + ((size_t)l * 2 + 0) * M * dim, w->x, sizeof(float) * (size_t)M * dim);

        vox_rms_norm(w->xn, w->x, L->ffn_norm, M, dim, d->eps);
        vox_linear_bf16(w->gate, w->xn, L->w1, NULL, M, dim, d->hidden);
        vox_linear_bf16(w->up, w->xn, L->w3, NULL, M, dim, d->hidden);
        vox_silu_mul(w->gate, w->up, M * d->hidden);
        vox_linear_bf16(w->ffn, w->gate, L->w2, NULL, M, d->hidden, dim);
        add_rows(w->x, w->ffn, (size_t)M * dim);
        if (tap) memcpy(tap + ((size_t)l * 2 + 1) * M * dim, w->x, sizeof(float) * (size_t)M * dim);
    }
    free(pos);
    free(cs);
}

/* tts_llm_forward, voxtral_tts_llm.c:171-271 (ends with the final RMSNorm :267;
 * no vocabulary projection is computed). */
void vox_llm_forward(const vox_decoder_t *dec, float *kv_k, float *kv_v, int kv_max,
                     int pos, const float *input_embed, float *out_hidden, float *tap) {
    work_t w;
    if (work_alloc(&w, &dec->d, 1) != 0) { work_free(&w); return; }
    memcpy(w.x, input_embed, sizeof(float) * dec->d.dim);
    decoder_layers(dec, kv_k, kv_v, kv_max, pos, 1, &w, tap);
    vox_rms_norm(out_hidden, w.x, dec->final_norm, 1, dec->d.dim, dec->d.eps);
    work_free(&w);
}

/* tts_llm_prefill, voxtral_tts_llm.c:277-373 (hidden states discarded, only the
 * cache rows are kept). */
void vox_llm_prefill(const vox_decoder_t *dec, float *kv_k, float *kv_v, int kv_max,
                     int start_pos, const float *embeds, int seq_len, float *tap) {
    work_t w;
    if (work_alloc(&w, &dec->d, seq_len) != 0) { work_free(&w); return; }
    memcpy(w.x, embeds, sizeof(float) * (size_t)seq_len * dec->d.dim);
    decoder_layers(dec, kv_k, kv_v, kv_max, start_pos, seq_len, &w, tap);
    work_free(&w);
}

/* ---- acoustic ---- */

/* predict_velocity, voxtral_tts_acoustic.c:182-262: three tokens
 * [input_proj(x_t), time_proj(temb(t)), llm_proj(h)], three unmasked layers
 * without RoPE, final norm of token 0 only, 36-wide velocity head. */
void vox_predict_velocity(const vox_acoustic_t *ac, const float *x_t,
                          const float *llm_hidden, float t, float *out_v) {
    const vox_dims_t *d = &ac->d;
    int dim = d->dim, qd = d->n_heads * d->head_dim, kd = d->n_kv_heads * d->head_dim;
    const int S = 3;
    float scale = 1.0f / sqrtf((float)d->head_dim);
    work_t w;
    if (work_alloc(&w, d, S) != 0) { work_free(&w); return; }
    float *temb = malloc(sizeof(float) * dim);

    vox_linear_bf16(w.x + 0 * dim, x_t, ac->input_proj, NULL, 1, ac->n_acoustic, dim);
    vox_time_embedding(temb, ac->time_inv_freq, t, dim);
    vox_linear_bf16(w.x + 1 * dim, temb, ac->time_proj, NULL, 1, dim, dim);
    vox_linear_bf16(w.x + 2 * dim, llm_hidden, ac->llm_proj, NULL, 1, dim, dim);

    for (int l = 0; l < d->n_layers; l++) {
        const vox_layer_t *L = &ac->layers[l];
        vox_rms_norm(w.xn, w.x, L->attn_norm, S, dim, d->eps);
        vox_linear_bf16(w.q, w.xn, L->wq, NULL, S, dim, qd);
        vox_linear_bf16(w.k, w.xn, L->wk, NULL, S, dim, kd);
        vox_linear_bf16(w.v, w.xn, L->wv, NULL, S, dim, kd);
        vox_attention_full(w.attn, w.q, w.k, w.v, S, d->n_heads, d->n_kv_heads, d->head_dim, scale);
        vox_linear_bf16(w.proj, w.attn, L->wo, NULL, S, qd, dim);
        add_rows(w.x, w.proj, (size_t)S * dim);
        vox_rms_norm(w.xn, w.x, L->ffn_norm, S, dim, d->eps);
        vox_linear_bf16(w.gate, w.xn, L->w1, NULL, S, dim, d->hidden);
        vox_linear_bf16(w.up, w.xn, L->w3, NULL, S, dim, d->hidden);
        vox_silu_mul(w.gate, w.up, S * d->hidden);
        vox_linear_bf16(w.ffn, w.gate, L->w2, NULL, S, d->hidden, dim);
        add_rows(w.x, w.ffn, (size_t)S * dim);
    }
    vox_rms_norm(w.xn, w.x, ac->final_norm, 1, dim, d->eps);
    vox_linear_bf16(out_v, w.xn, ac->acoustic_out, NULL, 1, dim, ac->n_acoustic);
    free(temb);
    work_free(&w);
}

/* tts_acoustic_forward, voxtral_tts_acoustic.c:268-373.
 *  - semantic logits (+bias), index 0 and indices >= sem_valid_end set to -1e30,
 *    first strict maximum wins (:283-309);
 *  - code 1 (END) fills the 36 acoustic codes with 2 and leaves the RNG alone
 *    (:312-320);
 *  - otherwise 36 normals, timesteps i/(steps-1), per interval a conditional and
 *    a zero-conditioned pass, v = a*vc + (1-a)*vu, x += v*dt (:329-355);
 *  - FSQ: clamp to [-1,1], (x+1)/2*(levels-1), add 0.5 and truncate, clamp,
 *    add 2 (:358-372). */
void vox_acoustic_forward(const vox_acoustic_t *ac, uint64_t *rng, const float *llm_hidden,
                          int *out_codes, float *logits_out, float *x_final) {
    int dim = ac->d.dim, A = ac->n_acoustic;
    float *logits = malloc(sizeof(float) * ac->sem_padded);
    vox_linear_bf16(logits, llm_hidden, ac->semantic_out, ac->semantic_bias, 1, dim, ac->sem_padded);
    logits[0] = -1e30f;
    for (int i = ac->sem_valid_end; i < ac->sem_padded; i++) logits[i] = -1e30f;
    int best_i = 0;
    float best = logits[0];
    for (int i = 1; i < ac->sem_padded; i++)
        if (logits[i] > best) { best = logits[i]; best_i = i; }
    if (logits_out) memcpy(logits_out, logits, sizeof(float) * ac->sem_padded);
    free(logits);
    out_codes[0] = best_i;

    if (best_i == 1) {
        for (int i = 1; i <= A; i++) out_codes[i] = 2;
        if (x_final) memset(x_final, 0, sizeof(float) * A);
        return;
    }

    float *x = malloc(sizeof(float) * A), *vc = malloc(sizeof(float) * A), *vu = malloc(sizeof(float) * A);
    float *zero = calloc(dim, sizeof(float));
    float *ts = malloc(sizeof(float) * ac->flow_steps);
    vox_randn_fill(rng, x, A);
    for (int i = 0; i < A; i++) x[i] *= ac->noise_scale;
    for (int i = 0; i < ac->flow_steps; i++) ts[i] = (float)i / (float)(ac->flow_steps - 1);

    for (int s = 0; s < ac->flow_steps - 1; s++) {
        float t = ts[s], dt = ts[s + 1] - ts[s];
        vox_predict_velocity(ac, x, llm_hidden, t, vc);
        vox_predict_velocity(ac, x, zero, t, vu);
        for (int i = 0; i < A; i++) {
            float v = ac->cfg_alpha * vc[i] + (1.0f - ac->cfg_alpha) * vu[i];
            x[i] += v * dt;
        }
    }
    if (x_final) memcpy(x_final, x, sizeof(float) * A);

    for (int i = 0; i < A; i++) {
        float val = x[i];
        if (val > 1.0f) val = 1.0f;
        if (val < -1.0f) val = -1.0f;
        float scaled = ((val + 1.0f) / 2.0f) * (float)(ac->fsq_levels - 1);
        int code = (int)(scaled + 0.5f);
        if (code < 0) code = 0;
        if (code >= ac->fsq_levels) code = ac->fsq_levels - 1;
        out_codes[i + 1] = code + 2;
    }
    free(x); free(vc); free(vu); free(zero); free(ts);
}

/* tts_embed_token_bf16, voxtral_tts_kernels.c:55-59. */
void vox_embed_row_bf16(float *out, const uint16_t *table, int row, int dim) {
    const uint16_t *src = table + (size_t)row * dim;
    for (int i = 0; i < dim; i++) out[i] = bf16_as_f32(src[i]);
}

/* tts_audio_embed_forward, voxtral_tts_voice.c:292-315 with the offsets of
 * tts_audio_embed_load (:275-283): codebook 0 starts at row 0 and has
 * semantic_rows (8194) rows, every later codebook has acoustic_rows (23);
 * rows are added in codebook order starting from zero. */
void vox_audio_embed(const uint16_t *table, int dim, const int *codes, int n_codebooks,
                     int semantic_rows, int acoustic_rows, float *out) {
    for (int i = 0; i < dim; i++) out[i] = 0.0f;
    int base = 0;
    for (int cb = 0; cb < n_codebooks; cb++) {
        const uint16_t *src = table + (size_t)(base + codes[cb]) * dim;
        for (int i = 0; i < dim; i++) out[i] += bf16_as_f32(src[i]);
        base += (cb == 0) ? semantic_rows : acoustic_rows;
    }
}
