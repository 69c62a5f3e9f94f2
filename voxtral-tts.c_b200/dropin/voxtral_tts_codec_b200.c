/*
 * voxtral_tts_codec_b200.c - replaces the reference's voxtral_tts_codec.c when the engine is
 * built against libvoxtral_b200.so.
 *
 *   tts_codec_load    the tensors of voxtral_tts_codec.c:177-262 under the same names: semantic
 *                     embedding = embedding_sum / max(cluster_usage, 1e-5), weight-normed or
 *                     plain convolutions, eight transformer layers with their optional QK-norm
 *                     and layer-scale vectors, ALiBi slopes 2^(-h-1)
 *   tts_codec_decode  37 codes per frame -> waveform (voxtral_tts_codec.c:389-510) in one call
 *                     to the library; the weights go to the GPU on the first call
 *
 * Compile with -I<reference> -DUSE_CUDA. No CPU path: when the GPU call fails the result is
 * NULL / 0 samples, as the reference reports an allocation failure.
 */
#include "voxtral_tts.h"
#include "voxtral_tts_safetensors.h"
#include "voxtral_b200_ext.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define BLK "audio_tokenizer.decoder_blocks"

static float *tensor(safetensors_file_t *sf, const char *fmt, const char *a, int i, int j, const char *b) {
    char name[512];
    snprintf(name, sizeof name, fmt, a, i, j, b);
    const safetensor_t *t = safetensors_find(sf, name);
    return t ? safetensors_get_f32(sf, t) : NULL;
}

/* v scaled slice by slice to the length g[slice] (weight normalisation over everything but the
 * leading dimension; float accumulation in index order, as voxtral_tts_codec.c:38-61). */
static float *normed(const float *v, const float *g, int slices, int len) {
    float *w = (float *)malloc(sizeof(float) * (size_t)slices * len);
    if (!w) return NULL;
    for (int s = 0; s < slices; s++) {
        const float *row = v + (size_t)s * len;
        float ss = 0.0f;
        for (int i = 0; i < len; i++) ss += row[i] * row[i];
        const float k = g[s] / sqrtf(ss + 1e-12f);
        for (int i = 0; i < len; i++) w[(size_t)s * len + i] = row[i] * k;
    }
    return w;
}

/* "<prefix>.conv.parametrizations.weight.original{0,1}" (g, v) or "<prefix>.conv.weight". */
static int load_conv(safetensors_file_t *sf, const char *prefix, tts_conv_t *c, int in_ch, int out_ch, int kernel,
                     int stride, int transposed) {
    float *g = tensor(sf, "%s.conv.parametrizations.weight.original%d%.0d%s", prefix, 0, 0, "");
    float *v = tensor(sf, "%s.conv.parametrizations.weight.original%d%.0d%s", prefix, 1, 0, "");
    if (g && v) {
        /* conv: [out, in, k] normed per output channel; transposed conv: [in, out, k] per input channel */
        c->weight = transposed ? normed(v, g, in_ch, out_ch * kernel) : normed(v, g, out_ch, in_ch * kernel);
    } else {
        c->weight = tensor(sf, "%s.conv.weight%.0d%.0d%s", prefix, 0, 0, "");
    }
    free(g);
    free(v);
    if (!c->weight) {
        fprintf(stderr, "codec: no weight for %s\n", prefix);
        return -1;
    }
    c->bias = tensor(sf, "%s.conv.bias%.0d%.0d%s", prefix, 0, 0, "");
    c->in_ch = in_ch; c->out_ch = out_ch; c->kernel = kernel; c->stride = stride; c->is_transpose = transposed;
    return 0;
}

int tts_codec_load(tts_codec_t *codec, void *sf_ptr) {
    safetensors_file_t *sf = (safetensors_file_t *)sf_ptr;
    const char *Q = "audio_tokenizer.quantizer.semantic_codebook";
    float *sum = tensor(sf, "%s.embedding_sum%.0d%.0d%s", Q, 0, 0, "");
    float *use = tensor(sf, "%s.cluster_usage%.0d%.0d%s", Q, 0, 0, "");
    if (!sum || !use) {
        fprintf(stderr, "codec: semantic codebook not found\n");
        free(sum); free(use);
        return -1;
    }
    for (int i = 0; i < TTS_SEMANTIC_CB_SIZE; i++) {
        const float u = use[i] < 1e-5f ? 1e-5f : use[i];
        for (int j = 0; j < TTS_SEMANTIC_CB_DIM; j++) sum[(size_t)i * TTS_SEMANTIC_CB_DIM + j] /= u;
    }
    free(use);
    codec->semantic_embedding = sum;
    for (int h = 0; h < TTS_CODEC_HEADS; h++)
        codec->alibi_slopes[h] = powf(2.0f, -8.0f / (float)TTS_CODEC_HEADS * (float)(h + 1));

    /* blocks: 0 conv in, then (transformer, transposed conv) x 3, transformer; windows double per stage */
    if (load_conv(sf, BLK ".0", &codec->input_conv, TTS_EMBED_DIM, TTS_CODEC_DIM, 3, 1, 0)) return -1;
    static const char *const vec[6] = {"attention.q_norm.weight", "attention.k_norm.weight", "attention_norm.weight",
                                       "ffn_norm.weight", "attention_scale", "ffn_scale"};
    static const char *const mat[7] = {"attention.wq.weight", "attention.wk.weight", "attention.wv.weight",
                                       "attention.wo.weight", "feed_forward.w1.weight", "feed_forward.w2.weight",
                                       "feed_forward.w3.weight"};
    for (int stage = 0, layer = 0; stage < TTS_CODEC_STAGES; stage++) {
        const int block = 1 + 2 * stage;
        for (int l = 0; l < TTS_CODEC_LAYERS_PER_STAGE; l++, layer++) {
            tts_codec_layer_t *L = &codec->transformers[layer];
            float **m[7] = {&L->wq, &L->wk, &L->wv, &L->wo, &L->w1, &L->w2, &L->w3};
            float **v[6] = {&L->q_norm, &L->k_norm, &L->attention_norm, &L->ffn_norm, &L->attn_scale, &L->ffn_scale};
            int missing = 0;
            for (int k = 0; k < 7; k++) missing |= !(*m[k] = tensor(sf, "%s.%d.layers.%d.%s", BLK, block, l, mat[k]));
            for (int k = 0; k < 6; k++) *v[k] = tensor(sf, "%s.%d.layers.%d.%s", BLK, block, l, vec[k]);
            if (missing || !L->attention_norm || !L->ffn_norm) {
                fprintf(stderr, "codec: transformer weights missing at %s.%d.layers.%d\n", BLK, block, l);
                return -1;
            }
            L->window_size = 2 << stage;
        }
        if (stage < TTS_CODEC_STAGES - 1) {
            char prefix[128];
            snprintf(prefix, sizeof prefix, BLK ".%d", block + 1);
            if (load_conv(sf, prefix, &codec->stage_convs[stage], TTS_CODEC_DIM, TTS_CODEC_DIM, 4, 2, 1)) return -1;
        }
    }
    return load_conv(sf, "audio_tokenizer.output_proj", &codec->output_proj, TTS_CODEC_DIM, TTS_PATCH_SIZE, 7, 1, 0);
}

void tts_codec_decode(tts_ctx_t *ctx, const int *codes, int n_frames, float **out_samples, int *out_n_samples) {
    static const tts_codec_t *on_gpu = NULL;
    *out_samples = NULL;
    *out_n_samples = 0;
    if (n_frames <= 0) return;
    if (on_gpu != &ctx->codec) {
        /* tts_codec_t and vb200_codec_weights_t have the same layout (checked at build time below) */
        if (vb200_codec_upload((const vb200_codec_weights_t *)&ctx->codec) != 0) {
            fprintf(stderr, "codec: upload to the GPU failed\n");
            return;
        }
        on_gpu = &ctx->codec;
    }
    const int max_samples = n_frames * 8 * TTS_PATCH_SIZE;
    float *samples = (float *)malloc(sizeof(float) * (size_t)max_samples);
    int n = 0;
    if (!samples || vb200_codec_decode(codes, n_frames, samples, max_samples, &n) != 0) {
        fprintf(stderr, "codec: decode failed\n");
        free(samples);
        return;
    }
    *out_samples = samples;
    *out_n_samples = n;
}

typedef char vb200_codec_layout_check[sizeof(tts_codec_t) == sizeof(vb200_codec_weights_t) &&
                                      sizeof(tts_conv_t) == sizeof(vb200_conv_t) &&
                                      sizeof(tts_codec_layer_t) == sizeof(vb200_codec_layer_t) ? 1 : -1];
