/*
 * dropin_harness.c - runs the stage entry points of voxtral_tts.h:360-377 the way the
 * reference's orchestrator does (tts_load, voxtral_tts.c:22-107, and the frame loop of
 * tts_generate, voxtral_tts.c:279-321), on a synthetic checkpoint file.
 *
 * TEST INFRASTRUCTURE ONLY. oracle/build_oracle.py compiles this file twice, each time with the
 * reference's own voxtral_tts_kernels.c, voxtral_tts_voice.c and voxtral_tts_safetensors.c taken
 * by path from the reference checkout:
 *   oracle/_ref/dropin_run_ref   + the reference's voxtral_tts_llm.c and voxtral_tts_acoustic.c
 *                                (CPU; the checker)
 *   oracle/_ref/dropin_run_b200  + the two replacement files of voxtral-tts.c_b200/dropin/,
 *                                -DUSE_CUDA, linked against libvoxtral_b200.so (the candidate)
 * Both binaries print the same report; a test compares the two reports.
 *
 * tts_load itself is not called: it insists on a tokenizer file and on the codec's tensors
 * (voxtral_tts.c:47-91), which are outside the hot path. Everything it does for the decoder
 * and acoustic stages is done here in the same order.
 *
 * usage: dropin_run_* <file.safetensors> <prompt.f32> <n_prompt_rows> <seed> <n_frames> <kv_max> <force_end>
 *   prompt.f32   n_prompt_rows x 3072 raw fp32 rows (what voxtral_tts.c:230-272 assembles)
 *   force_end    1: give the semantic head a bias that makes END (code 1) win every frame
 * report (stdout): one line "frame <i> rng <state> codes <37 ints>" per frame produced, an END
 * frame included, then "done frames <n> rng <state> kv_len <n>".
 */
#include "voxtral_tts.h"
#include "voxtral_tts_kernels.h"
#include "voxtral_tts_safetensors.h"
/* with -DUSE_CUDA voxtral_tts_kernels.h pulls in the reference's voxtral_tts_cuda.h, whose
 * entry points libvoxtral_b200.so exports under the same names */

#include <inttypes.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

int tts_verbose = 0; /* defined in voxtral_tts.c, which is not linked here */

static float *read_rows(const char *path, int rows) {
    FILE *f = fopen(path, "rb");
    if (!f) return NULL;
    const size_t n = (size_t)rows * TTS_DEC_DIM;
    float *buf = (float *)malloc(n * sizeof(float));
    if (buf && fread(buf, sizeof(float), n, f) != n) { free(buf); buf = NULL; }
    fclose(f);
    return buf;
}

int main(int argc, char **argv) {
    if (argc != 8) {
        fprintf(stderr, "usage: %s file.safetensors prompt.f32 rows seed frames kv_max force_end\n", argv[0]);
        return 2;
    }
    const int n_prompt = atoi(argv[3]);
    const uint64_t seed = strtoull(argv[4], NULL, 10);
    const int n_frames = atoi(argv[5]), kv_max = atoi(argv[6]), force_end = atoi(argv[7]);

    tts_ctx_t *ctx = (tts_ctx_t *)calloc(1, sizeof(tts_ctx_t));
    if (!ctx) return 1;
    safetensors_file_t *sf = safetensors_open(argv[1]);
    if (!sf) { fprintf(stderr, "cannot open %s\n", argv[1]); return 1; }
    ctx->safetensors = sf;
    if (tts_llm_load(&ctx->decoder, sf) != 0) { fprintf(stderr, "tts_llm_load failed\n"); return 1; }
    if (tts_llm_kv_cache_alloc(ctx, kv_max) != 0) { fprintf(stderr, "tts_llm_kv_cache_alloc failed\n"); return 1; }
    if (tts_acoustic_load(&ctx->acoustic, sf) != 0) { fprintf(stderr, "tts_acoustic_load failed\n"); return 1; }
    if (tts_audio_embed_load(&ctx->audio_embed, sf) != 0) { fprintf(stderr, "tts_audio_embed_load failed\n"); return 1; }
    if (force_end) {
        float *bias = (float *)calloc(TTS_SEMANTIC_CB_PADDED, sizeof(float));
        if (!bias) return 1;
        bias[TTS_AUDIO_SPECIAL_END] = 1e6f;
        ctx->acoustic.semantic_out_bias = bias;
    }
#ifdef USE_CUDA
    if (tts_cuda_init(ctx->kv_cache_max) != 0) { fprintf(stderr, "tts_cuda_init failed\n"); return 1; }
    tts_cuda_upload_llm_weights(&ctx->decoder);
    tts_cuda_upload_acoustic_weights(&ctx->acoustic);
    if (!tts_cuda_available()) { fprintf(stderr, "weight upload failed\n"); return 1; }
#endif
    tts_rng_seed(&ctx->rng_state, seed);

    float *prompt = read_rows(argv[2], n_prompt);
    if (!prompt) { fprintf(stderr, "cannot read %d prompt rows from %s\n", n_prompt, argv[2]); return 1; }
    ctx->kv_cache_len = 0;
    tts_llm_prefill(ctx, prompt, n_prompt);
    free(prompt);

    float next_embed[TTS_DEC_DIM], hidden[TTS_DEC_DIM];
    tts_embed_token_bf16(next_embed, ctx->decoder.tok_embeddings_bf16, TTS_TOK_AUDIO, TTS_DEC_DIM);
    int produced = 0;
    for (int f = 0; f < n_frames; f++) {
        int codes[TTS_CODES_PER_FRAME];
        tts_llm_forward(ctx, next_embed, hidden);
        tts_acoustic_forward(ctx, hidden, codes);
        printf("frame %d rng %" PRIu64 " codes", f, ctx->rng_state);
        for (int i = 0; i < TTS_CODES_PER_FRAME; i++) printf(" %d", codes[i]);
        printf("\n");
        produced++;
        if (codes[0] == TTS_AUDIO_SPECIAL_END) break;       /* voxtral_tts.c:307 */
        tts_audio_embed_forward(ctx, codes, next_embed);
    }
    printf("done frames %d rng %" PRIu64 " kv_len %d\n", produced, ctx->rng_state, ctx->kv_cache_len);
#ifdef USE_CUDA
    tts_cuda_free();
#endif
    safetensors_close(sf);
    return 0;
}
