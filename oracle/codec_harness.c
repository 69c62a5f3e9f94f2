/*
 * codec_harness.c - runs tts_codec_load and tts_codec_decode (voxtral_tts.h:370-373) on a synthetic
 * safetensors file, the way tts_load and tts_generate do (voxtral_tts.c:86-91, :333-334).
 *
 * TEST INFRASTRUCTURE ONLY. oracle/build_oracle.py compiles this file twice with the reference's
 * own voxtral_tts_kernels.c and voxtral_tts_safetensors.c taken by path from the reference checkout:
 *   oracle/_ref/codec_run_ref   + the reference's voxtral_tts_codec.c (CPU; the checker)
 *   oracle/_ref/codec_run_b200  + voxtral-tts.c_b200/dropin/voxtral_tts_codec_b200.c, -DUSE_CUDA,
 *                               linked against libvoxtral_b200.so (the candidate)
 * usage: codec_run_* <codec.safetensors> <codes.i32> <n_frames> <out.f32>
 *   codes.i32  n_frames x 37 raw int32
 *   out.f32    the waveform as raw fp32; stdout: "samples <n>"
 */
#include "voxtral_tts.h"
#include "voxtral_tts_kernels.h"
#include "voxtral_tts_safetensors.h"

#include <stdio.h>
#include <stdlib.h>

int tts_verbose = 0; /* defined in voxtral_tts.c, which is not linked here */

int main(int argc, char **argv) {
    if (argc != 5) {
        fprintf(stderr, "usage: %s codec.safetensors codes.i32 n_frames out.f32\n", argv[0]);
        return 2;
    }
    const int n_frames = atoi(argv[3]);
    tts_ctx_t *ctx = (tts_ctx_t *)calloc(1, sizeof(tts_ctx_t));
    safetensors_file_t *sf = safetensors_open(argv[1]);
    if (!ctx || !sf || n_frames < 1) { fprintf(stderr, "cannot open %s\n", argv[1]); return 1; }
    if (tts_codec_load(&ctx->codec, sf) != 0) { fprintf(stderr, "tts_codec_load failed\n"); return 1; }
    int *codes = (int *)malloc(sizeof(int) * (size_t)n_frames * TTS_CODES_PER_FRAME);
    FILE *f = fopen(argv[2], "rb");
    if (!codes || !f || fread(codes, sizeof(int), (size_t)n_frames * TTS_CODES_PER_FRAME, f) !=
                            (size_t)n_frames * TTS_CODES_PER_FRAME) {
        fprintf(stderr, "cannot read %d frames of codes from %s\n", n_frames, argv[2]);
        return 1;
    }
    fclose(f);
#ifdef USE_CUDA
    if (tts_cuda_init(64) != 0) { fprintf(stderr, "tts_cuda_init failed\n"); return 1; }
#endif
    float *samples = NULL;
    int n = 0;
    tts_codec_decode(ctx, codes, n_frames, &samples, &n);
    if (!samples || n <= 0) { fprintf(stderr, "tts_codec_decode produced nothing\n"); return 1; }
    f = fopen(argv[4], "wb");
    if (!f || fwrite(samples, sizeof(float), (size_t)n, f) != (size_t)n) { fprintf(stderr, "cannot write %s\n", argv[4]); return 1; }
    fclose(f);
    printf("samples %d\n", n);
#ifdef USE_CUDA
    tts_cuda_free();
#endif
    safetensors_close(sf);
    return 0;
}
