/*
 * voxtral_b200_ext.h - additions to the reference-compatible ABI.
 *
 * None of these has a counterpart in mudler/voxtral-tts.c. They exist so that a
 * replacement for the reference's decoder / acoustic stages can run a whole
 * audio frame in one launch instead of 15 host round trips, and so that tests
 * and benchmarks can reach state the reference keeps private. The
 * reference-compatible surface in voxtral_b200.h is unaffected.
 *
 * All pointers are host memory unless named d_*. Calls return 0 on success and
 * a negative value on failure; vb200_last_status() gives the device status word
 * (0 = fine) of the most recent launch.
 */
#ifndef VOXTRAL_B200_EXT_H
#define VOXTRAL_B200_EXT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* One whole frame as the orchestrator's loop body runs it
 * (voxtral_tts.c:301-318): decoder step on `embed` at cache row `pos`, then
 * semantic argmax, 7 Euler steps with both guidance branches batched, FSQ.
 * noise36: the 36 normals tts_randn_fill would draw for this frame
 * (voxtral_tts_acoustic.c:329); the caller owns the RNG and advances it only if
 * codes[0] != 1, which reproduces the reference's "END frame draws nothing".
 * hidden_out (3072, optional) receives the decoder output. */
int vb200_frame(const float *embed, const float *noise36, int pos, float *hidden_out, int *codes37);

/* The acoustic half alone (tts_acoustic_forward, voxtral_tts_acoustic.c:268-373)
 * on a host hidden state. latent_out (36, optional): latent before quantisation. */
int vb200_acoustic_frame(const float *llm_hidden, const float *noise36, int *codes37,
                         float *latent_out);

/* Same as vb200_frame, but the next decoder input is taken from the previous
 * frame's codes on the device (sum of the 37 codebook rows,
 * voxtral_tts_voice.c:292-315); needs vb200_upload_audio_embed first. */
int vb200_frame_chained(const float *noise36, int pos, float *hidden_out, int *codes37);
int vb200_upload_audio_embed(const uint16_t *table_bf16, int rows);

/* What the weight uploads since tts_cuda_init have cost: wall-clock seconds inside the upload
 * calls (host -> device copies through a ring of pinned staging buffers filled by
 * VB200_UPLOAD_THREADS host threads, repacking kernels behind them on the same stream, one
 * wait at the end of each call) and the bytes copied. The reference's counterpart is one
 * blocking cudaMemcpy per matrix (voxtral_tts_cuda.cu:223-310). Either pointer may be null. */
void vb200_upload_stats(double *seconds, double *bytes);

/* The prompt of voxtral_tts.c:230-272 assembled on the device and prefilled:
 *   [BOS=1] [BEGIN_AUDIO=25] voice rows [/INST=36] text tokens [INST=35] [BEGIN_AUDIO=25]
 * Token rows come from the token table that tts_cuda_upload_llm_weights uploaded (the decoder
 * struct's tok_embeddings must have been set), voice rows from `voice_bf16` ([n_voice, 3072] BF16 in
 * host memory, the payload of a voice file; tts_voice_embed, voxtral_tts_voice.c:228-248). Only
 * ids and BF16 rows cross to the device; nothing is expanded to fp32 on the host. The rows land in
 * the cache from row start_pos. Returns the number of prompt rows (n_voice + n_text + 5) or -1. */
int vb200_prefill_prompt(const int *text_ids, int n_text, const uint16_t *voice_bf16, int n_voice, int start_pos);

/* The orchestrator's frame loop (voxtral_tts.c:301-321) kept on the device: no host
 * round trip per frame. begin: first decoder input, first cache row, and the noise
 * of all n_frames frames ([n_frames, 36]; the reference RNG draws 36 normals per
 * frame in sequence). run: queue up to n more frames and return at once. end: wait,
 * fetch codes [frames_done, 37] (an END frame is included and flagged through
 * hit_end; the reference discards it) and the device time of the last run call. */
int vb200_utterance_begin(const float *first_embed, int start_pos, const float *noise, int n_frames);
int vb200_utterance_run(int n_frames);
int vb200_utterance_end(int *codes_out, int *frames_done, int *hit_end, float *device_ms);
/* Device time (ms, CUDA events) spent inside the frame-kernel launches of the last
 * vb200_utterance_run batch, and how many launches that was. */
double vb200_utterance_engine_ms(int *launches);
/* Several independent utterances decoded in lock step on this GPU (no counterpart in the
 * reference, which synthesises one utterance per process: voxtral_tts.c:301-321 run once
 * per utterance). Every weight matrix is read once per frame for all utterances: the decoder
 * step runs as an n-row and the acoustic passes as a 6n-row tensor-core GEMM. Each utterance
 * has its own cache slab, position, noise and END state.
 *   open:    1..8 utterances, cache rows per utterance, frames the code/noise arrays hold
 *   prefill: prompt rows [n_rows, 3072] of one utterance into its cache rows 0..n_rows-1
 *   begin:   first decoder input rows [n, 3072], first cache row per utterance [n], noise
 *            [n, max_frames, 36]
 *   run:     queue up to n_frames more frames for every utterance still running
 *   end:     wait; codes [n, max_frames, 37] (zero past frames_done[u]), frames_done [n],
 *            hit_end [n], device time of the last run call
 *   hidden:  decoder output rows of the last frame [n, 3072] */
int vb200_batch_open(int n_utterances, int kv_max, int max_frames);
int vb200_batch_prefill(int utterance, const float *embeds, int n_rows);
int vb200_batch_begin(const float *first_embeds, const int *start_pos, const float *noise);
int vb200_batch_run(int n_frames);
int vb200_batch_end(int *codes_out, int *frames_done, int *hit_end, float *device_ms);
int vb200_batch_hidden(float *out);
int vb200_batch_launches_per_frame(void);
void vb200_batch_close(void);

/* Tensor parallelism over the GPUs of one node, one process per GPU (no counterpart in the
 * reference, which is single-GPU: voxtral_tts_cuda.cu:103). Every rank uploads all weights and
 * makes the same vb200_frame / vb200_utterance_* calls with the same inputs; each decoder-layer
 * GEMM then covers only the rank's slice of output tiles and stores its results into every
 * rank's buffers over NVLink, ordered by per-site sequence flags (bounded waits).
 *   arena:   after tts_cuda_init; allocates the exchange arena, returns its CUDA IPC handle
 *            (64 bytes). world must divide 24 (1, 2, 3, 4, 6, 8).
 *   connect: handles = world x 64 bytes, rank order, gathered by the caller (e.g. an
 *            all-gather over the launcher's process group); maps the peers' arenas. The
 *            caller puts a host barrier between connect and the first frame.
 *   close:   back to single-GPU launches. */
int vb200_tp_arena(int rank, int world, void *handle_out64);
int vb200_tp_connect(const void *handles);
void vb200_tp_close(void);
/* Host arithmetic only: the slices rank `rank` of `world` computes. out9 = first tile and tile
 * count (tiles of 128 output rows) of the QKV, O/down and gate/up GEMMs, then the split-K
 * factors of QKV, O and down. -1 when world does not divide the tile counts. */
int vb200_tp_plan(int rank, int world, int n_sm, int *out9);
/* 1 when vb200_frame / vb200_utterance_* run as the graph of tensor-core GEMM launches, 0 when
 * they run on the streaming frame kernel (VB200_NO_TC=1, or per-layer taps enabled). */
int vb200_frame_on_tensor_cores(void);

/* 1 when the decoder step of vb200_frame / vb200_utterance_* runs as one launch of the
 * persistent streaming kernel (option "decoder_kernel" = 1), 0 when it runs as GEMM launches of the
 * frame graph (the default). */
int vb200_frame_on_stream_kernel(void);

/* Options by name. "ignore_end" (0/1): a device-resident run started after this call
 * treats END as an ordinary code, for fixed-length timing runs. "decoder_kernel" (0/1): the
 * decoder step of vb200_frame / vb200_utterance_* runs as GEMM launches inside the frame graph
 * (0, default) or as one launch of the persistent streaming kernel (1; one GPU only). Both give
 * the same results within the summation-order tolerance. "wait_limit_us": the limit of
 * every wait inside the streaming decoder kernel (default about one second); when a wait runs
 * out the call returns -1 and vb200_last_status() names the wait. "codec_block_frames" (64 ..
 * 2048, default 2048): vb200_codec_decode takes longer utterances block by block (see there).
 * Returns -1 for an unknown name or value. */
int vb200_set_option(const char *name, int value);

/* Copy rows [pos0, pos0+n) of one layer's K and V cache to / from the host
 * ([n, 1024] fp32 each), e.g. to pre-fill a cache prefix. */
int vb200_kv_write(int layer, int pos0, int n, const float *k_rows, const float *v_rows);
int vb200_kv_read(int layer, int pos0, int n, float *k_rows, float *v_rows);

/* Residual-stream tap for per-layer parity checks: when enabled, every decode
 * step also stores the stream after attention and after the FFN of each layer.
 * vb200_tap_read copies [26, 2, 3072] floats. */
int vb200_tap_enable(int on);
int vb200_tap_read(float *out);

/* y[seq,out] = x[seq,in] . W[out,in]^T like tts_cuda_linear_bf16, for callers that may
 * not allocate device memory at the time of the call: plugins inside a host that owns
 * the whole GPU heap, real-time audio threads that cannot afford cudaMalloc's implicit
 * synchronisation, code that must leave a tracked allocator untouched. No counterpart
 * in the reference. It calls no cudaMalloc / cudaFree (nor anything that does) and
 * does not need tts_cuda_init. All three pointers are device memory supplied by the
 * caller. The few hundred bytes per row block that the kernel needs besides its
 * operands (op descriptors, barrier counters, status) live in a fixed 10 KB device
 * array inside the library, present on every GPU that loads it until exit.
 *  - Limit: seq_len <= 512 per call (64 descriptors of 8 rows); more returns -2 and
 *    does nothing. Other failures return -1; 0 means the work was queued.
 *  - Asynchronous on the default stream; tts_cuda_sync() (or any device
 *    synchronisation) before reading y. vb200_linear_bf16_static_status() then gives
 *    the kernel's status word (0 = fine).
 *  - The first call on each device looks up the array's address and zeroes it with
 *    synchronous runtime calls: make that first call before starting a stream capture.
 *  - One array per device is shared by all calls and keeps what the last call left
 *    (the counters are re-zeroed by every launch); two calls in flight on the same
 *    GPU at once would race on it, so issue them from one thread / one stream. */
int vb200_linear_bf16_static(float *d_y, const float *d_x, const uint16_t *d_W, int seq_len,
                             int in_dim, int out_dim);
int vb200_linear_bf16_static_status(void);

int vb200_last_status(void);
int vb200_sm_count(void);
/* Average device time, in milliseconds, of the engine launches since the last
 * call with reset != 0 (CUDA events on the library's stream); n receives the
 * number of launches averaged. */
double vb200_engine_ms(int reset, int *n);

/* Deterministic synthetic tensors (integer hash -> sum of 16 uniform bytes ->
 * approximately normal), identical on every machine. value = mean + sigma * z.
 * `stream` separates tensors (e.g. a CRC of the tensor name); `first` is the
 * index of dst[0] inside the tensor, so rows can be produced on demand. */
void vb200_synth_bf16(uint16_t *dst, size_t n, uint64_t seed, uint64_t stream, uint64_t first,
                      float sigma);
void vb200_synth_f32(float *dst, size_t n, uint64_t seed, uint64_t stream, uint64_t first,
                     float mean, float sigma);

/* The reference's noise generator (tts_rng_seed / tts_randn_fill, voxtral_tts_kernels.c:640-669),
 * bit for bit: n normals, *state advanced in place (a zero state is replaced by the reference's
 * default seed). One frame that is not END consumes 36 of them (voxtral_tts_acoustic.c:329). */
void vb200_randn_fill(uint64_t *state, float *out, size_t n);

/* ---- codec decoder on the GPU (tts_codec_decode, voxtral_tts_codec.c:389-510) ----
 * 37 codes per frame -> 24 kHz waveform, 1920 samples per frame: code embedding, causal
 * convolution 292 -> 1024, four stages of two transformer layers (ALiBi sliding-window
 * attention, QK norm, layer scale; voxtral_tts_codec.c:306-383) with three stride-2 transposed
 * convolutions between them, causal convolution 1024 -> 240. The three structs mirror tts_conv_t,
 * tts_codec_layer_t and tts_codec_t (voxtral_tts.h:172-225) field by field, so a host that has run
 * the reference's tts_codec_load passes &ctx->codec. All pointers are host fp32 arrays.
 *
 * The transformer matrices must be exactly representable in BF16 (they are when the checkpoint
 * stores them as BF16, which safetensors_get_f32 merely widens): they are kept as BF16 on the
 * device and multiplied on the tensor cores; vb200_codec_upload returns -1 and says so when a
 * value would be rounded. The (weight-normed) convolution weights stay fp32. */
typedef struct {
    float *weight;              /* conv: [out_ch, in_ch, kernel]; transposed conv: [in_ch, out_ch, kernel] */
    float *bias;                /* [out_ch] or NULL */
    int in_ch, out_ch, kernel, stride, is_transpose;
} vb200_conv_t;

typedef struct {
    float *wq, *wk, *wv, *wo;   /* [1024, 1024] */
    float *q_norm, *k_norm;     /* [1024] or NULL */
    float *attention_norm;      /* [1024] */
    float *w1, *w2, *w3;        /* [4096, 1024], [1024, 4096], [4096, 1024] */
    float *ffn_norm;            /* [1024] */
    float *attn_scale, *ffn_scale; /* [1024] or NULL */
    int window_size;
} vb200_codec_layer_t;

typedef struct {
    float *semantic_embedding;  /* [8192, 256] */
    vb200_conv_t input_conv;    /* 292 -> 1024, kernel 3 */
    vb200_codec_layer_t transformers[8];
    vb200_conv_t stage_convs[4];/* [0..2]: transposed, 1024 -> 1024, kernel 4, stride 2; [3] unused */
    vb200_conv_t output_proj;   /* 1024 -> 240, kernel 7 */
    float alibi_slopes[8];
} vb200_codec_weights_t;

/* Needs tts_cuda_init. 0 on success. */
int vb200_codec_upload(const vb200_codec_weights_t *w);
/* codes: [n_frames, 37] host ints. Writes n_frames * 1920 samples to samples_out (host) when
 * max_samples allows, stores the count in *n_samples; -1 on any failure. Any number of frames:
 * up to 2048 frames (164 s of audio; the reference's generation limit is 2000) go through in one
 * piece, longer inputs block by block with 32 frames of left context that is decoded again and
 * dropped - the decoder looks back less than 17 frames, so the result is that of one piece. */
int vb200_codec_decode(const int *codes, int n_frames, float *samples_out, int max_samples, int *n_samples);
/* Device time of the last vb200_codec_decode in milliseconds (CUDA events around its kernels). */
float vb200_codec_last_ms(void);

#ifdef __cplusplus
}
#endif
#endif
