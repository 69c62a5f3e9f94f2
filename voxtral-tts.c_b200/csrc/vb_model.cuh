/*
 * vb_model.cuh - host-side state of the library: device buffers, repacked
 * weights, op programs and the calls that run them.
 */
#ifndef VB_MODEL_CUH
#define VB_MODEL_CUH

#include <cuda_runtime.h>
#include <stdint.h>
#include <vector>

#include "../../include/voxtral_b200.h"
#include "../../include/voxtral_b200_ext.h"
#include "vb_engine.cuh"

namespace vb {

/* One transformer layer in HBM. QKV rows are concatenated ([q | k | v] x dim) and
 * gate/up rows interleaved (2i = gate_i, 2i+1 = up_i) so each is one GEMV. */
struct LayerDev {
    uint16_t *wqkv = nullptr;  /* [6144, 3072] */
    uint16_t *wo = nullptr;    /* [3072, 4096] */
    uint16_t *w13 = nullptr;   /* [18432, 3072] */
    uint16_t *w2 = nullptr;    /* [3072, 9216] */
    float *attn_norm = nullptr, *ffn_norm = nullptr;
};

/* Host -> device input block of one launch (one pinned copy). lat[0] is the noise. */
struct DevIn {
    VbDyn dyn;
    float embed[VB200_DIM];
    float lat[VB200_FLOW_STEPS][VB200_ACOUSTIC_DIM];
    float hidden_in[VB200_DIM];   /* acoustic-only entry: hidden state from the host */
    float temb[VB200_DIM];        /* single-pass entry: time embedding from the host */
};

/* Device -> host result block of one launch. */
struct DevOut {
    int status;
    int codes[VB200_CODES + 3];
    alignas(16) float hidden[VB200_DIM];   /* read back with 128-bit loads by the acoustic ops */
    alignas(16) float vel[2][VB200_ACOUSTIC_DIM];
};

struct Program {
    VbOp *d_ops = nullptr;
    int n = 0;
};

struct Model {
    bool inited = false;
    bool llm_ready = false, ac_ready = false, embed_ready = false;
    int device = 0, n_cta = 0, sm_count = 0;
    cudaStream_t st = nullptr;
    std::vector<void *> allocs;
    unsigned char *lin_terms = nullptr, *lin_part = nullptr;   /* scratch of tts_cuda_linear_bf16 on many rows (grow-only) */
    size_t lin_terms_cap = 0, lin_part_cap = 0;
    double upload_seconds = 0.0, upload_bytes = 0.0;   /* host -> device weight copies so far */

    LayerDev dec[VB200_DEC_LAYERS], ac[VB200_AC_LAYERS];
    uint16_t *tok_emb = nullptr;
    float *dec_norm = nullptr;
    uint16_t *ac_input_proj = nullptr, *ac_time_proj = nullptr, *ac_llm_proj = nullptr;
    uint16_t *ac_sem_out = nullptr, *ac_out = nullptr;
    float *ac_sem_bias = nullptr, *ac_norm = nullptr;
    uint16_t *audio_table = nullptr;
    float dt[VB200_FLOW_STEPS];
    std::vector<float> inv_freq;   /* host copy, for the time embedding */

    float *kv_k = nullptr, *kv_v = nullptr;
    int kv_max = 0;

    /* activations */
    float *x = nullptr, *qkv = nullptr, *attn = nullptr, *h = nullptr;
    float *logits = nullptr, *ltok = nullptr, *ttok = nullptr;
    float *X6 = nullptr, *qkv6 = nullptr, *attn6 = nullptr, *h6 = nullptr;
    float *attn_scratch = nullptr, *tap = nullptr;
    unsigned *tickets = nullptr, *bar = nullptr, *exitc = nullptr;
    DevIn *d_in = nullptr;
    DevOut *d_out = nullptr;
    DevIn *h_in = nullptr;     /* pinned */
    DevOut *h_out = nullptr;   /* pinned */
    VbOp *d_op1 = nullptr;     /* slots for single-op programs */

    bool tap_on = false;
    int prefetch_chunks = kPrefetchChunks;   /* VB200_PREFETCH overrides */
    bool ignore_end = false;      /* timed runs: an END code does not stop a device-resident run */
    bool decoder_stream = false;  /* decoder step of the single-utterance calls on the persistent streaming kernel */
    long long wait_cycles = 2000000000LL;   /* limit of the waits inside the streaming decoder kernel (~1 s) */
    Program p_llm, p_ac, p_frame, p_chain, p_pv, p_run_first, p_run_next;
    float *noise_all = nullptr;   /* device-resident run: [frames, 36] */
    int *codes_all = nullptr;     /* [frames, 37] */
    int run_cap = 0, run_launched = 0;
    bool run_on_tc = false;       /* the current device-resident run uses the tensor-core frame graph */
    std::vector<cudaEvent_t> run_ev;   /* event pairs around the frame-kernel launches of a run */
    int run_ev_used = 0, run_engine_n = 0;
    double run_engine_ms = 0.0;

    cudaEvent_t ev0 = nullptr, ev1 = nullptr, evr0 = nullptr, evr1 = nullptr;
    double ms_sum = 0.0;
    int ms_n = 0;
    bool timing = false, time_pending = false;
    int last_status = 0;
};

Model &model();

int model_init(int kv_cache_max);
void model_free();
int model_upload_llm(const vb200_decoder_weights_t *w);
int model_upload_acoustic(const vb200_acoustic_weights_t *w);
int model_upload_audio_embed(const uint16_t *table, int rows);
int model_rebuild_programs();

void flush_launch_time();
int run_program(const Program &p);   /* launch + status */
int run_ops(const std::vector<VbOp> &ops);

int llm_forward(float *out_hidden, const float *embed, int pos);
int frame(const float *embed, const float *noise, int pos, float *hidden_out, int *codes, bool chained);
int acoustic_frame(const float *hidden, const float *noise, int *codes, float *latent_out);
int predict_velocity(float *out_v, const float *x_t, const float *hidden, float t);
int linear(float *y, const float *x, const uint16_t *W_host, int M, int K, int N, const void *W_gpu);
int linear_device(float *d_y, const float *d_x, const uint16_t *d_W, int M, int K, int N);
int prefill(const float *embeds, int seq_len, int start_pos);
int prefill_prompt(const int *text_ids, int n_text, const uint16_t *voice_bf16, int n_voice, int start_pos);
int prefill_tc_setup();
void prefill_free_all();
/* tensor-core acoustic path (vb_acoustic_tc.cu) */
int acoustic_tc_setup();
bool acoustic_tc_ready();
void acoustic_tc_free_all();
int acoustic_tc_enqueue(const float *noise_all, int *codes_all, int frame_cap, bool advance, bool ignore_end);

/* several utterances in lock step (vb_batch.cu) */
int batch_open(int n_utt, int kv_max, int max_frames);
int batch_prefill(int utt, const float *embeds, int n_rows);
int batch_begin(const float *first_embeds, const int *start_pos, const float *noise);
int batch_run(int n);
int batch_end(int *codes_out, int *frames_done, int *hit_end, float *device_ms);
int batch_hidden(float *out);
int batch_launches_per_frame();
/* one utterance on the library's cache, same launches (vb_batch.cu) */
bool single_tc_usable();
int single_frame(const float *embed, const float *noise, int pos, float *hidden_out, int *codes, bool chained);
int single_begin(const float *first_embed, int start_pos, const float *noise_all, int n_frames);
int single_run(int n);
int single_end(int *codes_out, int *frames_done, int *hit_end, float *device_ms);
int gemm_sweep(int which, int iters, float *ms_out, double *bytes_per_sweep, int *launches_per_sweep);
int stream_step_time(int pos, int iters, float *ms_out, double *bytes_per_launch);
int stream_wait_expiry(int limit_us);
bool single_on_stream();
int tp_arena(int rank, int world, void *handle_out);
int tp_connect(const void *handles);
int tp_plan(int rank, int world, int n_sm, int *out);
void tp_close();
void batch_close();
void batch_invalidate();
struct TcWeight;
int batch_tiled_decoder(const TcWeight **wqkv, const TcWeight **wo, const TcWeight **w13, const TcWeight **w2);
void batch_options_changed();
void single_path_changed();
void batch_free_all();
/* vb_codec.cu */
void codec_free_all();
int codec_upload(const vb200_codec_weights_t *w);
int codec_decode(const int *codes, int n_frames, float *samples_out, int max_samples, int *n_samples);
float codec_last_ms();
int codec_set_block_frames(int frames);

int utterance_begin(const float *first_embed, int start_pos, const float *noise_all, int n_frames);
int utterance_run(int n);
int utterance_end(int *codes_out, int *frames_done, int *hit_end, float *device_ms);

} // namespace vb

#endif
