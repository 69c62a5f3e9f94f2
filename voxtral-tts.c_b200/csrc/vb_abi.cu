/*
 * vb_abi.cu - the exported C symbols: the reference-compatible surface
 * (include/voxtral_b200.h, names and meaning of voxtral_tts_cuda.h:82-185) and
 * the additions of include/voxtral_b200_ext.h.
 */
#include "../../include/voxtral_b200.h"
#include "../../include/voxtral_b200_ext.h"
#include "../../include/voxtral_b200_probe.h"
#include "vb_model.cuh"
#include "vb_simple.cuh"
#include "vb_tc.cuh"
#include "vb_stream.cuh"

#include <stddef.h>
#include <stdio.h>
#include <string.h>

static_assert(sizeof(vb200_ref_cuda_ctx_t) == 2400, "must match tts_cuda_ctx_t (voxtral_tts_cuda.h:28-79)");
static_assert(offsetof(vb200_ref_cuda_ctx_t, kv_k) == 2184, "K cache pointer offset of tts_cuda_ctx_t");
static_assert(offsetof(vb200_ref_cuda_ctx_t, initialized) == 2396, "initialized flag offset of tts_cuda_ctx_t");
static_assert(sizeof(vb200_layer_weights_t) == 72, "must match tts_dec_layer_t (voxtral_tts.h:101-114)");
static_assert(sizeof(vb200_decoder_weights_t) == 8 + 26 * 72 + 8, "must match tts_decoder_t");
static_assert(sizeof(vb200_acoustic_weights_t) == 8 * 8 + 3 * 72, "must match tts_acoustic_t");

using namespace vb;

extern "C" {

vb200_ref_cuda_ctx_t g_cuda;

int tts_cuda_init(int kv_cache_max) { return model_init(kv_cache_max); }
int tts_cuda_upload_llm_weights(void *p) { return model_upload_llm((const vb200_decoder_weights_t *)p); }
int tts_cuda_upload_acoustic_weights(void *p) { return model_upload_acoustic((const vb200_acoustic_weights_t *)p); }
void tts_cuda_free(void) { model_free(); }
int tts_cuda_available(void) { return g_cuda.initialized; }

void tts_cuda_linear_bf16(float *y, const float *x, const uint16_t *W_bf16, int seq_len, int in_dim,
                          int out_dim, const void *W_gpu) {
    if (linear(y, x, W_bf16, seq_len, in_dim, out_dim, W_gpu))
        fprintf(stderr, "voxtral_b200: tts_cuda_linear_bf16(%d,%d,%d) failed\n", seq_len, in_dim, out_dim);
}

void tts_cuda_rms_norm(float *d_out, const float *d_x, const float *d_weight, int seq_len, int dim, float eps) {
    if (!model().inited) return;
    rms_norm(d_out, d_x, d_weight, seq_len, dim, eps, model().st);
}

void tts_cuda_apply_rope(float *d_x, const float *d_freqs, int seq, int heads, int head_dim) {
    if (!model().inited || !d_freqs) return;
    rope_apply(d_x, d_freqs, seq, heads, head_dim, heads * head_dim, model().st);
}

void tts_cuda_compute_rope_freqs(float *d_freqs, int start_pos, int seq, int dim, float theta) {
    if (!model().inited) return;
    rope_table(d_freqs, start_pos, seq, dim, theta, model().st);
}

void tts_cuda_silu_mul(float *d_gate, const float *d_up, int n) {
    if (!model().inited) return;
    silu_mul(d_gate, d_up, n, model().st);
}

void tts_cuda_add_inplace(float *d_a, const float *d_b, int n) {
    if (!model().inited) return;
    add_inplace(d_a, d_b, n, model().st);
}

void tts_cuda_causal_attention_decode(float *d_out, const float *d_Q, const float *d_K_cache,
                                      const float *d_V_cache, int seq_k, int n_heads, int n_kv_heads,
                                      int head_dim, float scale, int kv_cache_stride) {
    if (!model().inited || seq_k <= 0) return;
    const int ldk = kv_cache_stride > 0 ? kv_cache_stride : n_kv_heads * head_dim;
    if (attention_rows(d_out, d_Q, d_K_cache, d_V_cache, 1, seq_k, n_heads, n_kv_heads, head_dim, scale,
                       seq_k - 1, 1, n_heads * head_dim, ldk, n_heads * head_dim, model().st))
        fprintf(stderr, "voxtral_b200: unsupported attention shape (heads %d/%d, head_dim %d)\n", n_heads,
                n_kv_heads, head_dim);
}

void tts_cuda_causal_attention_prefill(float *d_out, const float *d_Q, const float *d_K, const float *d_V,
                                       int seq_len, int start_pos, int n_heads, int n_kv_heads, int head_dim,
                                       float scale) {
    if (!model().inited || seq_len <= 0) return;
    if (attention_rows(d_out, d_Q, d_K, d_V, seq_len, start_pos + seq_len, n_heads, n_kv_heads, head_dim, scale,
                       start_pos, 1, n_heads * head_dim, n_kv_heads * head_dim, n_heads * head_dim, model().st))
        fprintf(stderr, "voxtral_b200: unsupported attention shape (heads %d/%d, head_dim %d)\n", n_heads,
                n_kv_heads, head_dim);
}

void tts_cuda_bidirectional_attention(float *d_out, const float *d_Q, const float *d_K, const float *d_V,
                                      int seq_len, int n_heads, int n_kv_heads, int head_dim, float scale) {
    if (!model().inited || seq_len <= 0) return;
    if (attention_rows(d_out, d_Q, d_K, d_V, seq_len, seq_len, n_heads, n_kv_heads, head_dim, scale, 0, 0,
                       n_heads * head_dim, n_kv_heads * head_dim, n_heads * head_dim, model().st))
        fprintf(stderr, "voxtral_b200: unsupported attention shape (heads %d/%d, head_dim %d)\n", n_heads,
                n_kv_heads, head_dim);
}

void tts_cuda_embed_token(float *d_out, const void *d_embeddings_bf16, int token_id, int dim) {
    if (!model().inited) return;
    embed_token(d_out, (const uint16_t *)d_embeddings_bf16, token_id, dim, model().st);
}

void tts_cuda_llm_forward(float *out_hidden, const float *input_embed, int pos) {
    if (llm_forward(out_hidden, input_embed, pos))
        fprintf(stderr, "voxtral_b200: tts_cuda_llm_forward(pos=%d) failed\n", pos);
}

void tts_cuda_llm_prefill(const float *embeds, int seq_len, int start_pos) {
    if (prefill(embeds, seq_len, start_pos))
        fprintf(stderr, "voxtral_b200: tts_cuda_llm_prefill(%d rows at %d) failed\n", seq_len, start_pos);
}

void tts_cuda_predict_velocity(float *out_velocity, const float *x_t, const float *llm_hidden, float t_val) {
    if (predict_velocity(out_velocity, x_t, llm_hidden, t_val))
        fprintf(stderr, "voxtral_b200: tts_cuda_predict_velocity failed\n");
}

void tts_cuda_to_device(void *d_dst, const void *h_src, size_t bytes) {
    cudaError_t e = cudaMemcpy(d_dst, h_src, bytes, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) fprintf(stderr, "voxtral_b200: copy to device failed: %s\n", cudaGetErrorString(e));
}

void tts_cuda_to_host(void *h_dst, const void *d_src, size_t bytes) {
    cudaError_t e = cudaMemcpy(h_dst, d_src, bytes, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) fprintf(stderr, "voxtral_b200: copy to host failed: %s\n", cudaGetErrorString(e));
}

void tts_cuda_memset(void *d_ptr, int value, size_t bytes) { cudaMemset(d_ptr, value, bytes); }

void *tts_cuda_alloc(size_t bytes) {
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return p;
}

void tts_cuda_free_ptr(void *d_ptr) {
    if (d_ptr) cudaFree(d_ptr);
}

void tts_cuda_sync(void) { cudaDeviceSynchronize(); }

/* ---------------- additions ---------------- */

int vb200_frame(const float *embed, const float *noise36, int pos, float *hidden_out, int *codes37) {
    return frame(embed, noise36, pos, hidden_out, codes37, false);
}

int vb200_frame_chained(const float *noise36, int pos, float *hidden_out, int *codes37) {
    return frame(nullptr, noise36, pos, hidden_out, codes37, true);
}

int vb200_acoustic_frame(const float *llm_hidden, const float *noise36, int *codes37, float *latent_out) {
    return acoustic_frame(llm_hidden, noise36, codes37, latent_out);
}

int vb200_utterance_begin(const float *first_embed, int start_pos, const float *noise, int n_frames) {
    return utterance_begin(first_embed, start_pos, noise, n_frames);
}

int vb200_utterance_run(int n_frames) { return utterance_run(n_frames); }

int vb200_batch_open(int n_utterances, int kv_max, int max_frames) { return batch_open(n_utterances, kv_max, max_frames); }
int vb200_batch_prefill(int utterance, const float *embeds, int n_rows) { return batch_prefill(utterance, embeds, n_rows); }
int vb200_batch_begin(const float *first_embeds, const int *start_pos, const float *noise) {
    return batch_begin(first_embeds, start_pos, noise);
}
int vb200_batch_run(int n_frames) { return batch_run(n_frames); }
int vb200_batch_end(int *codes_out, int *frames_done, int *hit_end, float *device_ms) {
    return batch_end(codes_out, frames_done, hit_end, device_ms);
}
int vb200_batch_hidden(float *out) { return batch_hidden(out); }
int vb200_batch_launches_per_frame(void) { return batch_launches_per_frame(); }
void vb200_batch_close(void) { batch_close(); }
int vb200_gemm_sweep(int which, int iters, float *ms, double *bytes_per_sweep, int *launches_per_sweep) {
    return gemm_sweep(which, iters, ms, bytes_per_sweep, launches_per_sweep);
}
int vb200_tc_gemm_probe(int M, int N, int K, int swiglu, int tiled, int reps, float *ms, int *splits) {
    int dev = 0, n_sm = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    return tc_probe(M, N, K, swiglu ? TC_EPI_SWIGLU_TERMS : TC_EPI_PARTIAL, tiled, reps, n_sm, ms, splits);
}
int vb200_stream_step_ms(int pos, int iters, float *ms, double *bytes_per_launch) {
    return stream_step_time(pos, iters, ms, bytes_per_launch);
}
int vb200_stream_probe(int N, int K, int n_ops, int sync, int reps, float *ms, double *bytes_per_launch) {
    return stream_probe(N, K, n_ops, sync, reps, ms, bytes_per_launch);
}
int vb200_selftest_wait_expiry(int limit_us) { return stream_wait_expiry(limit_us); }
int vb200_frame_on_stream_kernel(void) { return single_on_stream() ? 1 : 0; }
int vb200_tp_arena(int rank, int world, void *handle_out64) { return tp_arena(rank, world, handle_out64); }
int vb200_tp_connect(const void *handles) { return tp_connect(handles); }
void vb200_tp_close(void) { tp_close(); }
int vb200_tp_plan(int rank, int world, int n_sm, int *out9) { return tp_plan(rank, world, n_sm, out9); }
int vb200_frame_on_tensor_cores(void) { return single_tc_usable() ? 1 : 0; }

double vb200_utterance_engine_ms(int *launches) {
    if (launches) *launches = model().run_engine_n;
    return model().run_engine_ms;
}

int vb200_set_option(const char *name, int value) {
    if (!name) return -1;
    if (!strcmp(name, "ignore_end")) {
        const bool v = value != 0;
        if (v != model().ignore_end) {
            if (model().st) cudaStreamSynchronize(model().st);
            model().ignore_end = v;
            batch_options_changed();
        }
        return 0;
    }
    if (!strcmp(name, "decoder_kernel")) {
        if (value != 0 && value != 1) return -1;
        if ((value != 0) != model().decoder_stream) {
            if (model().st) cudaStreamSynchronize(model().st);
            model().decoder_stream = value != 0;
            single_path_changed();
        }
        return 0;
    }
    if (!strcmp(name, "codec_block_frames")) return codec_set_block_frames(value);
    if (!strcmp(name, "wait_limit_us")) {
        if (value < 1) return -1;
        model().wait_cycles = (long long)value * 2000;   /* SM clock, about 2 GHz */
        return 0;
    }
    return -1;
}

int vb200_utterance_end(int *codes_out, int *frames_done, int *hit_end, float *device_ms) {
    return utterance_end(codes_out, frames_done, hit_end, device_ms);
}

int vb200_prefill_prompt(const int *text_ids, int n_text, const uint16_t *voice_bf16, int n_voice, int start_pos) {
    return prefill_prompt(text_ids, n_text, voice_bf16, n_voice, start_pos);
}

int vb200_upload_audio_embed(const uint16_t *table_bf16, int rows) {
    return model_upload_audio_embed(table_bf16, rows);
}

int vb200_codec_upload(const vb200_codec_weights_t *w) { return codec_upload(w); }
int vb200_codec_decode(const int *codes, int n_frames, float *samples_out, int max_samples, int *n_samples) {
    return codec_decode(codes, n_frames, samples_out, max_samples, n_samples);
}
float vb200_codec_last_ms(void) { return codec_last_ms(); }

void vb200_upload_stats(double *seconds, double *bytes) {
    if (seconds) *seconds = model().upload_seconds;
    if (bytes) *bytes = model().upload_bytes;
}

static int kv_rows(int layer, int pos0, int n, float *k_rows, float *v_rows, bool to_device) {
    Model &m = model();
    if (!m.inited || layer < 0 || layer >= VB200_DEC_LAYERS || pos0 < 0 || n < 0 || pos0 + n > m.kv_max) return -1;
    const size_t off = ((size_t)layer * m.kv_max + pos0) * VB200_KV_DIM;
    const size_t bytes = (size_t)n * VB200_KV_DIM * sizeof(float);
    cudaError_t e1, e2;
    if (to_device) {
        e1 = cudaMemcpy(m.kv_k + off, k_rows, bytes, cudaMemcpyHostToDevice);
        e2 = cudaMemcpy(m.kv_v + off, v_rows, bytes, cudaMemcpyHostToDevice);
    } else {
        e1 = cudaMemcpy(k_rows, m.kv_k + off, bytes, cudaMemcpyDeviceToHost);
        e2 = cudaMemcpy(v_rows, m.kv_v + off, bytes, cudaMemcpyDeviceToHost);
    }
    return (e1 == cudaSuccess && e2 == cudaSuccess) ? 0 : -1;
}

int vb200_kv_write(int layer, int pos0, int n, const float *k_rows, const float *v_rows) {
    return kv_rows(layer, pos0, n, (float *)k_rows, (float *)v_rows, true);
}

int vb200_kv_read(int layer, int pos0, int n, float *k_rows, float *v_rows) {
    return kv_rows(layer, pos0, n, k_rows, v_rows, false);
}

int vb200_tap_enable(int on) {
    Model &m = model();
    if (!m.inited) return -1;
    m.tap_on = on != 0;
    return model_rebuild_programs();
}

int vb200_tap_read(float *out) {
    Model &m = model();
    if (!m.inited) return -1;
    return cudaMemcpy(out, m.tap, sizeof(float) * VB200_DEC_LAYERS * 2 * VB200_DIM, cudaMemcpyDeviceToHost) ==
                   cudaSuccess
               ? 0
               : -1;
}

int vb200_debug_gemv_plan(int N, int K, int M, int swiglu, int cta, int n_cta, int *out) {
    const int epi = swiglu ? VB_EPI_SWIGLU : VB_EPI_STORE;
    const int rc = gemv_validate(N, K, M, epi, n_cta);
    if (rc) return rc;
    const GemvPlan p = gemv_plan(N, K, M, epi, cta, n_cta);
    out[0] = p.r0; out[1] = p.r1; out[2] = p.passes; out[3] = p.seg_cols;
    out[4] = p.rows_per_chunk; out[5] = p.row_blocks; out[6] = p.n_chunks;
    return 0;
}

int vb200_last_status(void) { return model().last_status; }
int vb200_sm_count(void) { return model().sm_count; }

double vb200_engine_ms(int reset, int *n) {
    Model &m = model();
    flush_launch_time();
    const double avg = m.ms_n > 0 ? m.ms_sum / m.ms_n : 0.0;
    if (n) *n = m.ms_n;
    if (reset) {
        m.ms_sum = 0.0;
        m.ms_n = 0;
        m.timing = true;
    }
    return avg;
}

} /* extern "C" */
