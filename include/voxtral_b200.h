/*
 * voxtral_b200.h - the reference-compatible C ABI of libvoxtral_b200.so.
 *
 * Every symbol below has the name, argument meaning and error behaviour of the
 * entry point it replaces in mudler/voxtral-tts.c, so that the reference's
 * orchestrator (voxtral_tts.c), its decoder/acoustic stages and its kernel test
 * harness (test_kernels.c) link against this library unchanged. Each
 * declaration cites the reference interface it stands in for.
 *
 * Plain C: pointers and sizes only. "d_" arguments are device pointers obtained
 * from tts_cuda_alloc; everything else is host memory.
 *
 * The library is built for sm_100a only. tts_cuda_init returns -1 (and the
 * forward calls do nothing) when no such GPU is present; there is no CPU
 * fallback inside the library.
 */
#ifndef VOXTRAL_B200_H
#define VOXTRAL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Model dimensions, as fixed at compile time by the reference (voxtral_tts.h:19-79). */
#define VB200_DIM            3072
#define VB200_DEC_LAYERS     26
#define VB200_AC_LAYERS      3
#define VB200_HEADS          32
#define VB200_KV_HEADS       8
#define VB200_HEAD_DIM       128
#define VB200_HIDDEN         9216
#define VB200_Q_DIM          (VB200_HEADS * VB200_HEAD_DIM)
#define VB200_KV_DIM         (VB200_KV_HEADS * VB200_HEAD_DIM)
#define VB200_VOCAB          131072
#define VB200_NORM_EPS       1e-5f
#define VB200_ROPE_THETA     1000000.0f
#define VB200_ACOUSTIC_DIM   36
#define VB200_SEM_PADDED     8320
#define VB200_SEM_VALID_END  8194
#define VB200_FLOW_STEPS     8
#define VB200_FSQ_LEVELS     21
#define VB200_CFG_ALPHA      1.2f
#define VB200_CODES          37
#define VB200_CODE_END       1
#define VB200_AUDIO_ROWS     (8194 + 36 * 23)

/* Host-side weight tables handed to the upload calls. Field order and types are
 * those of tts_dec_layer_t / tts_ac_layer_t (voxtral_tts.h:101-114, :131-144),
 * tts_decoder_t (:116-125) and tts_acoustic_t (:146-165); a pointer to the
 * reference's struct can be passed as it is. BF16 matrices are row-major
 * [out, in]; gains are fp32. */
typedef struct {
    const uint16_t *wq, *wk, *wv, *wo;
    const float *attention_norm;
    const uint16_t *w1, *w2, *w3;       /* gate, down, up */
    const float *ffn_norm;
} vb200_layer_weights_t;

typedef struct {
    const uint16_t *tok_embeddings;     /* [131072, 3072], lookup only */
    vb200_layer_weights_t layers[VB200_DEC_LAYERS];
    const float *norm;
} vb200_decoder_weights_t;

typedef struct {
    const float *time_inv_freq;         /* [1536] */
    const uint16_t *input_proj;         /* [3072, 36] */
    const uint16_t *time_proj;          /* [3072, 3072] */
    const uint16_t *llm_proj;           /* [3072, 3072] */
    const uint16_t *semantic_out;       /* [8320, 3072] */
    const float *semantic_out_bias;     /* [8320] or NULL */
    const uint16_t *acoustic_out;       /* [36, 3072] */
    const float *norm;
    vb200_layer_weights_t layers[VB200_AC_LAYERS];
} vb200_acoustic_weights_t;

/* Device-side mirror with the size and field offsets of tts_cuda_ctx_t
 * (voxtral_tts_cuda.h:21-79): 2400 bytes, K cache pointer at offset 2184. The
 * reference's own decoder stage writes the cache through these pointers after a
 * CPU prefill (voxtral_tts_llm.c:379-381), so kv_k / kv_v / kv_max and
 * `initialized` are kept meaningful; the per-layer weight slots are left NULL
 * (this library stores fused QKV and gate/up matrices instead). */
typedef struct {
    void *dev_layer_slots[9];
} vb200_ref_layer_slots_t;

typedef struct {
    void *blas_handle;                  /* always NULL: no cuBLAS here */
    int sm_major, sm_minor, has_bf16;
    void *tok_embeddings_gpu;
    float *dec_norm_gpu;
    vb200_ref_layer_slots_t dec_layers[VB200_DEC_LAYERS];
    void *ac_proj_slots[5];
    float *ac_norm_gpu;
    float *ac_time_inv_freq_gpu;
    vb200_ref_layer_slots_t ac_layers[VB200_AC_LAYERS];
    float *kv_k;                        /* [26, kv_max, 1024] fp32 */
    float *kv_v;
    int kv_max;
    float *dec_buffers[12];
    float *ac_buffers[10];
    float *embed_buffer;
    int max_alloc_seq;
    int initialized;
} vb200_ref_cuda_ctx_t;

/* voxtral_tts_cuda.h:82 */
extern vb200_ref_cuda_ctx_t g_cuda;

/* ---- lifetime (voxtral_tts_cuda.h:88-99; voxtral_tts_cuda.cu:92-243) ---- */

/* Selects the GPU, allocates the K/V cache for kv_cache_max positions and all
 * activation buffers. 0 on success (also when already initialised), -1 when no
 * sm_100 GPU is usable or an allocation fails. */
int tts_cuda_init(int kv_cache_max);
/* Copy (and repack) the BF16 weights out of the caller's mapping into HBM.
 * decoder_ptr / acoustic_ptr: vb200_decoder_weights_t* / vb200_acoustic_weights_t*
 * (equivalently the reference's tts_decoder_t* / tts_acoustic_t*). 0 or -1; on
 * failure tts_cuda_available() turns 0 because the reference ignores the
 * return value (voxtral_tts.c:96-99). */
int tts_cuda_upload_llm_weights(void *decoder_ptr);
int tts_cuda_upload_acoustic_weights(void *acoustic_ptr);
void tts_cuda_free(void);
int tts_cuda_available(void);

/* ---- linear (voxtral_tts_cuda.h:105-111; voxtral_tts_cuda.cu:364-431) ----
 * y[seq,out] = x[seq,in] . W[out,in]^T with BF16 W and fp32 x, y. x and y may
 * each be host or device memory; W_gpu is the device copy of W, or NULL to have
 * W_bf16 (host) uploaded for this call. */
void tts_cuda_linear_bf16(float *y, const float *x, const uint16_t *W_bf16,
                          int seq_len, int in_dim, int out_dim, const void *W_gpu);

/* ---- single ops on device buffers (voxtral_tts_cuda.h:117-154) ---- */
/* voxtral_tts_cuda.cu:468-478 */
void tts_cuda_rms_norm(float *d_out, const float *d_x, const float *d_weight,
                       int seq_len, int dim, float eps);
/* voxtral_tts_cuda.cu:504-509. d_freqs is the (cos,sin) table written by
 * tts_cuda_compute_rope_freqs, [seq, head_dim/2, 2] as in tts_apply_rope
 * (voxtral_tts_kernels.c:616-634). The reference's GPU version ignores the table
 * and rotates by position 0; this one applies the table. */
void tts_cuda_apply_rope(float *d_x, const float *d_freqs, int seq, int heads, int head_dim);
/* voxtral_tts_cuda.cu:511-515 (a stub there); fills the table for positions
 * start_pos .. start_pos+seq-1 like tts_compute_rope_freqs
 * (voxtral_tts_kernels.c:602-614). dim is the head dimension. */
void tts_cuda_compute_rope_freqs(float *d_freqs, int start_pos, int seq, int dim, float theta);
/* voxtral_tts_cuda.cu:521-533 */
void tts_cuda_silu_mul(float *d_gate, const float *d_up, int n);
/* voxtral_tts_cuda.cu:539-548 */
void tts_cuda_add_inplace(float *d_a, const float *d_b, int n);
/* voxtral_tts_cuda.cu:644-657: one query row against seq_k cached keys;
 * kv_cache_stride is the row pitch of the caches in floats (0 = n_kv_heads*head_dim). */
void tts_cuda_causal_attention_decode(float *d_out, const float *d_Q, const float *d_K_cache,
                                      const float *d_V_cache, int seq_k, int n_heads,
                                      int n_kv_heads, int head_dim, float scale,
                                      int kv_cache_stride);
/* voxtral_tts_cuda.cu:937-995: seq_len query rows at positions start_pos.. against
 * keys 0..start_pos+seq_len-1 with the causal mask. */
void tts_cuda_causal_attention_prefill(float *d_out, const float *d_Q, const float *d_K,
                                       const float *d_V, int seq_len, int start_pos,
                                       int n_heads, int n_kv_heads, int head_dim, float scale);
/* voxtral_tts_cuda.cu:663-684 */
void tts_cuda_bidirectional_attention(float *d_out, const float *d_Q, const float *d_K,
                                      const float *d_V, int seq_len, int n_heads,
                                      int n_kv_heads, int head_dim, float scale);
/* voxtral_tts_cuda.cu:706-712 */
void tts_cuda_embed_token(float *d_out, const void *d_embeddings_bf16, int token_id, int dim);

/* ---- decoder (voxtral_tts_cuda.h:160-165) ---- */
/* voxtral_tts_cuda.cu:710-797: one decode step at cache row `pos`; host in, host out. */
void tts_cuda_llm_forward(float *out_hidden, const float *input_embed, int pos);
/* voxtral_tts_cuda.cu:806-893 (never called by the reference, which prefills on
 * the CPU): seq_len rows of embeddings fill cache rows start_pos.. on the GPU. */
void tts_cuda_llm_prefill(const float *embeds, int seq_len, int start_pos);

/* ---- acoustic (voxtral_tts_cuda.h:172-174; voxtral_tts_cuda.cu:1016-1100) ---- */
void tts_cuda_predict_velocity(float *out_velocity, const float *x_t, const float *llm_hidden,
                               float t_val);

/* ---- memory helpers (voxtral_tts_cuda.h:180-185; voxtral_tts_cuda.cu:52-86) ---- */
void tts_cuda_to_device(void *d_dst, const void *h_src, size_t bytes);
void tts_cuda_to_host(void *h_dst, const void *d_src, size_t bytes);
void tts_cuda_memset(void *d_ptr, int value, size_t bytes);
void *tts_cuda_alloc(size_t bytes);
void tts_cuda_free_ptr(void *d_ptr);
void tts_cuda_sync(void);

#ifdef __cplusplus
}
#endif
#endif
