/*
 * vb_model.cu - host side of the library: device state, weight repacking, the op
 * programs for a decoder step / acoustic frame / whole frame, and the calls that
 * run them. Mirrors what voxtral_tts_cuda.cu:92-310 (init, upload) and
 * :710-797, :1016-1100 (forward passes) do for the reference, with a different
 * device layout and one kernel launch per call.
 */
#include "vb_model.cuh"
#include "vb_simple.cuh"
#include "vb_tc.cuh"

#include <math.h>
#include <stddef.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <thread>
#include <vector>

namespace vb {

#define VB_CHECK(call)                                                                         \
    do {                                                                                       \
        cudaError_t e_ = (call);                                                               \
        if (e_ != cudaSuccess) {                                                               \
            fprintf(stderr, "voxtral_b200: %s failed at %s:%d: %s\n", #call, __FILE__, __LINE__, \
                    cudaGetErrorString(e_));                                                   \
            return -1;                                                                         \
        }                                                                                      \
    } while (0)

static Model g_model;
Model &model() { return g_model; }

static const int D = VB200_DIM, QD = VB200_Q_DIM, KVD = VB200_KV_DIM, HID = VB200_HIDDEN;
static const int QKV = QD + 2 * KVD;
static const int A = VB200_ACOUSTIC_DIM;

template <typename T>
static int dev_alloc(T **p, size_t count) {
    void *q = nullptr;
    cudaError_t e = cudaMalloc(&q, count * sizeof(T));
    if (e != cudaSuccess) {
        fprintf(stderr, "voxtral_b200: cudaMalloc(%zu bytes) failed: %s\n", count * sizeof(T),
                cudaGetErrorString(e));
        *p = nullptr;
        return -1;
    }
    g_model.allocs.push_back(q);
    *p = (T *)q;
    return 0;
}

static void dev_release(void *p) {
    if (!p) return;
    for (size_t i = 0; i < g_model.allocs.size(); i++)
        if (g_model.allocs[i] == p) {
            g_model.allocs[i] = g_model.allocs.back();
            g_model.allocs.pop_back();
            break;
        }
    cudaFree(p);
}

int model_init(int kv_cache_max) {
    Model &m = g_model;
    if (m.inited) return 0;
    if (kv_cache_max <= 0) return -1;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        fprintf(stderr, "voxtral_b200: no CUDA device\n");
        return -1;
    }
    const char *env = getenv("VB200_DEVICE");
    m.device = env ? atoi(env) : 0;
    if (m.device < 0 || m.device >= count) m.device = 0;
    VB_CHECK(cudaSetDevice(m.device));
    cudaDeviceProp prop;
    VB_CHECK(cudaGetDeviceProperties(&prop, m.device));
    if (prop.major != 10) {
        fprintf(stderr, "voxtral_b200: %s is sm_%d%d; this library is built for sm_100a only\n", prop.name,
                prop.major, prop.minor);
        return -1;
    }
    m.sm_count = prop.multiProcessorCount;
    VB_CHECK(cudaStreamCreate(&m.st));
    VB_CHECK(cudaEventCreate(&m.ev0));
    VB_CHECK(cudaEventCreate(&m.ev1));
    VB_CHECK(cudaEventCreate(&m.evr0));
    VB_CHECK(cudaEventCreate(&m.evr1));
    m.n_cta = engine_max_ctas(m.device);
    if (m.n_cta <= 0) {
        fprintf(stderr, "voxtral_b200: frame kernel does not fit on this device\n");
        return -1;
    }
    if (getenv("VB200_PREFETCH")) m.prefetch_chunks = atoi(getenv("VB200_PREFETCH"));
    if (getenv("VB200_STREAM")) m.decoder_stream = atoi(getenv("VB200_STREAM")) != 0;
    const char *cta_env = getenv("VB200_CTAS");
    if (cta_env && atoi(cta_env) > 0 && atoi(cta_env) < m.n_cta) m.n_cta = atoi(cta_env);

    m.kv_max = kv_cache_max;
    const size_t kv_elems = (size_t)VB200_DEC_LAYERS * kv_cache_max * KVD;
    if (dev_alloc(&m.kv_k, kv_elems) || dev_alloc(&m.kv_v, kv_elems)) return -1;
    VB_CHECK(cudaMemset(m.kv_k, 0, kv_elems * sizeof(float)));
    VB_CHECK(cudaMemset(m.kv_v, 0, kv_elems * sizeof(float)));

    const int max_s = m.n_cta / VB200_KV_HEADS > 0 ? m.n_cta / VB200_KV_HEADS : 1;
    int rc = 0;
    rc |= dev_alloc(&m.x, D);
    rc |= dev_alloc(&m.qkv, QKV);
    rc |= dev_alloc(&m.attn, QD);
    rc |= dev_alloc(&m.h, HID);
    rc |= dev_alloc(&m.logits, VB200_SEM_PADDED);
    rc |= dev_alloc(&m.ltok, D);
    rc |= dev_alloc(&m.ttok, (size_t)(VB200_FLOW_STEPS - 1) * D);
    rc |= dev_alloc(&m.X6, (size_t)6 * D);
    rc |= dev_alloc(&m.qkv6, (size_t)6 * QKV);
    rc |= dev_alloc(&m.attn6, (size_t)6 * QD);
    rc |= dev_alloc(&m.h6, (size_t)6 * HID);
    rc |= dev_alloc(&m.attn_scratch, (size_t)VB200_KV_HEADS * max_s * 4 * (VB200_HEAD_DIM + 2));
    rc |= dev_alloc(&m.tap, (size_t)VB200_DEC_LAYERS * 2 * D);
    rc |= dev_alloc(&m.tickets, 64);
    rc |= dev_alloc(&m.bar, 16);
    rc |= dev_alloc(&m.exitc, 16);
    rc |= dev_alloc(&m.d_in, 1);
    rc |= dev_alloc(&m.d_out, 1);
    rc |= dev_alloc(&m.d_op1, 64);
    if (rc) return -1;
    VB_CHECK(cudaMemset(m.tickets, 0, 64 * sizeof(unsigned)));
    VB_CHECK(cudaMemset(m.bar, 0, 16 * sizeof(unsigned)));
    VB_CHECK(cudaMemset(m.exitc, 0, 16 * sizeof(unsigned)));
    VB_CHECK(cudaMemset(m.d_in, 0, sizeof(DevIn)));
    VB_CHECK(cudaMemset(m.d_out, 0, sizeof(DevOut)));
    VB_CHECK(cudaMemset(m.tap, 0, (size_t)VB200_DEC_LAYERS * 2 * D * sizeof(float)));
    VB_CHECK(cudaMallocHost((void **)&m.h_in, sizeof(DevIn)));
    VB_CHECK(cudaMallocHost((void **)&m.h_out, sizeof(DevOut)));
    memset(m.h_in, 0, sizeof(DevIn));
    memset(m.h_out, 0, sizeof(DevOut));

    for (int i = 0; i < VB200_FLOW_STEPS - 1; i++) {
        /* timesteps i/(steps-1) and their differences, as voxtral_tts_acoustic.c:336-342 */
        const float t0 = (float)i / (float)(VB200_FLOW_STEPS - 1);
        const float t1 = (float)(i + 1) / (float)(VB200_FLOW_STEPS - 1);
        m.dt[i] = t1 - t0;
    }

    memset(&g_cuda, 0, sizeof(g_cuda));
    g_cuda.sm_major = prop.major;
    g_cuda.sm_minor = prop.minor;
    g_cuda.has_bf16 = 1;
    g_cuda.kv_k = m.kv_k;
    g_cuda.kv_v = m.kv_v;
    g_cuda.kv_max = kv_cache_max;
    g_cuda.max_alloc_seq = 1;
    g_cuda.initialized = 1;
    m.inited = true;
    fprintf(stderr, "  voxtral_b200: %s (sm_%d%d), %d SMs, frame kernel on %d CTAs, KV cache %d positions\n",
            prop.name, prop.major, prop.minor, m.sm_count, m.n_cta, kv_cache_max);
    return 0;
}

void model_free() {
    Model &m = g_model;
    if (!m.inited) return;
    cudaDeviceSynchronize();
    batch_free_all();
    acoustic_tc_free_all();
    codec_free_all();
    prefill_free_all();
    for (void *p : m.allocs) cudaFree(p);
    m.allocs.clear();
    if (m.h_in) cudaFreeHost(m.h_in);
    if (m.h_out) cudaFreeHost(m.h_out);
    if (m.ev0) cudaEventDestroy(m.ev0);
    if (m.ev1) cudaEventDestroy(m.ev1);
    if (m.evr0) cudaEventDestroy(m.evr0);
    if (m.evr1) cudaEventDestroy(m.evr1);
    if (m.st) cudaStreamDestroy(m.st);
    m = Model();
    memset(&g_cuda, 0, sizeof(g_cuda));
}

/* ------------------------------------------------------------------ */
/* weights                                                             */
/* ------------------------------------------------------------------ */
/* Uploads replace whatever an earlier upload left in the same slot. */
template <typename T>
static void drop(T **p) {
    if (*p) { dev_release(*p); *p = nullptr; }
}

/* Host -> device copies of the weights go through a small ring of pinned staging buffers:
 * a few host threads fill buffer n + 1 from the caller's (pageable, usually memory-mapped:
 * voxtral_tts_safetensors.c:400-405) memory while the copy engine drains buffer n, and the
 * repacking kernels run behind the copies on the same stream. Nothing waits for the device
 * except a buffer that is still being drained; the upload call synchronises once at its end.
 * The reference copies every matrix with a blocking cudaMemcpy (voxtral_tts_cuda.cu:223-310). */
struct Stager {
    static const int kBufs = 3;
    size_t cap = (size_t)64 << 20;
    void *pin[kBufs] = {};
    cudaEvent_t drained[kBufs] = {};
    bool busy[kBufs] = {};
    int next = 0, threads = 4;
    bool ok = false;
};
static Stager g_stage;

static void stage_open() {
    Stager &s = g_stage;
    if (s.ok) return;
    const char *env = getenv("VB200_UPLOAD_THREADS");
    unsigned hc = std::thread::hardware_concurrency();
    s.threads = env ? atoi(env) : (hc >= 4 ? 4 : 1);   /* four saturate the host's copy bandwidth where measured */
    if (s.threads < 1) s.threads = 1;
    if (s.threads > 32) s.threads = 32;
    for (int i = 0; i < Stager::kBufs; i++) {
        if (cudaHostAlloc(&s.pin[i], s.cap, cudaHostAllocDefault) != cudaSuccess ||
            cudaEventCreateWithFlags(&s.drained[i], cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            return;   /* no pinned memory: stage_copy() falls back to plain copies */
        }
        s.busy[i] = false;
    }
    s.ok = true;
}

static void stage_close() {
    Stager &s = g_stage;
    for (int i = 0; i < Stager::kBufs; i++) {
        if (s.pin[i]) cudaFreeHost(s.pin[i]);
        if (s.drained[i]) cudaEventDestroy(s.drained[i]);
        s.pin[i] = nullptr; s.drained[i] = nullptr; s.busy[i] = false;
    }
    s.ok = false;
}

static void fill_parallel(char *dst, const char *src, size_t n, int threads) {
    const size_t min_part = (size_t)4 << 20;
    int parts = (int)((n + min_part - 1) / min_part);
    if (parts > threads) parts = threads;
    if (parts <= 1) { memcpy(dst, src, n); return; }
    const size_t per = ((n / parts) + 4095) & ~(size_t)4095;
    std::vector<std::thread> pool;
    for (int i = 1; i < parts; i++) {
        const size_t off = per * i;
        if (off >= n) break;
        const size_t len = off + per < n ? per : n - off;
        pool.emplace_back([=] { memcpy(dst + off, src + off, len); });
    }
    memcpy(dst, src, per < n ? per : n);
    for (auto &t : pool) t.join();
}

/* Asynchronous on m.st as far as the device goes; the source may be reused on return. */
static int stage_copy(void *dst, const void *src, size_t bytes) {
    Model &m = g_model;
    Stager &s = g_stage;
    m.upload_bytes += (double)bytes;
    if (!s.ok) {
        VB_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, m.st));
        VB_CHECK(cudaStreamSynchronize(m.st));
        return 0;
    }
    for (size_t off = 0; off < bytes; off += s.cap) {
        const size_t n = bytes - off < s.cap ? bytes - off : s.cap;
        const int b = s.next;
        s.next = (s.next + 1) % Stager::kBufs;
        if (s.busy[b]) VB_CHECK(cudaEventSynchronize(s.drained[b]));
        fill_parallel((char *)s.pin[b], (const char *)src + off, n, s.threads);
        VB_CHECK(cudaMemcpyAsync((char *)dst + off, s.pin[b], n, cudaMemcpyHostToDevice, m.st));
        VB_CHECK(cudaEventRecord(s.drained[b], m.st));
        s.busy[b] = true;
    }
    return 0;
}

static int upload_bf16(uint16_t **dst, const uint16_t *src, size_t n) {
    if (!src) return -1;
    drop(dst);
    if (dev_alloc(dst, n)) return -1;
    return stage_copy(*dst, src, n * 2);
}

static int upload_f32(float **dst, const float *src, size_t n) {
    if (!src) return -1;
    drop(dst);
    if (dev_alloc(dst, n)) return -1;
    return stage_copy(*dst, src, n * 4);
}

/* Column-split projections of one layer become single matrices: [wq; wk; wv] and
 * gate/up interleaved row by row. tmp_a / tmp_b hold the staged gate and up; everything is
 * ordered by the stream, so they are reused from layer to layer without a host wait. */
static int upload_layer(LayerDev &L, const vb200_layer_weights_t &w, uint16_t *tmp_a, uint16_t *tmp_b) {
    Model &m = g_model;
    if (!w.wq || !w.wk || !w.wv || !w.wo || !w.w1 || !w.w2 || !w.w3 || !w.attention_norm || !w.ffn_norm)
        return -1;
    drop(&L.wqkv);
    drop(&L.w13);
    if (dev_alloc(&L.wqkv, (size_t)QKV * D)) return -1;
    if (stage_copy(L.wqkv, w.wq, (size_t)QD * D * 2)) return -1;
    if (stage_copy(L.wqkv + (size_t)QD * D, w.wk, (size_t)KVD * D * 2)) return -1;
    if (stage_copy(L.wqkv + (size_t)(QD + KVD) * D, w.wv, (size_t)KVD * D * 2)) return -1;
    if (upload_bf16(&L.wo, w.wo, (size_t)D * QD)) return -1;
    if (upload_bf16(&L.w2, w.w2, (size_t)D * HID)) return -1;
    if (dev_alloc(&L.w13, (size_t)2 * HID * D)) return -1;
    if (stage_copy(tmp_a, w.w1, (size_t)HID * D * 2)) return -1;
    if (stage_copy(tmp_b, w.w3, (size_t)HID * D * 2)) return -1;
    interleave_rows(L.w13, tmp_a, tmp_b, HID, D, m.st);
    if (upload_f32(&L.attn_norm, w.attention_norm, D)) return -1;
    if (upload_f32(&L.ffn_norm, w.ffn_norm, D)) return -1;
    return 0;
}

/* Brackets one upload call: opens the staging ring, and on the way out waits for the stream
 * once, releases the ring and adds the call's wall-clock time to the model's upload record. */
struct UploadScope {
    std::chrono::steady_clock::time_point t0;
    UploadScope() : t0(std::chrono::steady_clock::now()) { stage_open(); }
    int finish(int rc) {
        if (cudaStreamSynchronize(g_model.st) != cudaSuccess) rc = -1;
        stage_close();
        g_model.upload_seconds += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        return rc;
    }
};

static void upload_failed() {
    g_model.llm_ready = g_model.ac_ready = false;
    g_cuda.initialized = 0; /* the caller ignores our return value (voxtral_tts.c:96-99) */
}

int model_upload_llm(const vb200_decoder_weights_t *w) {
    Model &m = g_model;
    if (!m.inited || !w) return -1;
    uint16_t *ta = nullptr, *tb = nullptr;
    if (dev_alloc(&ta, (size_t)HID * D) || dev_alloc(&tb, (size_t)HID * D)) { upload_failed(); return -1; }
    UploadScope scope;
    int rc = 0;
    for (int i = 0; i < VB200_DEC_LAYERS && !rc; i++) rc = upload_layer(m.dec[i], w->layers[i], ta, tb);
    if (!rc) rc = upload_f32(&m.dec_norm, w->norm, D);
    if (!rc && w->tok_embeddings) rc = upload_bf16(&m.tok_emb, w->tok_embeddings, (size_t)VB200_VOCAB * D);
    rc = scope.finish(rc);
    dev_release(ta);
    dev_release(tb);
    if (rc) {
        fprintf(stderr, "voxtral_b200: decoder weight upload failed\n");
        upload_failed();
        return -1;
    }
    g_cuda.tok_embeddings_gpu = m.tok_emb;
    g_cuda.dec_norm_gpu = m.dec_norm;
    m.llm_ready = true;
    batch_invalidate();
    prefill_tc_setup();
    return model_rebuild_programs();
}

int model_upload_acoustic(const vb200_acoustic_weights_t *w) {
    Model &m = g_model;
    if (!m.inited || !w) return -1;
    uint16_t *ta = nullptr, *tb = nullptr;
    if (dev_alloc(&ta, (size_t)HID * D) || dev_alloc(&tb, (size_t)HID * D)) { upload_failed(); return -1; }
    UploadScope scope;
    int rc = 0;
    for (int i = 0; i < VB200_AC_LAYERS && !rc; i++) rc = upload_layer(m.ac[i], w->layers[i], ta, tb);
    if (!rc) rc = upload_bf16(&m.ac_input_proj, w->input_proj, (size_t)D * A);
    if (!rc) rc = upload_bf16(&m.ac_time_proj, w->time_proj, (size_t)D * D);
    if (!rc) rc = upload_bf16(&m.ac_llm_proj, w->llm_proj, (size_t)D * D);
    if (!rc) rc = upload_bf16(&m.ac_sem_out, w->semantic_out, (size_t)VB200_SEM_PADDED * D);
    if (!rc) rc = upload_bf16(&m.ac_out, w->acoustic_out, (size_t)A * D);
    if (!rc) rc = upload_f32(&m.ac_norm, w->norm, D);
    if (!w->semantic_out_bias) drop(&m.ac_sem_bias);
    if (!rc && w->semantic_out_bias) rc = upload_f32(&m.ac_sem_bias, w->semantic_out_bias, VB200_SEM_PADDED);
    if (!rc && !w->time_inv_freq) rc = -1;
    rc = scope.finish(rc);
    dev_release(ta);
    dev_release(tb);
    if (rc) {
        fprintf(stderr, "voxtral_b200: acoustic weight upload failed\n");
        upload_failed();
        return -1;
    }
    g_cuda.ac_norm_gpu = m.ac_norm;
    m.inv_freq.assign(w->time_inv_freq, w->time_inv_freq + D / 2);

    /* The time token depends only on the step index: time_proj(temb(t_i)) for the
     * 7 timesteps is computed once here (voxtral_tts_acoustic.c:166-176,205-208).
     * cos/sin run on the host so they are the host libm's, like the reference's. */
    const int steps = VB200_FLOW_STEPS - 1;
    float *temb_h = (float *)malloc(sizeof(float) * steps * D);
    float *temb_d = nullptr;
    if (!temb_h || dev_alloc(&temb_d, (size_t)steps * D)) { free(temb_h); upload_failed(); return -1; }
    for (int i = 0; i < steps; i++) {
        const float t = (float)i / (float)(VB200_FLOW_STEPS - 1);
        for (int k = 0; k < D / 2; k++) {
            const float ang = t * m.inv_freq[k];
            temb_h[(size_t)i * D + k] = cosf(ang);
            temb_h[(size_t)i * D + D / 2 + k] = sinf(ang);
        }
    }
    cudaError_t ce = cudaMemcpy(temb_d, temb_h, sizeof(float) * steps * D, cudaMemcpyHostToDevice);
    free(temb_h);
    if (ce != cudaSuccess) { upload_failed(); return -1; }
    std::vector<VbOp> ops(1);
    VbOp &o = ops[0];
    memset(&o, 0, sizeof(o));
    o.type = VB_OP_GEMV; o.M = steps; o.N = D; o.K = D; o.epi = VB_EPI_STORE;
    o.W = m.ac_time_proj; o.x = temb_d; o.ldx = D; o.y = m.ttok; o.ldy = D;
    rc = run_ops(ops);
    if (!rc && cudaStreamSynchronize(m.st) != cudaSuccess) rc = -1;
    dev_release(temb_d);
    if (rc) { upload_failed(); return -1; }
    if (acoustic_tc_setup()) { upload_failed(); return -1; }
    batch_invalidate();
    m.ac_ready = true;
    return model_rebuild_programs();
}

int model_upload_audio_embed(const uint16_t *table, int rows) {
    Model &m = g_model;
    if (!m.inited || !table || rows < VB200_AUDIO_ROWS) return -1;
    if (m.audio_table) { dev_release(m.audio_table); m.audio_table = nullptr; }
    UploadScope scope;
    if (scope.finish(upload_bf16(&m.audio_table, table, (size_t)rows * D))) return -1;
    m.embed_ready = true;
    return model_rebuild_programs();
}

/* ------------------------------------------------------------------ */
/* programs                                                            */
/* ------------------------------------------------------------------ */
static VbOp op_zero() {
    VbOp o;
    memset(&o, 0, sizeof(o));
    return o;
}

static VbOp op_gemv(int M, int N, int K, const uint16_t *W, const float *x, int ldx, float *y, int ldy, int epi) {
    VbOp o = op_zero();
    o.type = VB_OP_GEMV; o.M = M; o.N = N; o.K = K; o.W = W; o.x = x; o.ldx = ldx; o.y = y; o.ldy = ldy;
    o.epi = epi; o.eps = VB200_NORM_EPS;
    return o;
}

/* Decoder step: per layer  norm+QKV | RoPE+append+attention | O+residual |
 * norm+gate/up+SwiGLU | down+residual ; then the final norm
 * (voxtral_tts_llm.c:205-267). `in` is the input embedding, `hidden` the output. */
static void build_llm(std::vector<VbOp> &ops, const float *in, float *hidden) {
    Model &m = g_model;
    const float scale = 1.0f / sqrtf((float)VB200_HEAD_DIM);
    for (int l = 0; l < VB200_DEC_LAYERS; l++) {
        const LayerDev &L = m.dec[l];
        const float *res = (l == 0) ? in : m.x;
        VbOp o = op_gemv(1, QKV, D, L.wqkv, res, D, m.qkv, QKV, VB_EPI_STORE);
        o.norm_w = L.attn_norm;
        ops.push_back(o);

        o = op_zero();
        o.type = VB_OP_ATTN_DECODE; o.M = 1; o.x = m.qkv; o.y = m.attn;
        o.p0 = m.attn_scratch; o.p1 = m.tickets;
        o.p2 = m.kv_k + (size_t)l * m.kv_max * KVD;
        o.p3 = m.kv_v + (size_t)l * m.kv_max * KVD;
        o.i0 = VB200_HEADS; o.i1 = VB200_KV_HEADS; o.f0 = scale; o.f1 = VB200_ROPE_THETA;
        ops.push_back(o);

        o = op_gemv(1, D, QD, L.wo, m.attn, QD, m.x, D, VB_EPI_ADD);
        o.res = res;
        if (m.tap_on) o.tap = m.tap + (size_t)(2 * l) * D;
        ops.push_back(o);

        o = op_gemv(1, 2 * HID, D, L.w13, m.x, D, m.h, HID, VB_EPI_SWIGLU);
        o.norm_w = L.ffn_norm;
        ops.push_back(o);

        o = op_gemv(1, D, HID, L.w2, m.h, HID, m.x, D, VB_EPI_ADD);
        o.res = m.x;
        if (m.tap_on) o.tap = m.tap + (size_t)(2 * l + 1) * D;
        ops.push_back(o);
    }
    VbOp o = op_zero();
    o.type = VB_OP_NORM; o.M = 1; o.K = D; o.x = m.x; o.ldx = D; o.y = hidden; o.ldy = D;
    o.norm_w = m.dec_norm; o.eps = VB200_NORM_EPS;
    ops.push_back(o);
}

/* Three acoustic layers on `rows` token rows (voxtral_tts_acoustic.c:215-253). */
static void build_ac_layers(std::vector<VbOp> &ops, int rows) {
    Model &m = g_model;
    const float scale = 1.0f / sqrtf((float)VB200_HEAD_DIM);
    for (int l = 0; l < VB200_AC_LAYERS; l++) {
        const LayerDev &L = m.ac[l];
        VbOp o = op_gemv(rows, QKV, D, L.wqkv, m.X6, D, m.qkv6, QKV, VB_EPI_STORE);
        o.norm_w = L.attn_norm;
        ops.push_back(o);

        o = op_zero();
        o.type = VB_OP_ATTN_AC; o.M = rows; o.x = m.qkv6; o.ldx = QKV; o.y = m.attn6; o.ldy = QD;
        o.i0 = VB200_HEADS; o.i1 = VB200_KV_HEADS; o.f0 = scale;
        ops.push_back(o);

        o = op_gemv(rows, D, QD, L.wo, m.attn6, QD, m.X6, D, VB_EPI_ADD);
        o.res = m.X6;
        ops.push_back(o);

        o = op_gemv(rows, 2 * HID, D, L.w13, m.X6, D, m.h6, HID, VB_EPI_SWIGLU);
        o.norm_w = L.ffn_norm;
        ops.push_back(o);

        o = op_gemv(rows, D, HID, L.w2, m.h6, HID, m.X6, D, VB_EPI_ADD);
        o.res = m.X6;
        ops.push_back(o);
    }
}

/* Acoustic frame (voxtral_tts_acoustic.c:283-372) with both guidance branches of
 * each Euler step batched as six rows. `hidden` is the decoder output on the
 * device; latents and velocities live in d_in / d_out. */
static void build_acoustic(std::vector<VbOp> &ops, const float *hidden, const float *noise_all = nullptr,
                           int *codes_all = nullptr) {
    Model &m = g_model;
    VbOp o = op_gemv(1, VB200_SEM_PADDED, D, m.ac_sem_out, hidden, D, m.logits, VB200_SEM_PADDED, VB_EPI_STORE);
    o.bias = m.ac_sem_bias;
    o.flags = VB_F_NOSYNC;
    ops.push_back(o);
    o = op_gemv(1, D, D, m.ac_llm_proj, hidden, D, m.ltok, D, VB_EPI_STORE);
    ops.push_back(o);
    o = op_zero();
    o.type = VB_OP_ARGMAX; o.N = VB200_SEM_PADDED; o.x = m.logits; o.i0 = VB200_SEM_VALID_END;
    o.p2 = m.d_out->codes; o.flags = VB_F_NOSYNC;
    ops.push_back(o);
    /* With the tensor-core path up, the Euler steps run as their own kernels after this
     * program (vb_acoustic_tc.cu); the program ends with the semantic head. */
    if (acoustic_tc_ready()) return;

    const int steps = VB200_FLOW_STEPS - 1;
    float *lat = &m.d_in->lat[0][0];
    float *vel = &m.d_out->vel[0][0];
    for (int s = 0; s < steps; s++) {
        o = op_zero();
        o.type = VB_OP_AC_TOKENS; o.N = D; o.K = A; o.W = m.ac_input_proj; o.x = lat; o.p0 = vel;
        o.p1 = m.ttok; o.p2 = m.ltok; o.y = m.X6; o.ldy = D; o.i0 = s; o.i1 = 0;
        o.f0 = VB200_CFG_ALPHA; o.f1 = (s > 0) ? m.dt[s - 1] : 0.0f;
        if (s == 0) o.p3 = (void *)noise_all;
        ops.push_back(o);
        build_ac_layers(ops, 6);
        /* final norm of token 0 of each branch (rows 0 and 3), then the velocity head */
        o = op_gemv(2, A, D, m.ac_out, m.X6, 3 * D, vel, A, VB_EPI_STORE);
        o.norm_w = m.ac_norm;
        ops.push_back(o);
    }
    o = op_zero();
    o.type = VB_OP_FSQ; o.K = A; o.x = lat; o.p0 = vel; o.p2 = m.d_out->codes;
    o.i0 = steps; o.i1 = VB200_FSQ_LEVELS; o.f0 = VB200_CFG_ALPHA; o.f1 = m.dt[steps - 1];
    o.p3 = codes_all;
    ops.push_back(o);
}

/* One velocity prediction exactly as the reference's entry point asks for it
 * (voxtral_tts_acoustic.c:182-262): three rows, arbitrary t. */
static void build_predict_velocity(std::vector<VbOp> &ops) {
    Model &m = g_model;
    VbOp o = op_gemv(1, D, D, m.ac_time_proj, m.d_in->temb, D, m.X6 + D, D, VB_EPI_STORE);
    o.flags = VB_F_NOSYNC;
    ops.push_back(o);
    o = op_gemv(1, D, D, m.ac_llm_proj, m.d_in->hidden_in, D, m.X6 + 2 * D, D, VB_EPI_STORE);
    o.flags = VB_F_NOSYNC;
    ops.push_back(o);
    o = op_zero();
    o.type = VB_OP_AC_TOKENS; o.N = D; o.K = A; o.W = m.ac_input_proj; o.x = &m.d_in->lat[0][0];
    o.y = m.X6; o.ldy = D; o.i0 = 0; o.i1 = 1;
    ops.push_back(o);
    build_ac_layers(ops, 3);
    o = op_gemv(1, A, D, m.ac_out, m.X6, D, &m.d_out->vel[0][0], A, VB_EPI_STORE);
    o.norm_w = m.ac_norm;
    ops.push_back(o);
}

static int validate(const std::vector<VbOp> &ops) {
    for (size_t i = 0; i < ops.size(); i++)
        if (ops[i].type == VB_OP_GEMV) {
            int rc = gemv_validate(ops[i].N, ops[i].K, ops[i].M, ops[i].epi, g_model.n_cta);
            /* bulk copies and 128-bit loads need 16-byte aligned rows */
            if (!rc && (((uintptr_t)ops[i].W | (uintptr_t)ops[i].x | (uintptr_t)ops[i].norm_w) & 15)) rc = -20;
            if (!rc && ops[i].M > 1 && (ops[i].ldx & 3)) rc = -21;
            if (rc) {
                fprintf(stderr, "voxtral_b200: op %zu (M=%d N=%d K=%d) not runnable: %d\n", i, ops[i].M, ops[i].N,
                        ops[i].K, rc);
                return -1;
            }
        }
    return 0;
}

static int upload_program(Program &p, const std::vector<VbOp> &ops) {
    if (validate(ops)) return -1;
    if (p.d_ops) { dev_release(p.d_ops); p.d_ops = nullptr; p.n = 0; }
    if (dev_alloc(&p.d_ops, ops.size())) return -1;
    VB_CHECK(cudaMemcpy(p.d_ops, ops.data(), ops.size() * sizeof(VbOp), cudaMemcpyHostToDevice));
    p.n = (int)ops.size();
    return 0;
}

int model_rebuild_programs() {
    Model &m = g_model;
    std::vector<VbOp> ops;
    if (m.llm_ready) {
        build_llm(ops, m.d_in->embed, m.d_out->hidden);
        if (upload_program(m.p_llm, ops)) return -1;
    }
    if (m.ac_ready) {
        ops.clear();
        build_acoustic(ops, m.d_in->hidden_in);
        if (upload_program(m.p_ac, ops)) return -1;
        ops.clear();
        build_predict_velocity(ops);
        if (upload_program(m.p_pv, ops)) return -1;
    }
    if (m.llm_ready && m.ac_ready) {
        ops.clear();
        build_llm(ops, m.d_in->embed, m.d_out->hidden);
        build_acoustic(ops, m.d_out->hidden);
        if (upload_program(m.p_frame, ops)) return -1;
        if (m.embed_ready) {
            ops.clear();
            VbOp o = op_zero();
            o.type = VB_OP_EMBED; o.N = D; o.W = m.audio_table; o.p0 = m.d_out->codes; o.y = m.d_in->embed;
            o.i0 = VB200_CODES; o.i1 = 8194; o.i2 = 23;
            ops.push_back(o);
            build_llm(ops, m.d_in->embed, m.d_out->hidden);
            build_acoustic(ops, m.d_out->hidden);
            if (upload_program(m.p_chain, ops)) return -1;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------ */
/* running                                                             */
/* ------------------------------------------------------------------ */
/* Per-launch device time (only while vb200_engine_ms has switched timing on): the
 * event pair of the previous launch is read before the next one reuses it. */
void flush_launch_time() {
    Model &m = g_model;
    if (!m.time_pending) return;
    m.time_pending = false;
    float ms = 0.0f;
    if (cudaEventSynchronize(m.ev1) == cudaSuccess && cudaEventElapsedTime(&ms, m.ev0, m.ev1) == cudaSuccess) {
        m.ms_sum += ms;
        m.ms_n++;
    }
}

static int launch(const VbOp *d_ops, int n) {
    Model &m = g_model;
    EngineArgs a;
    a.ops = d_ops; a.n_ops = n; a.dyn = &m.d_in->dyn;
    a.bar_counter = m.bar; a.exit_counter = m.exitc; a.status = &m.d_out->status;
    a.prefetch_chunks = m.prefetch_chunks;
    if (m.timing) {
        flush_launch_time();
        cudaEventRecord(m.ev0, m.st);
    }
    VB_CHECK(engine_launch(a, m.n_cta, m.st));
    if (m.timing) {
        cudaEventRecord(m.ev1, m.st);
        m.time_pending = true;
    }
    return 0;
}

static void account_time() { flush_launch_time(); }

/* Reads back the status word after a synchronised launch; a non-zero status
 * means a bounded wait ran out inside the kernel. The counters are re-zeroed so
 * that the next launch starts clean. */
static int check_status() {
    Model &m = g_model;
    m.last_status = m.h_out->status;
    if (m.last_status == 0) return 0;
    fprintf(stderr, "voxtral_b200: frame kernel gave up with status %d\n", m.last_status);
    cudaMemsetAsync(m.bar, 0, 16 * sizeof(unsigned), m.st);
    cudaMemsetAsync(m.exitc, 0, 16 * sizeof(unsigned), m.st);
    cudaMemsetAsync(m.tickets, 0, 64 * sizeof(unsigned), m.st);
    cudaMemsetAsync(&m.d_out->status, 0, sizeof(int), m.st);
    cudaStreamSynchronize(m.st);
    return -1;
}

int run_program(const Program &p) {
    if (!p.d_ops || p.n <= 0) return -1;
    return launch(p.d_ops, p.n);
}

int run_ops(const std::vector<VbOp> &ops) {
    Model &m = g_model;
    if (ops.empty() || ops.size() > 64) return -1;
    if (validate(ops)) return -1;
    VB_CHECK(cudaMemcpyAsync(m.d_op1, ops.data(), ops.size() * sizeof(VbOp), cudaMemcpyHostToDevice, m.st));
    return launch(m.d_op1, (int)ops.size());
}

static int finish(size_t out_bytes) {
    Model &m = g_model;
    VB_CHECK(cudaMemcpyAsync(m.h_out, m.d_out, out_bytes, cudaMemcpyDeviceToHost, m.st));
    VB_CHECK(cudaStreamSynchronize(m.st));
    account_time();
    return check_status();
}

int llm_forward(float *out_hidden, const float *embed, int pos) {
    Model &m = g_model;
    if (!m.inited || !m.llm_ready) return -1;
    if (pos < 0 || pos >= m.kv_max) {
        fprintf(stderr, "voxtral_b200: position %d outside the %d-row cache\n", pos, m.kv_max);
        return -1;
    }
    m.h_in->dyn.pos = pos; m.h_in->dyn.kv_max = m.kv_max; m.h_in->dyn.frame = 0; m.h_in->dyn.done = 0;
    memcpy(m.h_in->embed, embed, sizeof(float) * D);
    VB_CHECK(cudaMemcpyAsync(m.d_in, m.h_in, offsetof(DevIn, lat), cudaMemcpyHostToDevice, m.st));
    if (run_program(m.p_llm)) return -1;
    if (finish(offsetof(DevOut, vel))) return -1;
    memcpy(out_hidden, m.h_out->hidden, sizeof(float) * D);
    return 0;
}

int frame(const float *embed, const float *noise, int pos, float *hidden_out, int *codes, bool chained) {
    Model &m = g_model;
    if (!m.inited || !m.llm_ready || !m.ac_ready) return -1;
    if (chained && !m.embed_ready) return -1;
    if (pos < 0 || pos >= m.kv_max) {
        fprintf(stderr, "voxtral_b200: position %d outside the %d-row cache\n", pos, m.kv_max);
        return -1;
    }
    /* the whole frame as one graph of tensor-core GEMM launches; the streaming kernel serves
     * when that path is off or per-layer taps are wanted */
    if (single_tc_usable()) return single_frame(embed, noise, pos, hidden_out, codes, chained);
    m.h_in->dyn.pos = pos; m.h_in->dyn.kv_max = m.kv_max; m.h_in->dyn.frame = 0; m.h_in->dyn.done = 0;
    memcpy(m.h_in->lat[0], noise, sizeof(float) * A);
    if (chained) {
        VB_CHECK(cudaMemcpyAsync(&m.d_in->dyn, &m.h_in->dyn, sizeof(VbDyn), cudaMemcpyHostToDevice, m.st));
        VB_CHECK(cudaMemcpyAsync(m.d_in->lat[0], m.h_in->lat[0], sizeof(float) * A, cudaMemcpyHostToDevice, m.st));
        if (run_program(m.p_chain)) return -1;
        if (acoustic_tc_ready() && acoustic_tc_enqueue(nullptr, nullptr, 0, false, false)) return -1;
    } else {
        memcpy(m.h_in->embed, embed, sizeof(float) * D);
        VB_CHECK(cudaMemcpyAsync(m.d_in, m.h_in, offsetof(DevIn, lat) + sizeof(float) * A, cudaMemcpyHostToDevice,
                                 m.st));
        if (run_program(m.p_frame)) return -1;
        if (acoustic_tc_ready() && acoustic_tc_enqueue(nullptr, nullptr, 0, false, false)) return -1;
    }
    if (finish(offsetof(DevOut, vel))) return -1;
    memcpy(codes, m.h_out->codes, sizeof(int) * VB200_CODES);
    if (hidden_out) memcpy(hidden_out, m.h_out->hidden, sizeof(float) * D);
    return 0;
}

int acoustic_frame(const float *hidden, const float *noise, int *codes, float *latent_out) {
    Model &m = g_model;
    if (!m.inited || !m.ac_ready) return -1;
    memcpy(m.h_in->lat[0], noise, sizeof(float) * A);
    memcpy(m.h_in->hidden_in, hidden, sizeof(float) * D);
    VB_CHECK(cudaMemcpyAsync(m.d_in, m.h_in, offsetof(DevIn, temb), cudaMemcpyHostToDevice, m.st));
    if (run_program(m.p_ac)) return -1;
    if (acoustic_tc_ready() && acoustic_tc_enqueue(nullptr, nullptr, 0, false, false)) return -1;
    if (latent_out)
        VB_CHECK(cudaMemcpyAsync(m.h_in->lat[VB200_FLOW_STEPS - 1], m.d_in->lat[VB200_FLOW_STEPS - 1],
                                 sizeof(float) * A, cudaMemcpyDeviceToHost, m.st));
    if (finish(offsetof(DevOut, hidden))) return -1;
    memcpy(codes, m.h_out->codes, sizeof(int) * VB200_CODES);
    if (latent_out) memcpy(latent_out, m.h_in->lat[VB200_FLOW_STEPS - 1], sizeof(float) * A);
    return 0;
}

int predict_velocity(float *out_v, const float *x_t, const float *hidden, float t) {
    Model &m = g_model;
    if (!m.inited || !m.ac_ready) return -1;
    memcpy(m.h_in->lat[0], x_t, sizeof(float) * A);
    memcpy(m.h_in->hidden_in, hidden, sizeof(float) * D);
    for (int k = 0; k < D / 2; k++) {
        const float ang = t * m.inv_freq[k];
        m.h_in->temb[k] = cosf(ang);
        m.h_in->temb[D / 2 + k] = sinf(ang);
    }
    VB_CHECK(cudaMemcpyAsync(m.d_in, m.h_in, sizeof(DevIn), cudaMemcpyHostToDevice, m.st));
    if (run_program(m.p_pv)) return -1;
    if (finish(sizeof(DevOut))) return -1;
    memcpy(out_v, m.h_out->vel[0], sizeof(float) * A);
    return 0;
}

/* ------------------------------------------------------------------ */
/* device-resident frame loop                                          */
/* ------------------------------------------------------------------ */
/* The orchestrator's loop (voxtral_tts.c:301-321) without host round trips: the
 * noise of every frame is uploaded up front (the reference RNG is sequential and
 * draws 36 values per frame that is not END), codes are re-embedded on the device,
 * position and frame index advance in device memory, and an END code turns the
 * remaining queued launches into no-ops. */
int utterance_begin(const float *first_embed, int start_pos, const float *noise_all, int n_frames) {
    Model &m = g_model;
    if (!m.inited || !m.llm_ready || !m.ac_ready || !m.embed_ready) return -1;
    if (n_frames <= 0 || start_pos < 0 || start_pos >= m.kv_max) return -1;
    m.run_on_tc = single_tc_usable();
    if (m.run_on_tc) return single_begin(first_embed, start_pos, noise_all, n_frames);
    drop(&m.noise_all);
    drop(&m.codes_all);
    if (dev_alloc(&m.noise_all, (size_t)n_frames * A) || dev_alloc(&m.codes_all, (size_t)n_frames * VB200_CODES))
        return -1;
    VB_CHECK(cudaMemcpy(m.noise_all, noise_all, sizeof(float) * (size_t)n_frames * A, cudaMemcpyHostToDevice));
    VB_CHECK(cudaMemset(m.codes_all, 0, sizeof(int) * (size_t)n_frames * VB200_CODES));
    m.run_cap = n_frames;
    m.run_launched = 0;

    std::vector<VbOp> ops;
    VbOp adv = op_zero();
    adv.type = VB_OP_ADVANCE; adv.p0 = m.d_out->codes; adv.i0 = n_frames; adv.i1 = m.ignore_end ? 1 : 0;
    build_llm(ops, m.d_in->embed, m.d_out->hidden);
    build_acoustic(ops, m.d_out->hidden, m.noise_all, m.codes_all);
    if (!acoustic_tc_ready()) ops.push_back(adv);
    if (upload_program(m.p_run_first, ops)) return -1;
    ops.clear();
    VbOp e = op_zero();
    e.type = VB_OP_EMBED; e.N = D; e.W = m.audio_table; e.p0 = m.d_out->codes; e.y = m.d_in->embed;
    e.i0 = VB200_CODES; e.i1 = 8194; e.i2 = 23;
    ops.push_back(e);
    build_llm(ops, m.d_in->embed, m.d_out->hidden);
    build_acoustic(ops, m.d_out->hidden, m.noise_all, m.codes_all);
    if (!acoustic_tc_ready()) ops.push_back(adv);
    if (upload_program(m.p_run_next, ops)) return -1;

    m.h_in->dyn.pos = start_pos; m.h_in->dyn.kv_max = m.kv_max; m.h_in->dyn.frame = 0; m.h_in->dyn.done = 0;
    memcpy(m.h_in->embed, first_embed, sizeof(float) * D);
    VB_CHECK(cudaMemcpyAsync(m.d_in, m.h_in, offsetof(DevIn, lat), cudaMemcpyHostToDevice, m.st));
    VB_CHECK(cudaStreamSynchronize(m.st));
    return 0;
}

/* Queues n more frames; returns without waiting. */
int utterance_run(int n) {
    Model &m = g_model;
    if (m.run_on_tc) return single_run(n);
    if (!m.noise_all || n < 0) return -1;
    const bool timing = m.timing;
    m.timing = false;                      /* one event pair around the whole batch instead */
    m.run_ev_used = 0;
    cudaEventRecord(m.evr0, m.st);
    for (int i = 0; i < n; i++) {
        if (m.run_launched >= m.run_cap) break;
        /* the frame kernel's own device time: one event pair per launch */
        cudaEvent_t e0 = nullptr, e1 = nullptr;
        if (m.run_ev.size() < 2 * (size_t)(m.run_ev_used + 1)) {
            if (cudaEventCreate(&e0) == cudaSuccess && cudaEventCreate(&e1) == cudaSuccess) {
                m.run_ev.push_back(e0);
                m.run_ev.push_back(e1);
            }
        }
        const bool timed = m.run_ev.size() >= 2 * (size_t)(m.run_ev_used + 1);
        if (timed) cudaEventRecord(m.run_ev[2 * m.run_ev_used], m.st);
        if (run_program(m.run_launched == 0 ? m.p_run_first : m.p_run_next)) return -1;
        if (timed) cudaEventRecord(m.run_ev[2 * m.run_ev_used++ + 1], m.st);
        if (acoustic_tc_ready() && acoustic_tc_enqueue(m.noise_all, m.codes_all, m.run_cap, true, m.ignore_end))
            return -1;
        m.run_launched++;
    }
    cudaEventRecord(m.evr1, m.st);
    m.timing = timing;
    return 0;
}

/* Waits for the queued frames; codes_out receives [frames_done, 37]. A run that hit
 * END reports the END frame too (the reference drops it, voxtral_tts.c:307-311). */
int utterance_end(int *codes_out, int *frames_done, int *hit_end, float *device_ms) {
    Model &m = g_model;
    if (m.run_on_tc) {
        m.run_engine_ms = 0.0;
        m.run_engine_n = 0;
        return single_end(codes_out, frames_done, hit_end, device_ms);
    }
    if (!m.noise_all) return -1;
    VB_CHECK(cudaMemcpyAsync(m.h_out, m.d_out, offsetof(DevOut, hidden), cudaMemcpyDeviceToHost, m.st));
    VB_CHECK(cudaMemcpyAsync(&m.h_in->dyn, &m.d_in->dyn, sizeof(VbDyn), cudaMemcpyDeviceToHost, m.st));
    VB_CHECK(cudaStreamSynchronize(m.st));
    if (device_ms && cudaEventElapsedTime(device_ms, m.evr0, m.evr1) != cudaSuccess) *device_ms = -1.0f;
    m.run_engine_ms = 0.0;
    m.run_engine_n = 0;
    for (int i = 0; i < m.run_ev_used; i++) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, m.run_ev[2 * i], m.run_ev[2 * i + 1]) == cudaSuccess) {
            m.run_engine_ms += ms;
            m.run_engine_n++;
        }
    }
    const int done = m.h_in->dyn.frame;
    const int end = m.h_in->dyn.done;
    if (frames_done) *frames_done = done;
    if (hit_end) *hit_end = (end == 2) ? 1 : 0;
    if (codes_out && done > 0)
        VB_CHECK(cudaMemcpy(codes_out, m.codes_all, sizeof(int) * (size_t)done * VB200_CODES, cudaMemcpyDeviceToHost));
    m.h_in->dyn.done = 0;
    m.h_in->dyn.frame = 0;
    VB_CHECK(cudaMemcpy(&m.d_in->dyn, &m.h_in->dyn, sizeof(VbDyn), cudaMemcpyHostToDevice));
    return check_status();
}

/* y[M,N] = x[M,K] . W[N,K]^T for host or device x / y (cudaPointerGetAttributes
 * decides, as voxtral_tts_cuda.cu:374,399 does). Rows go through the streaming
 * engine eight at a time; shapes it does not take use the generic kernel. */
static bool is_device_ptr(const void *p) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

int linear_device(float *d_y, const float *d_x, const uint16_t *d_W, int M, int K, int N) {
    Model &m = g_model;
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const bool aligned = ((uintptr_t)d_x % 16 == 0) && ((uintptr_t)d_W % 16 == 0);
    const bool tc_rows = M >= 2 && (K % kTcBlockK) == 0 && !getenv("VB200_NO_TC");
    /* the streaming engine is checked for the widest row block it would get (8 rows, unless the
     * tensor-core GEMM takes the multi-row case) */
    const int m_engine = tc_rows ? 1 : (M < kMaxM ? M : kMaxM);
    if (!aligned || (m_engine > 1 && (K & 3)) || gemv_validate(N, K, m_engine, VB_EPI_STORE, m.n_cta) != 0) {
        linear_generic(d_y, d_x, d_W, nullptr, M, K, N, m.st);
        return 0;
    }
    /* Two or more rows: the tensor-core GEMMs (fp32 rows as BF16 terms, vb_tc.cu), all rows of a
     * block of up to kTcMaxRows in one launch. The term and split-K buffers are kept between
     * calls and only ever grow; everything is ordered by the stream. */
    if (tc_rows && tc_init() == 0) {
        TcWeight w;
        if (tc_weight(&w, d_W, N, K) == 0) {
            int rc = 0;
            for (int r = 0; r < M && !rc; r += kTcMaxRows) {
                const int rows = (M - r < kTcMaxRows) ? M - r : kTcMaxRows;
                const int rp = tc_rows_pad_any(rows);
                int splits = tc_pick_splits(N, K, m.sm_count);
                if (rows > 256) {   /* many row blocks fill the GPU by themselves */
                    const int ctas = ((N + 255) / 256) * ((rows + 127) / 128);
                    splits = m.sm_count / ctas < 1 ? 1 : (m.sm_count / ctas < splits ? m.sm_count / ctas : splits);
                }
                const size_t need_t = tc_acts_bytes(rp, K), need_p = splits > 1 ? sizeof(float) * (size_t)splits * rows * N : 0;
                if (need_t > m.lin_terms_cap) {
                    if (m.lin_terms) dev_release(m.lin_terms);
                    m.lin_terms = nullptr; m.lin_terms_cap = 0;
                    if (dev_alloc((unsigned char **)&m.lin_terms, need_t)) return -1;
                    m.lin_terms_cap = need_t;
                }
                if (need_p > m.lin_part_cap) {
                    if (m.lin_part) dev_release(m.lin_part);
                    m.lin_part = nullptr; m.lin_part_cap = 0;
                    if (dev_alloc((unsigned char **)&m.lin_part, need_p)) return -1;
                    m.lin_part_cap = need_p;
                }
                TcActs a;
                cudaMemsetAsync(m.lin_terms, 0, need_t, m.st);       /* padding rows stay finite */
                if (tc_acts(&a, (uint16_t *)m.lin_terms, rp, K)) rc = -1;
                if (!rc) tc_prepare(a, d_x + (size_t)r * K, K, rows, nullptr, 0, 0, nullptr, nullptr, nullptr, nullptr, m.st);
                TcGemm g;
                g.M = rows; g.status = &m.d_out->status; g.ld_out = N; g.splits = splits;
                if (!rc && splits == 1) {
                    g.epi = TC_EPI_STORE; g.out = d_y + (size_t)r * N;
                    rc = tc_gemm(w, a, g, m.st);
                } else if (!rc) {
                    g.epi = TC_EPI_PARTIAL; g.out = (float *)m.lin_part;
                    rc = tc_gemm(w, a, g, m.st);
                    if (!rc) tc_reduce(d_y + (size_t)r * N, (const float *)m.lin_part, splits, (size_t)rows * N,
                                       (size_t)rows * N, nullptr, N, m.st);
                }
            }
            if (cudaStreamSynchronize(m.st) != cudaSuccess) rc = -1;
            return rc;
        }
    }
    if (gemv_validate(N, K, M < kMaxM ? M : kMaxM, VB_EPI_STORE, m.n_cta) != 0 || (M > 1 && (K & 3))) {
        linear_generic(d_y, d_x, d_W, nullptr, M, K, N, m.st);
        return 0;
    }
    for (int r = 0; r < M; r += kMaxM) {
        const int rows = (M - r < kMaxM) ? M - r : kMaxM;
        std::vector<VbOp> ops(1, op_gemv(rows, N, K, d_W, d_x + (size_t)r * K, K, d_y + (size_t)r * N, N,
                                         VB_EPI_STORE));
        if (run_ops(ops)) return -1;
    }
    return 0;
}

int linear(float *y, const float *x, const uint16_t *W_host, int M, int K, int N, const void *W_gpu) {
    Model &m = g_model;
    if (!m.inited) return -1;
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const bool x_dev = is_device_ptr(x), y_dev = is_device_ptr(y);
    float *d_x = (float *)x, *d_y = y;
    uint16_t *d_W = (uint16_t *)W_gpu;
    void *tmp_x = nullptr, *tmp_y = nullptr, *tmp_W = nullptr;
    int rc = 0;
    if (!x_dev) {
        if (cudaMalloc(&tmp_x, (size_t)M * K * 4) != cudaSuccess) return -1;
        cudaMemcpyAsync(tmp_x, x, (size_t)M * K * 4, cudaMemcpyHostToDevice, m.st);
        d_x = (float *)tmp_x;
    }
    if (!y_dev) {
        if (cudaMalloc(&tmp_y, (size_t)M * N * 4) != cudaSuccess) rc = -1;
        d_y = (float *)tmp_y;
    }
    if (!rc && !d_W) {
        if (!W_host || cudaMalloc(&tmp_W, (size_t)N * K * 2) != cudaSuccess) rc = -1;
        else cudaMemcpyAsync(tmp_W, W_host, (size_t)N * K * 2, cudaMemcpyHostToDevice, m.st);
        d_W = (uint16_t *)tmp_W;
    }
    if (!rc) rc = linear_device(d_y, d_x, d_W, M, K, N);
    if (!rc && !y_dev) cudaMemcpyAsync(y, d_y, (size_t)M * N * 4, cudaMemcpyDeviceToHost, m.st);
    if (tmp_x || tmp_y || tmp_W) {
        cudaStreamSynchronize(m.st);
        cudaFree(tmp_x); cudaFree(tmp_y); cudaFree(tmp_W);
    }
    return rc;
}

} // namespace vb
