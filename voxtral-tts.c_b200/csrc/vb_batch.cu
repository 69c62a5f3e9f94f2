/*
 * vb_batch.cu - the frame as a CUDA graph of tensor-core GEMM launches, for one utterance or
 * for several independent utterances decoded in lock step on one GPU.
 *
 * The reference synthesises one utterance at a time (voxtral_tts.c:301-321: decoder step,
 * acoustic frame, re-embedding, per frame). Frames of different utterances do not depend on
 * one another, so B of them share every weight read: the decoder step becomes a B-row GEMM
 * and the acoustic passes a 6B-row GEMM on the tcgen05 kernel (vb_tc.cu); weights cross HBM
 * once per frame for all B utterances. Each utterance has its own KV cache slab, position,
 * noise rows and END state. B = 1 on the library's own cache serves the single-utterance calls
 * (vb200_frame, vb200_utterance_*, the drop-in's tts_llm_forward).
 *
 * One frame is a fixed sequence of launches (captured as a CUDA graph):
 *   embed (from the previous frame's codes)
 *   26 x [prepare, QKV GEMM, decode attention, O GEMM, prepare, gate/up GEMM, down GEMM]
 *   final norm, semantic-head GEMM + argmax, llm_proj GEMM
 *   7 Euler steps + FSQ (vb_acoustic_tc.cu), which also advances every utterance.
 *
 * Also here: the tensor-parallel variant of the decoder layers over the GPUs of a node
 * (struct Tp), and a measurement aid (gemm_sweep).
 */
#include "vb_acoustic_tc.cuh"
#include "vb_common.cuh"
#include "vb_stream.cuh"
#include "vb_umma.cuh"

#include <math.h>
#include <stdio.h>
#include <string.h>

namespace vb {

static const int D = VB200_DIM, QD = VB200_Q_DIM, KVD = VB200_KV_DIM, HID = VB200_HIDDEN;
static const int QKV = QD + 2 * KVD;
static const int A = VB200_ACOUSTIC_DIM;
static const int NSEM = VB200_SEM_PADDED;
constexpr int kHD = VB200_HEAD_DIM;        /* 128 */
constexpr int kGroup = VB200_HEADS / VB200_KV_HEADS;   /* 4 query heads per KV head */
constexpr int kBtMaxUtt = 8;
constexpr int kBtKeySplits = 16;           /* CTAs sharing one (utterance, KV head) */
constexpr int kBtSubsets = 4;              /* warp subsets of a CTA's key range */
constexpr int kBtAttnThreads = 512;
constexpr int kCodeStride = 40;            /* ints per utterance in the codes block */

/* Decoder weights on the tensor-core path (tile-contiguous copies), shared by every context. */
struct BtWeights {
    bool ready = false;
    TcWeight wqkv[VB200_DEC_LAYERS], wo[VB200_DEC_LAYERS], w13[VB200_DEC_LAYERS], w2[VB200_DEC_LAYERS];
    TcWeight wsem, wllm;
    std::vector<void *> allocs;
    int s_qkv = 1, s_wo = 1, s_w2 = 1, s_sem = 1, s_llm = 1;
};
static BtWeights g_w;

/* Slab-order copies of the decoder's matrices and of the two M = 1 heads, made once per
 * weight upload, for a grid of g_sw.n_cta CTAs. */
struct StreamWeights {
    bool ready = false;
    int n_cta = 0;
    uint16_t *wqkv[VB200_DEC_LAYERS] = {}, *wo[VB200_DEC_LAYERS] = {}, *w13[VB200_DEC_LAYERS] = {}, *w2[VB200_DEC_LAYERS] = {};
    uint16_t *wsem = nullptr, *wllm = nullptr;
    std::vector<void *> allocs;
};
static StreamWeights g_sw;


/* Host <-> device blocks of the single-utterance context: one copy each way per frame. */
struct OneIn {
    VbDyn dyn;
    alignas(16) float X[VB200_DIM];
    alignas(16) float noise[VB200_ACOUSTIC_DIM];
};
struct OneOut {
    int status[4];
    int codes[40];
    alignas(16) float hidden[VB200_DIM];
};

/* How a frame gets its decoder input row. */
enum EmbedMode {
    EMBED_HOST = 0,        /* the host wrote it */
    EMBED_CODES = 1,       /* always from the previous frame's codes */
    EMBED_CODES_AFTER0 = 2 /* from the codes, except for frame 0 of a run */
};

constexpr int kVariants = 3;   /* captured graphs: run loop, single frame, single chained frame */

struct Batch {
    bool open = false, begun = false, single = false;
    int B = 0, kv_max = 0, cap = 0, launched = 0;
    int alloc_cap = 0;                          /* frames the noise / code arrays were allocated for */
    std::vector<void *> allocs;
    /* per-utterance state */
    float *kv_k = nullptr, *kv_v = nullptr;     /* [B][layers][kv_max][1024] (single: the library's cache) */
    size_t slab = 0;                            /* floats per utterance */
    VbDyn *dyn = nullptr;                       /* [B] */
    float *X = nullptr, *hidden = nullptr;      /* [B][3072] */
    float *lat = nullptr, *vel = nullptr, *ltok = nullptr;
    int *codes = nullptr, *status = nullptr;
    float *noise_all = nullptr;                 /* [B][cap][36] */
    int *codes_all = nullptr;                   /* [B][cap][37] */
    float *noise1 = nullptr;                    /* single context: the noise row of a single-frame call */
    OneIn *d_in = nullptr, *h_in = nullptr;     /* single context */
    OneOut *d_out = nullptr, *h_out = nullptr;
    /* decoder-step activations */
    TcActs aD, aQ, aH;
    uint16_t *bD = nullptr, *bQ = nullptr, *bH = nullptr;
    float *part = nullptr, *ssq = nullptr, *logit_part = nullptr;
    float *part_qkv = nullptr, *part_wo = nullptr, *part_w2 = nullptr;   /* = part, or the tensor-parallel arena's */
    bool tp = false;                            /* this context runs tensor-parallel */
    float *attn_scratch = nullptr;
    unsigned *tickets = nullptr;
    AcBuffers ac;
    /* the decoder step as one launch of the persistent streaming kernel (vb_stream.cu) */
    bool stream = false, s_tap = false;
    const uint16_t *s_table = nullptr;          /* audio table the op lists were built with */
    stag_t *s_qkv = nullptr, *s_attn = nullptr, *s_h = nullptr, *s_xa = nullptr, *s_xb = nullptr;   /* tagged vectors */
    stag_t *s_scratch = nullptr;                /* attention key-slice partials, tagged */
    float *s_logits = nullptr;
    unsigned *s_counters = nullptr;             /* [0] grid barrier, [16] exit counter */
    unsigned *s_seq = nullptr;                  /* launch sequence number (never reset: tags must not repeat) */
    SOp *s_prog[kVariants] = {};
    SWeights *s_wl[kVariants] = {};             /* the producer's view of each op list: its GEMV weights in order */
    int s_n[kVariants] = {}, s_nw[kVariants] = {};
    cudaGraphExec_t exec[kVariants] = {};
    int direct_calls[kVariants] = {};
    int graph_cap = 0;                          /* frame cap baked into exec[0] */
    cudaEvent_t e0 = nullptr, e1 = nullptr;
};
static Batch g_bt;    /* vb200_batch_*: up to 8 utterances, own cache slabs */
static Batch g_one;   /* the single-utterance calls on the library's cache */

/* Tensor parallelism over the GPUs of one node, one process per GPU (single-utterance calls).
 * Every rank holds all weights and runs the same launches, but each GEMM of a decoder or
 * acoustic layer covers only this rank's slice of output tiles and stores its results into
 * every rank's buffers over NVLink; the small kernels between the GEMMs run redundantly on
 * identical data, so the residual stream and the caches stay bit-identical on all ranks. The
 * exchanged buffers (split-K partials per GEMM type, the SwiGLU terms) and the flag words lie
 * in one arena per rank at identical offsets; peers map it through CUDA IPC.
 *
 * Why a fast rank never overwrites data a slow rank still reads, with one buffer per GEMM type:
 * rank q stores exchange v+1 of a buffer only after its own consumer of exchange v of the
 * NEXT buffer in the layer cycle (QKV -> O -> gate/up -> down -> QKV ...) has passed its wait,
 * i.e. after every rank p has finished the GEMM that fills that next buffer; on p that GEMM is
 * stream-ordered after p's reads of exchange v of the first buffer. */
enum TpSlot { TP_QKV = 0, TP_WO = 1, TP_W13 = 2, TP_W2 = 3 };
struct TpSet {                 /* exchanged buffers of one context (decoder rows / acoustic rows) */
    size_t part[4];            /* byte offsets in the arena: partials of QKV, O, (unused), down */
    size_t bH;                 /* SwiGLU terms [3][16][9216] */
};
struct Tp {
    bool on = false;
    int rank = 0, world = 1;
    unsigned char *arena = nullptr;
    unsigned char *peer[kTpMaxRanks] = {};
    size_t bytes = 0, off_flags = 0;
    TpSet ll, ac;              /* decoder rows; acoustic rows (reserved: the acoustic layers are not sliced) */
    unsigned *epoch = nullptr, *tickets = nullptr;   /* local words */
};
static Tp g_tp;
constexpr int kTpRowsLl = 1, kTpRowsAc = 6;

static void tp_layout(Tp &t) {
    size_t o = 4096;            /* flags: 8 slots x 8 ranks */
    t.off_flags = 0;
    auto take = [&](size_t bytes) { const size_t at = o; o += (bytes + 1023) & ~(size_t)1023; return at; };
    for (int c = 0; c < 2; c++) {
        TpSet &st = c == 0 ? t.ll : t.ac;
        const size_t rows = c == 0 ? kTpRowsLl : kTpRowsAc;
        st.part[TP_QKV] = take(sizeof(float) * kTcMaxSplits * rows * QKV);
        st.part[TP_WO] = take(sizeof(float) * kTcMaxSplits * rows * D);
        st.part[TP_W13] = 0;
        st.part[TP_W2] = take(sizeof(float) * kTcMaxSplits * rows * D);
        st.bH = take(tc_acts_bytes(16, HID));
    }
    t.bytes = o;
}

/* Slice of `tiles` output tiles this rank computes. */
static void tp_slice(int tiles, int *t0, int *n) {
    const int a = (int)((long long)tiles * g_tp.rank / g_tp.world), b = (int)((long long)tiles * (g_tp.rank + 1) / g_tp.world);
    *t0 = a;
    *n = b - a;
}

/* Producer side of visit `visit` (1-based, of visits_per_frame per frame) of an exchanged buffer. */
static TcPush tp_push(int ctx, int slot, int visits_per_frame, int visit) {
    TcPush p;
    if (!g_tp.on) return p;
    p.n_dst = g_tp.world;
    /* destination 0 is the local copy (the kernel's plain store); the others follow */
    int d = 1;
    p.flag[0] = (unsigned *)(g_tp.arena + g_tp.off_flags) + (ctx * 4 + slot) * kTpMaxRanks + g_tp.rank;
    for (int r = 0; r < g_tp.world; r++) {
        if (r == g_tp.rank) continue;
        p.dst_off[d] = (long long)(g_tp.peer[r] - g_tp.arena);
        p.flag[d] = (unsigned *)(g_tp.peer[r] + g_tp.off_flags) + (ctx * 4 + slot) * kTpMaxRanks + g_tp.rank;
        d++;
    }
    p.ticket = g_tp.tickets + (ctx * 4 + slot);
    p.epoch = g_tp.epoch;
    p.visits_per_frame = visits_per_frame; p.visit = visit;
    return p;
}

static TcWait tp_wait_for(int ctx, int slot, int visits_per_frame, int visit, int *status) {
    TcWait w;
    if (!g_tp.on) return w;
    w.flags = (const unsigned *)(g_tp.arena + g_tp.off_flags) + (ctx * 4 + slot) * kTpMaxRanks;
    w.n = g_tp.world;
    w.epoch = g_tp.epoch;
    w.visits_per_frame = visits_per_frame; w.visit = visit;
    w.status = status;
    return w;
}

__global__ void tp_epoch_kernel(unsigned *epoch) { *epoch += 1u; }

/* ------------------------------------------------------------------ kernels */

/* Next decoder input of every utterance: the sum of the 37 code rows of the audio table in
 * codebook order (voxtral_tts_voice.c:292-315, offsets :275-283). Frame 0 of a run keeps the
 * row the host supplied. grid = (dim / 256, B). */
__global__ void bt_embed_kernel(float *X, const uint16_t *table, const int *codes, const VbDyn *dyn, int n_codes,
                                int rows0, int rows_other, int mode) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    if (dyn[b].done || (mode == EMBED_CODES_AFTER0 && dyn[b].frame == 0)) return;
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= D) return;
    const int *cb = codes + (size_t)b * kCodeStride;
    /* the 37 code loads, then the 37 table loads, are each in flight together; the sum keeps
     * the codebook order */
    constexpr int kMaxCodes = VB200_CODES;
    int rowi[kMaxCodes];
    uint16_t val[kMaxCodes];
#pragma unroll
    for (int c = 0; c < kMaxCodes; c++) rowi[c] = c < n_codes ? __ldcg(cb + c) : 0;
#pragma unroll
    for (int c = 0; c < kMaxCodes; c++) {
        const int base = c == 0 ? 0 : rows0 + (c - 1) * rows_other;
        val[c] = c < n_codes ? __ldg(table + (size_t)(base + rowi[c]) * D + n) : (uint16_t)0;
    }
    float acc = 0.0f;
#pragma unroll
    for (int c = 0; c < kMaxCodes; c++)
        if (c < n_codes) acc += __uint_as_float((uint32_t)val[c] << 16);
    X[(size_t)b * D + n] = acc;
}

/* Decode attention for one new token per utterance: split-K reduction of the QKV GEMM's
 * partials, RoPE on q and k, cache append, GQA attention over the utterance's own cache
 * (voxtral_tts_llm.c:221-238; tts_apply_rope / tts_causal_attention,
 * voxtral_tts_kernels.c:403-465, 602-634). grid = (key splits, KV heads, B); a CTA serves the
 * four query heads of its KV head on one slice of the keys; the last CTA of a (utterance,
 * KV head) to finish merges the slices in fixed order and writes the result as the three
 * BF16 terms the O projection's GEMM consumes. */
template <bool TP, int KP>
__global__ void __launch_bounds__(kBtAttnThreads)
bt_attn_kernel(uint16_t *terms, int rows_pad, const float *part, int n_part, size_t part_stride, float *kv_k,
               float *kv_v, size_t slab, int layer, const VbDyn *dyn, float scale, float theta, float *scratch,
               unsigned *tickets, int *status, const typename TcWaitSel<TP>::type wait) {
    __shared__ float cs[kHD];
    __shared__ __align__(16) float qraw[kGroup * kHD];
    __shared__ float kraw[kHD], vraw[kHD];
    __shared__ __align__(16) float qs[kGroup][kHD];
    __shared__ __align__(16) float attn_o[kBtSubsets][kGroup][kHD];
    __shared__ float attn_ml[kBtSubsets][kGroup][2];
    __shared__ float cmb_m[kBtKeySplits * kGroup], cmb_l[kBtKeySplits * kGroup];
    __shared__ int last_flag;
    pdl_launch_dependents();
    pdl_wait();
    if constexpr (TP) {   /* tensor parallelism: the QKV partials come from every rank */
        if (threadIdx.x == 0) tp_wait(wait);
        __syncthreads();
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int sp = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
    const int max_s = gridDim.x, G = gridDim.y;
    /* The split-K partials of q (and, for the first 128 threads, of the new k and v) are requested
     * before anything else: they depend on nothing this kernel reads, and the utterance's state
     * below is a second trip to L2 that now overlaps the first. */
    const float *row = part + (size_t)b * QKV;
    const bool kv_lane = tid < kHD;
    float pq[kTcMaxSplits], pk[kTcMaxSplits], pv[kTcMaxSplits];
#pragma unroll
    for (int p = 0; p < kTcMaxSplits; p++) {
        const bool on = p < n_part;
        pq[p] = on ? __ldcg(row + p * part_stride + (size_t)g * kGroup * kHD + tid) : 0.0f;
        pk[p] = (on && kv_lane) ? __ldcg(row + p * part_stride + QD + g * kHD + tid) : 0.0f;
        pv[p] = (on && kv_lane) ? __ldcg(row + p * part_stride + QD + KVD + g * kHD + tid) : 0.0f;
    }
    if (dyn[b].done) return;
    const int pos = dyn[b].pos, kv_max = dyn[b].kv_max;
    if (pos < 0 || pos >= kv_max) {
        if (tid == 0) atomicCAS(status, 0, (int)VB_ERR_POS_RANGE);
        return;
    }
    const int nk = pos + 1;
    int S = (nk + 31) / 32;
    if (S > max_s) S = max_s;
    if (S < 1) S = 1;
    if (sp >= S) return;
    const int j0 = (int)((long long)nk * sp / S), j1 = (int)((long long)nk * (sp + 1) / S);
    float *Kc = kv_k + (size_t)b * slab + (size_t)layer * kv_max * KVD;
    float *Vc = kv_v + (size_t)b * slab + (size_t)layer * kv_max * KVD;
    const bool writer = sp == S - 1;   /* its key range ends with the new token */

    {
        /* split-K sums in split order */
        const bool kv = writer && kv_lane;
        /* the rotation table is worked out while those loads are in flight */
        if (tid < kHD / 2) {
            const float freq = 1.0f / powf(theta, (float)(2 * tid) / (float)kHD);
            const float ang = (float)pos * freq;
            cs[2 * tid] = cosf(ang);
            cs[2 * tid + 1] = sinf(ang);
        }
        float v = 0.0f, kk = 0.0f, vv = 0.0f;
#pragma unroll
        for (int p = 0; p < kTcMaxSplits; p++) { v += pq[p]; kk += pk[p]; vv += pv[p]; }
        qraw[tid] = v;
        if (kv) { kraw[tid] = kk; vraw[tid] = vv; }
    }
    __syncthreads();
    const int half = kHD / 2;
    if (tid < kGroup * half) {
        const int hh = tid / half, d = tid % half;
        const float a = qraw[hh * kHD + 2 * d], bb = qraw[hh * kHD + 2 * d + 1];
        const float cv = cs[2 * d], sv = cs[2 * d + 1];
        qs[hh][2 * d] = a * cv - bb * sv;
        qs[hh][2 * d + 1] = a * sv + bb * cv;
    } else if (writer && tid < kGroup * half + half) {
        const int d = tid - kGroup * half;
        const float a = kraw[2 * d], bb = kraw[2 * d + 1];
        const float cv = cs[2 * d], sv = cs[2 * d + 1];
        float *dst = Kc + (size_t)pos * KVD + g * kHD;
        dst[2 * d] = a * cv - bb * sv;
        dst[2 * d + 1] = a * sv + bb * cv;
        __threadfence();
    } else if (writer && tid >= 384 && tid < 384 + kHD) {
        const int d = tid - 384;
        Vc[(size_t)pos * KVD + g * kHD + d] = vraw[d];
        __threadfence();
    }
    __syncthreads();

    const int hh = warp & 3, ss = warp >> 2;
    const float4 q4 = *reinterpret_cast<const float4 *>(&qs[hh][4 * lane]);
    float mx = -1e30f, den = 0.0f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    /* KP keys per pass: their 2 KP loads are in flight together, the running-maximum update then
     * takes them in key order as the reference does. Eight for a single utterance (one pass instead
     * of two at 256+ cached rows; its 80 CTAs have an SM each anyway), four for several (82
     * registers would leave one CTA per SM and a second wave of CTAs) */
    constexpr int kKeysPerPass = KP;
    for (int jb = j0 + ss; jb < j1; jb += kKeysPerPass * kBtSubsets) {
        float4 kq[kKeysPerPass], vq[kKeysPerPass];
#pragma unroll
        for (int u = 0; u < kKeysPerPass; u++) {
            const int j = jb + u * kBtSubsets;
            if (j < j1) {
                kq[u] = vb_ldcg4(Kc + (size_t)j * KVD + g * kHD + 4 * lane);
                vq[u] = vb_ldcg4(Vc + (size_t)j * KVD + g * kHD + 4 * lane);
            } else {
                kq[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                vq[u] = kq[u];
            }
        }
        float dq[kKeysPerPass];
#pragma unroll
        for (int u = 0; u < kKeysPerPass; u++)
            dq[u] = q4.x * kq[u].x + q4.y * kq[u].y + q4.z * kq[u].z + q4.w * kq[u].w;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
            for (int u = 0; u < kKeysPerPass; u++) dq[u] += __shfl_xor_sync(0xffffffffu, dq[u], off);
        }
#pragma unroll
        for (int u = 0; u < kKeysPerPass; u++) {
            if (jb + u * kBtSubsets >= j1) break;
            const float d = dq[u] * scale;
            const float4 vv = vq[u];
            if (d > mx) {
                const float corr = expf(mx - d);
                den = den * corr + 1.0f;
                o.x = o.x * corr + vv.x; o.y = o.y * corr + vv.y;
                o.z = o.z * corr + vv.z; o.w = o.w * corr + vv.w;
                mx = d;
            } else {
                const float w = expf(d - mx);
                den += w;
                o.x += w * vv.x; o.y += w * vv.y; o.z += w * vv.z; o.w += w * vv.w;
            }
        }
    }
    *reinterpret_cast<float4 *>(&attn_o[ss][hh][4 * lane]) = o;
    if (lane == 0) { attn_ml[ss][hh][0] = mx; attn_ml[ss][hh][1] = den; }
    __syncthreads();

    /* merge the four key subsets: thread = (head, dim) */
    const int th = tid / kHD, td = tid % kHD;
    float M0 = -1e30f;
#pragma unroll
    for (int u = 0; u < kBtSubsets; u++) M0 = fmaxf(M0, attn_ml[u][th][0]);
    float L = 0.0f, O = 0.0f;
#pragma unroll
    for (int u = 0; u < kBtSubsets; u++) {
        const float w = (attn_ml[u][th][1] > 0.0f) ? expf(attn_ml[u][th][0] - M0) : 0.0f;
        L += attn_ml[u][th][1] * w;
        O += attn_o[u][th][td] * w;
    }
    float result;
    if (S == 1) {
        result = (L > 0.0f) ? O * (1.0f / L) : 0.0f;
    } else {
        /* several CTAs share this KV head: publish the slice, the last arrival merges */
        const int stride = kHD + 2;
        float *po = scratch + (size_t)(b * G + g) * max_s * kGroup * stride;   /* [max_s][group][kHD + 2] */
        float *mine = po + ((size_t)sp * kGroup + th) * stride;
        mine[td] = O;
        if (td == 0) { mine[kHD] = M0; mine[kHD + 1] = L; }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned t = atomicAdd(&tickets[b * G + g], 1u);
            last_flag = (t == (unsigned)(S - 1));
            if (last_flag) tickets[b * G + g] = 0u;
        }
        __syncthreads();
        if (!last_flag) return;
        __threadfence();
        /* merge the S slices in slice order. All loads are issued before anything waits on them:
         * the (max, sum) pairs go through shared memory, the S output values of this thread's
         * (head, dim) are fetched in one unrolled batch. */
        if (tid < S * kGroup) {
            const float *pu = po + (size_t)tid * stride;           /* (slice, head) = tid / kGroup, tid % kGroup */
            cmb_m[tid] = __ldcg(pu + kHD);
            cmb_l[tid] = __ldcg(pu + kHD + 1);
        }
        float ov[kBtKeySplits];
#pragma unroll
        for (int u = 0; u < kBtKeySplits; u++)
            ov[u] = u < S ? __ldcg(po + ((size_t)u * kGroup + th) * stride + td) : 0.0f;
        __syncthreads();
        float Mg = -1e30f;
        for (int u = 0; u < S; u++) Mg = fmaxf(Mg, cmb_m[u * kGroup + th]);
        float Lg = 0.0f, Og = 0.0f;
#pragma unroll
        for (int u = 0; u < kBtKeySplits; u++) {
            if (u < S) {
                const float lu = cmb_l[u * kGroup + th];
                const float w = (lu > 0.0f) ? expf(cmb_m[u * kGroup + th] - Mg) : 0.0f;
                Lg += lu * w;
                Og += ov[u] * w;
            }
        }
        result = (Lg > 0.0f) ? Og * (1.0f / Lg) : 0.0f;
    }
    uint16_t t0, t1, t2;
    vb_split3(result, t0, t1, t2);
    const size_t off = (size_t)b * QD + (size_t)(g * kGroup + th) * kHD + td, term = (size_t)rows_pad * QD;
    terms[off] = t0;
    terms[term + off] = t1;
    terms[2 * term + off] = t2;
}

/* End of the decoder step: last residual add (split-K partials of the last down projection),
 * final RMSNorm (voxtral_tts_llm.c:267), hidden rows out as fp32 and as BF16 terms for the two
 * head GEMMs. grid = B, 1024 threads. */
template <bool TP>
__global__ void __launch_bounds__(1024)
bt_final_kernel(float *hidden, uint16_t *terms, int rows_pad, const float *X, const float *part, int n_part,
                size_t part_stride, const float *gain, float eps, float *tap, const typename TcWaitSel<TP>::type wait) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    if constexpr (TP) {
        if (threadIdx.x == 0) tp_wait(wait);
        __syncthreads();
    }
    const int b = blockIdx.x, tid = threadIdx.x;
    float v[3];
    float ss = 0.0f;
    {
        float pp[3][kTcMaxSplits], xv[3];
#pragma unroll
        for (int i = 0; i < 3; i++) {
            const int c = tid + i * 1024;
            xv[i] = __ldcg(X + (size_t)b * D + c);
#pragma unroll
            for (int p = 0; p < kTcMaxSplits; p++)
                pp[i][p] = p < n_part ? __ldcg(part + p * part_stride + (size_t)b * D + c) : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 3; i++) {
            float s = 0.0f;
#pragma unroll
            for (int p = 0; p < kTcMaxSplits; p++) s += pp[i][p];     /* split order; unused splits add 0 */
            v[i] = xv[i] + s;
            if (tap) tap[(size_t)b * D + tid + i * 1024] = v[i];       /* residual stream after the last layer */
            ss += v[i] * v[i];
        }
    }
    ss = vb_warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    float t = 0.0f;
    for (int w = 0; w < 32; w++) t += red[w];
    const float inv = 1.0f / sqrtf(t / (float)D + eps);
#pragma unroll
    for (int i = 0; i < 3; i++) {
        const int c = tid + i * 1024;
        const float h = v[i] * inv * __ldg(gain + c);
        hidden[(size_t)b * D + c] = h;
        uint16_t t0, t1, t2;
        vb_split3(h, t0, t1, t2);
        const size_t off = (size_t)b * D + c, term = (size_t)rows_pad * D;
        terms[off] = t0;
        terms[term + off] = t1;
        terms[2 * term + off] = t2;
    }
}

/* Masked greedy argmax over every utterance's semantic logits (voxtral_tts_acoustic.c:290-309):
 * index 0 and indices >= valid_end are excluded, the first strict maximum wins. The logits
 * arrive as split-K partials. grid = B, 1024 threads. */
__global__ void __launch_bounds__(1024)
bt_argmax_kernel(int *codes, const float *part, int n_part, size_t part_stride, const float *bias, int N,
                 int valid_end) {
    __shared__ float rv[32];
    __shared__ int ri[32];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x, tid = threadIdx.x;
    float best = -1e30f;
    int bi = 0;
    for (int i = tid; i < N; i += 1024) {
        float v = -1e30f;
        if (i != 0 && i < valid_end) {
            v = 0.0f;
            for (int p = 0; p < n_part; p++) v += __ldcg(part + p * part_stride + (size_t)b * N + i);
            if (bias) v += __ldg(bias + i);
        }
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if ((tid & 31) == 0) { rv[tid >> 5] = best; ri[tid >> 5] = bi; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 0; w < 32; w++)
            if (rv[w] > best || (rv[w] == best && ri[w] < bi)) { best = rv[w]; bi = ri[w]; }
        codes[(size_t)b * kCodeStride] = bi;
    }
}

/* ------------------------------------------------------------------ host */
static int bt_alloc(void **p, size_t bytes, std::vector<void *> *owner) {
    if (cudaMalloc(p, bytes) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    owner->push_back(*p);
    return cudaMemset(*p, 0, bytes) == cudaSuccess ? 0 : -1;
}

static void bt_free(std::vector<void *> *owner) {
    for (void *p : *owner) cudaFree(p);
    owner->clear();
}

static void drop_graphs(Batch &t) {
    for (int v = 0; v < kVariants; v++) {
        if (t.exec[v]) cudaGraphExecDestroy(t.exec[v]);
        t.exec[v] = nullptr;
        t.direct_calls[v] = 0;
    }
}

/* Tile-contiguous copies of the decoder's matrices and of the two heads, made once per
 * weight upload. */
static int bt_weights() {
    Model &m = model();
    BtWeights &w = g_w;
    if (w.ready) return 0;
    if (tc_init()) return -1;
    bt_free(&w.allocs);
    auto tiled = [&](TcWeight *tw, const uint16_t *src, int N, int K) -> int {
        void *dst = nullptr;
        if (bt_alloc(&dst, tc_tiled_bytes(N, K), &w.allocs)) return -1;
        return tc_weight_tiled(tw, src, N, K, (uint16_t *)dst, m.st);
    };
    for (int l = 0; l < VB200_DEC_LAYERS; l++) {
        const LayerDev &L = m.dec[l];
        if (tiled(&w.wqkv[l], L.wqkv, QKV, D) || tiled(&w.wo[l], L.wo, D, QD) || tiled(&w.w13[l], L.w13, 2 * HID, D) ||
            tiled(&w.w2[l], L.w2, D, HID))
            return -1;
    }
    /* the two heads belong to the acoustic upload; a decoder-only model (prefill) does without */
    w.wsem.ok = w.wllm.ok = false;
    if (m.ac_ready && (tiled(&w.wsem, m.ac_sem_out, NSEM, D) || tiled(&w.wllm, m.ac_llm_proj, D, D))) return -1;
    if (cudaStreamSynchronize(m.st) != cudaSuccess) return -1;
    w.s_qkv = tc_pick_splits(QKV, D, m.sm_count);
    w.s_wo = tc_pick_splits(D, QD, m.sm_count);
    w.s_w2 = tc_pick_splits(D, HID, m.sm_count);
    w.s_sem = tc_pick_splits(NSEM, D, m.sm_count);
    w.s_llm = tc_pick_splits(D, D, m.sm_count);
    w.ready = true;
    return 0;
}

/* The decoder's tile-contiguous matrices for the prefill: [26] each, in layer order. */
int batch_tiled_decoder(const TcWeight **wqkv, const TcWeight **wo, const TcWeight **w13, const TcWeight **w2) {
    if (!model().llm_ready || bt_weights()) return -1;
    *wqkv = g_w.wqkv; *wo = g_w.wo; *w13 = g_w.w13; *w2 = g_w.w2;
    return 0;
}

static void ctx_close(Batch &t) {
    drop_graphs(t);
    if (model().st) cudaStreamSynchronize(model().st);
    bt_free(&t.allocs);
    if (t.h_in) cudaFreeHost(t.h_in);
    if (t.h_out) cudaFreeHost(t.h_out);
    if (t.e0) cudaEventDestroy(t.e0);
    if (t.e1) cudaEventDestroy(t.e1);
    t = Batch();
}

/* Called when weights are uploaded again: the copies and every captured graph are stale. */
void batch_invalidate() {
    drop_graphs(g_bt);
    drop_graphs(g_one);
    g_w.ready = false;
    g_sw.ready = false;
    /* the op lists of an open context point at the old copies */
    if (g_one.open && g_one.stream) ctx_close(g_one);
}

/* Called when an option that is baked into captured launches as a kernel argument changes
 * (ignore_end): the run-loop graphs are captured again on their next use. */
void batch_options_changed() {
    for (Batch *t : {&g_bt, &g_one}) {
        if (t->exec[0]) { cudaGraphExecDestroy(t->exec[0]); t->exec[0] = nullptr; }
        if (t->direct_calls[0] > 1) t->direct_calls[0] = 1;
    }
}

static void ctx_close(Batch &t);
void batch_close() { ctx_close(g_bt); }

/* The decoder-step kernel of the single-utterance calls was switched: reopen that context on
 * its next use. */
void single_path_changed() {
    if (g_one.open) ctx_close(g_one);
}

/* ---- tensor parallelism: set-up ---- */
void tp_close() {
    Tp &t = g_tp;
    if (model().st) cudaStreamSynchronize(model().st);
    ctx_close(g_one);
    for (int r = 0; r < t.world; r++)
        if (t.peer[r] && r != t.rank) cudaIpcCloseMemHandle(t.peer[r]);
    if (t.arena) cudaFree(t.arena);
    if (t.epoch) cudaFree(t.epoch);
    cudaGetLastError();
    t = Tp();
}

/* Step 1 (every rank): allocate this rank's exchange arena and return its IPC handle (64 bytes). */
int tp_arena(int rank, int world, void *handle_out) {
    Model &m = model();
    if (!m.inited || !handle_out || world < 1 || world > kTpMaxRanks || rank < 0 || rank >= world) return -1;
    if ((QKV / kTcTileN) % world || (D / kTcTileN) % world || (2 * HID / kTcTileN) % world) return -1;
    tp_close();
    Tp &t = g_tp;
    t.rank = rank; t.world = world;
    tp_layout(t);
    if (cudaMalloc((void **)&t.arena, t.bytes) != cudaSuccess || cudaMemset(t.arena, 0, t.bytes) != cudaSuccess ||
        cudaMalloc((void **)&t.epoch, 64 * sizeof(unsigned)) != cudaSuccess ||
        cudaMemset(t.epoch, 0, 64 * sizeof(unsigned)) != cudaSuccess ||
        cudaIpcGetMemHandle((cudaIpcMemHandle_t *)handle_out, t.arena) != cudaSuccess) {
        tp_close();
        return -1;
    }
    t.tickets = t.epoch + 16;
    return 0;
}

/* The tile slices and split-K factors a rank would use: out[0..8] = first tile and tile count of
 * the QKV, O/down and gate/up GEMMs, then the split-K factors of QKV, O, down. Host arithmetic
 * only (no GPU needed): lets a test check that the slices of all ranks tile every matrix. */
int tp_plan(int rank, int world, int n_sm, int *out) {
    if (!out || world < 1 || world > kTpMaxRanks || rank < 0 || rank >= world) return -1;
    if ((QKV / kTcTileN) % world || (D / kTcTileN) % world || (2 * HID / kTcTileN) % world) return -1;
    const int tiles[3] = {QKV / kTcTileN, D / kTcTileN, 2 * HID / kTcTileN};
    for (int i = 0; i < 3; i++) {
        out[2 * i] = (int)((long long)tiles[i] * rank / world);
        out[2 * i + 1] = (int)((long long)tiles[i] * (rank + 1) / world) - out[2 * i];
    }
    out[6] = tc_pick_splits(out[1] * kTcTileN, D, n_sm);
    out[7] = tc_pick_splits(out[3] * kTcTileN, QD, n_sm);
    out[8] = tc_pick_splits(out[3] * kTcTileN, HID, n_sm);
    return 0;
}

/* Step 2 (every rank, after the handles of all ranks were gathered by the caller): map the
 * peers' arenas and switch the single-utterance calls to tensor-parallel launches. The caller
 * synchronises the ranks (a host barrier) before the first frame and keeps them in lock step:
 * every rank makes the same frame calls with the same inputs. */
int tp_connect(const void *handles) {
    Tp &t = g_tp;
    if (!t.arena || !handles) return -1;
    const cudaIpcMemHandle_t *h = (const cudaIpcMemHandle_t *)handles;
    for (int r = 0; r < t.world; r++) {
        if (r == t.rank) { t.peer[r] = t.arena; continue; }
        void *p = nullptr;
        if (cudaIpcOpenMemHandle(&p, h[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            cudaGetLastError();
            tp_close();
            return -1;
        }
        t.peer[r] = (unsigned char *)p;
    }
    ctx_close(g_one);       /* reopened on first use with its exchanged buffers inside the arena */
    t.on = t.world > 1;
    return 0;
}

void batch_free_all() {
    ctx_close(g_bt);
    ctx_close(g_one);
    tp_close();
    bt_free(&g_w.allocs);
    g_w.ready = false;
    bt_free(&g_sw.allocs);
    g_sw.ready = false;
}

/* ---- the streaming decoder step (vb_stream.cu) ---- */
/* Which kernel runs the decoder step of the single-utterance calls: the GEMM graph (default) or
 * the persistent streaming kernel (vb200_set_option("decoder_kernel", 1), or VB200_STREAM=1). */
static bool stream_wanted() { return model().decoder_stream; }

static int stream_weights() {
    Model &m = model();
    StreamWeights &w = g_sw;
    if (w.ready) return 0;
    bt_free(&w.allocs);
    w.n_cta = stream_max_ctas(m.device);
    if (w.n_cta <= 0) return -1;
    const struct { int N, K, epi; } shp[6] = {{QKV, D, S_EPI_STORE}, {D, QD, S_EPI_ADD}, {2 * HID, D, S_EPI_SWIGLU},
                                              {D, HID, S_EPI_ADD}, {NSEM, D, S_EPI_STORE}, {D, D, S_EPI_STORE}};
    for (int i = 0; i < 6; i++)
        if (stream_validate(shp[i].N, shp[i].K, shp[i].epi, w.n_cta)) return -1;
    auto slab = [&](uint16_t **dst, const uint16_t *src, int i) -> int {
        void *p = nullptr;
        if (bt_alloc(&p, stream_slab_bytes(shp[i].N, shp[i].K), &w.allocs)) return -1;
        *dst = (uint16_t *)p;
        return stream_make_slabs(*dst, src, shp[i].N, shp[i].K, shp[i].epi, w.n_cta, m.st);
    };
    for (int l = 0; l < VB200_DEC_LAYERS; l++) {
        const LayerDev &L = m.dec[l];
        if (slab(&w.wqkv[l], L.wqkv, 0) || slab(&w.wo[l], L.wo, 1) || slab(&w.w13[l], L.w13, 2) || slab(&w.w2[l], L.w2, 3))
            return -1;
    }
    if (slab(&w.wsem, m.ac_sem_out, 4) || slab(&w.wllm, m.ac_llm_proj, 5)) return -1;
    if (cudaStreamSynchronize(m.st) != cudaSuccess) return -1;
    w.ready = true;
    return 0;
}

static SOp sop_zero() {
    SOp o;
    memset(&o, 0, sizeof(o));
    return o;
}

static SOp sop_gemv(int N, int K, int epi, const uint16_t *W, const float *x, float *y) {
    SOp o = sop_zero();
    o.type = S_OP_GEMV; o.N = N; o.K = K; o.epi = epi; o.W = W; o.x = x; o.y = y; o.eps = VB200_NORM_EPS;
    return o;
}

static std::vector<SWeights> stream_weight_list(const std::vector<SOp> &ops) {
    std::vector<SWeights> wl;
    for (const SOp &o : ops)
        if (o.type == S_OP_GEMV) wl.push_back(SWeights{o.W, o.N, o.K, o.epi, 0});
    return wl;
}

/* The op lists of the three frame variants (they differ in how the input row is made). */
static int stream_programs(Batch &t) {
    Model &m = model();
    const StreamWeights &w = g_sw;
    const float scale = 1.0f / sqrtf((float)kHD);
    for (int v = 0; v < kVariants; v++) {
        std::vector<SOp> ops;
        if (v != 1) {
            SOp e = sop_zero();
            e.type = S_OP_EMBED; e.N = D; e.W = m.audio_table; e.p0 = t.codes; e.y = t.X;
            e.i0 = VB200_CODES; e.i1 = 8194; e.i2 = 23;
            if (v == 0) e.flags = S_F_SKIP_FRAME0;
            ops.push_back(e);
        }
        /* The residual stream alternates between two tagged vectors: the O projection writes
         * xb = x + ..., the down projection writes xa = xb + ... (the input row itself stays
         * plain: the host or the embed op wrote it). Every vector a GEMV or attention op hands on
         * is tagged with (launch, producing op), so these ops need no grid barrier between them. */
        int tag = 0;
        const float *x_cur = t.X;               /* the layer's input: plain for layer 0, then xa */
        int x_cur_tag = 0;
        for (int l = 0; l < VB200_DEC_LAYERS; l++) {
            const LayerDev &L = m.dec[l];
            const int in_flag = x_cur_tag ? S_F_X_TAGGED : 0;
            SOp o = sop_gemv(QKV, D, S_EPI_STORE, w.wqkv[l], x_cur, (float *)t.s_qkv);
            o.gain = L.attn_norm;
            o.flags = S_F_NOSYNC | S_F_Y_TAGGED | in_flag; o.x_tag = x_cur_tag; o.y_tag = ++tag;
            const int qkv_tag = tag;
            ops.push_back(o);
            o = sop_zero();
            o.type = S_OP_ATTN; o.x = (const float *)t.s_qkv; o.y = (float *)t.s_attn;
            o.p2 = t.kv_k + (size_t)l * t.kv_max * KVD;
            o.p3 = t.kv_v + (size_t)l * t.kv_max * KVD;
            o.i0 = VB200_HEADS; o.i1 = VB200_KV_HEADS; o.f0 = scale; o.f1 = VB200_ROPE_THETA;
            o.p0 = t.s_scratch;
            o.flags = S_F_NOSYNC | S_F_X_TAGGED | S_F_Y_TAGGED; o.x_tag = qkv_tag; o.y_tag = ++tag;
            const int part_tag = tag;
            o.i2 = part_tag + 1;            /* with a single key slice it writes the final output itself */
            ops.push_back(o);
            o = sop_zero();
            o.type = S_OP_ATTN_MERGE; o.p0 = t.s_scratch; o.y = (float *)t.s_attn;
            o.i0 = VB200_HEADS; o.i1 = VB200_KV_HEADS;
            o.flags = S_F_NOSYNC | S_F_X_TAGGED | S_F_Y_TAGGED; o.x_tag = part_tag; o.y_tag = ++tag;
            const int attn_tag = tag;
            ops.push_back(o);
            o = sop_gemv(D, QD, S_EPI_ADD, w.wo[l], (const float *)t.s_attn, (float *)t.s_xb);
            o.res = x_cur;
            o.flags = S_F_NOSYNC | S_F_X_TAGGED | S_F_Y_TAGGED | (x_cur_tag ? S_F_RES_TAGGED : 0);
            o.x_tag = attn_tag; o.y_tag = ++tag;
            const int xb_tag = tag;
            if (m.tap_on) o.tap = m.tap + (size_t)(2 * l) * D;
            ops.push_back(o);
            o = sop_gemv(2 * HID, D, S_EPI_SWIGLU, w.w13[l], (const float *)t.s_xb, (float *)t.s_h);
            o.gain = L.ffn_norm;
            o.flags = S_F_NOSYNC | S_F_X_TAGGED | S_F_Y_TAGGED; o.x_tag = xb_tag; o.y_tag = ++tag;
            const int h_tag = tag;
            ops.push_back(o);
            o = sop_gemv(D, HID, S_EPI_ADD, w.w2[l], (const float *)t.s_h, (float *)t.s_xa);
            o.res = (const float *)t.s_xb;
            o.flags = S_F_NOSYNC | S_F_X_TAGGED | S_F_Y_TAGGED | S_F_RES_TAGGED; o.x_tag = h_tag; o.y_tag = ++tag;
            if (m.tap_on) o.tap = m.tap + (size_t)(2 * l + 1) * D;
            ops.push_back(o);
            x_cur = (const float *)t.s_xa;
            x_cur_tag = tag;
        }
        /* final RMSNorm (voxtral_tts_llm.c:267) folded into the two heads that read it; the
         * hidden row itself goes out through xn_out. Their outputs are plain vectors: a grid
         * barrier separates them from the argmax. */
        SOp o = sop_gemv(NSEM, D, S_EPI_STORE, w.wsem, x_cur, t.s_logits);
        o.gain = m.dec_norm; o.bias = m.ac_sem_bias; o.xn_out = t.hidden;
        o.flags = S_F_NOSYNC | S_F_X_TAGGED; o.x_tag = x_cur_tag;
        ops.push_back(o);
        o = sop_gemv(D, D, S_EPI_STORE, w.wllm, x_cur, t.ltok);
        o.gain = m.dec_norm;
        o.flags = S_F_X_TAGGED; o.x_tag = x_cur_tag;
        ops.push_back(o);
        o = sop_zero();
        o.type = S_OP_ARGMAX; o.N = NSEM; o.x = t.s_logits; o.i0 = VB200_SEM_VALID_END; o.p2 = t.codes;
        ops.push_back(o);
        if (tag > 255) return -1;
        if (!t.s_prog[v] && (bt_alloc((void **)&t.s_prog[v], sizeof(SOp) * 200, &t.allocs) ||
                             bt_alloc((void **)&t.s_wl[v], sizeof(SWeights) * 200, &t.allocs)))
            return -1;
        if (ops.size() > 200) return -1;
        const std::vector<SWeights> wl = stream_weight_list(ops);
        if (cudaMemcpyAsync(t.s_prog[v], ops.data(), sizeof(SOp) * ops.size(), cudaMemcpyHostToDevice, m.st) != cudaSuccess ||
            cudaMemcpyAsync(t.s_wl[v], wl.data(), sizeof(SWeights) * wl.size(), cudaMemcpyHostToDevice, m.st) != cudaSuccess ||
            cudaStreamSynchronize(m.st) != cudaSuccess)
            return -1;
        t.s_n[v] = (int)ops.size();
        t.s_nw[v] = (int)wl.size();
    }
    t.s_tap = m.tap_on;
    t.s_table = m.audio_table;
    return 0;
}

static int stream_step(Batch &t, int variant) {
    Model &m = model();
    SArgs a;
    a.ops = t.s_prog[variant]; a.n_ops = t.s_n[variant]; a.dyn = t.dyn;
    a.wl = t.s_wl[variant]; a.n_wl = t.s_nw[variant];
    a.bar_counter = t.s_counters; a.exit_counter = t.s_counters + 16; a.status = t.status;
    a.seq = t.s_seq;
    a.wait_cycles = m.wait_cycles;
    return stream_launch(a, g_sw.n_cta, m.st) == cudaSuccess ? 0 : -1;
}

/* Buffers of a context. single: one utterance on the library's own cache, with pinned
 * staging blocks; otherwise n_utt cache slabs of kv_max rows. */
static int ctx_open(Batch &t, bool single, int n_utt, int kv_max, int max_frames) {
    Model &m = model();
    ctx_close(t);
    /* one utterance on one GPU: the decoder step runs on the streaming kernel and needs the slab
     * copies; everything else (batches, tensor parallelism) runs the GEMM graph on the tile copies */
    const bool stream = single && !g_tp.on && stream_wanted() && stream_weights() == 0;
    if (!stream && bt_weights()) return -1;
    t.single = single;
    t.B = n_utt; t.kv_max = kv_max; t.cap = max_frames; t.alloc_cap = max_frames;
    t.slab = (size_t)VB200_DEC_LAYERS * kv_max * KVD;
    const int B = n_utt;
    int rc = 0;
    if (single) {
        t.kv_k = m.kv_k; t.kv_v = m.kv_v;
        rc |= bt_alloc((void **)&t.d_in, sizeof(OneIn), &t.allocs);
        rc |= bt_alloc((void **)&t.d_out, sizeof(OneOut), &t.allocs);
        if (!rc) {
            t.dyn = &t.d_in->dyn; t.X = t.d_in->X; t.noise1 = t.d_in->noise;
            t.status = t.d_out->status; t.codes = t.d_out->codes; t.hidden = t.d_out->hidden;
            if (cudaMallocHost((void **)&t.h_in, sizeof(OneIn)) != cudaSuccess ||
                cudaMallocHost((void **)&t.h_out, sizeof(OneOut)) != cudaSuccess)
                rc = -1;
            else { memset(t.h_in, 0, sizeof(OneIn)); memset(t.h_out, 0, sizeof(OneOut)); }
        }
    } else {
        rc |= bt_alloc((void **)&t.kv_k, sizeof(float) * t.slab * B, &t.allocs);
        rc |= bt_alloc((void **)&t.kv_v, sizeof(float) * t.slab * B, &t.allocs);
        rc |= bt_alloc((void **)&t.dyn, sizeof(VbDyn) * B, &t.allocs);
        rc |= bt_alloc((void **)&t.X, sizeof(float) * B * D, &t.allocs);
        rc |= bt_alloc((void **)&t.hidden, sizeof(float) * B * D, &t.allocs);
        rc |= bt_alloc((void **)&t.codes, sizeof(int) * B * kCodeStride, &t.allocs);
        rc |= bt_alloc((void **)&t.status, sizeof(int) * 4, &t.allocs);
    }
    rc |= bt_alloc((void **)&t.lat, sizeof(float) * B * VB200_FLOW_STEPS * A, &t.allocs);
    rc |= bt_alloc((void **)&t.vel, sizeof(float) * B * 2 * A, &t.allocs);
    rc |= bt_alloc((void **)&t.ltok, sizeof(float) * B * D, &t.allocs);
    if (max_frames > 0) {
        rc |= bt_alloc((void **)&t.noise_all, sizeof(float) * (size_t)B * max_frames * A, &t.allocs);
        rc |= bt_alloc((void **)&t.codes_all, sizeof(int) * (size_t)B * max_frames * VB200_CODES, &t.allocs);
    }
    rc |= bt_alloc((void **)&t.bD, tc_acts_bytes(16, D), &t.allocs);
    rc |= bt_alloc((void **)&t.bQ, tc_acts_bytes(16, QD), &t.allocs);
    rc |= bt_alloc((void **)&t.bH, tc_acts_bytes(16, HID), &t.allocs);
    if (single && g_tp.on) t.bH = (uint16_t *)(g_tp.arena + g_tp.ll.bH);
    rc |= bt_alloc((void **)&t.part, sizeof(float) * kTcMaxSplits * B * QKV, &t.allocs);
    t.part_qkv = t.part_wo = t.part_w2 = t.part;
    t.tp = single && g_tp.on;
    if (t.tp) {
        t.part_qkv = (float *)(g_tp.arena + g_tp.ll.part[TP_QKV]);
        t.part_wo = (float *)(g_tp.arena + g_tp.ll.part[TP_WO]);
        t.part_w2 = (float *)(g_tp.arena + g_tp.ll.part[TP_W2]);
    }
    rc |= bt_alloc((void **)&t.ssq, sizeof(float) * 16 * 16, &t.allocs);
    rc |= bt_alloc((void **)&t.logit_part, sizeof(float) * kTcMaxSplits * B * NSEM, &t.allocs);
    rc |= bt_alloc((void **)&t.attn_scratch,
                   sizeof(float) * (size_t)B * VB200_KV_HEADS * kBtKeySplits * kGroup * (kHD + 2), &t.allocs);
    rc |= bt_alloc((void **)&t.tickets, sizeof(unsigned) * B * VB200_KV_HEADS, &t.allocs);
    if (stream) {
        rc |= bt_alloc((void **)&t.s_qkv, sizeof(stag_t) * QKV, &t.allocs);
        rc |= bt_alloc((void **)&t.s_attn, sizeof(stag_t) * QD, &t.allocs);
        rc |= bt_alloc((void **)&t.s_h, sizeof(stag_t) * HID, &t.allocs);
        rc |= bt_alloc((void **)&t.s_xa, sizeof(stag_t) * D, &t.allocs);
        rc |= bt_alloc((void **)&t.s_xb, sizeof(stag_t) * D, &t.allocs);
        rc |= bt_alloc((void **)&t.s_seq, sizeof(unsigned) * 16, &t.allocs);
        rc |= bt_alloc((void **)&t.s_scratch, sizeof(stag_t) * (size_t)VB200_KV_HEADS * 16 * kGroup * (kHD + 2), &t.allocs);
        rc |= bt_alloc((void **)&t.s_logits, sizeof(float) * NSEM, &t.allocs);
        rc |= bt_alloc((void **)&t.s_counters, sizeof(unsigned) * 64, &t.allocs);
    }
    if (rc) { ctx_close(t); return -1; }
    if (tc_acts(&t.aD, t.bD, 16, D) || tc_acts(&t.aQ, t.bQ, 16, QD) || tc_acts(&t.aH, t.bH, 16, HID)) {
        ctx_close(t);
        return -1;
    }
    t.ac = AcBuffers();
    if (acoustic_buffers_alloc(&t.ac, B, &t.allocs)) { ctx_close(t); return -1; }
    t.ac.lat = t.lat; t.ac.vel = t.vel; t.ac.ltok = t.ltok; t.ac.codes = t.codes; t.ac.dyn = t.dyn;
    t.ac.status = t.status;
    t.ac.sd.lat = VB200_FLOW_STEPS * A; t.ac.sd.vel = 2 * A; t.ac.sd.codes = kCodeStride;
    t.ac.sd.noise = (size_t)max_frames * A; t.ac.sd.codes_all = (size_t)max_frames * VB200_CODES;
    if (cudaEventCreate(&t.e0) != cudaSuccess || cudaEventCreate(&t.e1) != cudaSuccess) { ctx_close(t); return -1; }
    t.stream = stream;
    t.s_tap = m.tap_on;
    if (stream && stream_programs(t)) { ctx_close(t); return -1; }
    t.open = true;
    return 0;
}

/* One frame of every utterance of the context, enqueued launch by launch. */
static int enqueue_frame(Batch &t, int embed_mode, bool advance, const float *noise, int *codes_log, int cap) {
    Model &m = model();
    const BtWeights &w = g_w;
    cudaStream_t st = m.st;
    const int B = t.B;
    const float scale = 1.0f / sqrtf((float)kHD);
    const int chunksD = tc_prepare_chunks(D);
    const size_t psD = (size_t)B * D, psQ = (size_t)B * QKV;
    if (t.stream) {
        /* decoder step, semantic head + argmax and llm token: one launch */
        const int variant = embed_mode == EMBED_CODES_AFTER0 ? 0 : embed_mode == EMBED_HOST ? 1 : 2;
        if (stream_step(t, variant)) return -1;
        if (acoustic_tc_enqueue_on(t.ac, noise, codes_log, cap, advance, m.ignore_end)) return -1;
        return cudaGetLastError() == cudaSuccess ? 0 : -1;
    }
    if (embed_mode != EMBED_HOST)
        launch_pdl(bt_embed_kernel, dim3((D + 255) / 256, B), dim3(256), 0, st, t.X, (const uint16_t *)m.audio_table,
                   (const int *)t.codes, (const VbDyn *)t.dyn, VB200_CODES, 8194, 23, embed_mode);
    /* Tensor parallelism: this rank's tile slice of each layer GEMM, split-K chosen for the slice. */
    const bool tp = t.tp;
    int q0 = 0, qn = 0, o0 = 0, on = 0, h0 = 0, hn = 0;
    int s_qkv = w.s_qkv, s_wo = w.s_wo, s_w2 = w.s_w2;
    if (tp) {
        tp_slice(QKV / kTcTileN, &q0, &qn);
        tp_slice(D / kTcTileN, &o0, &on);
        tp_slice(2 * HID / kTcTileN, &h0, &hn);
        s_qkv = tc_pick_splits(qn * kTcTileN, D, m.sm_count);
        s_wo = tc_pick_splits(on * kTcTileN, QD, m.sm_count);
        s_w2 = tc_pick_splits(on * kTcTileN, HID, m.sm_count);
        tp_epoch_kernel<<<1, 1, 0, st>>>(g_tp.epoch);
    }
    /* Key splits of the decode attention: as many as fit the GPU in one wave. A CTA of this kernel
     * takes 28 K registers, two fit an SM; beyond that the extra CTAs queue up behind the first
     * wave (8 utterances x 8 KV heads x 9 splits ran as two waves: 22 us instead of 12 per layer). */
    int attn_splits = (2 * m.sm_count) / (VB200_KV_HEADS * B);
    if (attn_splits > kBtKeySplits) attn_splits = kBtKeySplits;
    if (attn_splits < 1) attn_splits = 1;
    for (int l = 0; l < VB200_DEC_LAYERS; l++) {
        const LayerDev &L = m.dec[l];
        const int NL = VB200_DEC_LAYERS;      /* every exchanged buffer is filled once per layer */
        /* residual-stream taps (single utterance only): after the attention half and after the
         * FFN half of every layer, as the parity tests read them (voxtral_tts_llm.c:245,263) */
        float *const tap_base = (t.single && m.tap_on) ? m.tap : nullptr;
        if (l == 0) tc_prepare(t.aD, t.X, D, B, nullptr, 0, 0, nullptr, nullptr, L.attn_norm, t.ssq, st);
        else tc_prepare(t.aD, nullptr, D, B, t.part_w2, s_w2, psD, t.X, t.X, L.attn_norm, t.ssq, st,
                        tp_wait_for(0, TP_W2, NL, l, t.status), tap_base ? tap_base + (size_t)(2 * l - 1) * D : nullptr);
        TcGemm g;
        g.M = B; g.status = t.status; g.eps = VB200_NORM_EPS;
        g.epi = TC_EPI_PARTIAL; g.out = t.part_qkv; g.splits = s_qkv; g.ld_out = QKV;
        g.ssq = t.ssq; g.ssq_chunks = chunksD;
        if (tp) { g.tile0 = q0; g.n_tiles = qn; g.push = tp_push(0, TP_QKV, NL, l + 1); }
        if (tc_gemm(w.wqkv[l], t.aD, g, st)) return -1;
        if (tp)
            launch_pdl(bt_attn_kernel<true, 4>, dim3(kBtKeySplits, VB200_KV_HEADS, B), dim3(kBtAttnThreads), 0, st, t.bQ,
                       16, (const float *)t.part_qkv, s_qkv, psQ, t.kv_k, t.kv_v, t.slab, l, (const VbDyn *)t.dyn,
                       scale, VB200_ROPE_THETA, t.attn_scratch, t.tickets, t.status,
                       tp_wait_for(0, TP_QKV, NL, l + 1, t.status));
        else if (B == 1)   /* one utterance: one CTA per SM at most, so eight keys per pass cost no occupancy */
            launch_pdl(bt_attn_kernel<false, 8>, dim3(attn_splits, VB200_KV_HEADS, B), dim3(kBtAttnThreads), 0, st, t.bQ,
                       16, (const float *)t.part_qkv, s_qkv, psQ, t.kv_k, t.kv_v, t.slab, l, (const VbDyn *)t.dyn,
                       scale, VB200_ROPE_THETA, t.attn_scratch, t.tickets, t.status, TcNoWait());
        else
            launch_pdl(bt_attn_kernel<false, 4>, dim3(attn_splits, VB200_KV_HEADS, B), dim3(kBtAttnThreads), 0, st, t.bQ,
                       16, (const float *)t.part_qkv, s_qkv, psQ, t.kv_k, t.kv_v, t.slab, l, (const VbDyn *)t.dyn,
                       scale, VB200_ROPE_THETA, t.attn_scratch, t.tickets, t.status, TcNoWait());
        g = TcGemm();
        g.M = B; g.status = t.status; g.eps = VB200_NORM_EPS;
        g.epi = TC_EPI_PARTIAL; g.out = t.part_wo; g.splits = s_wo; g.ld_out = D;
        if (tp) { g.tile0 = o0; g.n_tiles = on; g.push = tp_push(0, TP_WO, NL, l + 1); }
        if (tc_gemm(w.wo[l], t.aQ, g, st)) return -1;
        tc_prepare(t.aD, nullptr, D, B, t.part_wo, s_wo, psD, t.X, t.X, L.ffn_norm, t.ssq, st,
                   tp_wait_for(0, TP_WO, NL, l + 1, t.status), tap_base ? tap_base + (size_t)(2 * l) * D : nullptr);
        g = TcGemm();
        g.M = B; g.status = t.status; g.eps = VB200_NORM_EPS;
        g.epi = TC_EPI_SWIGLU_TERMS; g.out_terms = t.bH; g.out_rows_pad = 16;
        g.splits = 1; g.ld_out = HID; g.ssq = t.ssq; g.ssq_chunks = chunksD;
        if (tp) { g.tile0 = h0; g.n_tiles = hn; g.push = tp_push(0, TP_W13, NL, l + 1); }
        if (tc_gemm(w.w13[l], t.aD, g, st)) return -1;
        g = TcGemm();
        g.M = B; g.status = t.status; g.eps = VB200_NORM_EPS;
        g.epi = TC_EPI_PARTIAL; g.out = t.part_w2; g.splits = s_w2; g.ld_out = D;
        if (tp) {
            g.tile0 = o0; g.n_tiles = on; g.push = tp_push(0, TP_W2, NL, l + 1);
            g.wait = tp_wait_for(0, TP_W13, NL, l + 1, t.status);     /* the SwiGLU terms come from every rank */
        }
        if (tc_gemm(w.w2[l], t.aH, g, st)) return -1;
    }
    float *const last_tap = (t.single && m.tap_on) ? m.tap + (size_t)(2 * VB200_DEC_LAYERS - 1) * D : nullptr;
    if (tp)
        launch_pdl(bt_final_kernel<true>, dim3(B), dim3(1024), 0, st, t.hidden, t.bD, 16, (const float *)t.X,
                   (const float *)t.part_w2, s_w2, psD, (const float *)m.dec_norm, VB200_NORM_EPS, last_tap,
                   tp_wait_for(0, TP_W2, VB200_DEC_LAYERS, VB200_DEC_LAYERS, t.status));
    else
        launch_pdl(bt_final_kernel<false>, dim3(B), dim3(1024), 0, st, t.hidden, t.bD, 16, (const float *)t.X,
                   (const float *)t.part_w2, s_w2, psD, (const float *)m.dec_norm, VB200_NORM_EPS, last_tap, TcNoWait());
    TcGemm g;
    g.M = B; g.status = t.status;
    /* semantic head + argmax (voxtral_tts_acoustic.c:283-309), llm token (:204) */
    g.epi = TC_EPI_PARTIAL; g.out = t.logit_part; g.splits = w.s_sem; g.ld_out = NSEM; g.ssq = nullptr; g.ssq_chunks = 0;
    if (tc_gemm(w.wsem, t.aD, g, st)) return -1;
    launch_pdl(bt_argmax_kernel, dim3(B), dim3(1024), 0, st, t.codes, (const float *)t.logit_part, w.s_sem,
               (size_t)B * NSEM, (const float *)m.ac_sem_bias, NSEM, VB200_SEM_VALID_END);
    g.out = t.part; g.splits = w.s_llm; g.ld_out = D;
    if (tc_gemm(w.wllm, t.aD, g, st)) return -1;
    tc_reduce(t.ltok, t.part, w.s_llm, psD, psD, nullptr, D, st);
    if (acoustic_tc_enqueue_on(t.ac, noise, codes_log, cap, advance, m.ignore_end)) return -1;
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

/* Variant v of the frame: 0 = a frame of a device-resident run, 1 = single frame with the
 * host's input row, 2 = single frame re-embedding the previous codes. */
static int enqueue_variant(Batch &t, int v) {
    switch (v) {
    case 0: return enqueue_frame(t, EMBED_CODES_AFTER0, true, t.noise_all, t.codes_all, t.cap);
    case 1: return enqueue_frame(t, EMBED_HOST, false, t.noise1, nullptr, 0);
    default: return enqueue_frame(t, EMBED_CODES, false, t.noise1, nullptr, 0);
    }
}

/* The first call of a variant runs launch by launch (kernel attributes are set on first use,
 * which must not happen inside a capture), the second is captured as a CUDA graph and every
 * later call replays it. */
static int launch_variant(Batch &t, int v) {
    Model &m = model();
    static const bool no_graph = getenv("VB200_NO_GRAPH") != nullptr;
    if (t.exec[v]) return cudaGraphLaunch(t.exec[v], m.st) == cudaSuccess ? 0 : -1;
    if (no_graph || t.direct_calls[v]++ == 0) return enqueue_variant(t, v);
    cudaGraph_t graph = nullptr;
    if (cudaStreamBeginCapture(m.st, cudaStreamCaptureModeRelaxed) != cudaSuccess) {
        cudaGetLastError();
        return enqueue_variant(t, v);
    }
    const int rc = enqueue_variant(t, v);
    const cudaError_t ee = cudaStreamEndCapture(m.st, &graph);
    if (rc || ee != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        return -1;
    }
    const cudaError_t ie = cudaGraphInstantiate(&t.exec[v], graph, 0);
    cudaGraphDestroy(graph);
    if (ie != cudaSuccess) {
        t.exec[v] = nullptr;
        cudaGetLastError();
        return -1;
    }
    return cudaGraphLaunch(t.exec[v], m.st) == cudaSuccess ? 0 : -1;
}

static int ctx_run(Batch &t, int n) {
    Model &m = model();
    if (!t.begun || n < 0) return -1;
    cudaEventRecord(t.e0, m.st);
    for (int i = 0; i < n && t.launched < t.cap; i++, t.launched++)
        if (launch_variant(t, 0)) return -1;
    cudaEventRecord(t.e1, m.st);
    return 0;
}

/* ---- several utterances ---- */
int batch_open(int n_utt, int kv_max, int max_frames) {
    Model &m = model();
    if (!m.inited || !m.llm_ready || !m.ac_ready || !m.embed_ready || !acoustic_tc_ready()) return -1;
    if (n_utt < 1 || n_utt > kBtMaxUtt || kv_max < 1 || max_frames < 1) return -1;
    return ctx_open(g_bt, false, n_utt, kv_max, max_frames);
}

/* Prompt rows of one utterance into its own cache slab (the single-utterance prefill,
 * pointed at the slab for the duration of the call). */
int batch_prefill(int utt, const float *embeds, int n_rows) {
    Model &m = model();
    Batch &t = g_bt;
    if (!t.open || !embeds || utt < 0 || utt >= t.B || n_rows < 1 || n_rows > t.kv_max) return -1;
    float *k0 = m.kv_k, *v0 = m.kv_v;
    const int max0 = m.kv_max;
    m.kv_k = t.kv_k + (size_t)utt * t.slab;
    m.kv_v = t.kv_v + (size_t)utt * t.slab;
    m.kv_max = t.kv_max;
    const int rc = prefill(embeds, n_rows, 0);
    m.kv_k = k0; m.kv_v = v0; m.kv_max = max0;
    return rc;
}

int batch_begin(const float *first_embeds, const int *start_pos, const float *noise) {
    Model &m = model();
    Batch &t = g_bt;
    if (!t.open || !first_embeds || !start_pos || !noise) return -1;
    std::vector<VbDyn> d(t.B);
    for (int b = 0; b < t.B; b++) {
        if (start_pos[b] < 0 || start_pos[b] >= t.kv_max) return -1;
        d[b].pos = start_pos[b]; d[b].kv_max = t.kv_max; d[b].frame = 0; d[b].done = 0;
    }
    if (cudaStreamSynchronize(m.st) != cudaSuccess) return -1;
    if (cudaMemcpy(t.dyn, d.data(), sizeof(VbDyn) * t.B, cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemcpy(t.X, first_embeds, sizeof(float) * t.B * D, cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemcpy(t.noise_all, noise, sizeof(float) * (size_t)t.B * t.cap * A, cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemset(t.codes_all, 0, sizeof(int) * (size_t)t.B * t.cap * VB200_CODES) != cudaSuccess ||
        cudaMemset(t.status, 0, sizeof(int) * 4) != cudaSuccess ||
        cudaMemset(t.tickets, 0, sizeof(unsigned) * t.B * VB200_KV_HEADS) != cudaSuccess)
        return -1;
    t.launched = 0;
    t.begun = true;
    return 0;
}

/* Queues n more frames; returns without waiting. */
int batch_run(int n) { return ctx_run(g_bt, n); }

/* Waits for the queued frames. codes_out [B][max_frames][37] (rows past frames_done[b] are
 * zero), frames_done[b], hit_end[b] (1 when the utterance produced END; that frame is counted),
 * device_ms = device time of the last batch_run. */
int batch_end(int *codes_out, int *frames_done, int *hit_end, float *device_ms) {
    Model &m = model();
    Batch &t = g_bt;
    if (!t.begun) return -1;
    if (cudaStreamSynchronize(m.st) != cudaSuccess) return -1;
    std::vector<VbDyn> d(t.B);
    int status = 0;
    if (cudaMemcpy(d.data(), t.dyn, sizeof(VbDyn) * t.B, cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(&status, t.status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
        return -1;
    m.last_status = status;
    if (codes_out &&
        cudaMemcpy(codes_out, t.codes_all, sizeof(int) * (size_t)t.B * t.cap * VB200_CODES, cudaMemcpyDeviceToHost) !=
            cudaSuccess)
        return -1;
    for (int b = 0; b < t.B; b++) {
        if (frames_done) frames_done[b] = d[b].frame;
        if (hit_end) hit_end[b] = d[b].done == 2 ? 1 : 0;
    }
    if (device_ms) {
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, t.e0, t.e1);
        *device_ms = ms;
    }
    return status ? -2 : 0;
}

/* The decoder's hidden rows of the last frame decoded [B][3072]. */
int batch_hidden(float *out) {
    Model &m = model();
    Batch &t = g_bt;
    if (!t.open || !out) return -1;
    if (cudaStreamSynchronize(m.st) != cudaSuccess) return -1;
    return cudaMemcpy(out, t.hidden, sizeof(float) * t.B * D, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : -1;
}

int batch_launches_per_frame() { return 1 + VB200_DEC_LAYERS * 7 + 5 + (VB200_FLOW_STEPS - 1) * (2 + VB200_AC_LAYERS * 7) + 1; }

/* The decoder's 104 layer GEMMs (QKV, O, gate/up, down x 26 layers: every decoder weight byte
 * once) launched back to back on the stream, `iters` times, between two events: the GEMM
 * kernel's own average launch time at the shapes and row count the frame uses, without the
 * glue kernels. which = 0: the single-utterance context, 1: the open batch. */
static int one_ready(int frames);
int gemm_sweep(int which, int iters, float *ms_out, double *bytes_per_sweep, int *launches_per_sweep) {
    Model &m = model();
    if (which == 0 && one_ready(0)) return -1;
    Batch &t = which == 0 ? g_one : g_bt;
    if (!t.open || iters < 1 || bt_weights()) return -1;
    const BtWeights &w = g_w;
    const int chunksD = tc_prepare_chunks(D);
    TcGemm g;
    g.M = t.B; g.status = t.status; g.eps = VB200_NORM_EPS;
    cudaEventRecord(t.e0, m.st);
    for (int it = 0; it < iters; it++) {
        for (int l = 0; l < VB200_DEC_LAYERS; l++) {
            g.epi = TC_EPI_PARTIAL; g.out = t.part; g.out_terms = nullptr;
            g.splits = w.s_qkv; g.ld_out = QKV; g.ssq = t.ssq; g.ssq_chunks = chunksD;
            if (tc_gemm(w.wqkv[l], t.aD, g, m.st)) return -1;
            g.splits = w.s_wo; g.ld_out = D; g.ssq = nullptr; g.ssq_chunks = 0;
            if (tc_gemm(w.wo[l], t.aQ, g, m.st)) return -1;
            g.epi = TC_EPI_SWIGLU_TERMS; g.out = nullptr; g.out_terms = t.bH; g.out_rows_pad = 16;
            g.splits = 1; g.ld_out = HID; g.ssq = t.ssq; g.ssq_chunks = chunksD;
            if (tc_gemm(w.w13[l], t.aD, g, m.st)) return -1;
            g.epi = TC_EPI_PARTIAL; g.out = t.part; g.out_terms = nullptr;
            g.splits = w.s_w2; g.ld_out = D; g.ssq = nullptr; g.ssq_chunks = 0;
            if (tc_gemm(w.w2[l], t.aH, g, m.st)) return -1;
        }
    }
    cudaEventRecord(t.e1, m.st);
    if (cudaStreamSynchronize(m.st) != cudaSuccess) return -1;
    if (ms_out && cudaEventElapsedTime(ms_out, t.e0, t.e1) != cudaSuccess) return -1;
    if (bytes_per_sweep)
        *bytes_per_sweep = 2.0 * VB200_DEC_LAYERS * ((double)QKV * D + (double)D * QD + 2.0 * HID * D + (double)D * HID);
    if (launches_per_sweep) *launches_per_sweep = 4 * VB200_DEC_LAYERS;
    return 0;
}

/* The streaming decoder step (26 layers, both heads, argmax: one launch) `iters` times back to
 * back at cache row `pos`, between two events: the kernel's own launch time. Every launch reads
 * every decoder weight byte once; the cache row `pos` is rewritten with the same values. */
static int one_status(Batch &t);
int stream_step_time(int pos, int iters, float *ms_out, double *bytes_per_launch) {
    Model &m = model();
    if (!m.inited || !m.llm_ready || !m.ac_ready || iters < 1 || pos < 0 || pos >= m.kv_max || one_ready(0)) return -1;
    Batch &t = g_one;
    if (!t.stream) return -1;
    t.h_in->dyn.pos = pos; t.h_in->dyn.kv_max = m.kv_max; t.h_in->dyn.frame = 0; t.h_in->dyn.done = 0;
    if (cudaMemcpyAsync(&t.d_in->dyn, &t.h_in->dyn, sizeof(VbDyn), cudaMemcpyHostToDevice, m.st) != cudaSuccess) return -1;
    for (int i = 0; i < 2; i++)
        if (stream_step(t, 1)) return -1;
    cudaEventRecord(t.e0, m.st);
    for (int i = 0; i < iters; i++)
        if (stream_step(t, 1)) return -1;
    cudaEventRecord(t.e1, m.st);
    if (cudaMemcpyAsync(t.h_out, t.d_out, sizeof(OneOut), cudaMemcpyDeviceToHost, m.st) != cudaSuccess ||
        cudaStreamSynchronize(m.st) != cudaSuccess)
        return -1;
    if (ms_out && cudaEventElapsedTime(ms_out, t.e0, t.e1) != cudaSuccess) return -1;
    if (bytes_per_launch)
        *bytes_per_launch = 2.0 * VB200_DEC_LAYERS * ((double)QKV * D + (double)D * QD + 2.0 * HID * D + (double)D * HID) +
                            2.0 * ((double)NSEM * D + (double)D * D) +
                            2.0 * VB200_DEC_LAYERS * (double)(pos + 1) * KVD * sizeof(float);
    return one_status(t);
}

/* A wait inside the streaming kernel that nothing ever satisfies, with a short limit: the kernel
 * must record its status, leave through the abort path by itself and leave the library usable.
 * Host-safe by construction (the kernel returns; nothing faults, nothing is killed). Returns the
 * status word the kernel left (S_ERR_FLAG_WAIT when all is well), or -1. */
int stream_wait_expiry(int limit_us) {
    Model &m = model();
    if (!m.inited || limit_us < 1 || limit_us > 1000000) return -1;
    const int n_cta = stream_max_ctas(m.device);
    if (n_cta <= 0) return -1;
    std::vector<void *> own;
    unsigned *words = nullptr;      /* [0] the flag nobody sets, [16] barrier, [32] exit, [48] status, [52..56) dyn */
    SOp *d_ops = nullptr;
    if (bt_alloc((void **)&words, sizeof(unsigned) * 64, &own) || bt_alloc((void **)&d_ops, sizeof(SOp) * 2, &own)) {
        bt_free(&own);
        return -1;
    }
    SOp ops[2];
    for (SOp &o : ops) {
        o = sop_zero();
        o.type = S_OP_WAIT; o.p0 = words; o.i0 = 1; o.i1 = limit_us;
    }
    int st = -1;
    SArgs a;
    a.ops = d_ops; a.n_ops = 2; a.dyn = (VbDyn *)(words + 52);
    a.wl = nullptr; a.n_wl = 0;
    a.bar_counter = words + 16; a.exit_counter = words + 32; a.status = (int *)(words + 48);
    a.seq = words + 60;
    a.wait_cycles = m.wait_cycles;       /* the other waits keep the ordinary limit: the flag wait runs out first */
    if (cudaMemcpyAsync(d_ops, ops, sizeof(ops), cudaMemcpyHostToDevice, m.st) == cudaSuccess &&
        stream_launch(a, n_cta, m.st) == cudaSuccess && cudaStreamSynchronize(m.st) == cudaSuccess)
        cudaMemcpy(&st, words + 48, sizeof(int), cudaMemcpyDeviceToHost);
    cudaGetLastError();
    bt_free(&own);
    return st;
}

/* ---- one utterance on the library's own cache ---- */
bool single_tc_usable() {
    Model &m = model();
    static const bool off = getenv("VB200_NO_TC") != nullptr;
    if (off || !m.inited || !m.llm_ready || !m.ac_ready || !acoustic_tc_ready()) return false;
    return true;     /* per-layer taps exist on both decoder-step paths */
}

/* 1 when the single-utterance calls run their decoder step on the streaming kernel. */
bool single_on_stream() { return single_tc_usable() && !g_tp.on && stream_wanted() && (!g_one.open || g_one.stream); }

/* (Re)creates the single-utterance context when needed; the code / noise arrays grow on demand. */
static int one_ready(int frames) {
    Model &m = model();
    Batch &t = g_one;
    if (t.open && t.kv_k == m.kv_k && t.kv_max == m.kv_max && frames <= t.alloc_cap) {
        if (!t.stream) {
            if (t.s_tap != m.tap_on) {          /* the tap pointers are arguments of the captured launches */
                if (cudaStreamSynchronize(m.st) != cudaSuccess) return -1;
                drop_graphs(t);
                t.s_tap = m.tap_on;
            }
            return bt_weights();
        }
        if (t.s_tap != m.tap_on || t.s_table != m.audio_table) {   /* both are part of the op lists */
            if (cudaStreamSynchronize(m.st) != cudaSuccess) return -1;
            drop_graphs(t);
            return stream_programs(t);
        }
        return 0;
    }
    const int cap = frames > t.alloc_cap ? frames : t.alloc_cap;
    return ctx_open(t, true, 1, m.kv_max, cap);
}

static int one_status(Batch &t) {
    Model &m = model();
    m.last_status = t.h_out->status[0];
    if (m.last_status == 0) return 0;
    fprintf(stderr, "voxtral_b200: a frame kernel gave up with status %d\n", m.last_status);
    cudaMemsetAsync(t.tickets, 0, sizeof(unsigned) * VB200_KV_HEADS, m.st);
    if (t.s_counters) cudaMemsetAsync(t.s_counters, 0, sizeof(unsigned) * 64, m.st);
    cudaMemsetAsync(t.status, 0, sizeof(int) * 4, m.st);
    cudaStreamSynchronize(m.st);
    return -1;
}

/* tts_llm_forward + tts_acoustic_forward of one frame (voxtral_tts.c:303-318) as one graph
 * launch between one copy in and one copy out. */
int single_frame(const float *embed, const float *noise, int pos, float *hidden_out, int *codes, bool chained) {
    Model &m = model();
    if (one_ready(0)) return -1;
    Batch &t = g_one;
    if (chained && !m.embed_ready) return -1;
    t.h_in->dyn.pos = pos; t.h_in->dyn.kv_max = m.kv_max; t.h_in->dyn.frame = 0; t.h_in->dyn.done = 0;
    memcpy(t.h_in->noise, noise, sizeof(float) * A);
    if (chained) {
        if (cudaMemcpyAsync(&t.d_in->dyn, &t.h_in->dyn, sizeof(VbDyn), cudaMemcpyHostToDevice, m.st) != cudaSuccess ||
            cudaMemcpyAsync(t.d_in->noise, t.h_in->noise, sizeof(float) * A, cudaMemcpyHostToDevice, m.st) != cudaSuccess)
            return -1;
    } else {
        memcpy(t.h_in->X, embed, sizeof(float) * D);
        if (cudaMemcpyAsync(t.d_in, t.h_in, sizeof(OneIn), cudaMemcpyHostToDevice, m.st) != cudaSuccess) return -1;
    }
    if (m.timing) {
        flush_launch_time();
        cudaEventRecord(m.ev0, m.st);
    }
    if (launch_variant(t, chained ? 2 : 1)) return -1;
    if (m.timing) {
        cudaEventRecord(m.ev1, m.st);
        m.time_pending = true;
    }
    if (cudaMemcpyAsync(t.h_out, t.d_out, sizeof(OneOut), cudaMemcpyDeviceToHost, m.st) != cudaSuccess ||
        cudaStreamSynchronize(m.st) != cudaSuccess)
        return -1;
    flush_launch_time();
    if (one_status(t)) return -1;
    memcpy(codes, t.h_out->codes, sizeof(int) * VB200_CODES);
    if (hidden_out) memcpy(hidden_out, t.h_out->hidden, sizeof(float) * D);
    return 0;
}

int single_begin(const float *first_embed, int start_pos, const float *noise_all, int n_frames) {
    Model &m = model();
    if (!m.embed_ready || one_ready(n_frames)) return -1;
    Batch &t = g_one;
    if (t.graph_cap != n_frames) {
        /* the frame cap is an argument of the captured launches */
        if (t.exec[0]) { cudaGraphExecDestroy(t.exec[0]); t.exec[0] = nullptr; }
        if (t.direct_calls[0] > 1) t.direct_calls[0] = 1;
        t.graph_cap = n_frames;
    }
    t.cap = n_frames;
    t.ac.sd.noise = (size_t)n_frames * A; t.ac.sd.codes_all = (size_t)n_frames * VB200_CODES;
    t.h_in->dyn.pos = start_pos; t.h_in->dyn.kv_max = m.kv_max; t.h_in->dyn.frame = 0; t.h_in->dyn.done = 0;
    memcpy(t.h_in->X, first_embed, sizeof(float) * D);
    if (cudaStreamSynchronize(m.st) != cudaSuccess) return -1;
    if (cudaMemcpy(t.d_in, t.h_in, sizeof(OneIn), cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemcpy(t.noise_all, noise_all, sizeof(float) * (size_t)n_frames * A, cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemset(t.codes_all, 0, sizeof(int) * (size_t)n_frames * VB200_CODES) != cudaSuccess)
        return -1;
    t.launched = 0;
    t.begun = true;
    return 0;
}

int single_run(int n) { return ctx_run(g_one, n); }

int single_end(int *codes_out, int *frames_done, int *hit_end, float *device_ms) {
    Model &m = model();
    Batch &t = g_one;
    if (!t.begun) return -1;
    if (cudaMemcpyAsync(t.h_out, t.d_out, sizeof(OneOut), cudaMemcpyDeviceToHost, m.st) != cudaSuccess ||
        cudaMemcpyAsync(&t.h_in->dyn, &t.d_in->dyn, sizeof(VbDyn), cudaMemcpyDeviceToHost, m.st) != cudaSuccess ||
        cudaStreamSynchronize(m.st) != cudaSuccess)
        return -1;
    if (device_ms && cudaEventElapsedTime(device_ms, t.e0, t.e1) != cudaSuccess) *device_ms = -1.0f;
    const int done = t.h_in->dyn.frame;
    if (frames_done) *frames_done = done;
    if (hit_end) *hit_end = t.h_in->dyn.done == 2 ? 1 : 0;
    if (codes_out && done > 0 &&
        cudaMemcpy(codes_out, t.codes_all, sizeof(int) * (size_t)done * VB200_CODES, cudaMemcpyDeviceToHost) != cudaSuccess)
        return -1;
    return one_status(t);
}

} // namespace vb
