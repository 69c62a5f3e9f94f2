/*
 * vb_acoustic_tc.cu - the acoustic frame on the tensor-core path.
 *
 * tts_acoustic_forward (voxtral_tts_acoustic.c:268-373): semantic head + argmax, then 7
 * Euler steps; both guidance branches of a step run together as six token rows
 * (voxtral_tts_acoustic.c:198-212, :345-348), so every layer matrix is streamed once per
 * step by the tcgen05 GEMM (vb_tc.cu). Around the GEMMs sit small kernels: token
 * build + Euler update, 3-token attention, split-K reduction + residual + RMSNorm +
 * BF16 term split ("prepare"), velocity head, FSQ. The sequence (about 200 launches) is
 * captured once as a CUDA graph and replayed per frame.
 */
#include "vb_acoustic_tc.cuh"
#include "vb_common.cuh"

#include <math.h>
#include <stdio.h>
#include <string.h>

namespace vb {

static const int D = VB200_DIM, QD = VB200_Q_DIM, KVD = VB200_KV_DIM, HID = VB200_HIDDEN;
static const int QKV = QD + 2 * KVD;
static const int A = VB200_ACOUSTIC_DIM;
static const int ROWS1 = 6;    /* rows per utterance: 2 guidance branches x 3 tokens */

struct AcTc {
    bool ready = false;
    TcWeight wqkv[VB200_AC_LAYERS], wo[VB200_AC_LAYERS], w13[VB200_AC_LAYERS], w2[VB200_AC_LAYERS];
    uint16_t *tiled[VB200_AC_LAYERS][4] = {};   /* tile-contiguous weight copies */
    int s_qkv = 1, s_wo = 1, s_w2 = 1;
    AcBuffers one;              /* the single-utterance buffers */
};
static AcTc g_ac;
void acoustic_tc_drop_graphs();

/* ---- small kernels ---- */

__device__ __forceinline__ float euler_step(float x, float vc, float vu, float alpha, float dt) {
    /* v = alpha*vc + (1-alpha)*vu; x += v*dt  without fused multiply-adds
     * (voxtral_tts_acoustic.c:350-354) */
    const float v = __fadd_rn(__fmul_rn(alpha, vc), __fmul_rn(__fsub_rn(1.0f, alpha), vu));
    return __fadd_rn(x, __fmul_rn(v, dt));
}

/* Euler update of the latent (step > 0) and the six input rows of a pass
 * (voxtral_tts_acoustic.c:198-212): rows 0,3 input_proj(x_t); 1,4 the precomputed time token;
 * 2 llm_proj(h); 5 zero. */
__global__ void ac_tokens_kernel(float *X6, float *lat, const float *vel, const uint16_t *Wip, const float *ttok,
                                 const float *ltok, int step, float alpha, float dt_prev, const float *noise_all,
                                 const VbDyn *dyn, AcStrides sd) {
    __shared__ float xs[64];
    pdl_launch_dependents();
    pdl_wait();
    /* utterance blockIdx.y of the batch */
    const int b = blockIdx.y;
    X6 += (size_t)b * ROWS1 * D;
    lat += (size_t)b * sd.lat;
    vel += (size_t)b * sd.vel;
    ltok += (size_t)b * D;
    dyn += b;
    if (noise_all) noise_all += (size_t)b * sd.noise;
    if (noise_all && dyn->done) return;   /* device-resident run already ended */
    if (threadIdx.x < A) {
        float xv;
        if (step == 0) {
            if (noise_all) {
                xv = noise_all[(size_t)dyn->frame * A + threadIdx.x];
                if (blockIdx.x == 0) lat[threadIdx.x] = xv;
            } else {
                xv = lat[threadIdx.x];
            }
        } else {
            xv = euler_step(lat[(step - 1) * A + threadIdx.x], vel[threadIdx.x], vel[A + threadIdx.x], alpha, dt_prev);
            if (blockIdx.x == 0) lat[step * A + threadIdx.x] = xv;
        }
        xs[threadIdx.x] = xv;
    }
    __syncthreads();
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= D) return;
    const uint16_t *wr = Wip + (size_t)n * A;
    float acc = 0.0f;
    for (int k = 0; k < A; k++) acc = __fadd_rn(acc, __fmul_rn(__uint_as_float((uint32_t)wr[k] << 16), xs[k]));
    const float tt = ttok[(size_t)step * D + n];
    X6[n] = acc;
    X6[3 * D + n] = acc;
    X6[1 * D + n] = tt;
    X6[4 * D + n] = tt;
    X6[2 * D + n] = ltok[n];
    X6[5 * D + n] = 0.0f;
}

/* Unmasked attention inside each 3-token sequence (tts_bidirectional_attention,
 * voxtral_tts_kernels.c:467-525) on q/k/v given as split-K partials [n_part][6][6144].
 * One warp per (row, head). The result goes out as the three BF16 terms the O projection's
 * GEMM consumes ([3][rows_pad][4096]). */
__global__ void ac_attention_kernel(uint16_t *terms, const float *part, int n_part, float scale, int ROWS,
                                    int rows_pad) {
    pdl_launch_dependents();
    pdl_wait();
    const int task = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (task >= ROWS * VB200_HEADS) return;
    const int row = task / VB200_HEADS, h = task % VB200_HEADS, kvh = h / (VB200_HEADS / VB200_KV_HEADS);
    const int seq0 = (row / 3) * 3;
    const size_t ps = (size_t)ROWS * QKV;
    /* every load of the task is issued before anything is summed: 7 x n_part float4 per lane */
    constexpr int kMaxPart = kTcMaxSplits;
    const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 tq[kMaxPart], tk[3][kMaxPart], tv[3][kMaxPart];
#pragma unroll
    for (int p = 0; p < kMaxPart; p++) {
        const bool on = p < n_part;
        tq[p] = on ? __ldcg(reinterpret_cast<const float4 *>(part + p * ps + (size_t)row * QKV + h * 128 + 4 * lane)) : z4;
#pragma unroll
        for (int j = 0; j < 3; j++) {
            const float *b = part + p * ps + (size_t)(seq0 + j) * QKV + QD + kvh * 128 + 4 * lane;
            tk[j][p] = on ? __ldcg(reinterpret_cast<const float4 *>(b)) : z4;
            tv[j][p] = on ? __ldcg(reinterpret_cast<const float4 *>(b + KVD)) : z4;
        }
    }
    float4 q = z4;
#pragma unroll
    for (int p = 0; p < kMaxPart; p++) {
        if (p < n_part) { q.x += tq[p].x; q.y += tq[p].y; q.z += tq[p].z; q.w += tq[p].w; }
    }
    float mx = -1e30f, den = 0.0f;
    float4 o = z4;
#pragma unroll
    for (int j = 0; j < 3; j++) {
        float4 k = z4, v = z4;
#pragma unroll
        for (int p = 0; p < kMaxPart; p++) {
            if (p < n_part) {
                k.x += tk[j][p].x; k.y += tk[j][p].y; k.z += tk[j][p].z; k.w += tk[j][p].w;
                v.x += tv[j][p].x; v.y += tv[j][p].y; v.z += tv[j][p].z; v.w += tv[j][p].w;
            }
        }
        float d = q.x * k.x + q.y * k.y + q.z * k.z + q.w * k.w;
        d = vb_warp_sum(d) * scale;
        if (d > mx) {
            const float corr = expf(mx - d);
            den = den * corr + 1.0f;
            o.x = o.x * corr + v.x; o.y = o.y * corr + v.y; o.z = o.z * corr + v.z; o.w = o.w * corr + v.w;
            mx = d;
        } else {
            const float w = expf(d - mx);
            den += w;
            o.x += w * v.x; o.y += w * v.y; o.z += w * v.z; o.w += w * v.w;
        }
    }
    const float inv = den > 0.0f ? 1.0f / den : 0.0f;
    const float e[4] = {o.x * inv, o.y * inv, o.z * inv, o.w * inv};
    uint16_t t0[4], t1[4], t2[4];
#pragma unroll
    for (int i = 0; i < 4; i++) vb_split3(e[i], t0[i], t1[i], t2[i]);
    const size_t off = (size_t)row * QD + h * 128 + 4 * lane, term = (size_t)rows_pad * QD;
    *reinterpret_cast<uint2 *>(terms + off) = make_uint2(t0[0] | ((uint32_t)t0[1] << 16), t0[2] | ((uint32_t)t0[3] << 16));
    *reinterpret_cast<uint2 *>(terms + term + off) = make_uint2(t1[0] | ((uint32_t)t1[1] << 16), t1[2] | ((uint32_t)t1[3] << 16));
    *reinterpret_cast<uint2 *>(terms + 2 * term + off) = make_uint2(t2[0] | ((uint32_t)t2[1] << 16), t2[2] | ((uint32_t)t2[3] << 16));
}

/* Last residual add, final RMSNorm of token 0 of each branch (rows 0 and 3) and the 36-wide
 * velocity head (voxtral_tts_acoustic.c:255-261). grid = (9, 2 * utterances): blockIdx.y =
 * 2 * utterance + branch, four of the 36 outputs per CTA (every CTA re-derives the normalised
 * row; it is 12 KB). */
__global__ void ac_velocity_kernel(float *vel, const float *X6, const float *part, int n_part, const float *gain,
                                   float eps, const uint16_t *Wout, int ROWS, int vel_stride) {
    __shared__ float xn[VB200_DIM];
    __shared__ float red[32];
    pdl_launch_dependents();
    /* this warp's slice of its output row of acoustic_out: static data, fetched before the wait
     * for the previous kernel (24 BF16 values per lane) */
    constexpr int kWPerLane = VB200_DIM / 4 / 32;
    uint16_t wv[kWPerLane];
    {
        const int pw = threadIdx.x >> 5, pl = threadIdx.x & 31;
        const uint16_t *pr = Wout + (size_t)(blockIdx.x * 4 + (pw >> 2)) * VB200_DIM + (pw & 3) * (VB200_DIM / 4) + pl;
#pragma unroll
        for (int i = 0; i < kWPerLane; i++) wv[i] = __ldg(pr + 32 * i);
    }
    pdl_wait();
    const int row = blockIdx.y * 3;
    const size_t ps = (size_t)ROWS * D;
    float ss = 0.0f;
    /* 512 threads x 6 columns; the 6 x (n_part + 1) loads of a thread are issued together */
    {
        constexpr int kCols = VB200_DIM / 512;
        float pv[kCols][kTcMaxSplits], xv[kCols];
#pragma unroll
        for (int i = 0; i < kCols; i++) {
            const int c = threadIdx.x + i * 512;
            xv[i] = __ldcg(X6 + (size_t)row * D + c);
#pragma unroll
            for (int p = 0; p < kTcMaxSplits; p++) pv[i][p] = p < n_part ? __ldcg(part + p * ps + (size_t)row * D + c) : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < kCols; i++) {
            float s = 0.0f;
#pragma unroll
            for (int p = 0; p < kTcMaxSplits; p++) s += pv[i][p];     /* split order; unused splits add 0 */
            const float v = xv[i] + s;
            xn[threadIdx.x + i * 512] = v;
            ss += v * v;
        }
    }
    ss = vb_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float t = 0.0f;
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) t += red[w];
    const float inv = 1.0f / sqrtf(t / (float)D + eps);
    for (int c = threadIdx.x; c < D; c += blockDim.x) xn[c] = xn[c] * inv * gain[c];
    __syncthreads();
    /* 4 outputs per CTA, 4 warps per output, then a fixed-order sum of the 4 warp partials */
    __shared__ float wsum[16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q = warp & 3;   /* quarter of the row this warp sums; output blockIdx.x * 4 + (warp >> 2) */
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < kWPerLane; i++)
        acc = fmaf(__uint_as_float((uint32_t)wv[i] << 16), xn[q * (D / 4) + lane + 32 * i], acc);
    acc = vb_warp_sum(acc);
    if (lane == 0) wsum[warp] = acc;
    __syncthreads();
    if (threadIdx.x < 4) {
        const int o = threadIdx.x;
        vel[(size_t)(blockIdx.y >> 1) * vel_stride + (blockIdx.y & 1) * A + blockIdx.x * 4 + o] =
            ((wsum[4 * o] + wsum[4 * o + 1]) + wsum[4 * o + 2]) + wsum[4 * o + 3];
    }
}

/* Last Euler update and FSQ (voxtral_tts_acoustic.c:358-372); END forces code 2 (:312-320).
 * In a device-resident run it also logs the frame's codes and advances position and frame
 * counter (the loop of voxtral_tts.c:301-321). */
__global__ void ac_fsq_kernel(int *codes, float *lat, const float *vel, int steps, int levels, float alpha, float dt,
                              int *codes_all, VbDyn *dyn, int frame_cap, int advance, int ignore_end, AcStrides sd) {
    const int i = threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x;   /* utterance */
    codes += (size_t)b * sd.codes;
    lat += (size_t)b * sd.lat;
    vel += (size_t)b * sd.vel;
    dyn += b;
    if (codes_all) codes_all += (size_t)b * sd.codes_all;
    if (advance && dyn->done) return;
    const int sem = codes[0];
    const int frame = advance ? dyn->frame : 0;
    __syncthreads();
    if (advance && i == 0) {
        if (codes_all) codes_all[(size_t)frame * (A + 1)] = sem;
        const int nf = frame + 1, np = dyn->pos + 1;
        dyn->frame = nf;
        dyn->pos = np;
        if (sem == 1 && !ignore_end) dyn->done = 2;
        else if (nf >= frame_cap || np >= dyn->kv_max) dyn->done = 1;
    }
    if (i >= A) return;
    float xv = euler_step(lat[(steps - 1) * A + i], vel[i], vel[A + i], alpha, dt);
    lat[steps * A + i] = xv;
    if (xv > 1.0f) xv = 1.0f;
    if (xv < -1.0f) xv = -1.0f;
    const float scaled = __fmul_rn(__fdiv_rn(__fadd_rn(xv, 1.0f), 2.0f), (float)(levels - 1));
    int code = (int)__fadd_rn(scaled, 0.5f);
    if (code < 0) code = 0;
    if (code >= levels) code = levels - 1;
    const int out = (sem == 1) ? 2 : code + 2;
    codes[1 + i] = out;
    if (advance && codes_all) codes_all[(size_t)frame * (A + 1) + 1 + i] = out;
}

/* ---- set-up ---- */
static int alloc_zero(void **p, size_t bytes, std::vector<void *> *owner) {
    if (cudaMalloc(p, bytes) != cudaSuccess) return -1;
    owner->push_back(*p);
    return cudaMemset(*p, 0, bytes) == cudaSuccess ? 0 : -1;
}

int acoustic_buffers_alloc(AcBuffers *b, int B, std::vector<void *> *owner) {
    const int rows = ROWS1 * B, rp = tc_rows_pad_frame(rows);
    if (B < 1 || rp == 0) return -1;
    b->B = B; b->rows = rows; b->rows_pad = rp;
    if (alloc_zero((void **)&b->bD, tc_acts_bytes(rp, D), owner) || alloc_zero((void **)&b->bQ, tc_acts_bytes(rp, QD), owner) ||
        alloc_zero((void **)&b->bH, tc_acts_bytes(rp, HID), owner) ||
        alloc_zero((void **)&b->part, sizeof(float) * kTcMaxSplits * rows * QKV, owner) ||
        alloc_zero((void **)&b->ssq, sizeof(float) * rows * 16, owner))
        return -1;
    if (!b->X6 && alloc_zero((void **)&b->X6, sizeof(float) * rows * D, owner)) return -1;
    if (tc_acts(&b->aD, b->bD, rp, D) || tc_acts(&b->aQ, b->bQ, rp, QD) || tc_acts(&b->aH, b->bH, rp, HID)) return -1;
    return 0;
}

int acoustic_tc_setup() {
    Model &m = model();
    AcTc &t = g_ac;
    t.ready = false;
    acoustic_tc_drop_graphs();   /* captured launches hold the old weight pointers */
    if (getenv("VB200_NO_TC")) return 0;
    if (tc_init()) {
        fprintf(stderr, "voxtral_b200: cuTensorMapEncodeTiled unavailable; acoustic frame stays on the streaming kernel\n");
        return 0;
    }
    for (int l = 0; l < VB200_AC_LAYERS; l++) {
        const LayerDev &L = m.ac[l];
        if (getenv("VB200_TC_UNTILED")) {
            if (tc_weight(&t.wqkv[l], L.wqkv, QKV, D) || tc_weight(&t.wo[l], L.wo, D, QD) ||
                tc_weight(&t.w13[l], L.w13, 2 * HID, D) || tc_weight(&t.w2[l], L.w2, D, HID))
                return -1;
            continue;
        }
        /* tile-contiguous copies for the tensor-core path (the row-major originals stay for the
         * streaming kernel's single-pass entry point) */
        const struct { TcWeight *w; const uint16_t *src; int N, K; uint16_t **dst; } jobs[4] = {
            {&t.wqkv[l], L.wqkv, QKV, D, &t.tiled[l][0]}, {&t.wo[l], L.wo, D, QD, &t.tiled[l][1]},
            {&t.w13[l], L.w13, 2 * HID, D, &t.tiled[l][2]}, {&t.w2[l], L.w2, D, HID, &t.tiled[l][3]}};
        for (int j = 0; j < 4; j++) {
            if (!*jobs[j].dst && alloc_zero((void **)jobs[j].dst, tc_tiled_bytes(jobs[j].N, jobs[j].K), &m.allocs)) return -1;
            if (tc_weight_tiled(jobs[j].w, jobs[j].src, jobs[j].N, jobs[j].K, *jobs[j].dst, m.st)) return -1;
        }
        if (cudaStreamSynchronize(m.st) != cudaSuccess) return -1;
    }
    AcBuffers &o = t.one;
    if (!o.bD) {
        o.X6 = m.X6;
        if (acoustic_buffers_alloc(&o, 1, &m.allocs)) return -1;
    }
    o.lat = &m.d_in->lat[0][0];
    o.vel = &m.d_out->vel[0][0];
    o.ltok = m.ltok;
    o.codes = m.d_out->codes;
    o.dyn = &m.d_in->dyn;
    o.status = &m.d_out->status;
    t.s_qkv = tc_pick_splits(QKV, D, m.sm_count);
    t.s_wo = tc_pick_splits(D, QD, m.sm_count);
    t.s_w2 = tc_pick_splits(D, HID, m.sm_count);
    t.ready = true;
    return 0;
}

bool acoustic_tc_ready() { return g_ac.ready; }

/* Enqueues the 7 Euler steps + FSQ on the library's stream. The semantic head, llm token
 * and argmax have already run; the llm token rows are in b.ltok. */
int acoustic_tc_enqueue_on(const AcBuffers &b, const float *noise_all, int *codes_all, int frame_cap, bool advance,
                           bool ignore_end) {
    Model &m = model();
    AcTc &t = g_ac;
    if (!t.ready) return -1;
    cudaStream_t st = m.st;
    const float scale = 1.0f / sqrtf((float)VB200_HEAD_DIM);
    const int steps = VB200_FLOW_STEPS - 1;
    const int ROWS = b.rows;
    const size_t psD = (size_t)ROWS * D;
    const int chunksD = tc_prepare_chunks(D);
    TcGemm g;
    g.M = ROWS; g.status = b.status;
    for (int s = 0; s < steps; s++) {
        launch_pdl(ac_tokens_kernel, dim3((D + 127) / 128, b.B), dim3(128), 0, st, b.X6, b.lat, (const float *)b.vel,
                   (const uint16_t *)m.ac_input_proj, (const float *)m.ttok, (const float *)b.ltok, s,
                   VB200_CFG_ALPHA, s > 0 ? m.dt[s - 1] : 0.0f, noise_all, (const VbDyn *)b.dyn, b.sd);
        for (int l = 0; l < VB200_AC_LAYERS; l++) {
            const LayerDev &L = m.ac[l];
            /* attention half: (reduce + residual +) gain -> QKV -> attention -> O */
            if (l == 0) tc_prepare(b.aD, b.X6, D, ROWS, nullptr, 0, 0, nullptr, nullptr, L.attn_norm, b.ssq, st);
            else tc_prepare(b.aD, nullptr, D, ROWS, b.part, t.s_w2, psD, b.X6, b.X6, L.attn_norm, b.ssq, st);
            g.epi = TC_EPI_PARTIAL; g.out = b.part; g.out_terms = nullptr;
            g.splits = t.s_qkv; g.ld_out = QKV; g.ssq = b.ssq; g.ssq_chunks = chunksD; g.eps = VB200_NORM_EPS;
            if (tc_gemm(t.wqkv[l], b.aD, g, st)) return -1;
            launch_pdl(ac_attention_kernel, dim3((ROWS * VB200_HEADS * 32 + 255) / 256), dim3(256), 0, st, b.bQ,
                       (const float *)b.part, t.s_qkv, scale, ROWS, b.rows_pad);
            g.splits = t.s_wo; g.ld_out = D; g.ssq = nullptr; g.ssq_chunks = 0;
            if (tc_gemm(t.wo[l], b.aQ, g, st)) return -1;
            /* FFN half: reduce + residual + gain -> gate/up with SwiGLU (terms out) -> down */
            tc_prepare(b.aD, nullptr, D, ROWS, b.part, t.s_wo, psD, b.X6, b.X6, L.ffn_norm, b.ssq, st);
            g.epi = TC_EPI_SWIGLU_TERMS; g.out = nullptr; g.out_terms = b.bH; g.out_rows_pad = b.rows_pad;
            g.splits = 1; g.ld_out = HID; g.ssq = b.ssq; g.ssq_chunks = chunksD;
            if (tc_gemm(t.w13[l], b.aD, g, st)) return -1;
            g.epi = TC_EPI_PARTIAL; g.out = b.part; g.out_terms = nullptr;
            g.splits = t.s_w2; g.ld_out = D; g.ssq = nullptr; g.ssq_chunks = 0;
            if (tc_gemm(t.w2[l], b.aH, g, st)) return -1;
        }
        launch_pdl(ac_velocity_kernel, dim3(9, 2 * b.B), dim3(512), 0, st, b.vel, (const float *)b.X6,
                   (const float *)b.part, t.s_w2, (const float *)m.ac_norm, VB200_NORM_EPS, (const uint16_t *)m.ac_out,
                   ROWS, b.sd.vel);
    }
    launch_pdl(ac_fsq_kernel, dim3(b.B), dim3(64), 0, st, b.codes, b.lat, (const float *)b.vel, steps,
               VB200_FSQ_LEVELS, VB200_CFG_ALPHA, m.dt[steps - 1], codes_all, b.dyn, frame_cap,
               advance ? 1 : 0, ignore_end ? 1 : 0, b.sd);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

static int enqueue_direct(const float *noise_all, int *codes_all, int frame_cap, bool advance, bool ignore_end) {
    return acoustic_tc_enqueue_on(g_ac.one, noise_all, codes_all, frame_cap, advance, ignore_end);
}

/* The ~200 launches of a frame are captured once per argument set as a CUDA graph and
 * replayed; the first call with a new argument set runs directly (it also sets the
 * kernels' shared-memory attributes, which must not happen inside a capture). */
struct GraphSlot {
    const float *noise_all = nullptr;
    int *codes_all = nullptr;
    int cap = 0;
    bool advance = false, ignore_end = false, used = false;
    int calls = 0;
    cudaGraphExec_t exec = nullptr;
};
static GraphSlot g_slots[2];

void acoustic_tc_drop_graphs() {
    for (GraphSlot &s : g_slots) {
        if (s.exec) cudaGraphExecDestroy(s.exec);
        s = GraphSlot();
    }
}

/* Called when the device context goes away: the tiled copies and buffers were the context's. */
void acoustic_tc_free_all() {
    acoustic_tc_drop_graphs();
    g_ac = AcTc();
}

int acoustic_tc_enqueue(const float *noise_all, int *codes_all, int frame_cap, bool advance, bool ignore_end) {
    Model &m = model();
    if (getenv("VB200_NO_GRAPH")) return enqueue_direct(noise_all, codes_all, frame_cap, advance, ignore_end);
    GraphSlot &s = g_slots[advance ? 1 : 0];
    const bool same = s.used && s.noise_all == noise_all && s.codes_all == codes_all && s.cap == frame_cap &&
                      s.advance == advance && s.ignore_end == ignore_end;
    if (!same) {
        if (s.exec) cudaGraphExecDestroy(s.exec);
        s = GraphSlot();
        s.noise_all = noise_all; s.codes_all = codes_all; s.cap = frame_cap;
        s.advance = advance; s.ignore_end = ignore_end; s.used = true;
    }
    if (s.exec) return cudaGraphLaunch(s.exec, m.st) == cudaSuccess ? 0 : -1;
    if (s.calls++ == 0) return enqueue_direct(noise_all, codes_all, frame_cap, advance, ignore_end);
    cudaGraph_t graph = nullptr;
    if (cudaStreamBeginCapture(m.st, cudaStreamCaptureModeRelaxed) != cudaSuccess) {
        cudaGetLastError();
        return enqueue_direct(noise_all, codes_all, frame_cap, advance, ignore_end);
    }
    const int rc = enqueue_direct(noise_all, codes_all, frame_cap, advance, ignore_end);
    const cudaError_t ee = cudaStreamEndCapture(m.st, &graph);
    if (rc || ee != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        return -1;
    }
    const cudaError_t ie = cudaGraphInstantiate(&s.exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ie != cudaSuccess) {
        s.exec = nullptr;
        cudaGetLastError();
        return -1;
    }
    return cudaGraphLaunch(s.exec, m.st) == cudaSuccess ? 0 : -1;
}

} // namespace vb
