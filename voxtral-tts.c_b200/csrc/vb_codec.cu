/*
 * vb_codec.cu - the audio codec decoder on the GPU: 37 codes per frame -> 24 kHz waveform
 * (tts_codec_decode, voxtral_tts_codec.c:389-510).
 *
 *   codes -> embedding [T, 292] (voxtral_tts_codec.c:276-300)
 *         -> causal conv 292 -> 1024, kernel 3 (voxtral_tts_kernels.c:217-270)
 *         -> 4 stages x 2 transformer layers (voxtral_tts_codec.c:306-383: RMSNorm eps 1e-2, QK norm
 *            over the whole row, ALiBi sliding-window causal attention, voxtral_tts_kernels.c:527-596,
 *            layer scale, SwiGLU) with a stride-2 transposed conv (kernel 4,
 *            voxtral_tts_kernels.c:272-327) after stages 0..2: T -> 2T -> 4T -> 8T rows
 *         -> causal conv 1024 -> 240, kernel 7 -> [8T, 240] = the waveform
 *
 * Rows stay row-major [time, channel] throughout (the reference transposes to channel-first
 * around every convolution). The transformer linears run on the tensor-core row-block GEMM
 * (vb_tc.cu) with BF16 weights - exact, because the checkpoint's BF16 values were only widened to
 * fp32 by the loader - and the activations as hi + lo BF16 terms. The convolutions keep their
 * fp32 (weight-normed) weights and run as implicit GEMMs on the fp32 pipes: a convolution is
 * C[t][oc] = bias[oc] + sum over taps and input channels of X[src(t, tap)][ic] * W[oc][tap][ic],
 * and a stride-2 transposed convolution is two such products, one per output parity.
 */
#include "vb_common.cuh"
#include "vb_model.cuh"
#include "vb_tc.cuh"

#include <math.h>
#include <stdio.h>
#include <string.h>
#include <vector>

namespace vb {

namespace {

constexpr int CD = 1024, CH = 4096, CQKV = 3 * CD, CHEADS = 8, CHD = 128;
constexpr int CEMB = 292, CSEM = 256, CSEM_ROWS = 8192, CPATCH = 240, CLAYERS = 8, CSTAGES = 4;
constexpr float CEPS = 1e-2f, CQK_EPS = 1e-6f;
constexpr int CFSQ = 21, CSPECIAL = 2, CCODES = 37;

struct CodecLayer {
    TcWeight wqkv, wo, w13, w2;
    float *attn_norm = nullptr, *ffn_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr;
    float *attn_scale = nullptr, *ffn_scale = nullptr;
    int window = 0;
};

struct Codec {
    bool ready = false;
    std::vector<void *> allocs;          /* weights */
    float *sem = nullptr;
    float *in_w = nullptr, *in_b = nullptr;          /* [1024][3][292] */
    float *up_w[3] = {}, *up_b[3] = {};              /* [2 parities][1024][2 taps][1024] */
    float *out_w = nullptr, *out_b = nullptr;        /* [240][7][1024] */
    CodecLayer L[CLAYERS];
    float *d_slopes = nullptr;
    /* activations, sized for cap_rows = 8 * frames */
    std::vector<void *> act_allocs;
    int cap_frames = 0, rows_pad = 0;
    int *codes = nullptr;
    float *emb = nullptr, *x = nullptr, *x2 = nullptr, *y = nullptr, *qkv = nullptr, *attn = nullptr, *ssq = nullptr;
    float *pcm = nullptr;
    uint16_t *tD = nullptr, *tH = nullptr;
    TcActs aD, aH;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    float last_ms = 0.0f;
};
Codec g_codec;

int c_alloc(void **p, size_t bytes, std::vector<void *> *owner) {
    if (cudaMalloc(p, bytes) != cudaSuccess) {
        cudaGetLastError();
        fprintf(stderr, "voxtral_b200: codec: cudaMalloc(%zu bytes) failed\n", bytes);
        *p = nullptr;
        return -1;
    }
    owner->push_back(*p);
    return 0;
}
void c_free(std::vector<void *> *owner) {
    for (void *p : *owner) cudaFree(p);
    owner->clear();
}

/* ---------------------------------------------------------------- upload kernels */

/* dst[r0 + r][c] = BF16(src[r][c]); *inexact counts the values BF16 cannot hold. */
__global__ void to_bf16_kernel(uint16_t *dst, const float *src, size_t n, unsigned *inexact) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t u = __float_as_uint(src[i]);
    if (u & 0xffffu) atomicAdd(inexact, 1u);
    dst[i] = (uint16_t)(u >> 16);
}
/* rows 2i / 2i+1 <- gate row i / up row i (the SwiGLU pair layout of the GEMM epilogue) */
__global__ void to_bf16_interleaved_kernel(uint16_t *dst, const float *gate, const float *up, int rows, int cols,
                                           unsigned *inexact) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * cols) return;
    const size_t r = i / cols, c = i % cols;
    const uint32_t a = __float_as_uint(gate[i]), b = __float_as_uint(up[i]);
    if ((a | b) & 0xffffu) atomicAdd(inexact, 1u);
    dst[(2 * r) * cols + c] = (uint16_t)(a >> 16);
    dst[(2 * r + 1) * cols + c] = (uint16_t)(b >> 16);
}
/* conv weight [oc][ic][k] -> [oc][k][ic] */
__global__ void conv_w_kernel(float *dst, const float *src, int oc, int ic, int k) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)oc * ic * k) return;
    const int kk = (int)(i % k), c = (int)((i / k) % ic), o = (int)(i / ((size_t)k * ic));
    dst[((size_t)o * k + kk) * ic + c] = src[i];
}
/* transposed-conv weight [ic][oc][k], k = parity + 2 * tap -> [parity][oc][tap][ic] */
__global__ void convt_w_kernel(float *dst, const float *src, int ic, int oc, int k) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)oc * ic * k) return;
    const int kk = (int)(i % k), o = (int)((i / k) % oc), c = (int)(i / ((size_t)k * oc));
    const int parity = kk & 1, tap = kk >> 1, taps = k / 2;
    dst[(((size_t)parity * oc + o) * taps + tap) * ic + c] = src[i];
}

/* ---------------------------------------------------------------- decode kernels */

/* emb[t][0..255] = semantic_embedding[code], emb[t][256 + i] = FSQ level -> [-1, 1]
 * (voxtral_tts_codec.c:276-300). grid = frames, 320 threads. */
__global__ void codec_embed_kernel(float *emb, const int *codes, const float *sem) {
    const int t = blockIdx.x, d = threadIdx.x;
    const int *fc = codes + t * CCODES;
    if (d < CSEM) {
        int s = fc[0] - CSPECIAL;
        s = s < 0 ? 0 : (s >= CSEM_ROWS ? CSEM_ROWS - 1 : s);
        emb[(size_t)t * CEMB + d] = sem[(size_t)s * CSEM + d];
    } else if (d < CEMB) {
        int a = fc[d - CSEM + 1] - CSPECIAL;
        a = a < 0 ? 0 : (a >= CFSQ ? CFSQ - 1 : a);
        emb[(size_t)t * CEMB + d] = (float)a * 2.0f / (float)(CFSQ - 1) - 1.0f;
    }
}

/* Implicit GEMM on the fp32 pipes:
 *   C[out_row(m)][n] = bias[n] + sum_tap sum_ic X[src(m, tap)][ic] * W[n][tap * Cin + ic]
 * MODE 0, causal convolution with the reference's reflect rule (voxtral_tts_kernels.c:246-262):
 *   src = m + tap - left_pad; src < 0 -> -src; src >= T -> 2T - 2 - src; outside [0, T) -> 0;
 *   out_row = m.
 * MODE 1, one output parity (blockIdx.z) of a stride-2 transposed convolution
 *   (voxtral_tts_kernels.c:272-327; kernel 4: no left trim, the last two raw outputs dropped):
 *   src = m - tap (>= 0), out_row = 2 m + parity, W advanced by parity * N * taps * Cin.
 * 64 x 64 output tile per CTA, 16-wide k steps, 256 threads x (4 x 4) outputs. */
template <int MODE>
__global__ void __launch_bounds__(256)
codec_conv_kernel(float *C, int ldc, const float *X, int ldx, const float *W, const float *bias, int T, int N, int Cin,
                  int taps, int left_pad) {
    __shared__ float As[16][64 + 4];
    __shared__ float Bs[16][64 + 4];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    const int K = taps * Cin;
    const float *Wp = W + (MODE == 1 ? (size_t)blockIdx.z * N * K : 0);
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        /* 64 x 16 elements of each operand, 4 per thread: thread -> (row = tid / 4 .. , 4 k's) */
        {
            const int r = tid >> 2, kq = (tid & 3) * 4;
            const int m = m0 + r;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int kk = k0 + kq + i;
                float a = 0.0f, b = 0.0f;
                if (kk < K) {
                    const int tap = kk / Cin, ic = kk - tap * Cin;
                    if (m < T) {
                        int src;
                        bool ok;
                        if (MODE == 0) {
                            src = m + tap - left_pad;
                            if (src < 0) src = -src;
                            else if (src >= T) src = 2 * T - 2 - src;
                            ok = src >= 0 && src < T;
                        } else {
                            src = m - tap;
                            ok = src >= 0;
                        }
                        if (ok) a = X[(size_t)src * ldx + ic];
                    }
                    const int n = n0 + r;
                    if (n < N) b = __ldg(Wp + (size_t)n * K + kk);
                }
                As[kq + i][r] = a;
                Bs[kq + i][r] = b;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; kk++) {
            const float4 a4 = *reinterpret_cast<const float4 *>(&As[kk][ty * 4]);
            const float4 b4 = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4]);
            const float a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] += a[i] * b[j];
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty * 4 + i;
        if (m >= T) continue;
        const size_t row = MODE == 1 ? (size_t)(2 * m + blockIdx.z) : (size_t)m;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[row * ldc + n] = acc[i][j] + (bias ? __ldg(bias + n) : 0.0f);
        }
    }
}

/* Rows -> BF16 terms for the next GEMM, with the residual update folded in:
 *   v = x[m][c] (+ y[m][c] * yscale[c], or + y[m][c] without a layer scale);  x_out[m][c] = v
 *   terms = v * gain (or v), ssq[m] = sum v^2 (the GEMM applies 1/sqrt(ssq/K + eps))
 * grid = (K / 1024, rows), 256 threads x 4 columns; `buf` may be null (residual update only). */
__global__ void codec_prepare_kernel(uint16_t *buf, int rows_pad, int K, const float *x, const float *y,
                                     const float *yscale, float *x_out, const float *gain, float *ssq) {
    __shared__ float red[8];
    const int m = blockIdx.y, c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    float ss = 0.0f;
    if (c < K) {
        float4 v = *reinterpret_cast<const float4 *>(x + (size_t)m * K + c);
        if (y) {
            const float4 u = *reinterpret_cast<const float4 *>(y + (size_t)m * K + c);
            if (yscale) {
                const float4 s = __ldg(reinterpret_cast<const float4 *>(yscale + c));
                v.x += u.x * s.x; v.y += u.y * s.y; v.z += u.z * s.z; v.w += u.w * s.w;
            } else {
                v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
            }
        }
        if (x_out) *reinterpret_cast<float4 *>(x_out + (size_t)m * K + c) = v;
        ss = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        if (buf) {
            if (gain) {
                const float4 g = __ldg(reinterpret_cast<const float4 *>(gain + c));
                v.x *= g.x; v.y *= g.y; v.z *= g.z; v.w *= g.w;
            }
            const float e[4] = {v.x, v.y, v.z, v.w};
            uint16_t t0[4], t1[4], t2[4];
#pragma unroll
            for (int i = 0; i < 4; i++) vb_split3(e[i], t0[i], t1[i], t2[i]);
            const size_t o = (size_t)m * K + c, term = (size_t)rows_pad * K;
            *reinterpret_cast<uint2 *>(buf + o) = make_uint2(t0[0] | ((uint32_t)t0[1] << 16), t0[2] | ((uint32_t)t0[3] << 16));
            *reinterpret_cast<uint2 *>(buf + term + o) = make_uint2(t1[0] | ((uint32_t)t1[1] << 16), t1[2] | ((uint32_t)t1[3] << 16));
            *reinterpret_cast<uint2 *>(buf + 2 * term + o) = make_uint2(t2[0] | ((uint32_t)t2[1] << 16), t2[2] | ((uint32_t)t2[3] << 16));
        }
    }
    if (ssq) {
        ss = vb_warp_sum(ss);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.0f;
            for (int w = 0; w < (int)(blockDim.x >> 5); w++) t += red[w];
            ssq[m * gridDim.x + blockIdx.x] = t;
        }
    }
}

/* QK norm in place: RMSNorm over the whole 1024-wide q row and k row (tts_qk_norm,
 * voxtral_tts_kernels.c:351-355). grid = (rows, 2), 256 threads. */
__global__ void codec_qknorm_kernel(float *qkv, const float *qw, const float *kw, float eps) {
    __shared__ float red[8];
    const float *w = blockIdx.y == 0 ? qw : kw;
    if (!w) return;
    float *row = qkv + (size_t)blockIdx.x * CQKV + blockIdx.y * CD;
    float4 v = *reinterpret_cast<float4 *>(row + threadIdx.x * 4);
    float ss = vb_warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < 8; i++) t += red[i];
    const float inv = 1.0f / sqrtf(t / (float)CD + eps);
    const float4 g = __ldg(reinterpret_cast<const float4 *>(w + threadIdx.x * 4));
    v.x = v.x * inv * g.x; v.y = v.y * inv * g.y; v.z = v.z * inv * g.z; v.w = v.w * inv * g.w;
    *reinterpret_cast<float4 *>(row + threadIdx.x * 4) = v;
}

/* ALiBi sliding-window causal attention (tts_alibi_attention, voxtral_tts_kernels.c:527-596): one
 * warp per (row, head), a lane owns 4 of the 128 dims, keys max(0, i - window + 1) .. i taken in
 * order with the reference's running-maximum update. */
__global__ void codec_attention_kernel(float *out, const float *qkv, int rows, int window, float scale,
                                       const float *slopes8) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows * CHEADS) return;
    const int i = warp / CHEADS, h = warp % CHEADS;
    const float slope = slopes8[h];
    const float4 q = *reinterpret_cast<const float4 *>(qkv + (size_t)i * CQKV + h * CHD + lane * 4);
    int j0 = 0;
    if (window > 0 && i - window + 1 > 0) j0 = i - window + 1;
    float mx = -1e30f, den = 0.0f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = j0; j <= i; j++) {
        const float4 k = *reinterpret_cast<const float4 *>(qkv + (size_t)j * CQKV + CD + h * CHD + lane * 4);
        const float4 v = *reinterpret_cast<const float4 *>(qkv + (size_t)j * CQKV + 2 * CD + h * CHD + lane * 4);
        float s = vb_warp_sum(q.x * k.x + q.y * k.y + q.z * k.z + q.w * k.w);
        s = __shfl_sync(0xffffffffu, s, 0);
        s = s * scale + slope * (float)(j - i);
        if (s > mx) {
            const float corr = expf(mx - s);
            den = den * corr + 1.0f;
            o.x = o.x * corr + v.x; o.y = o.y * corr + v.y; o.z = o.z * corr + v.z; o.w = o.w * corr + v.w;
            mx = s;
        } else {
            const float w = expf(s - mx);
            den += w;
            o.x += w * v.x; o.y += w * v.y; o.z += w * v.z; o.w += w * v.w;
        }
    }
    const float inv = den > 0.0f ? 1.0f / den : 0.0f;
    *reinterpret_cast<float4 *>(out + (size_t)i * CD + h * CHD + lane * 4) = make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv);
}

/* ---------------------------------------------------------------- host side */

int up_f32(float **dst, const float *src, size_t n, std::vector<void *> *owner) {
    if (!src) { *dst = nullptr; return 0; }
    if (c_alloc((void **)dst, n * 4, owner)) return -1;
    return cudaMemcpy(*dst, src, n * 4, cudaMemcpyHostToDevice) == cudaSuccess ? 0 : -1;
}

/* fp32 host matrices -> one BF16 device matrix (rows stacked), tile-contiguous for the GEMM. */
int up_matrix(TcWeight *tw, const float *const *parts, const int *part_rows, int n_parts, int cols, bool interleave,
              float *stage, unsigned *inexact, std::vector<void *> *owner, cudaStream_t st) {
    int rows = 0;
    for (int i = 0; i < n_parts; i++) rows += part_rows[i];
    uint16_t *plain = nullptr, *tiled = nullptr;
    if (cudaMalloc((void **)&plain, (size_t)rows * cols * 2) != cudaSuccess) return -1;
    int rc = 0;
    if (interleave) {
        /* two parts of equal height: gate rows and up rows */
        const size_t n = (size_t)part_rows[0] * cols;
        if (cudaMemcpyAsync(stage, parts[0], n * 4, cudaMemcpyHostToDevice, st) != cudaSuccess ||
            cudaMemcpyAsync(stage + n, parts[1], n * 4, cudaMemcpyHostToDevice, st) != cudaSuccess)
            rc = -1;
        if (!rc)
            to_bf16_interleaved_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(plain, stage, stage + n, part_rows[0],
                                                                                  cols, inexact);
    } else {
        size_t off = 0;
        for (int i = 0; i < n_parts && !rc; i++) {
            const size_t n = (size_t)part_rows[i] * cols;
            if (cudaMemcpyAsync(stage, parts[i], n * 4, cudaMemcpyHostToDevice, st) != cudaSuccess) { rc = -1; break; }
            to_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(plain + off, stage, n, inexact);
            off += n;
        }
    }
    if (!rc && c_alloc((void **)&tiled, tc_tiled_bytes(rows, cols), owner)) rc = -1;
    if (!rc && tc_weight_tiled(tw, plain, rows, cols, tiled, st)) rc = -1;
    if (cudaStreamSynchronize(st) != cudaSuccess) rc = -1;
    cudaFree(plain);
    return rc;
}

int ensure_buffers(int frames) {
    Codec &c = g_codec;
    if (frames <= c.cap_frames) return 0;
    c_free(&c.act_allocs);
    c.cap_frames = 0;
    const int rows = 8 * frames;
    const int rp = tc_rows_pad_any(rows);
    if (!rp) return -1;
    int rc = 0;
    rc |= c_alloc((void **)&c.codes, sizeof(int) * (size_t)frames * CCODES, &c.act_allocs);
    rc |= c_alloc((void **)&c.emb, sizeof(float) * (size_t)frames * CEMB, &c.act_allocs);
    rc |= c_alloc((void **)&c.x, sizeof(float) * (size_t)rows * CD, &c.act_allocs);
    rc |= c_alloc((void **)&c.x2, sizeof(float) * (size_t)rows * CD, &c.act_allocs);
    rc |= c_alloc((void **)&c.y, sizeof(float) * (size_t)rows * CD, &c.act_allocs);
    rc |= c_alloc((void **)&c.qkv, sizeof(float) * (size_t)rows * CQKV, &c.act_allocs);
    rc |= c_alloc((void **)&c.attn, sizeof(float) * (size_t)rows * CD, &c.act_allocs);
    rc |= c_alloc((void **)&c.ssq, sizeof(float) * (size_t)rows * 4, &c.act_allocs);
    rc |= c_alloc((void **)&c.pcm, sizeof(float) * (size_t)rows * CPATCH, &c.act_allocs);
    rc |= c_alloc((void **)&c.tD, tc_acts_bytes(rp, CD), &c.act_allocs);
    rc |= c_alloc((void **)&c.tH, tc_acts_bytes(rp, CH), &c.act_allocs);
    if (rc) { c_free(&c.act_allocs); return -1; }
    /* rows of the padding are multiplied like any other (their results are never stored):
     * keep them finite */
    cudaMemset(c.tD, 0, tc_acts_bytes(rp, CD));
    cudaMemset(c.tH, 0, tc_acts_bytes(rp, CH));
    if (tc_acts(&c.aD, c.tD, rp, CD) || tc_acts(&c.aH, c.tH, rp, CH)) { c_free(&c.act_allocs); return -1; }
    c.rows_pad = rp;
    c.cap_frames = frames;
    return 0;
}

/* One GEMM on `rows` rows of the padded term buffers. The term buffers are laid out for
 * c.rows_pad rows whatever `rows` is, so the same tensor maps serve every stage. */
int gemm(const TcWeight &w, const TcActs &a, int rows, int epi, float *out, int ld_out, const float *ssq, float eps,
         uint16_t *out_terms, cudaStream_t st) {
    TcGemm g;
    g.M = rows; g.splits = 1; g.epi = epi; g.out = out; g.ld_out = ld_out;
    g.ssq = ssq; g.ssq_chunks = ssq ? 1 : 0; g.eps = eps;
    g.out_terms = out_terms; g.out_rows_pad = g_codec.rows_pad;
    g.status = &model().d_out->status;
    return tc_gemm(w, a, g, st);
}

int layer_forward(const CodecLayer &L, int rows, const float *y_prev, const float *yscale_prev, cudaStream_t st) {
    Codec &c = g_codec;
    const float scale = 1.0f / sqrtf((float)CHD);
    /* x (+ the previous layer's FFN update) -> attention-norm terms */
    codec_prepare_kernel<<<dim3(1, rows), 256, 0, st>>>(c.tD, c.rows_pad, CD, c.x, y_prev, yscale_prev,
                                                        y_prev ? c.x : nullptr, L.attn_norm, c.ssq);
    if (gemm(L.wqkv, c.aD, rows, TC_EPI_STORE, c.qkv, CQKV, c.ssq, CEPS, nullptr, st)) return -1;
    if (L.q_norm || L.k_norm) codec_qknorm_kernel<<<dim3(rows, 2), 256, 0, st>>>(c.qkv, L.q_norm, L.k_norm, CQK_EPS);
    codec_attention_kernel<<<(rows * CHEADS * 32 + 255) / 256, 256, 0, st>>>(c.attn, c.qkv, rows, L.window, scale,
                                                                            c.d_slopes);
    codec_prepare_kernel<<<dim3(1, rows), 256, 0, st>>>(c.tD, c.rows_pad, CD, c.attn, nullptr, nullptr, nullptr, nullptr,
                                                        nullptr);
    if (gemm(L.wo, c.aD, rows, TC_EPI_STORE, c.y, CD, nullptr, 0.0f, nullptr, st)) return -1;
    /* x += proj * attn_scale -> FFN-norm terms */
    codec_prepare_kernel<<<dim3(1, rows), 256, 0, st>>>(c.tD, c.rows_pad, CD, c.x, c.y, L.attn_scale, c.x, L.ffn_norm,
                                                        c.ssq);
    if (gemm(L.w13, c.aD, rows, TC_EPI_SWIGLU_TERMS, nullptr, CH, c.ssq, CEPS, c.tH, st)) return -1;
    if (gemm(L.w2, c.aH, rows, TC_EPI_STORE, c.y, CD, nullptr, 0.0f, nullptr, st)) return -1;
    return 0;   /* the caller folds x += y * ffn_scale into the next step */
}

int conv_reorder(float **dst, const vb200_conv_t &cv, bool transposed, float *stage, std::vector<void *> *owner,
                 cudaStream_t st) {
    const size_t n = (size_t)cv.in_ch * cv.out_ch * cv.kernel;
    if (!cv.weight || c_alloc((void **)dst, n * 4, owner)) return -1;
    if (cudaMemcpyAsync(stage, cv.weight, n * 4, cudaMemcpyHostToDevice, st) != cudaSuccess) return -1;
    if (transposed) convt_w_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(*dst, stage, cv.in_ch, cv.out_ch, cv.kernel);
    else conv_w_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(*dst, stage, cv.out_ch, cv.in_ch, cv.kernel);
    return cudaStreamSynchronize(st) == cudaSuccess ? 0 : -1;
}

} // namespace

void codec_free_all() {
    Codec &c = g_codec;
    c_free(&c.allocs);
    c_free(&c.act_allocs);
    if (c.e0) cudaEventDestroy(c.e0);
    if (c.e1) cudaEventDestroy(c.e1);
    c = Codec();
}

int codec_upload(const vb200_codec_weights_t *w) {
    Model &m = model();
    Codec &c = g_codec;
    if (!m.inited || !w) return -1;
    codec_free_all();
    if (tc_init()) return -1;
    /* the shapes this decoder is written for (voxtral_tts_codec.c:204-262) */
    const vb200_conv_t &ic = w->input_conv, &oc = w->output_proj;
    bool ok = w->semantic_embedding && ic.in_ch == CEMB && ic.out_ch == CD && ic.kernel == 3 && ic.stride == 1 &&
              !ic.is_transpose && oc.in_ch == CD && oc.out_ch == CPATCH && oc.kernel == 7 && oc.stride == 1 && !oc.is_transpose;
    for (int s = 0; s < CSTAGES - 1 && ok; s++) {
        const vb200_conv_t &u = w->stage_convs[s];
        ok = u.in_ch == CD && u.out_ch == CD && u.kernel == 4 && u.stride == 2 && u.is_transpose && u.weight;
    }
    for (int l = 0; l < CLAYERS && ok; l++) {
        const vb200_codec_layer_t &L = w->transformers[l];
        ok = L.wq && L.wk && L.wv && L.wo && L.w1 && L.w2 && L.w3 && L.attention_norm && L.ffn_norm;
    }
    if (!ok) {
        fprintf(stderr, "voxtral_b200: codec: weights missing or of an unexpected shape\n");
        return -1;
    }
    cudaStream_t st = m.st;
    float *stage = nullptr;
    unsigned *inexact = nullptr;
    if (cudaMalloc((void **)&stage, sizeof(float) * (size_t)2 * CH * CD) != cudaSuccess ||
        cudaMalloc((void **)&inexact, sizeof(unsigned)) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(stage);
        return -1;
    }
    cudaMemset(inexact, 0, sizeof(unsigned));
    int rc = 0;
    rc |= up_f32(&c.sem, w->semantic_embedding, (size_t)CSEM_ROWS * CSEM, &c.allocs);
    rc |= conv_reorder(&c.in_w, ic, false, stage, &c.allocs, st);
    rc |= up_f32(&c.in_b, ic.bias, CD, &c.allocs);
    rc |= conv_reorder(&c.out_w, oc, false, stage, &c.allocs, st);
    rc |= up_f32(&c.out_b, oc.bias, CPATCH, &c.allocs);
    for (int s = 0; s < CSTAGES - 1 && !rc; s++) {
        rc |= conv_reorder(&c.up_w[s], w->stage_convs[s], true, stage, &c.allocs, st);
        rc |= up_f32(&c.up_b[s], w->stage_convs[s].bias, CD, &c.allocs);
    }
    for (int l = 0; l < CLAYERS && !rc; l++) {
        const vb200_codec_layer_t &L = w->transformers[l];
        CodecLayer &d = c.L[l];
        const float *qkv[3] = {L.wq, L.wk, L.wv};
        const int r3[3] = {CD, CD, CD};
        const float *gu[2] = {L.w1, L.w3};
        const int r2[2] = {CH, CH};
        const float *one[1];
        const int rD[1] = {CD};
        rc |= up_matrix(&d.wqkv, qkv, r3, 3, CD, false, stage, inexact, &c.allocs, st);
        one[0] = L.wo;
        rc |= up_matrix(&d.wo, one, rD, 1, CD, false, stage, inexact, &c.allocs, st);
        rc |= up_matrix(&d.w13, gu, r2, 2, CD, true, stage, inexact, &c.allocs, st);
        one[0] = L.w2;
        rc |= up_matrix(&d.w2, one, rD, 1, CH, false, stage, inexact, &c.allocs, st);
        rc |= up_f32(&d.attn_norm, L.attention_norm, CD, &c.allocs);
        rc |= up_f32(&d.ffn_norm, L.ffn_norm, CD, &c.allocs);
        rc |= up_f32(&d.q_norm, L.q_norm, CD, &c.allocs);
        rc |= up_f32(&d.k_norm, L.k_norm, CD, &c.allocs);
        rc |= up_f32(&d.attn_scale, L.attn_scale, CD, &c.allocs);
        rc |= up_f32(&d.ffn_scale, L.ffn_scale, CD, &c.allocs);
        d.window = L.window_size;
    }
    float *slopes = nullptr;
    if (!rc) rc = up_f32(&slopes, w->alibi_slopes, CHEADS, &c.allocs);
    c.d_slopes = slopes;
    unsigned bad = 0;
    if (!rc && cudaMemcpy(&bad, inexact, sizeof(unsigned), cudaMemcpyDeviceToHost) != cudaSuccess) rc = -1;
    cudaFree(stage);
    cudaFree(inexact);
    if (!rc && bad) {
        fprintf(stderr, "voxtral_b200: codec: %u transformer weights are not exactly representable in BF16; "
                        "this decoder keeps them as BF16 and refuses to round\n", bad);
        rc = -1;
    }
    if (!rc && (cudaEventCreate(&c.e0) != cudaSuccess || cudaEventCreate(&c.e1) != cudaSuccess)) rc = -1;
    if (rc) {
        codec_free_all();
        return -1;
    }
    c.ready = true;
    return 0;
}

int codec_decode(const int *codes, int n_frames, float *samples_out, int max_samples, int *n_samples) {
    Model &m = model();
    Codec &c = g_codec;
    if (n_samples) *n_samples = 0;
    if (!m.inited || !c.ready || !codes || n_frames < 1 || !samples_out) return -1;
    const long long total = (long long)n_frames * 8 * CPATCH;
    if (total > max_samples || 8 * n_frames > kTcMaxRows) return -1;
    if (ensure_buffers(n_frames)) return -1;
    cudaStream_t st = m.st;
    if (cudaMemcpyAsync(c.codes, codes, sizeof(int) * (size_t)n_frames * CCODES, cudaMemcpyHostToDevice, st) != cudaSuccess)
        return -1;
    cudaEventRecord(c.e0, st);
    codec_embed_kernel<<<n_frames, 320, 0, st>>>(c.emb, c.codes, c.sem);
    int rows = n_frames;
    codec_conv_kernel<0><<<dim3(CD / 64, (rows + 63) / 64, 1), 256, 0, st>>>(c.x, CD, c.emb, CEMB, c.in_w, c.in_b, rows, CD,
                                                                         CEMB, 3, 2);
    int l = 0;
    for (int stage = 0; stage < CSTAGES; stage++) {
        const float *y_prev = nullptr, *sc_prev = nullptr;
        for (int i = 0; i < 2; i++, l++) {
            if (layer_forward(c.L[l], rows, y_prev, sc_prev, st)) return -1;
            y_prev = c.y;
            sc_prev = c.L[l].ffn_scale;
        }
        /* the stage's last FFN update, no terms */
        codec_prepare_kernel<<<dim3(1, rows), 256, 0, st>>>(nullptr, c.rows_pad, CD, c.x, y_prev, sc_prev, c.x, nullptr,
                                                            nullptr);
        if (stage < CSTAGES - 1) {
            codec_conv_kernel<1><<<dim3(CD / 64, (rows + 63) / 64, 2), 256, 0, st>>>(c.x2, CD, c.x, CD, c.up_w[stage],
                                                                                 c.up_b[stage], rows, CD, CD, 2, 0);
            float *t = c.x; c.x = c.x2; c.x2 = t;
            rows *= 2;
        }
    }
    codec_conv_kernel<0><<<dim3((CPATCH + 63) / 64, (rows + 63) / 64, 1), 256, 0, st>>>(c.pcm, CPATCH, c.x, CD, c.out_w, c.out_b,
                                                                                    rows, CPATCH, CD, 7, 6);
    cudaEventRecord(c.e1, st);
    int status = 0;
    if (cudaMemcpyAsync(samples_out, c.pcm, sizeof(float) * (size_t)total, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaMemcpyAsync(&status, &m.d_out->status, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    cudaEventElapsedTime(&c.last_ms, c.e0, c.e1);
    m.last_status = status;
    if (status) {
        cudaMemset(&m.d_out->status, 0, sizeof(int));
        return -1;
    }
    if (n_samples) *n_samples = (int)total;
    return 0;
}

float codec_last_ms() { return g_codec.last_ms; }

} // namespace vb
