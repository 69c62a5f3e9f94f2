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
 * fp32 by the loader - and the activations as hi + lo BF16 terms. A convolution is a GEMM too,
 *   C[t][oc] = bias[oc] + sum over taps and input channels of X[src(t, tap)][ic] * W[oc][tap][ic],
 * and a stride-2 transposed convolution is one with both output parities as columns,
 *   C[m][parity * 1024 + oc] = sum over 2 taps of X[m - tap][ic] * W[ic][oc][parity + 2 tap],
 * whose row-major result [T][2048] IS the upsampled sequence [2T][1024]. Their (weight-normed)
 * weights are genuine fp32: they are split into W = hi + lo BF16 matrices (16 mantissa bits,
 * relative error 4e-6) and the row-block GEMM runs once on each, on the gathered activation
 * terms, into split-K partial buffers that one reduction sums together with the bias.
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
constexpr int kConvSplits = 4;      /* K splits per half (hi / lo) of a convolution GEMM */

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
    /* convolutions as GEMMs: hi / lo BF16 halves of W[N][Kpad], bias[N] */
    struct Conv {
        TcWeight hi, lo;
        float *bias = nullptr;
        int N = 0, K = 0, Kpad = 0, Cin = 0, taps = 0, mode = 0, left_pad = 0;
    } in_conv, up_conv[3], out_conv;
    CodecLayer L[CLAYERS];
    float *d_slopes = nullptr;
    /* activations, sized for cap_rows = 8 * frames */
    std::vector<void *> act_allocs;
    int cap_frames = 0, rows_pad = 0;
    int *codes = nullptr;
    float *emb = nullptr, *x = nullptr, *x2 = nullptr, *y = nullptr, *qkv = nullptr, *attn = nullptr, *ssq = nullptr;
    float *pcm = nullptr;
    uint16_t *tD = nullptr, *tH = nullptr, *tC = nullptr;
    float *part = nullptr;
    TcActs aD, aH, aIn, aUp, aOut;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    float last_ms = 0.0f;
};
Codec g_codec;
int g_block_frames = 0;   /* frames per decode block; 0: the largest the GEMM takes (an option, survives uploads) */

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
    pdl_launch_dependents();
    pdl_wait();
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

/* The A operand of a convolution GEMM: terms[m][tap * Cin + ic] = hi / lo BF16 of X[src(m, tap)][ic]
 * (columns from taps * Cin up to Kpad are zero).
 * MODE 0, causal convolution with the reference's reflect rule (voxtral_tts_kernels.c:246-262):
 *   src = m + tap - left_pad; src < 0 -> -src; src >= T -> 2T - 2 - src; outside [0, T) -> 0.
 * MODE 1, stride-2 transposed convolution, kernel 4 (voxtral_tts_kernels.c:272-327: no left
 *   trim, the last two raw outputs dropped): src = m - tap, zero when negative.
 * grid = (Kpad / 1024 rounded up, T), 256 threads x 4 columns. */
__global__ void codec_gather_kernel(uint16_t *buf, int rows_pad, int Kpad, const float *X, int ldx, int T, int Cin,
                                    int taps, int mode, int left_pad) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.y, k = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (k >= Kpad) return;
    float e[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int kk = k + i;
        float v = 0.0f;
        if (kk < taps * Cin) {
            const int tap = kk / Cin, ic = kk - tap * Cin;
            int src;
            bool ok;
            if (mode == 0) {
                src = m + tap - left_pad;
                if (src < 0) src = -src;
                else if (src >= T) src = 2 * T - 2 - src;
                ok = src >= 0 && src < T;
            } else {
                src = m - tap;
                ok = src >= 0;
            }
            if (ok) v = X[(size_t)src * ldx + ic];
        }
        e[i] = v;
    }
    uint16_t t0[4], t1[4], t2[4];
#pragma unroll
    for (int i = 0; i < 4; i++) vb_split3(e[i], t0[i], t1[i], t2[i]);
    const size_t o = (size_t)m * Kpad + k, term = (size_t)rows_pad * Kpad;
    *reinterpret_cast<uint2 *>(buf + o) = make_uint2(t0[0] | ((uint32_t)t0[1] << 16), t0[2] | ((uint32_t)t0[3] << 16));
    *reinterpret_cast<uint2 *>(buf + term + o) = make_uint2(t1[0] | ((uint32_t)t1[1] << 16), t1[2] | ((uint32_t)t1[3] << 16));
    *reinterpret_cast<uint2 *>(buf + 2 * term + o) = make_uint2(t2[0] | ((uint32_t)t2[1] << 16), t2[2] | ((uint32_t)t2[3] << 16));
}

/* W[N][K] fp32 -> hi[N][Kpad], lo[N][Kpad] BF16 with W = hi + lo up to 2^-17 (hi truncated, lo the
 * rounded remainder), zero beyond K. */
__global__ void split_w_kernel(uint16_t *hi, uint16_t *lo, const float *W, int N, int K, int Kpad) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)N * Kpad) return;
    const int n = (int)(i / Kpad), k = (int)(i % Kpad);
    uint16_t h = 0, l = 0;
    if (k < K) {
        const float w = W[(size_t)n * K + k];
        const uint32_t u = __float_as_uint(w) & 0xffff0000u;
        h = (uint16_t)(u >> 16);
        const float r = w - __uint_as_float(u);
        uint32_t ru = __float_as_uint(r);
        ru += 0x7fffu + ((ru >> 16) & 1u);                     /* round to nearest even */
        l = (uint16_t)(ru >> 16);
    }
    hi[i] = h;
    lo[i] = l;
}

/* Rows -> BF16 terms for the next GEMM, with the residual update folded in:
 *   v = x[m][c] (+ y[m][c] * yscale[c], or + y[m][c] without a layer scale);  x_out[m][c] = v
 *   terms = v * gain (or v), ssq[m] = sum v^2 (the GEMM applies 1/sqrt(ssq/K + eps))
 * grid = (K / 1024, rows), 256 threads x 4 columns; `buf` may be null (residual update only). */
__global__ void codec_prepare_kernel(uint16_t *buf, int rows_pad, int K, const float *x, const float *y,
                                     const float *yscale, float *x_out, const float *gain, float *ssq) {
    pdl_launch_dependents();
    pdl_wait();
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
    pdl_launch_dependents();
    pdl_wait();
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
    pdl_launch_dependents();
    pdl_wait();
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
    /* convolution operands: one buffer, laid out per convolution (every term is rewritten by the
     * gather before each use); split-K partials of the largest convolution GEMM */
    const int rp_in = tc_rows_pad_any(frames), rp_up = tc_rows_pad_any(4 * frames);
    size_t conv_bytes = tc_acts_bytes(rp, c.out_conv.Kpad);
    if (tc_acts_bytes(rp_up, c.up_conv[0].Kpad) > conv_bytes) conv_bytes = tc_acts_bytes(rp_up, c.up_conv[0].Kpad);
    if (tc_acts_bytes(rp_in, c.in_conv.Kpad) > conv_bytes) conv_bytes = tc_acts_bytes(rp_in, c.in_conv.Kpad);
    rc |= c_alloc((void **)&c.tC, conv_bytes, &c.act_allocs);
    rc |= c_alloc((void **)&c.part, sizeof(float) * (size_t)2 * kConvSplits * 4 * frames * 2 * CD, &c.act_allocs);
    if (rc) { c_free(&c.act_allocs); return -1; }
    cudaMemset(c.tC, 0, conv_bytes);
    if (tc_acts(&c.aIn, c.tC, rp_in, c.in_conv.Kpad) || tc_acts(&c.aUp, c.tC, rp_up, c.up_conv[0].Kpad) ||
        tc_acts(&c.aOut, c.tC, rp, c.out_conv.Kpad)) {
        c_free(&c.act_allocs);
        return -1;
    }
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
    launch_pdl(codec_prepare_kernel, dim3(1, rows), dim3(256), 0, st, c.tD, c.rows_pad, CD, c.x, y_prev, yscale_prev,
                                                        y_prev ? c.x : nullptr, L.attn_norm, c.ssq);
    if (gemm(L.wqkv, c.aD, rows, TC_EPI_STORE, c.qkv, CQKV, c.ssq, CEPS, nullptr, st)) return -1;
    if (L.q_norm || L.k_norm) launch_pdl(codec_qknorm_kernel, dim3(rows, 2), dim3(256), 0, st, c.qkv, L.q_norm, L.k_norm, CQK_EPS);
    launch_pdl(codec_attention_kernel, dim3((rows * CHEADS * 32 + 255) / 256), dim3(256), 0, st, c.attn, c.qkv, rows, L.window, scale,
                                                                            c.d_slopes);
    launch_pdl(codec_prepare_kernel, dim3(1, rows), dim3(256), 0, st, c.tD, c.rows_pad, CD, c.attn, nullptr, nullptr, nullptr, nullptr,
                                                        nullptr);
    if (gemm(L.wo, c.aD, rows, TC_EPI_STORE, c.y, CD, nullptr, 0.0f, nullptr, st)) return -1;
    /* x += proj * attn_scale -> FFN-norm terms */
    launch_pdl(codec_prepare_kernel, dim3(1, rows), dim3(256), 0, st, c.tD, c.rows_pad, CD, c.x, c.y, L.attn_scale, c.x, L.ffn_norm,
                                                        c.ssq);
    if (gemm(L.w13, c.aD, rows, TC_EPI_SWIGLU_TERMS, nullptr, CH, c.ssq, CEPS, c.tH, st)) return -1;
    if (gemm(L.w2, c.aH, rows, TC_EPI_STORE, c.y, CD, nullptr, 0.0f, nullptr, st)) return -1;
    return 0;   /* the caller folds x += y * ffn_scale into the next step */
}

/* One convolution made ready as a GEMM: weights reordered to [N][taps * Cin] (a transposed
 * convolution: both parities stacked, N = 2 * out_ch, 2 taps each), split into hi / lo BF16
 * matrices and tiled; bias (repeated per parity). */
int conv_setup(Codec::Conv *cv, const vb200_conv_t &w, float *stage, std::vector<void *> *owner, cudaStream_t st) {
    const bool tr = w.is_transpose != 0;
    const size_t n = (size_t)w.in_ch * w.out_ch * w.kernel;
    cv->Cin = w.in_ch;
    cv->taps = tr ? w.kernel / 2 : w.kernel;
    cv->N = tr ? 2 * w.out_ch : w.out_ch;
    cv->K = cv->taps * w.in_ch;
    cv->Kpad = (cv->K + 63) / 64 * 64;
    cv->mode = tr ? 1 : 0;
    cv->left_pad = tr ? 0 : w.kernel - w.stride;
    float *ordered = stage + n;                                  /* second half of the staging buffer */
    uint16_t *hi = nullptr, *lo = nullptr, *thi = nullptr, *tlo = nullptr;
    const size_t nk = (size_t)cv->N * cv->Kpad;
    int rc = 0;
    if (!w.weight || cudaMemcpyAsync(stage, w.weight, n * 4, cudaMemcpyHostToDevice, st) != cudaSuccess) return -1;
    if (tr) convt_w_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(ordered, stage, w.in_ch, w.out_ch, w.kernel);
    else conv_w_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(ordered, stage, w.out_ch, w.in_ch, w.kernel);
    if (cudaMalloc((void **)&hi, nk * 2) != cudaSuccess || cudaMalloc((void **)&lo, nk * 2) != cudaSuccess) rc = -1;
    if (!rc) split_w_kernel<<<(unsigned)((nk + 255) / 256), 256, 0, st>>>(hi, lo, ordered, cv->N, cv->K, cv->Kpad);
    if (!rc && (c_alloc((void **)&thi, tc_tiled_bytes(cv->N, cv->Kpad), owner) ||
                c_alloc((void **)&tlo, tc_tiled_bytes(cv->N, cv->Kpad), owner)))
        rc = -1;
    if (!rc && (tc_weight_tiled(&cv->hi, hi, cv->N, cv->Kpad, thi, st) || tc_weight_tiled(&cv->lo, lo, cv->N, cv->Kpad, tlo, st)))
        rc = -1;
    if (cudaStreamSynchronize(st) != cudaSuccess) rc = -1;
    cudaFree(hi);
    cudaFree(lo);
    if (!rc && w.bias) {
        if (c_alloc((void **)&cv->bias, sizeof(float) * cv->N, owner)) return -1;
        for (int p = 0; p < (tr ? 2 : 1) && !rc; p++)
            if (cudaMemcpy(cv->bias + (size_t)p * w.out_ch, w.bias, sizeof(float) * w.out_ch, cudaMemcpyHostToDevice) != cudaSuccess)
                rc = -1;
    }
    return rc;
}

/* Runs one convolution: gather -> GEMM on the hi and on the lo matrix (split-K partials) -> sum +
 * bias into out [T][N]. */
int conv_run(const Codec::Conv &cv, const TcActs &acts, const float *X, int ldx, int T, float *out, cudaStream_t st) {
    Codec &c = g_codec;
    launch_pdl(codec_gather_kernel, dim3((cv.Kpad + 1023) / 1024, T), dim3(256), 0, st, acts.buf, acts.rows_pad, cv.Kpad, X, ldx, T, cv.Cin,
                                                                          cv.taps, cv.mode, cv.left_pad);
    const int pairs = ((cv.N + kTcTileN - 1) / kTcTileN + 1) / 2, blocks = (T + 127) / 128;
    int splits = model().sm_count / (pairs * blocks);
    if (splits > kConvSplits) splits = kConvSplits;
    if (splits > cv.Kpad / kTcBlockK) splits = cv.Kpad / kTcBlockK;
    if (splits < 1) splits = 1;
    TcGemm g;
    g.M = T; g.splits = splits; g.epi = TC_EPI_PARTIAL; g.ld_out = cv.N; g.status = &model().d_out->status;
    g.out = c.part;
    if (tc_gemm(cv.hi, acts, g, st)) return -1;
    g.out = c.part + (size_t)splits * T * cv.N;
    if (tc_gemm(cv.lo, acts, g, st)) return -1;
    tc_reduce(out, c.part, 2 * splits, (size_t)T * cv.N, (size_t)T * cv.N, cv.bias, cv.N, st);
    return 0;
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
    rc |= conv_setup(&c.in_conv, ic, stage, &c.allocs, st);
    rc |= conv_setup(&c.out_conv, oc, stage, &c.allocs, st);
    for (int s = 0; s < CSTAGES - 1 && !rc; s++) rc |= conv_setup(&c.up_conv[s], w->stage_convs[s], stage, &c.allocs, st);
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

/* One block of at most kTcMaxRows / 8 frames: the samples of frames [skip, n_frames) go to
 * samples_out. */
static int decode_block(const int *codes, int n_frames, int skip, float *samples_out, float *ms) {
    Model &m = model();
    Codec &c = g_codec;
    if (8 * n_frames > kTcMaxRows || skip < 0 || skip >= n_frames) return -1;
    const size_t total = (size_t)(n_frames - skip) * 8 * CPATCH;
    if (ensure_buffers(n_frames)) return -1;
    cudaStream_t st = m.st;
    if (cudaMemcpyAsync(c.codes, codes, sizeof(int) * (size_t)n_frames * CCODES, cudaMemcpyHostToDevice, st) != cudaSuccess)
        return -1;
    cudaEventRecord(c.e0, st);
    launch_pdl(codec_embed_kernel, dim3(n_frames), dim3(320), 0, st, c.emb, c.codes, c.sem);
    int rows = n_frames;
    if (conv_run(c.in_conv, c.aIn, c.emb, CEMB, rows, c.x, st)) return -1;
    int l = 0;
    for (int stage = 0; stage < CSTAGES; stage++) {
        const float *y_prev = nullptr, *sc_prev = nullptr;
        for (int i = 0; i < 2; i++, l++) {
            if (layer_forward(c.L[l], rows, y_prev, sc_prev, st)) return -1;
            y_prev = c.y;
            sc_prev = c.L[l].ffn_scale;
        }
        /* the stage's last FFN update, no terms */
        launch_pdl(codec_prepare_kernel, dim3(1, rows), dim3(256), 0, st, nullptr, c.rows_pad, CD, c.x, y_prev, sc_prev, c.x, nullptr,
                                                            nullptr);
        if (stage < CSTAGES - 1) {
            /* [rows][2 x 1024] row-major = [2 rows][1024] */
            if (conv_run(c.up_conv[stage], c.aUp, c.x, CD, rows, c.x2, st)) return -1;
            float *t = c.x; c.x = c.x2; c.x2 = t;
            rows *= 2;
        }
    }
    if (conv_run(c.out_conv, c.aOut, c.x, CD, rows, c.pcm, st)) return -1;
    cudaEventRecord(c.e1, st);
    int status = 0;
    if (cudaMemcpyAsync(samples_out, c.pcm + (size_t)skip * 8 * CPATCH, sizeof(float) * total, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaMemcpyAsync(&status, &m.d_out->status, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    float t = 0.0f;
    cudaEventElapsedTime(&t, c.e0, c.e1);
    *ms += t;
    m.last_status = status;
    if (status) {
        cudaMemset(&m.d_out->status, 0, sizeof(int));
        return -1;
    }
    return 0;
}


/* The decoder only looks back: 2 frames in the input convolution, (window - 1) positions per
 * transformer layer at its stage's rate (2 + 3 + 3.5 + 3.75 frames), one position per transposed
 * convolution, 6/8 of a frame in the output convolution - under 17 frames in all. An utterance
 * longer than one block is therefore decoded block by block with 32 frames of left context whose
 * samples are dropped; what is kept equals the one-piece decode. */
constexpr int kCodecContext = 32;

int codec_set_block_frames(int frames) {
    if (frames < 2 * kCodecContext || frames > kTcMaxRows / 8) return -1;
    g_block_frames = frames;
    return 0;
}

int codec_decode(const int *codes, int n_frames, float *samples_out, int max_samples, int *n_samples) {
    Model &m = model();
    Codec &c = g_codec;
    if (n_samples) *n_samples = 0;
    if (!m.inited || !c.ready || !codes || n_frames < 1 || !samples_out) return -1;
    const long long total = (long long)n_frames * 8 * CPATCH;
    if (total > max_samples) return -1;
    const int block = g_block_frames > 0 ? g_block_frames : kTcMaxRows / 8;
    float ms = 0.0f;
    int pos = n_frames < block ? n_frames : block;
    if (decode_block(codes, pos, 0, samples_out, &ms)) return -1;
    while (pos < n_frames) {
        const int start = pos - kCodecContext;
        const int len = n_frames - start < block ? n_frames - start : block;
        if (decode_block(codes + (size_t)start * CCODES, len, kCodecContext, samples_out + (size_t)pos * 8 * CPATCH, &ms)) return -1;
        pos = start + len;
    }
    c.last_ms = ms;
    if (n_samples) *n_samples = (int)total;
    return 0;
}

float codec_last_ms() { return g_codec.last_ms; }

} // namespace vb
