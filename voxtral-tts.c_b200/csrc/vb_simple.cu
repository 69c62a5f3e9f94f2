/*
 * vb_simple.cu - stand-alone kernels behind the reference's single-op entry
 * points (voxtral_tts_cuda.h:118-154) and the multi-token (prefill) attention.
 * They are small, launch-bound ops; the frame kernel (vb_engine.cu) fuses their
 * work into its phases and does not call these.
 */
#include "vb_simple.cuh"
#include "vb_common.cuh"

namespace vb {

/* out[r,:] = x[r,:] * 1/sqrt(mean(x[r,:]^2)+eps) * w   (voxtral_tts_kernels.c:333-349) */
__global__ void rms_norm_kernel(float *out, const float *x, const float *w, int dim, float eps) {
    __shared__ float red[32];
    const float *xr = x + (size_t)blockIdx.x * dim;
    float *orow = out + (size_t)blockIdx.x * dim;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) { const float v = xr[i]; ss += v * v; }
    ss = vb_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float t = 0.0f;
    for (int wi = 0; wi < (int)(blockDim.x >> 5); wi++) t += red[wi];
    const float inv = 1.0f / sqrtf(t / (float)dim + eps);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) orow[i] = xr[i] * inv * w[i];
}

void rms_norm(float *out, const float *x, const float *w, int rows, int dim, float eps, cudaStream_t st) {
    if (rows <= 0 || dim <= 0) return;
    rms_norm_kernel<<<rows, 512, 0, st>>>(out, x, w, dim, eps);
}

/* gate = gate/(1+exp(-gate)) * up   (voxtral_tts_kernels.c:361-366, :29-31) */
__global__ void silu_mul_kernel(float *gate, const float *up, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float g = gate[i];
        gate[i] = (g / (1.0f + expf(-g))) * up[i];
    }
}
void silu_mul(float *gate, const float *up, int n, cudaStream_t st) {
    if (n <= 0) return;
    silu_mul_kernel<<<(n + 255) / 256, 256, 0, st>>>(gate, up, n);
}

/* a += b   (voxtral_tts_kernels.c:25-27) */
__global__ void add_kernel(float *a, const float *b, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] += b[i];
}
void add_inplace(float *a, const float *b, int n, cudaStream_t st) {
    if (n <= 0) return;
    add_kernel<<<(n + 255) / 256, 256, 0, st>>>(a, b, n);
}

/* (cos, sin) table for positions start..start+seq-1   (voxtral_tts_kernels.c:602-614) */
__global__ void rope_table_kernel(float *cs, int start, int seq, int head_dim, float theta) {
    const int half = head_dim / 2;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= seq * half) return;
    const int s = i / half, d = i % half;
    const float freq = 1.0f / powf(theta, (float)(2 * d) / (float)head_dim);
    const float ang = (float)(start + s) * freq;
    cs[2 * i] = cosf(ang);
    cs[2 * i + 1] = sinf(ang);
}
void rope_table(float *cs, int start, int seq, int head_dim, float theta, cudaStream_t st) {
    const int n = seq * (head_dim / 2);
    if (n <= 0) return;
    rope_table_kernel<<<(n + 255) / 256, 256, 0, st>>>(cs, start, seq, head_dim, theta);
}

/* rotate interleaved pairs with a table   (voxtral_tts_kernels.c:616-634) */
__global__ void rope_apply_kernel(float *x, const float *cs, int seq, int heads, int head_dim, int ld) {
    const int half = head_dim / 2;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= seq * heads * half) return;
    const int d = i % half, h = (i / half) % heads, s = i / (half * heads);
    float *v = x + (size_t)s * ld + h * head_dim + 2 * d;
    const float c = cs[((size_t)s * half + d) * 2], sn = cs[((size_t)s * half + d) * 2 + 1];
    const float a = v[0], b = v[1];
    v[0] = a * c - b * sn;
    v[1] = a * sn + b * c;
}
void rope_apply(float *x, const float *cs, int seq, int heads, int head_dim, int ld, cudaStream_t st) {
    const int n = seq * heads * (head_dim / 2);
    if (n <= 0) return;
    rope_apply_kernel<<<(n + 255) / 256, 256, 0, st>>>(x, cs, seq, heads, head_dim, ld);
}

/* out = BF16 row -> fp32   (voxtral_tts_kernels.c:55-59) */
__global__ void embed_rows_kernel(float *out, const uint16_t *table, const int *ids, int id0, int dim) {
    const int row = ids ? ids[blockIdx.y] : id0;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < dim) out[(size_t)blockIdx.y * dim + i] = __uint_as_float((uint32_t)table[(size_t)row * dim + i] << 16);
}
void embed_token(float *out, const uint16_t *table, int id, int dim, cudaStream_t st) {
    embed_rows_kernel<<<dim3((dim + 255) / 256, 1), 256, 0, st>>>(out, table, nullptr, id, dim);
}
void embed_rows(float *out, const uint16_t *table, const int *ids, int n, int dim, cudaStream_t st) {
    if (n <= 0) return;
    embed_rows_kernel<<<dim3((dim + 255) / 256, n), 256, 0, st>>>(out, table, ids, 0, dim);
}

/*
 * Attention of query rows against cached keys with the streaming softmax of
 * tts_causal_attention / tts_bidirectional_attention
 * (voxtral_tts_kernels.c:403-525). One warp per (query row, head); lane l owns
 * dims l, l+32, ... of the head. Keys 0..limit-1 where limit =
 * min(q_offset + row + 1, seq_k) when causal, seq_k otherwise.
 */
template <int DPL> /* dims per lane = head_dim / 32 */
__global__ void attention_rows_kernel(float *out, const float *Q, const float *K, const float *V,
                                      int seq_q, int seq_k, int n_heads, int n_kv_heads, float scale,
                                      int q_offset, int causal, int ldq, int ldk, int ldo) {
    const int head_dim = DPL * 32;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= seq_q * n_heads) return;
    const int row = warp / n_heads, h = warp % n_heads;
    const int kvh = h / (n_heads / n_kv_heads);
    int limit = seq_k;
    if (causal) { limit = q_offset + row + 1; if (limit > seq_k) limit = seq_k; }
    float q[DPL], o[DPL];
#pragma unroll
    for (int i = 0; i < DPL; i++) { q[i] = Q[(size_t)row * ldq + h * head_dim + lane + 32 * i]; o[i] = 0.0f; }
    float mx = -1e30f, den = 0.0f;
    /* four keys per pass: their loads and the four warp reductions overlap; the running
     * maximum then takes the keys in order, as the reference does */
    for (int jb = 0; jb < limit; jb += 4) {
        float kq[4][DPL], vq[4][DPL], dq[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int j = jb + u < limit ? jb + u : limit - 1;
            const float *kr = K + (size_t)j * ldk + kvh * head_dim;
            const float *vr = V + (size_t)j * ldk + kvh * head_dim;
#pragma unroll
            for (int i = 0; i < DPL; i++) { kq[u][i] = kr[lane + 32 * i]; vq[u][i] = vr[lane + 32 * i]; }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            float d = 0.0f;
#pragma unroll
            for (int i = 0; i < DPL; i++) d += q[i] * kq[u][i];
            dq[u] = d;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
            for (int u = 0; u < 4; u++) dq[u] += __shfl_xor_sync(0xffffffffu, dq[u], off);
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            if (jb + u >= limit) break;
            const float d = dq[u] * scale;
            if (d > mx) {
                const float corr = expf(mx - d);
                den = den * corr + 1.0f;
#pragma unroll
                for (int i = 0; i < DPL; i++) o[i] = o[i] * corr + vq[u][i];
                mx = d;
            } else {
                const float w = expf(d - mx);
                den += w;
#pragma unroll
                for (int i = 0; i < DPL; i++) o[i] += w * vq[u][i];
            }
        }
    }
    const float inv = den > 0.0f ? 1.0f / den : 0.0f;
#pragma unroll
    for (int i = 0; i < DPL; i++) out[(size_t)row * ldo + h * head_dim + lane + 32 * i] = o[i] * inv;
}

int attention_rows(float *out, const float *Q, const float *K, const float *V, int seq_q, int seq_k,
                   int n_heads, int n_kv_heads, int head_dim, float scale, int q_offset, int causal,
                   int ldq, int ldk, int ldo, cudaStream_t st) {
    if (seq_q <= 0 || n_heads <= 0) return 0;
    if (head_dim % 32 != 0 || head_dim > 256 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return -1;
    const int warps = seq_q * n_heads;
    const int threads = 256, blocks = (warps * 32 + threads - 1) / threads;
#define VB_ATTN_CASE(D)                                                                                   \
    case D:                                                                                               \
        attention_rows_kernel<D><<<blocks, threads, 0, st>>>(out, Q, K, V, seq_q, seq_k, n_heads,          \
                                                             n_kv_heads, scale, q_offset, causal, ldq,    \
                                                             ldk, ldo);                                   \
        break;
    switch (head_dim / 32) {
        VB_ATTN_CASE(1) VB_ATTN_CASE(2) VB_ATTN_CASE(3) VB_ATTN_CASE(4)
        VB_ATTN_CASE(5) VB_ATTN_CASE(6) VB_ATTN_CASE(7) VB_ATTN_CASE(8)
    default: return -1;
    }
#undef VB_ATTN_CASE
    return 0;
}

/* y[m,n] = sum_k x[m,k] * W[n,k] (+bias) for shapes the streaming engine does not
 * take (K not a multiple of 8). One warp per output element. */
__global__ void linear_generic_kernel(float *y, const float *x, const uint16_t *W, const float *bias,
                                      int M, int K, int N) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= M * N) return;
    const int m = warp / N, n = warp % N;
    float acc = 0.0f;
    for (int k = lane; k < K; k += 32)
        acc = fmaf(__uint_as_float((uint32_t)W[(size_t)n * K + k] << 16), x[(size_t)m * K + k], acc);
    acc = vb_warp_sum(acc);
    if (lane == 0) y[(size_t)m * N + n] = acc + (bias ? bias[n] : 0.0f);
}
void linear_generic(float *y, const float *x, const uint16_t *W, const float *bias, int M, int K, int N,
                    cudaStream_t st) {
    const long long warps = (long long)M * N;
    if (warps <= 0) return;
    const int threads = 256;
    const int blocks = (int)((warps * 32 + threads - 1) / threads);
    linear_generic_kernel<<<blocks, threads, 0, st>>>(y, x, W, bias, M, K, N);
}

/* dst rows 2i / 2i+1 <- gate row i / up row i: the SwiGLU pair layout the engine
 * streams (both halves of a pair land in the same chunk). */
__global__ void interleave_rows_kernel(uint4 *dst, const uint4 *a, const uint4 *b, int rows, int row_vec) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)rows * row_vec;
    if (i >= total) return;
    const size_t r = i / row_vec, c = i % row_vec;
    dst[(2 * r) * row_vec + c] = a[i];
    dst[(2 * r + 1) * row_vec + c] = b[i];
}
void interleave_rows(uint16_t *dst, const uint16_t *a, const uint16_t *b, int rows, int cols, cudaStream_t st) {
    const int row_vec = cols / 8;
    const size_t total = (size_t)rows * row_vec;
    if (total == 0) return;
    interleave_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((uint4 *)dst, (const uint4 *)a,
                                                                           (const uint4 *)b, rows, row_vec);
}

} // namespace vb
