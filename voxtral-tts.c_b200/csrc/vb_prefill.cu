/*
 * vb_prefill.cu - multi-token prefill of the decoder on the GPU
 * (tts_llm_prefill, voxtral_tts_llm.c:277-373): all prompt rows go through the
 * 26 layers, K and V of every row land in the cache, hidden states are dropped.
 *
 * The linears run on the tensor-core GEMM (vb_tc.cu; fp32 rows as three BF16 terms) in
 * blocks of up to 256 rows; RoPE, the cache write and the causal attention use the
 * stand-alone kernels. When the tensor maps cannot be made the same layer loop runs
 * on the streaming engine, eight rows at a time. Also here: the prompt assembled on
 * the device from token ids and BF16 voice rows (voxtral_tts.c:230-272).
 */
#include "vb_common.cuh"
#include "vb_model.cuh"
#include "vb_simple.cuh"
#include "vb_tc.cuh"

#include <math.h>
#include <stdio.h>
#include <string.h>
#include <vector>

namespace vb {

static const int D = VB200_DIM, QD = VB200_Q_DIM, KVD = VB200_KV_DIM, HID = VB200_HIDDEN;
static const int QKV = QD + 2 * KVD;

/* Runs `op` once per block of up to 8 rows; blocks are independent, so a launch
 * carries up to 64 of them without grid barriers in between. */
static int run_row_blocks(VbOp proto, int M, int x_ld, int y_ld, bool res_is_y) {
    std::vector<VbOp> ops;
    const float *x0 = proto.x;
    float *y0 = proto.y;
    for (int r = 0; r < M; r += kMaxM) {
        VbOp o = proto;
        o.M = (M - r < kMaxM) ? M - r : kMaxM;
        o.x = x0 + (size_t)r * x_ld;
        o.y = y0 + (size_t)r * y_ld;
        if (res_is_y) o.res = o.y;
        o.flags |= VB_F_NOSYNC;
        ops.push_back(o);
        if (ops.size() == 64) {
            if (run_ops(ops)) return -1;
            ops.clear();
        }
    }
    if (!ops.empty() && run_ops(ops)) return -1;
    return 0;
}

/* ---- glue kernels of the tensor-core prefill ---- */

/* QKV of a row block: sums the split-K partials in fixed order, rotates the q and k heads
 * (interleaved pairs, voxtral_tts_kernels.c:616-634), leaves q in `qkv` for the attention
 * and writes k and v straight into the cache rows (voxtral_tts_llm.c:318-330). One thread per
 * pair of columns. */
__global__ void pf_qkv_finish_kernel(float *qkv, const float *part, int n_part, size_t part_stride, const float *cs,
                                     float *k_rows, float *v_rows, int rows) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.y;
    const int col = 2 * (blockIdx.x * blockDim.x + threadIdx.x);
    if (col >= QKV || m >= rows) return;
    float2 v = make_float2(0.0f, 0.0f);
    for (int p = 0; p < n_part; p++) {
        const float2 t = __ldcg(reinterpret_cast<const float2 *>(part + (size_t)p * part_stride + (size_t)m * QKV + col));
        v.x += t.x; v.y += t.y;
    }
    if (col < QD + KVD) {
        const int d = (col % VB200_HEAD_DIM) >> 1;
        const float2 t = *reinterpret_cast<const float2 *>(cs + ((size_t)m * (VB200_HEAD_DIM / 2) + d) * 2);
        const float a = v.x, b = v.y;
        v.x = a * t.x - b * t.y;
        v.y = a * t.y + b * t.x;
    }
    if (col < QD) *reinterpret_cast<float2 *>(qkv + (size_t)m * QKV + col) = v;
    else if (col < QD + KVD) *reinterpret_cast<float2 *>(k_rows + (size_t)m * KVD + (col - QD)) = v;
    else *reinterpret_cast<float2 *>(v_rows + (size_t)m * KVD + (col - QD - KVD)) = v;
}

/* Causal attention of a block of prompt rows over the cache prefix (tts_causal_attention,
 * voxtral_tts_kernels.c:403-465) on the warp-level tensor cores; head_dim 128, four query heads
 * per KV head. A CTA owns one KV head and 16 query rows; warps w and w + 4 serve query head 4 g + w
 * on the first and on the second 16 keys of every 32-key tile (two partial softmax states merged at
 * the end), so the K and V rows are staged in shared memory once per KV head, 32 keys at a time, and
 * every SM sub-core has two warps' worth of independent MMAs to issue.
 *
 * fp32 accuracy from BF16 MMAs: every fp32 operand is split into hi + lo BF16 halves and a
 * product a.b is taken as a_hi.b_hi + a_hi.b_lo + a_lo.b_hi (the dropped lo.lo term is 2^-16 of
 * the product). Per 32-key tile a warp issues, with mma.sync.m16n8k16, for its 16 keys:
 *   S[16 x 16]  = Q[16 x 128] . K^T     2 key tiles x 8 k-steps x 3 products
 *   O[16 x 128] += P[16 x 16] . V      16 dim tiles x 1 k-step x 3 products
 * Q lives in registers as A fragments (scaled by 1/sqrt(128) before the split); K rows [key][dim]
 * are the "column-major" B operand of Q.K^T (ldmatrix), V rows [key][dim] the row-major B operand
 * of P.V (ldmatrix.trans); both sit in shared memory as BF16 with the 16-byte chunks of a row
 * XOR-swizzled by the key index. The running maximum / sum update is the usual one per tile;
 * S's accumulator fragments become P's A fragments without leaving registers. Row blocks are
 * issued heaviest (latest rows) first. */
constexpr int kFaRows = 16, kFaKeys = 32, kFaThreads = 256;

VB_DEVINL void fa_split(float v, uint32_t &hi, uint32_t &lo) {
    uint16_t a, b, c;
    vb_split3(v, a, b, c);
    hi = a;
    lo = b;
}
VB_DEVINL void fa_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
VB_DEVINL void fa_ldsm(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
VB_DEVINL void fa_ldsm_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
/* byte offset of 16-byte chunk `chunk` (0..15) of key row `key` in a [32][128] BF16 tile */
VB_DEVINL uint32_t fa_off(int key, int chunk) { return (uint32_t)(key * 256 + (((chunk & 8) | ((chunk ^ key) & 7)) << 4)); }

__global__ void __launch_bounds__(kFaThreads)
pf_attention_kernel(float *out, const float *q, const float *kc, const float *vc, int M, int start_pos, int ldq,
                    int ldkv, int ldo, float scale) {
    __shared__ __align__(128) unsigned char tiles[4 * kFaKeys * 256];   /* K hi, K lo, V hi, V lo; reused by the final merge */
    __shared__ float ml[4][32][4];                                      /* second half's (mA, mB, lA, lB) per head and lane */
    unsigned char *Kh = tiles, *Kl = tiles + kFaKeys * 256, *Vh = tiles + 2 * kFaKeys * 256, *Vl = tiles + 3 * kFaKeys * 256;
    pdl_launch_dependents();
    pdl_wait();
    const int g = blockIdx.y, r0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * kFaRows;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
    const int hw = warp & 3, half = warp >> 2;   /* head of the group; which 16 keys of every 32-key tile */
    const int h = g * 4 + hw;
    const int rowA = r0 + gq, rowB = rowA + 8;
    const bool validA = rowA < M, validB = rowB < M;
    const int limA = validA ? start_pos + rowA : 0, limB = validB ? start_pos + rowB : 0;   /* last key a row sees */
    const int rows_here = M - r0 < kFaRows ? M - r0 : kFaRows;
    const int n_keys = start_pos + r0 + rows_here;

    /* Q as A fragments: a0 (row A, k 2t..), a1 (row B, k 2t..), a2 (row A, k 8+2t..), a3 (row B, k 8+2t..) */
    uint32_t qh[8][4], ql[8][4];
#pragma unroll
    for (int ks = 0; ks < 8; ks++) {
#pragma unroll
        for (int half = 0; half < 2; half++) {
#pragma unroll
            for (int rr = 0; rr < 2; rr++) {
                const int row = rr ? rowB : rowA;
                float2 v = make_float2(0.f, 0.f);
                if (rr ? validB : validA)
                    v = *reinterpret_cast<const float2 *>(q + (size_t)row * ldq + h * VB200_HEAD_DIM + ks * 16 + half * 8 + 2 * tq);
                uint32_t h0, l0, h1, l1;
                fa_split(v.x * scale, h0, l0);
                fa_split(v.y * scale, h1, l1);
                qh[ks][half * 2 + rr] = h0 | (h1 << 16);
                ql[ks][half * 2 + rr] = l0 | (l1 << 16);
            }
        }
    }
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float mA = -1e30f, mB = -1e30f, lA = 0.0f, lB = 0.0f;
    const uint32_t sKh = vb_smem_u32(Kh), sKl = vb_smem_u32(Kl), sVh = vb_smem_u32(Vh), sVl = vb_smem_u32(Vl);
    const int mat = lane >> 3, mr = lane & 7;

    for (int k0 = 0; k0 < n_keys; k0 += kFaKeys) {
        __syncthreads();
        /* stage 32 keys of K and V: fp32 -> hi / lo BF16, 4 values (8 bytes) per piece */
        for (int i = tid; i < kFaKeys * 32; i += kFaThreads) {
            const int key = i >> 5, f = i & 31, kk = k0 + key;
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
            if (kk < n_keys) {
                a = __ldg(reinterpret_cast<const float4 *>(kc + (size_t)kk * ldkv + g * VB200_HEAD_DIM) + f);
                b = __ldg(reinterpret_cast<const float4 *>(vc + (size_t)kk * ldkv + g * VB200_HEAD_DIM) + f);
            }
            const float ea[4] = {a.x, a.y, a.z, a.w}, eb[4] = {b.x, b.y, b.z, b.w};
            uint32_t ah[4], al[4], bh[4], bl[4];
#pragma unroll
            for (int j = 0; j < 4; j++) { fa_split(ea[j], ah[j], al[j]); fa_split(eb[j], bh[j], bl[j]); }
            const uint32_t off = fa_off(key, f >> 1) + (uint32_t)(f & 1) * 8u;
            *reinterpret_cast<uint2 *>(Kh + off) = make_uint2(ah[0] | (ah[1] << 16), ah[2] | (ah[3] << 16));
            *reinterpret_cast<uint2 *>(Kl + off) = make_uint2(al[0] | (al[1] << 16), al[2] | (al[3] << 16));
            *reinterpret_cast<uint2 *>(Vh + off) = make_uint2(bh[0] | (bh[1] << 16), bh[2] | (bh[3] << 16));
            *reinterpret_cast<uint2 *>(Vl + off) = make_uint2(bl[0] | (bl[1] << 16), bl[2] | (bl[3] << 16));
        }
        __syncthreads();

        /* S = Q . K^T for this warp's 2 tiles of 8 keys */
        float s[2][4];
#pragma unroll
        for (int i = 0; i < 2; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            /* matrices: (keys half*16.., dims ks*16..), (same keys, dims +8), (keys +8, dims), (keys +8, dims +8) */
            const uint32_t off = fa_off(half * 16 + (mat >> 1) * 8 + mr, ks * 2 + (mat & 1));
            uint32_t bh[4], bl[4];
            fa_ldsm(bh, sKh + off);
            fa_ldsm(bl, sKl + off);
            fa_mma(s[0], qh[ks], bh[0], bh[1]);
            fa_mma(s[1], qh[ks], bh[2], bh[3]);
            fa_mma(s[0], qh[ks], bl[0], bl[1]);
            fa_mma(s[1], qh[ks], bl[2], bl[3]);
            fa_mma(s[0], ql[ks], bh[0], bh[1]);
            fa_mma(s[1], ql[ks], bh[2], bh[3]);
        }
        /* causal mask, running maximum and sum (rows A and B of this thread's quad) */
        float tmA = -1e30f, tmB = -1e30f;
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int key = k0 + half * 16 + nt * 8 + 2 * tq + (c & 1);
                if (key > (c < 2 ? limA : limB)) s[nt][c] = -1e30f;
            }
            tmA = fmaxf(tmA, fmaxf(s[nt][0], s[nt][1]));
            tmB = fmaxf(tmB, fmaxf(s[nt][2], s[nt][3]));
        }
        tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 1));
        tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 2));
        tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 1));
        tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 2));
        const float nA = fmaxf(mA, tmA), nB = fmaxf(mB, tmB);
        const float cA = expf(mA - nA), cB = expf(mB - nB);
        mA = nA; mB = nB;
        float sumA = 0.0f, sumB = 0.0f;
        uint32_t ph[4], pl[4];
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            float p[4];
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int key = k0 + half * 16 + nt * 8 + 2 * tq + (c & 1);
                p[c] = key > (c < 2 ? limA : limB) ? 0.0f : expf(s[nt][c] - (c < 2 ? nA : nB));
            }
            sumA += p[0] + p[1];
            sumB += p[2] + p[3];
            /* accumulator layout of key tile nt -> A fragment of the one k-step:
             * first tile: a0 (row A), a1 (row B); second tile: a2 (row A), a3 (row B) */
            uint32_t h0, l0, h1, l1;
            fa_split(p[0], h0, l0); fa_split(p[1], h1, l1);
            ph[nt * 2] = h0 | (h1 << 16);
            pl[nt * 2] = l0 | (l1 << 16);
            fa_split(p[2], h0, l0); fa_split(p[3], h1, l1);
            ph[nt * 2 + 1] = h0 | (h1 << 16);
            pl[nt * 2 + 1] = l0 | (l1 << 16);
        }
        lA = lA * cA + sumA;
        lB = lB * cB + sumB;
#pragma unroll
        for (int i = 0; i < 16; i++) { o[i][0] *= cA; o[i][1] *= cA; o[i][2] *= cB; o[i][3] *= cB; }
        /* O += P . V over this warp's 16 keys */
#pragma unroll
        for (int dp = 0; dp < 8; dp++) {
            /* matrices: (keys half*16.., dims dp*16..), (keys +8, dims), (keys, dims +8), (keys +8, dims +8) */
            const uint32_t off = fa_off(half * 16 + (mat & 1) * 8 + mr, dp * 2 + (mat >> 1));
            uint32_t vh[4], vl[4];
            fa_ldsm_t(vh, sVh + off);
            fa_ldsm_t(vl, sVl + off);
            fa_mma(o[2 * dp], ph, vh[0], vh[1]);
            fa_mma(o[2 * dp + 1], ph, vh[2], vh[3]);
            fa_mma(o[2 * dp], ph, vl[0], vl[1]);
            fa_mma(o[2 * dp + 1], ph, vl[2], vl[3]);
            fa_mma(o[2 * dp], pl, vh[0], vh[1]);
            fa_mma(o[2 * dp + 1], pl, vh[2], vh[3]);
        }
    }
    lA += __shfl_xor_sync(0xffffffffu, lA, 1);
    lA += __shfl_xor_sync(0xffffffffu, lA, 2);
    lB += __shfl_xor_sync(0xffffffffu, lB, 1);
    lB += __shfl_xor_sync(0xffffffffu, lB, 2);
    /* merge the two key halves of every head: the second half hands its (max, sum, O) over through
     * the tile memory, the first half combines them with the usual log-sum-exp weights */
    __syncthreads();
    float *xo = reinterpret_cast<float *>(tiles);                 /* [head][64 values][32 lanes] */
    if (half == 1) {
#pragma unroll
        for (int i = 0; i < 16; i++)
#pragma unroll
            for (int c = 0; c < 4; c++) xo[(hw * 64 + i * 4 + c) * 32 + lane] = o[i][c];
        ml[hw][lane][0] = mA; ml[hw][lane][1] = mB; ml[hw][lane][2] = lA; ml[hw][lane][3] = lB;
    }
    __syncthreads();
    if (half == 1) return;
    {
        const float m2A = ml[hw][lane][0], m2B = ml[hw][lane][1], l2A = ml[hw][lane][2], l2B = ml[hw][lane][3];
        const float MA = fmaxf(mA, m2A), MB = fmaxf(mB, m2B);
        const float w1A = expf(mA - MA), w2A = l2A > 0.0f ? expf(m2A - MA) : 0.0f;
        const float w1B = expf(mB - MB), w2B = l2B > 0.0f ? expf(m2B - MB) : 0.0f;
        lA = lA * w1A + l2A * w2A;
        lB = lB * w1B + l2B * w2B;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            o[i][0] = o[i][0] * w1A + xo[(hw * 64 + i * 4 + 0) * 32 + lane] * w2A;
            o[i][1] = o[i][1] * w1A + xo[(hw * 64 + i * 4 + 1) * 32 + lane] * w2A;
            o[i][2] = o[i][2] * w1B + xo[(hw * 64 + i * 4 + 2) * 32 + lane] * w2B;
            o[i][3] = o[i][3] * w1B + xo[(hw * 64 + i * 4 + 3) * 32 + lane] * w2B;
        }
    }
    const float iA = lA > 0.0f ? 1.0f / lA : 0.0f, iB = lB > 0.0f ? 1.0f / lB : 0.0f;
#pragma unroll
    for (int nt = 0; nt < 16; nt++) {
        const int d = nt * 8 + 2 * tq;
        if (validA) *reinterpret_cast<float2 *>(out + (size_t)rowA * ldo + h * VB200_HEAD_DIM + d) = make_float2(o[nt][0] * iA, o[nt][1] * iA);
        if (validB) *reinterpret_cast<float2 *>(out + (size_t)rowB * ldo + h * VB200_HEAD_DIM + d) = make_float2(o[nt][2] * iB, o[nt][3] * iB);
    }
}

/* ---- tensor-core prefill ---- */
struct PrefillTc {
    bool ready = false;
    /* the decoder's tile-contiguous matrices (shared with the frame graph), fetched per call */
    const TcWeight *wqkv = nullptr, *wo = nullptr, *w13 = nullptr, *w2 = nullptr;
    uint16_t *bD = nullptr, *bQ = nullptr, *bH = nullptr;
    float *part = nullptr, *ssq = nullptr;
    TcActs aD[3], aQ[3], aH[3];   /* for 16, 64 and 256 padded rows, over the same buffers */
    /* row buffers of a prefill call, kept between calls and only ever grown (allocating and
     * freeing them per call cost up to 10 ms of a 7.6 ms prefill) */
    float *x = nullptr, *qkv = nullptr, *attn = nullptr, *h = nullptr, *cs = nullptr;
    int cap_rows = 0;
};
static PrefillTc g_pf;

/* Called when the device context goes away: everything here pointed into it. */
void prefill_free_all() {
    PrefillTc &t = g_pf;
    cudaFree(t.x); cudaFree(t.qkv); cudaFree(t.attn); cudaFree(t.h); cudaFree(t.cs);
    t = PrefillTc();
}

static int prefill_rows(int M) {
    PrefillTc &t = g_pf;
    if (M <= t.cap_rows) return 0;
    cudaFree(t.x); cudaFree(t.qkv); cudaFree(t.attn); cudaFree(t.h); cudaFree(t.cs);
    t.x = t.qkv = t.attn = t.h = t.cs = nullptr;
    t.cap_rows = 0;
    const int cap = (M + 255) / 256 * 256;
    if (cudaMalloc((void **)&t.x, (size_t)cap * D * 4) != cudaSuccess || cudaMalloc((void **)&t.qkv, (size_t)cap * QKV * 4) != cudaSuccess ||
        cudaMalloc((void **)&t.attn, (size_t)cap * QD * 4) != cudaSuccess || cudaMalloc((void **)&t.h, (size_t)cap * HID * 4) != cudaSuccess ||
        cudaMalloc((void **)&t.cs, (size_t)cap * VB200_HEAD_DIM * 4) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(t.x); cudaFree(t.qkv); cudaFree(t.attn); cudaFree(t.h); cudaFree(t.cs);
        t.x = t.qkv = t.attn = t.h = t.cs = nullptr;
        return -1;
    }
    t.cap_rows = cap;
    return 0;
}
static const int kPfRows = 256;

static int pf_slot(int rows_pad) { return rows_pad == 16 ? 0 : rows_pad == 64 ? 1 : 2; }

/* The activation-term buffers and their tensor maps; called after the decoder upload. Failing here is not fatal: prefill() then uses the streaming kernel. */
int prefill_tc_setup() {
    Model &m = model();
    PrefillTc &t = g_pf;
    t.ready = false;
    if (getenv("VB200_NO_TC") || tc_init()) return 0;
    if (!t.bD) {
        void *p[5] = {};
        const size_t sz[5] = {tc_acts_bytes(kPfRows, D), tc_acts_bytes(kPfRows, QD), tc_acts_bytes(kPfRows, HID),
                              sizeof(float) * (size_t)kTcMaxSplits * kPfRows * QKV, sizeof(float) * kPfRows * 16};
        for (int i = 0; i < 5; i++) {
            if (cudaMalloc(&p[i], sz[i]) != cudaSuccess) return 0;
            m.allocs.push_back(p[i]);
            cudaMemset(p[i], 0, sz[i]);
        }
        t.bD = (uint16_t *)p[0]; t.bQ = (uint16_t *)p[1]; t.bH = (uint16_t *)p[2];
        t.part = (float *)p[3]; t.ssq = (float *)p[4];
    }
    const int pads[3] = {16, 64, 256};
    for (int i = 0; i < 3; i++)
        if (tc_acts(&t.aD[i], t.bD, pads[i], D) || tc_acts(&t.aQ[i], t.bQ, pads[i], QD) ||
            tc_acts(&t.aH[i], t.bH, pads[i], HID))
            return 0;
    t.ready = true;
    return 0;
}

/* Prefill with the tcgen05 GEMM (vb_tc.cu): per layer and per block of up to 256 rows
 * gain+terms -> QKV -> RoPE -> cache rows; causal attention over the whole cache prefix;
 * terms -> O -> residual+gain+terms -> gate/up with SwiGLU -> down -> residual. */
static int prefill_tc(float *x, float *qkv, float *attn, const float *cs, int M, int start_pos) {
    Model &m = model();
    PrefillTc &t = g_pf;
    cudaStream_t st = m.st;
    const float scale = 1.0f / sqrtf((float)VB200_HEAD_DIM);
    const int s_qkv = tc_pick_splits(QKV, D, m.sm_count), s_wo = tc_pick_splits(D, QD, m.sm_count),
              s_w2 = tc_pick_splits(D, HID, m.sm_count);
    const int chunksD = tc_prepare_chunks(D);
    for (int l = 0; l < VB200_DEC_LAYERS; l++) {
        const LayerDev &L = m.dec[l];
        for (int r0 = 0; r0 < M; r0 += kPfRows) {
            const int rows = M - r0 < kPfRows ? M - r0 : kPfRows;
            const int slot = pf_slot(tc_rows_pad(rows));
            float *xr = x + (size_t)r0 * D, *qr = qkv + (size_t)r0 * QKV;
            tc_prepare(t.aD[slot], xr, D, rows, nullptr, 0, 0, nullptr, nullptr, L.attn_norm, t.ssq, st);
            TcGemm g;
            g.M = rows; g.status = &m.d_out->status; g.epi = TC_EPI_PARTIAL; g.out = t.part; g.ld_out = QKV;
            g.splits = s_qkv; g.ssq = t.ssq; g.ssq_chunks = chunksD; g.eps = VB200_NORM_EPS;
            if (tc_gemm(t.wqkv[l], t.aD[slot], g, st)) return -1;
            float *ck = m.kv_k + ((size_t)l * m.kv_max + start_pos + r0) * KVD;
            float *cv = m.kv_v + ((size_t)l * m.kv_max + start_pos + r0) * KVD;
            launch_pdl(pf_qkv_finish_kernel, dim3(QKV / 2 / 256, rows), dim3(256), 0, st, qr, (const float *)t.part, s_qkv,
                       (size_t)rows * QKV, cs + (size_t)r0 * VB200_HEAD_DIM, ck, cv, rows);
        }
        const float *k0 = m.kv_k + (size_t)l * m.kv_max * KVD, *v0 = m.kv_v + (size_t)l * m.kv_max * KVD;
        launch_pdl(pf_attention_kernel, dim3((M + kFaRows - 1) / kFaRows, VB200_KV_HEADS), dim3(kFaThreads), 0, st, attn,
                   (const float *)qkv, k0, v0, M, start_pos, QKV, KVD, QD, scale);
        if (l == VB200_DEC_LAYERS - 1) break;   /* only the cache is kept (voxtral_tts_llm.c:281) */
        for (int r0 = 0; r0 < M; r0 += kPfRows) {
            const int rows = M - r0 < kPfRows ? M - r0 : kPfRows;
            const int rp = tc_rows_pad(rows), slot = pf_slot(rp);
            float *xr = x + (size_t)r0 * D;
            const size_t psD = (size_t)rows * D;
            tc_prepare(t.aQ[slot], attn + (size_t)r0 * QD, QD, rows, nullptr, 0, 0, nullptr, nullptr, nullptr, nullptr, st);
            TcGemm g;
            g.M = rows; g.status = &m.d_out->status; g.epi = TC_EPI_PARTIAL; g.out = t.part; g.ld_out = D;
            g.splits = s_wo;
            if (tc_gemm(t.wo[l], t.aQ[slot], g, st)) return -1;
            tc_prepare(t.aD[slot], nullptr, D, rows, t.part, s_wo, psD, xr, xr, L.ffn_norm, t.ssq, st);
            g.epi = TC_EPI_SWIGLU_TERMS; g.out = nullptr; g.out_terms = t.bH; g.out_rows_pad = rp; g.splits = 1;
            g.ld_out = HID; g.ssq = t.ssq; g.ssq_chunks = chunksD; g.eps = VB200_NORM_EPS;
            if (tc_gemm(t.w13[l], t.aD[slot], g, st)) return -1;
            g.epi = TC_EPI_PARTIAL; g.out = t.part; g.out_terms = nullptr; g.splits = s_w2; g.ld_out = D;
            g.ssq = nullptr; g.ssq_chunks = 0;
            if (tc_gemm(t.w2[l], t.aH[slot], g, st)) return -1;
            /* residual add (the terms it also writes are overwritten by the next layer's prepare) */
            tc_prepare(t.aD[slot], nullptr, D, rows, t.part, s_w2, psD, xr, xr, nullptr, nullptr, st);
        }
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int prefill(const float *embeds, int seq_len, int start_pos) {
    Model &m = model();
    if (!m.inited || !m.llm_ready) return -1;
    if (seq_len <= 0) return 0;
    if (start_pos < 0 || start_pos + seq_len > m.kv_max) {
        fprintf(stderr, "voxtral_b200: prefill of %d rows at %d exceeds the %d-row cache\n", seq_len, start_pos,
                m.kv_max);
        return -1;
    }
    const int M = seq_len;
    if (prefill_rows(M)) return -1;
    float *x = g_pf.x, *qkv = g_pf.qkv, *attn = g_pf.attn, *h = g_pf.h, *cs = g_pf.cs;
    int rc = 0;
    const float scale = 1.0f / sqrtf((float)VB200_HEAD_DIM);
    if (!rc && cudaMemcpyAsync(x, embeds, (size_t)M * D * 4, cudaMemcpyDefault, m.st) != cudaSuccess) rc = -1;
    if (!rc) rope_table(cs, start_pos, M, VB200_HEAD_DIM, VB200_ROPE_THETA, m.st);

    if (!rc && g_pf.ready && batch_tiled_decoder(&g_pf.wqkv, &g_pf.wo, &g_pf.w13, &g_pf.w2) == 0) {
        rc = prefill_tc(x, qkv, attn, cs, M, start_pos);
        if (cudaStreamSynchronize(m.st) != cudaSuccess) rc = -1;
        if (!rc) {
            int status = 0;
            cudaMemcpy(&status, &m.d_out->status, sizeof(int), cudaMemcpyDeviceToHost);
            m.last_status = status;
            if (status) {
                /* the word is sticky on the device (kernels only set it from 0): clear it so the
                 * next call starts clean */
                cudaMemset(&m.d_out->status, 0, sizeof(int));
                rc = -1;
            }
        }
        return rc;
    }
    for (int l = 0; l < VB200_DEC_LAYERS && !rc; l++) {
        const LayerDev &L = m.dec[l];
        float *ck = m.kv_k + ((size_t)l * m.kv_max + start_pos) * KVD;
        float *cv = m.kv_v + ((size_t)l * m.kv_max + start_pos) * KVD;

        VbOp o;
        memset(&o, 0, sizeof(o));
        o.type = VB_OP_GEMV; o.N = QKV; o.K = D; o.W = L.wqkv; o.x = x; o.ldx = D; o.y = qkv; o.ldy = QKV;
        o.epi = VB_EPI_STORE; o.norm_w = L.attn_norm; o.eps = VB200_NORM_EPS;
        rc = run_row_blocks(o, M, D, QKV, false);
        if (rc) break;

        rope_apply(qkv, cs, M, VB200_HEADS, VB200_HEAD_DIM, QKV, m.st);
        rope_apply(qkv + QD, cs, M, VB200_KV_HEADS, VB200_HEAD_DIM, QKV, m.st);
        if (cudaMemcpy2DAsync(ck, (size_t)KVD * 4, qkv + QD, (size_t)QKV * 4, (size_t)KVD * 4, M,
                              cudaMemcpyDeviceToDevice, m.st) != cudaSuccess ||
            cudaMemcpy2DAsync(cv, (size_t)KVD * 4, qkv + QD + KVD, (size_t)QKV * 4, (size_t)KVD * 4, M,
                              cudaMemcpyDeviceToDevice, m.st) != cudaSuccess) {
            rc = -1;
            break;
        }
        const float *k0 = m.kv_k + (size_t)l * m.kv_max * KVD;
        const float *v0 = m.kv_v + (size_t)l * m.kv_max * KVD;
        if (attention_rows(attn, qkv, k0, v0, M, start_pos + M, VB200_HEADS, VB200_KV_HEADS, VB200_HEAD_DIM,
                           scale, start_pos, 1, QKV, KVD, QD, m.st)) {
            rc = -1;
            break;
        }

        memset(&o, 0, sizeof(o));
        o.type = VB_OP_GEMV; o.N = D; o.K = QD; o.W = L.wo; o.x = attn; o.ldx = QD; o.y = x; o.ldy = D;
        o.epi = VB_EPI_ADD; o.eps = VB200_NORM_EPS;
        rc = run_row_blocks(o, M, QD, D, true);
        if (rc) break;

        memset(&o, 0, sizeof(o));
        o.type = VB_OP_GEMV; o.N = 2 * HID; o.K = D; o.W = L.w13; o.x = x; o.ldx = D; o.y = h; o.ldy = HID;
        o.epi = VB_EPI_SWIGLU; o.norm_w = L.ffn_norm; o.eps = VB200_NORM_EPS;
        rc = run_row_blocks(o, M, D, HID, false);
        if (rc) break;

        memset(&o, 0, sizeof(o));
        o.type = VB_OP_GEMV; o.N = D; o.K = HID; o.W = L.w2; o.x = h; o.ldx = HID; o.y = x; o.ldy = D;
        o.epi = VB_EPI_ADD; o.eps = VB200_NORM_EPS;
        rc = run_row_blocks(o, M, HID, D, true);
    }
    if (cudaStreamSynchronize(m.st) != cudaSuccess) rc = -1;
    if (!rc) {
        int status = 0;
        cudaMemcpy(&status, &m.d_out->status, sizeof(int), cudaMemcpyDeviceToHost);
        m.last_status = status;
        if (status) {
            cudaMemset(&m.d_out->status, 0, sizeof(int));
            cudaMemset(m.bar, 0, 16 * sizeof(unsigned));
            cudaMemset(m.exitc, 0, 16 * sizeof(unsigned));
            rc = -1;
        }
    }
    return rc;
}

/* ---- the prompt, assembled on the device ---- */
/* Row r of the prompt: a token-table row (ids[r] >= 0) or voice row -ids[r] - 1, BF16 -> fp32
 * (tts_embed_token_bf16, voxtral_tts_kernels.c:55-59; tts_voice_embed, voxtral_tts_voice.c:228-248). */
__global__ void prompt_rows_kernel(float *out, const uint16_t *table, const uint16_t *voice, const int *ids, int dim) {
    const int id = ids[blockIdx.y];
    const uint16_t *src = id >= 0 ? table + (size_t)id * dim : voice + (size_t)(-id - 1) * dim;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < dim) out[(size_t)blockIdx.y * dim + i] = __uint_as_float((uint32_t)src[i] << 16);
}

/* The prompt the orchestrator assembles on the host (voxtral_tts.c:230-272):
 *   [BOS=1] [BEGIN_AUDIO=25] voice rows [/INST=36] text tokens [INST=35] [BEGIN_AUDIO=25]
 * built on the device from the token table uploaded with the decoder weights and the BF16 voice
 * rows (host memory, [n_voice, 3072]), then prefilled from cache row start_pos. Only the token ids
 * and the BF16 voice rows cross PCIe (1.4 MB for 224 voice rows instead of 3 MB of fp32 rows, and
 * no BF16 -> fp32 pass on the host). Returns the number of prompt rows, or -1. */
int prefill_prompt(const int *text_ids, int n_text, const uint16_t *voice_bf16, int n_voice, int start_pos) {
    Model &m = model();
    if (!m.inited || !m.llm_ready || !m.tok_emb) {
        fprintf(stderr, "voxtral_b200: the prompt needs the decoder weights with the token table uploaded\n");
        return -1;
    }
    if (n_text < 0 || n_voice < 0 || (n_text > 0 && !text_ids) || (n_voice > 0 && !voice_bf16)) return -1;
    const int n = n_voice + n_text + 5;
    if (start_pos < 0 || start_pos + n > m.kv_max) {
        fprintf(stderr, "voxtral_b200: a prompt of %d rows at %d exceeds the %d-row cache\n", n, start_pos, m.kv_max);
        return -1;
    }
    std::vector<int> ids;
    ids.reserve(n);
    ids.push_back(1);
    ids.push_back(25);
    for (int i = 0; i < n_voice; i++) ids.push_back(-(i + 1));
    ids.push_back(36);
    for (int i = 0; i < n_text; i++) {
        if (text_ids[i] < 0 || text_ids[i] >= VB200_VOCAB) return -1;
        ids.push_back(text_ids[i]);
    }
    ids.push_back(35);
    ids.push_back(25);
    int *d_ids = nullptr;
    uint16_t *d_voice = nullptr;
    float *d_rows = nullptr;
    int rc = -1;
    do {
        if (cudaMalloc(&d_ids, sizeof(int) * n) != cudaSuccess || cudaMalloc(&d_rows, sizeof(float) * (size_t)n * D) != cudaSuccess)
            break;
        if (n_voice > 0 && cudaMalloc(&d_voice, (size_t)n_voice * D * 2) != cudaSuccess) break;
        if (cudaMemcpyAsync(d_ids, ids.data(), sizeof(int) * n, cudaMemcpyHostToDevice, m.st) != cudaSuccess) break;
        if (n_voice > 0 &&
            cudaMemcpyAsync(d_voice, voice_bf16, (size_t)n_voice * D * 2, cudaMemcpyHostToDevice, m.st) != cudaSuccess)
            break;
        prompt_rows_kernel<<<dim3((D + 255) / 256, n), 256, 0, m.st>>>(d_rows, m.tok_emb, d_voice, d_ids, D);
        if (cudaGetLastError() != cudaSuccess) break;
        rc = prefill(d_rows, n, start_pos) == 0 ? n : -1;    /* synchronises the stream */
    } while (0);
    cudaStreamSynchronize(m.st);
    cudaFree(d_ids); cudaFree(d_voice); cudaFree(d_rows);
    cudaGetLastError();
    return rc;
}

} // namespace vb

