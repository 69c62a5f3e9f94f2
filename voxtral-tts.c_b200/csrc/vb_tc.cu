/*
 * vb_tc.cu - tcgen05 / TMEM / TMA skinny GEMM (sm_100a) for M >= 2 activation rows:
 * the acoustic transformer's CFG-batched passes (M = 6) and the prompt prefill.
 *
 *   y[M,N] = x[M,K] . W[N,K]^T, BF16 W, fp32 x and y (tts_linear_nobias_bf16 with
 *   seq_len > 1, voxtral_tts_kernels.c:187-198, which the reference runs as
 *   weight expansion + SGEMM).
 *
 * Swap-AB: a 128-row weight tile is the UMMA A operand (K-major, 128-byte swizzle,
 * brought in by 2-D TMA), the activation rows are the narrow B operand (UMMA N =
 * 16 / 64 / 256), the fp32 accumulator tile [128 x N] sits in TMEM. The kernel is
 * HBM-bound (every weight byte is read once); tensor work is a few percent.
 *
 * fp32 fidelity: the reference multiplies fp32 activations by exactly expanded
 * BF16 weights. Each activation is split into three BF16 terms, x = hi + lo + lo2
 * (8 + 8 + 8 mantissa bits), and the three MMAs accumulate into the same TMEM
 * tile; BF16 x BF16 products are exact in fp32, so only the summation order
 * differs from the reference.
 *
 * Warp roles: warps 0-3 epilogue (TMEM lanes 32w..32w+31 -> registers -> global),
 * warp 4 lane 0 TMA producer, warp 5 lane 0 MMA issuer. No cluster, no multicast.
 * All waits are bounded; on expiry a status word is set, every role falls through,
 * and the TMEM columns are released before the CTA exits.
 */
#include "vb_tc.cuh"
#include "vb_common.cuh"

#include <cuda_bf16.h>
#include <stdio.h>

namespace vb {

/* ---------------------------------------------------------------- host: tensor maps */
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

int tc_init() {
    if (g_encode) return 0;
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess || !fn) {
        cudaGetLastError();
        return -1;
    }
    g_encode = (EncodeTiledFn)fn;
    return 0;
}

/* [rows, cols] BF16 row-major; box = 64 columns x box_rows rows, 128-byte swizzle. */
static int make_map(CUtensorMap *m, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    if (tc_init()) return -1;
    if (((uintptr_t)base & 15) || (cols * 2) % 16) return -1;
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)kTcBlockK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void *)base, gdim, gstride, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -1;
}

int tc_weight(TcWeight *w, const uint16_t *d_W, int N, int K) {
    w->ok = false;
    w->W = d_W; w->N = N; w->K = K;
    if (N <= 0 || K <= 0 || (K % kTcBlockK) != 0) return -1;
    if (make_map(&w->map, d_W, (uint64_t)N, (uint64_t)K, kTcTileN)) return -1;
    w->ok = true;
    return 0;
}

int tc_rows_pad(int M) { return M <= 16 ? 16 : M <= 64 ? 64 : M <= 256 ? 256 : 0; }

size_t tc_acts_bytes(int rows_pad, int K) { return (size_t)kTcTerms * rows_pad * K * 2; }

int tc_acts(TcActs *a, uint16_t *d_buf, int rows_pad, int K) {
    a->ok = false;
    a->buf = d_buf; a->rows_pad = rows_pad; a->K = K;
    if ((rows_pad != 16 && rows_pad != 64 && rows_pad != 256) || (K % kTcBlockK) != 0) return -1;
    if (make_map(&a->map, d_buf, (uint64_t)kTcTerms * rows_pad, (uint64_t)K, (uint32_t)rows_pad)) return -1;
    a->ok = true;
    return 0;
}

int tc_pick_splits(int N, int K, int n_sm) {
    const int tiles = (N + kTcTileN - 1) / kTcTileN;
    int s = n_sm / tiles;
    if (s < 1) s = 1;
    if (s > kTcMaxSplits) s = kTcMaxSplits;
    if (s > K / kTcBlockK) s = K / kTcBlockK;
    return s;
}

/* ---------------------------------------------------------------- device helpers */
VB_DEVINL void tma_load_2d(void *smem_dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            vb_smem_u32(smem_dst)),
        "l"(map), "r"(vb_smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

/* K-major operand tile with 128-byte swizzle: rows 128 B apart, 8-row groups 1024 B apart
 * (stride byte offset), descriptor version 1 (sm_100), layout type 2 (SWIZZLE_128B). */
VB_DEVINL uint64_t umma_desc_k_sw128(const void *smem_tile) {
    const uint32_t addr = vb_smem_u32(smem_tile);
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;                 /* leading byte offset: unused for swizzled K-major */
    d |= (uint64_t)(1024 >> 4) << 32;       /* stride byte offset */
    d |= (uint64_t)1 << 46;                 /* descriptor version */
    d |= (uint64_t)2 << 61;                 /* SWIZZLE_128B */
    return d;
}

/* kind::f16, BF16 x BF16 -> fp32, both operands K-major, M = 128, N = nb. */
VB_DEVINL uint32_t umma_idesc_bf16(int nb) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(nb >> 3) << 17) | ((uint32_t)(kTcTileN >> 4) << 24);
}

VB_DEVINL void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

VB_DEVINL void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     vb_smem_u32(bar))
                 : "memory");
}

VB_DEVINL void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

VB_DEVINL void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
VB_DEVINL void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

/* ---------------------------------------------------------------- the kernel */
template <int NB>
struct TcCfg {
    static constexpr int kStageA = kTcTileN * kTcBlockK * 2;        /* 16 KB */
    static constexpr int kTermB = NB * kTcBlockK * 2;               /* one BF16 term of the activations */
    static constexpr int kStage = kStageA + kTcTerms * kTermB;
    static constexpr int kStages = NB == 16 ? 8 : NB == 64 ? 5 : 2;
    static constexpr int kTmemCols = NB < 32 ? 32 : NB;
    static constexpr int kSmemBytes = kStages * kStage + 1024 /* alignment slack */ + 256 /* barriers */;
};

constexpr int kTcThreads = 192;

template <int NB>
__global__ void __launch_bounds__(kTcThreads, 1)
vb_tc_gemm_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, int N, int K,
                  int M, int rows_pad, float *out, int ld_out, int splits, int epi, const float *bias,
                  int *status) {
    using Cfg = TcCfg<NB>;
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char *base = (unsigned char *)(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char *stages = base;
    uint64_t *full = (uint64_t *)(base + Cfg::kStages * Cfg::kStage);
    uint64_t *empty = full + Cfg::kStages;
    uint64_t *accum = empty + Cfg::kStages;
    uint32_t *tmem_slot = (uint32_t *)(accum + 1);
    int *abort_flag = (int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / splits, sp = blockIdx.x % splits;
    const int kblocks = K / kTcBlockK;
    const int kb0 = (int)((long long)kblocks * sp / splits), kb1 = (int)((long long)kblocks * (sp + 1) / splits);
    const int n_it = kb1 - kb0;

    if (threadIdx.x == 0) {
        for (int i = 0; i < Cfg::kStages; i++) { vb_mbar_init(&full[i], 1); vb_mbar_init(&empty[i], 1); }
        vb_mbar_init(accum, 1);
        *abort_flag = 0;
        vb_mbar_init_fence();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(vb_smem_u32(tmem_slot)),
                     "r"((uint32_t)Cfg::kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *(volatile uint32_t *)tmem_slot;

    if (warp == 4 && lane == 0) {
        /* ---- TMA producer ---- */
        for (int it = 0; it < n_it; it++) {
            const int s = it % Cfg::kStages, use = it / Cfg::kStages;
            if (!vb_mbar_wait(&empty[s], (use & 1u) ^ 1u, abort_flag)) {
                atomicCAS(status, 0, 11);
                *(volatile int *)abort_flag = 1;
                break;
            }
            unsigned char *sa = stages + (size_t)s * Cfg::kStage;
            vb_mbar_arrive_expect_tx(&full[s], (uint32_t)Cfg::kStage);
            const int kx = (kb0 + it) * kTcBlockK;
            tma_load_2d(sa, &mapA, kx, tile * kTcTileN, &full[s]);
#pragma unroll
            for (int j = 0; j < kTcTerms; j++)
                tma_load_2d(sa + Cfg::kStageA + j * Cfg::kTermB, &mapB, kx, j * rows_pad, &full[s]);
        }
    } else if (warp == 5 && lane == 0) {
        /* ---- MMA issuer ---- */
        const uint32_t idesc = umma_idesc_bf16(NB);
        bool ok = true;
        for (int it = 0; it < n_it && ok; it++) {
            const int s = it % Cfg::kStages, use = it / Cfg::kStages;
            if (!vb_mbar_wait(&full[s], use & 1u, abort_flag)) {
                atomicCAS(status, 0, 12);
                *(volatile int *)abort_flag = 1;
                ok = false;
                break;
            }
            tc_fence_after();
            const unsigned char *sa = stages + (size_t)s * Cfg::kStage;
            const uint64_t adesc = umma_desc_k_sw128(sa);
#pragma unroll
            for (int j = 0; j < kTcTerms; j++) {
                const uint64_t bdesc = umma_desc_k_sw128(sa + Cfg::kStageA + j * Cfg::kTermB);
#pragma unroll
                for (int k = 0; k < kTcBlockK / 16; k++) {
                    /* 16 BF16 = 32 bytes further along K inside the swizzled row: +2 in 16-byte units */
                    umma_bf16(tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (it | j | k) != 0 ? 1u : 0u);
                }
            }
            umma_commit(&empty[s]);   /* stage reusable once these MMAs have read it */
        }
        umma_commit(accum);           /* accumulator complete (arrives at once when nothing was issued) */
    } else if (warp < 4) {
        /* ---- epilogue: TMEM -> registers -> global ---- */
        bool ok = vb_mbar_wait(accum, 0u, abort_flag);
        if (!ok) {
            atomicCAS(status, 0, 13);
            *(volatile int *)abort_flag = 1;
        }
        tc_fence_after();
        const int row = tile * kTcTileN + warp * 32 + lane;
        if (ok && n_it > 0) {
#pragma unroll 1
            for (int c0 = 0; c0 < NB && c0 < M; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const int m = c0 + i;
                    const float v = __uint_as_float(r[i]);
                    if (epi == TC_EPI_SWIGLU) {
                        const float other = __shfl_xor_sync(0xffffffffu, v, 1);
                        if (m < M && row < N && (lane & 1) == 0)
                            out[(size_t)m * ld_out + (row >> 1)] = (v / (1.0f + expf(-v))) * other;
                    } else if (m < M && row < N) {
                        if (epi == TC_EPI_STORE) out[(size_t)m * ld_out + row] = v + (bias ? __ldg(bias + row) : 0.0f);
                        else out[((size_t)sp * M + m) * ld_out + row] = v;
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    /* abort path: let copies already in flight land before the shared memory goes away */
    if (warp == 4 && lane == 0 && *(volatile int *)abort_flag) {
        for (int s = 0; s < Cfg::kStages; s++) {
            long long t0 = clock64();
            while (!vb_mbar_try_wait(&full[s], 0u) && !vb_mbar_try_wait(&full[s], 1u)) {
                if (clock64() - t0 > VB_WAIT_CYCLES / 8) break;
            }
        }
    }
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)Cfg::kTmemCols)
                     : "memory");
    }
}

template <int NB>
static int launch_tc(const TcWeight &w, const TcActs &a, int M, float *out, int ld_out, int splits, int epi,
                     const float *bias, int *d_status, cudaStream_t st) {
    using Cfg = TcCfg<NB>;
    static bool attr = false;
    if (!attr) {
        if (cudaFuncSetAttribute(vb_tc_gemm_kernel<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg::kSmemBytes) != cudaSuccess)
            return -1;
        attr = true;
    }
    const int tiles = (w.N + kTcTileN - 1) / kTcTileN;
    vb_tc_gemm_kernel<NB><<<tiles * splits, kTcThreads, Cfg::kSmemBytes, st>>>(
        w.map, a.map, w.N, w.K, M, a.rows_pad, out, ld_out, splits, epi, bias, d_status);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int tc_gemm(const TcWeight &w, const TcActs &a, int M, float *out, int ld_out, int splits, int epi,
            const float *bias, int *d_status, cudaStream_t st) {
    if (!w.ok || !a.ok || w.K != a.K || M < 1 || M > a.rows_pad) return -1;
    if (splits < 1 || splits > kTcMaxSplits || splits > w.K / kTcBlockK) return -1;
    if (epi != TC_EPI_PARTIAL && splits != 1) return -1;
    if (epi == TC_EPI_SWIGLU && (w.N & 1)) return -1;
    switch (a.rows_pad) {
    case 16: return launch_tc<16>(w, a, M, out, ld_out, splits, epi, bias, d_status, st);
    case 64: return launch_tc<64>(w, a, M, out, ld_out, splits, epi, bias, d_status, st);
    case 256: return launch_tc<256>(w, a, M, out, ld_out, splits, epi, bias, d_status, st);
    default: return -1;
    }
}

/* ---------------------------------------------------------------- prepare */
/* One CTA per activation row: v = x (or residual + sum of split-K partials), optional
 * RMSNorm (voxtral_tts_kernels.c:333-349), then the three BF16 terms. */
__global__ void vb_tc_prepare_kernel(uint16_t *buf, int rows_pad, int K, const float *x, int ldx,
                                     const float *partials, int n_part, size_t part_stride, int M,
                                     const float *residual, float *x_out, const float *gain, float eps) {
    extern __shared__ float row_smem[];
    __shared__ float red[32];
    const int m = blockIdx.x;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < K; c += blockDim.x) {
        float v;
        if (partials) {
            v = 0.0f;
            for (int p = 0; p < n_part; p++) v += partials[(size_t)p * part_stride + (size_t)m * K + c];
            if (residual) v = residual[(size_t)m * ldx + c] + v;
        } else {
            v = x[(size_t)m * ldx + c];
        }
        if (x_out) x_out[(size_t)m * ldx + c] = v;
        row_smem[c] = v;
        ss += v * v;
    }
    float inv = 1.0f;
    if (gain) {
        ss = vb_warp_sum(ss);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float t = 0.0f;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) t += red[w];
        inv = 1.0f / sqrtf(t / (float)K + eps);
    }
    __syncthreads();
    for (int c = threadIdx.x; c < K; c += blockDim.x) {
        float v = row_smem[c];
        if (gain) v = v * inv * gain[c];
        const __nv_bfloat16 h0 = __float2bfloat16_rn(v);
        const float r1 = v - __bfloat162float(h0);
        const __nv_bfloat16 h1 = __float2bfloat16_rn(r1);
        const float r2 = r1 - __bfloat162float(h1);
        const __nv_bfloat16 h2 = __float2bfloat16_rn(r2);
        buf[((size_t)0 * rows_pad + m) * K + c] = __bfloat16_as_ushort(h0);
        buf[((size_t)1 * rows_pad + m) * K + c] = __bfloat16_as_ushort(h1);
        buf[((size_t)2 * rows_pad + m) * K + c] = __bfloat16_as_ushort(h2);
    }
}

void tc_prepare(const TcActs &acts, const float *x, int ldx, int M, const float *partials, int n_part,
                size_t part_stride, const float *residual, float *x_out, const float *gain, float eps,
                cudaStream_t st) {
    if (M <= 0) return;
    static bool attr = false;
    if (!attr) {
        cudaFuncSetAttribute(vb_tc_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
        attr = true;
    }
    vb_tc_prepare_kernel<<<M, 512, (size_t)acts.K * sizeof(float), st>>>(acts.buf, acts.rows_pad, acts.K, x, ldx,
                                                                        partials, n_part, part_stride, M, residual,
                                                                        x_out, gain, eps);
}

/* y[i] = sum over the split-K partials in fixed order (+ bias[i % N]). */
__global__ void vb_tc_reduce_kernel(float *y, const float *partials, int n_part, size_t stride, size_t count,
                                    const float *bias, int N) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float v = 0.0f;
    for (int p = 0; p < n_part; p++) v += partials[(size_t)p * stride + i];
    if (bias) v += bias[i % N];
    y[i] = v;
}

void tc_reduce(float *y, const float *partials, int n_part, size_t stride, size_t count, const float *bias, int N,
               cudaStream_t st) {
    if (count == 0) return;
    vb_tc_reduce_kernel<<<(unsigned)((count + 255) / 256), 256, 0, st>>>(y, partials, n_part, stride, count, bias, N);
}

} // namespace vb
