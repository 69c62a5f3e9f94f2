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
#include "vb_umma.cuh"

#include <cuda_bf16.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <vector>

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
    w->W = d_W; w->N = N; w->K = K; w->tiled = false;
    if (N <= 0 || K <= 0 || (K % kTcBlockK) != 0) return -1;
    if (make_map(&w->map, d_W, (uint64_t)N, (uint64_t)K, kTcTileN)) return -1;
    w->ok = true;
    return 0;
}

/* Weights re-laid out so that every [128 rows x 64 columns] tile the kernel fetches is one
 * contiguous 16 KB block (tile-major, then k-block), instead of 128 pieces of 128 bytes that
 * sit a whole weight row apart: the TMA request becomes a single DRAM-friendly burst. */
__global__ void vb_tc_tile_weights_kernel(uint4 *dst, const uint4 *src, int N, int K) {
    const int kblocks = K / kTcBlockK;
    const size_t n_vec = (size_t)((N + kTcTileN - 1) / kTcTileN) * kblocks * kTcTileN * (kTcBlockK / 8);
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_vec) return;
    const int v = (int)(i % (kTcBlockK / 8));                 /* 16-byte vector inside the 128-byte row */
    const int r = (int)((i / (kTcBlockK / 8)) % kTcTileN);    /* row inside the tile */
    const size_t blk = i / ((kTcBlockK / 8) * kTcTileN);
    const int kb = (int)(blk % kblocks), t = (int)(blk / kblocks);
    const int row = t * kTcTileN + r;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (row < N) val = src[((size_t)row * K + (size_t)kb * kTcBlockK) / 8 + v];
    dst[i] = val;
}

size_t tc_tiled_bytes(int N, int K) {
    return (size_t)((N + kTcTileN - 1) / kTcTileN) * kTcTileN * K * 2;
}

int tc_weight_tiled(TcWeight *w, const uint16_t *d_W, int N, int K, uint16_t *d_tiled, cudaStream_t st) {
    w->ok = false;
    w->W = d_tiled; w->N = N; w->K = K; w->tiled = true;
    if (N <= 0 || K <= 0 || (K % kTcBlockK) != 0 || ((uintptr_t)d_W & 15) || ((uintptr_t)d_tiled & 15)) return -1;
    const size_t n_vec = tc_tiled_bytes(N, K) / 16;
    vb_tc_tile_weights_kernel<<<(unsigned)((n_vec + 255) / 256), 256, 0, st>>>((uint4 *)d_tiled, (const uint4 *)d_W, N, K);
    if (cudaGetLastError() != cudaSuccess) return -1;
    const uint64_t rows = (uint64_t)((N + kTcTileN - 1) / kTcTileN) * (K / kTcBlockK) * kTcTileN;
    if (make_map(&w->map, d_tiled, rows, (uint64_t)kTcBlockK, kTcTileN)) return -1;
    w->ok = true;
    return 0;
}

int tc_rows_pad(int M) { return M <= 16 ? 16 : M <= 64 ? 64 : M <= 256 ? 256 : 0; }

/* The tile a frame's GEMMs use for M rows: 17 .. 48 rows (the acoustic rows of 3 .. 8 utterances)
 * take the 48-row tile, whose stages are 6 KB smaller than the 64-row tile's, so that a sixth stage
 * fits and the weight stream keeps 96 KB in flight per SM. */
int tc_rows_pad_frame(int M) { return (M > 16 && M <= 48) ? 48 : tc_rows_pad(M); }

/* Any number of rows: beyond 256 the buffer is padded to whole 128-row blocks (row-block kernel). */
int tc_rows_pad_any(int M) {
    if (M <= 256) return tc_rows_pad(M);
    return M <= kTcMaxRows ? (M + 127) / 128 * 128 : 0;
}

size_t tc_acts_bytes(int rows_pad, int K) { return (size_t)kTcTerms * rows_pad * K * 2; }

int tc_acts(TcActs *a, uint16_t *d_buf, int rows_pad, int K) {
    a->ok = false;
    a->buf = d_buf; a->rows_pad = rows_pad; a->K = K;
    const bool big = rows_pad > 256 && rows_pad <= kTcMaxRows && rows_pad % 128 == 0;
    if ((rows_pad != 16 && rows_pad != 48 && rows_pad != 64 && rows_pad != 256 && !big) || (K % kTcBlockK) != 0) return -1;
    /* (a TMA box holds at most 256 rows: larger buffers only get the row-block kernel's map) */
    if (!big && make_map(&a->map, d_buf, (uint64_t)kTcTerms * rows_pad, (uint64_t)K, (uint32_t)rows_pad)) return -1;
    /* the row-block kernel fetches 128 rows of one term at a time */
    if (rows_pad >= 256 && make_map(&a->map_rows, d_buf, (uint64_t)kTcTerms * rows_pad, (uint64_t)K, 128u)) return -1;
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

/* ---------------------------------------------------------------- the kernel */
template <int NB, int ST>
struct TcCfg {
    static constexpr int kStageA = kTcTileN * kTcBlockK * 2;        /* 16 KB */
    static constexpr int kTermB = NB * kTcBlockK * 2;               /* one BF16 term of the activations */
    static constexpr int kStage = kStageA + kTcTerms * kTermB;
    static constexpr int kStages = ST;   /* NB=16: several CTAs fit one SM, so the next GEMMs of the stream fetch their first weight tiles under the tail of the running one */
    /* The three BF16 terms of the activations lie one after another in a stage, so for
     * NB <= 64 they form ONE B operand of 3*NB rows: a single MMA per 16-wide K step writes the
     * three partial products to separate TMEM column groups (summed in the epilogue) instead of
     * three narrow MMAs - the narrow ones are issue-latency bound, not throughput bound. */
    static constexpr bool kFusedTerms = (kTcTerms * NB) <= 256;
    static constexpr int kMmaN = kFusedTerms ? kTcTerms * NB : NB;
    static constexpr int kAccCols = kFusedTerms ? kTcTerms * NB : NB;
    static constexpr int kTmemCols = kAccCols <= 32 ? 32 : kAccCols <= 64 ? 64 : kAccCols <= 128 ? 128 : 256;
    static constexpr int kSmemBytes = kStages * kStage + 1024 /* alignment slack */ + 256 /* barriers */ + 4 * NB;
    static_assert(kSmemBytes <= 232448, "over the 227 KB a CTA may use");
};

constexpr int kTcThreads = 192;

/* Kernel-side scalars and pointers (everything but the two tensor maps). */
struct TcKernelArgs {
    int N, K, M, rows_pad, ld_out, splits, epi;
    int a_tiled;             /* weights in the tile-contiguous layout */
    float *out;
    const float *bias;
    const float *ssq;        /* optional [M][ssq_chunks] sums of squares: deferred RMSNorm row scale */
    int ssq_chunks;
    float eps;
    uint16_t *out_terms;     /* TC_EPI_SWIGLU_TERMS: BF16 terms of the result, [3][out_rows_pad][N/2] */
    int out_rows_pad;
    int *status;
    int tile0;               /* first output tile of this launch */
    int n_tiles_launch;      /* tiles this launch covers (host side: the grid) */
};

/* Tensor parallelism is a separate instantiation of every kernel that takes part in it, with
 * its arguments in a parameter of their own: the single-GPU kernels keep their parameter block
 * and code (carrying the extra 200 bytes and branches in every launch cost 0.3 ms per frame). */
struct TcTpArgs {
    TcPush push;             /* results also go to the peers' buffers */
    TcWait wait;             /* the activation terms may be exchanged data */
};
struct TcNoTpArgs {};
template <bool TP> struct TcTpSel { using type = TcNoTpArgs; };
template <> struct TcTpSel<true> { using type = TcTpArgs; };

template <int NB, int ST, bool TP>
__global__ void __launch_bounds__(kTcThreads, 1)
vb_tc_gemm_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                  const TcKernelArgs ka, const typename TcTpSel<TP>::type tp) {
    using Cfg = TcCfg<NB, ST>;
    /* the tensor maps are fetched while the first reads of the parameter block are on their way */
    if (threadIdx.x == 128) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&mapA) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&mapB) : "memory");
    }
    const int N = ka.N, K = ka.K, M = ka.M, rows_pad = ka.rows_pad, ld_out = ka.ld_out, splits = ka.splits,
              epi = ka.epi;
    float *const out = ka.out;
    const float *const bias = ka.bias;
    int *const status = ka.status;
    /* Programmatic dependent launch: the next kernel in the stream may start its own
     * prologue now; it waits (griddepcontrol.wait) before touching what this one writes. */
    pdl_launch_dependents();
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char *base = (unsigned char *)(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char *stages = base;
    uint64_t *full = (uint64_t *)(base + Cfg::kStages * Cfg::kStage);
    uint64_t *empty = full + Cfg::kStages;
    uint64_t *accum = empty + Cfg::kStages;
    uint32_t *tmem_slot = (uint32_t *)(accum + 1);
    int *abort_flag = (int *)(tmem_slot + 1);
    float *rscale = (float *)(abort_flag + 1);   /* [NB] per-row scales */

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int issued = 0;   /* producer thread only: pipeline iterations whose loads were requested */
    const int tile = ka.tile0 + blockIdx.x / splits, sp = blockIdx.x % splits;
    const int kblocks = K / kTcBlockK;
    const int kb0 = (int)((long long)kblocks * sp / splits), kb1 = (int)((long long)kblocks * (sp + 1) / splits);
    const int n_it = kb1 - kb0;

    int first = 0;   /* producer thread only: stages of the first ring-full */
    if (warp == 4 && lane == 0) {
        /* The TMA producer sets the barriers up itself and requests the first ring-full of weight
         * tiles at once - they depend on nothing, neither on the predecessor kernel nor on the
         * TMEM allocation and the CTA-wide barrier below. */
        for (int i = 0; i < Cfg::kStages; i++) { vb_mbar_init(&full[i], 1); vb_mbar_init(&empty[i], 1); }
        vb_mbar_init(accum, 1);
        *abort_flag = 0;
        vb_mbar_init_fence();
        first = n_it < Cfg::kStages ? n_it : Cfg::kStages;
        for (int it = 0; it < first; it++) {
            unsigned char *sa = stages + (size_t)it * Cfg::kStage;
            vb_mbar_arrive_expect_tx(&full[it], (uint32_t)Cfg::kStage);
            if (ka.a_tiled) tma_load_2d(sa, &mapA, 0, (tile * kblocks + kb0 + it) * kTcTileN, &full[it]);
            else tma_load_2d(sa, &mapA, (kb0 + it) * kTcBlockK, tile * kTcTileN, &full[it]);
        }
        issued = first;
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
        /* ---- TMA producer ----
         * The weights of the first ring-full are already on their way (above). Now the kernel
         * waits for its predecessor (griddepcontrol.wait) and only then fetches the activation
         * terms. */
        pdl_wait();
        if constexpr (TP) {
            if (tp.wait.n > 0) {
                /* the activation terms were written by other GPUs: wait for all of them, then make
                 * those writes visible to the TMA engine's proxy */
                if (!tp_wait(tp.wait)) *(volatile int *)abort_flag = 1;
                asm volatile("fence.proxy.async;" ::: "memory");
            }
        }
        for (int it = 0; it < first; it++) {
            unsigned char *sa = stages + (size_t)it * Cfg::kStage;
#pragma unroll
            for (int j = 0; j < kTcTerms; j++)
                tma_load_2d(sa + Cfg::kStageA + j * Cfg::kTermB, &mapB, (kb0 + it) * kTcBlockK, j * rows_pad, &full[it]);
        }
        for (int it = first; it < n_it; it++) {
            const int s = it % Cfg::kStages, use = it / Cfg::kStages;
            if (!vb_mbar_wait(&empty[s], (use & 1u) ^ 1u, abort_flag)) {
                atomicCAS(status, 0, 11);
                *(volatile int *)abort_flag = 1;
                break;
            }
            unsigned char *sa = stages + (size_t)s * Cfg::kStage;
            vb_mbar_arrive_expect_tx(&full[s], (uint32_t)Cfg::kStage);
            const int kx = (kb0 + it) * kTcBlockK;
            if (ka.a_tiled) tma_load_2d(sa, &mapA, 0, (tile * kblocks + kb0 + it) * kTcTileN, &full[s]);
            else tma_load_2d(sa, &mapA, kx, tile * kTcTileN, &full[s]);
#pragma unroll
            for (int j = 0; j < kTcTerms; j++)
                tma_load_2d(sa + Cfg::kStageA + j * Cfg::kTermB, &mapB, kx, j * rows_pad, &full[s]);
            issued = it + 1;
        }
    } else if (warp == 5 && lane == 0) {
        /* ---- MMA issuer ---- */
        const uint32_t idesc = umma_idesc_bf16(Cfg::kMmaN);
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
            /* 16 BF16 = 32 bytes further along K inside the swizzled row: +2 in 16-byte units */
            if (Cfg::kFusedTerms) {
                const uint64_t bdesc = umma_desc_k_sw128(sa + Cfg::kStageA);
#pragma unroll
                for (int k = 0; k < kTcBlockK / 16; k++)
                    umma_bf16(tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (it | k) != 0 ? 1u : 0u);
            } else {
#pragma unroll
                for (int j = 0; j < kTcTerms; j++) {
                    const uint64_t bdesc = umma_desc_k_sw128(sa + Cfg::kStageA + j * Cfg::kTermB);
#pragma unroll
                    for (int k = 0; k < kTcBlockK / 16; k++)
                        umma_bf16(tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (it | j | k) != 0 ? 1u : 0u);
                }
            }
            umma_commit(&empty[s]);   /* stage reusable once these MMAs have read it */
        }
        umma_commit(accum);           /* accumulator complete (arrives at once when nothing was issued) */
    } else if (warp < 4) {
        /* ---- epilogue: TMEM -> registers -> global ---- */
        /* Everything below reads or writes what earlier kernels of the stream own. While the main
         * loop runs, fetch the per-row RMSNorm scale: the activations went in as x*gain and
         * 1/sqrt(mean(x^2)+eps) is applied to the accumulators (voxtral_tts_kernels.c:333-349). */
        pdl_wait();
        if (ka.ssq) {
            for (int m = threadIdx.x; m < M; m += 128) {
                float t = 0.0f;
                for (int c = 0; c < ka.ssq_chunks; c++) t += __ldcg(ka.ssq + m * ka.ssq_chunks + c);
                rscale[m] = 1.0f / sqrtf(t / (float)K + ka.eps);
            }
            vb_named_bar(1, 128);
        }
        bool ok = vb_mbar_wait(accum, 0u, abort_flag);
        if (!ok) {
            atomicCAS(status, 0, 13);
            *(volatile int *)abort_flag = 1;
        }
        tc_fence_after();
        /* The results leave through shared memory (the pipeline stages are free once every MMA has
         * completed) as 16-byte stores along the output columns. Storing straight from the TMEM
         * layout - a lane owns one output column, one 4-byte store per activation row - was
         * measured at ~90 ns per store and 1.5 us per launch even with a single row. */
        float *stg = (float *)stages;                              /* [M][128 output columns] */
        if (ok && n_it > 0) {
#pragma unroll 1
            for (int c0 = 0; c0 < NB && c0 < M; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
                if (Cfg::kFusedTerms) {
                    /* column groups NB and 2*NB hold the lo and lo2 products: add them in */
                    uint32_t r1[16], r2[16];
                    tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(NB + c0), r1);
                    tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(2 * NB + c0), r2);
#pragma unroll
                    for (int i = 0; i < 16; i++)
                        r[i] = __float_as_uint((__uint_as_float(r[i]) + __uint_as_float(r1[i])) + __uint_as_float(r2[i]));
                }
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const int m = c0 + i;
                    float v = __uint_as_float(r[i]);
                    if (ka.ssq && m < M) v *= rscale[m];
                    if (m < M) stg[m * kTcTileN + warp * 32 + lane] = v;
                }
            }
            {
                vb_named_bar(1, 128);
                const int n = tile * kTcTileN + lane * 4;             /* this lane's four output columns */
                for (int m = warp; m < M; m += 4) {
                    const float4 v = *(const float4 *)(stg + m * kTcTileN + lane * 4);
                    if (epi == TC_EPI_SWIGLU || epi == TC_EPI_SWIGLU_TERMS) {
                        /* (gate, up, gate, up) -> two results at columns n / 2 and n / 2 + 1 */
                        const float res[2] = {(v.x / (1.0f + expf(-v.x))) * v.y, (v.z / (1.0f + expf(-v.z))) * v.w};
                        const int col = n >> 1;
                        const size_t ko = (size_t)(N >> 1);
                        if (n + 3 < N && ((ko | (size_t)ld_out) & 1) == 0) {
                            if (epi == TC_EPI_SWIGLU) {
                                *(float2 *)(out + (size_t)m * ld_out + col) = make_float2(res[0], res[1]);
                            } else {
                                uint16_t q[3][2];
                                vb_split3(res[0], q[0][0], q[1][0], q[2][0]);
                                vb_split3(res[1], q[0][1], q[1][1], q[2][1]);
                                const size_t o = (size_t)m * ko + col;
#pragma unroll
                                for (int j = 0; j < 3; j++) {
                                    const uint32_t pk = q[j][0] | ((uint32_t)q[j][1] << 16);
                                    *(uint32_t *)(ka.out_terms + (size_t)j * ka.out_rows_pad * ko + o) = pk;
                                    if constexpr (TP) {
                                        for (int d = 1; d < tp.push.n_dst; d++)
                                            *(uint32_t *)((char *)(ka.out_terms + (size_t)j * ka.out_rows_pad * ko + o) + tp.push.dst_off[d]) = pk;
                                    }
                                }
                            }
                        } else {
                            for (int i = 0; i < 2; i++) {
                                if (n + 2 * i + 1 >= N) break;
                                if (epi == TC_EPI_SWIGLU) {
                                    out[(size_t)m * ld_out + col + i] = res[i];
                                } else {
                                    uint16_t q0, q1, q2;
                                    vb_split3(res[i], q0, q1, q2);
                                    const size_t o = (size_t)m * ko + col + i;
                                    ka.out_terms[o] = q0;
                                    ka.out_terms[(size_t)ka.out_rows_pad * ko + o] = q1;
                                    ka.out_terms[(size_t)2 * ka.out_rows_pad * ko + o] = q2;
                                    if constexpr (TP) {
                                        for (int d = 1; d < tp.push.n_dst; d++) {
                                            uint16_t *pt = (uint16_t *)((char *)ka.out_terms + tp.push.dst_off[d]);
                                            pt[o] = q0;
                                            pt[(size_t)ka.out_rows_pad * ko + o] = q1;
                                            pt[(size_t)2 * ka.out_rows_pad * ko + o] = q2;
                                        }
                                    }
                                }
                            }
                        }
                    } else {
                        const size_t o = ((size_t)(epi == TC_EPI_STORE ? 0 : sp) * M + m) * ld_out + n;
                        if (n + 3 < N && (ld_out & 3) == 0) {
                            float4 w4 = v;
                            if (epi == TC_EPI_STORE && bias) {
                                w4.x += __ldg(bias + n); w4.y += __ldg(bias + n + 1);
                                w4.z += __ldg(bias + n + 2); w4.w += __ldg(bias + n + 3);
                            }
                            *(float4 *)(out + o) = w4;
                            if constexpr (TP) {
                                if (epi != TC_EPI_STORE)
                                    for (int d = 1; d < tp.push.n_dst; d++)
                                        *(float4 *)((char *)(out + o) + tp.push.dst_off[d]) = w4;
                            }
                        } else {
                            const float e[4] = {v.x, v.y, v.z, v.w};
                            for (int i = 0; i < 4 && n + i < N; i++) {
                                const float w1 = e[i] + (epi == TC_EPI_STORE && bias ? __ldg(bias + n + i) : 0.0f);
                                out[o + i] = w1;
                                if constexpr (TP) {
                                    if (epi != TC_EPI_STORE)
                                        for (int d = 1; d < tp.push.n_dst; d++)
                                            *(float *)((char *)(out + o + i) + tp.push.dst_off[d]) = w1;
                                }
                            }
                        }
                    }
                }
            }
        }
        if constexpr (TP) {
            if (tp.push.n_dst > 0) {
                /* once every CTA of this launch has its results in all ranks' buffers, the last one
                 * publishes the visit to every rank */
                vb_named_bar(1, 128);
                if (threadIdx.x == 0) tp_publish(tp.push, gridDim.x);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    /* abort path: let copies already in flight land before the shared memory goes away */
    if (warp == 4 && lane == 0 && *(volatile int *)abort_flag) {
        /* the last load issued into stage s was iteration `it` with it % kStages == s: wait for
         * exactly that phase of its barrier */
        const int first_it = issued > Cfg::kStages ? issued - Cfg::kStages : 0;
        for (int it = first_it; it < issued; it++) {
            const long long t0 = clock64();
            while (!vb_mbar_try_wait(&full[it % Cfg::kStages], (uint32_t)(it / Cfg::kStages) & 1u)) {
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

template <int NB, int ST, bool TP>
static int launch_tc_tp(const TcWeight &w, const TcActs &a, const TcKernelArgs &ka, const TcTpArgs &tpa,
                        cudaStream_t st) {
    using Cfg = TcCfg<NB, ST>;
    static bool attr = false;
    if (!attr) {
        if (cudaFuncSetAttribute(vb_tc_gemm_kernel<NB, ST, TP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg::kSmemBytes) != cudaSuccess) {
            cudaGetLastError();
            return -1;
        }
        attr = true;
    }
    const int tiles = ka.n_tiles_launch;
    typename TcTpSel<TP>::type arg;
    if constexpr (TP) arg = tpa;
    return launch_pdl(vb_tc_gemm_kernel<NB, ST, TP>, dim3(tiles * ka.splits), dim3(kTcThreads), (size_t)Cfg::kSmemBytes, st,
                      w.map, a.map, ka, arg) == cudaSuccess
               ? 0
               : -1;
}

template <int NB, int ST>
static int launch_tc(const TcWeight &w, const TcActs &a, const TcKernelArgs &ka, const TcTpArgs &tpa, cudaStream_t st) {
    if (tpa.push.n_dst > 0 || tpa.wait.n > 0) return launch_tc_tp<NB, ST, true>(w, a, ka, tpa, st);
    return launch_tc_tp<NB, ST, false>(w, a, ka, tpa, st);
}

/* ---------------------------------------------------------------- row-block kernel */
/* 65 .. 256 activation rows (the prompt prefill, tts_cuda_linear_bf16 on many rows). A CTA owns
 * TWO 128-row weight tiles and ONE block of 128 activation rows: per 64-column k-block it
 * fetches 2 x 16 KB of weights and the hi and lo BF16 terms of the activations (2 x 16 KB), and
 * issues 2 tiles x 2 terms x 4 MMAs of 128 x 128 x 16 into two 128-column accumulators. Against
 * one weight tile x 256 rows x 3 terms (16 KB + 96 KB per k-block for the same arithmetic per
 * term) this moves 64 KB instead of 112 KB from L2 per k-block, fits three stages instead of
 * two, and drops the third term: hi + lo carry 16 mantissa bits, a relative error of 4e-6 on the
 * result, against the 2e-3 the path is allowed. The decode path (1 .. 64 rows) keeps all three
 * terms. Grid: (tile pairs) x (row blocks) x (K splits), row blocks and splits adjacent so that
 * the CTAs that share weight tiles run together and the second read hits L2. */
constexpr int kRbRows = 128, kRbTiles = 2, kRbTerms = 2, kRbStages = 3;
constexpr int kRbStageW = kTcTileN * kTcBlockK * 2, kRbStageX = kRbRows * kTcBlockK * 2;
constexpr int kRbStage = kRbTiles * kRbStageW + kRbTerms * kRbStageX;
constexpr int kRbTmemCols = kRbTiles * kRbRows;
constexpr int kRbSmemBytes = kRbStages * kRbStage + 1024 + 256 + 4 * kRbRows;
static_assert(kRbSmemBytes <= 232448, "over the 227 KB a CTA may use");

__global__ void __launch_bounds__(kTcThreads, 1)
vb_tc_rows_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                  const TcKernelArgs ka) {
    const int N = ka.N, K = ka.K, M = ka.M, rows_pad = ka.rows_pad, ld_out = ka.ld_out, splits = ka.splits,
              epi = ka.epi;
    float *const out = ka.out;
    int *const status = ka.status;
    pdl_launch_dependents();
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char *base = (unsigned char *)(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char *stages = base;
    uint64_t *full = (uint64_t *)(base + kRbStages * kRbStage);
    uint64_t *empty = full + kRbStages;
    uint64_t *accum = empty + kRbStages;
    uint32_t *tmem_slot = (uint32_t *)(accum + 1);
    int *abort_flag = (int *)(tmem_slot + 1);
    float *rscale = (float *)(abort_flag + 1);   /* [128] per-row scales of this row block */

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int issued = 0;
    const int row_blocks = (M + kRbRows - 1) / kRbRows;
    const int sp = blockIdx.x % splits, rb = (blockIdx.x / splits) % row_blocks;
    const int pair = blockIdx.x / (splits * row_blocks);
    const int tiles_total = (N + kTcTileN - 1) / kTcTileN;
    const int t0 = pair * kRbTiles;
    const int nt = tiles_total - t0 < kRbTiles ? tiles_total - t0 : kRbTiles;
    const int kblocks = K / kTcBlockK;
    const int kb0 = (int)((long long)kblocks * sp / splits), kb1 = (int)((long long)kblocks * (sp + 1) / splits);
    const int n_it = kb1 - kb0;
    const int m0 = rb * kRbRows;
    const int Mb = M - m0 < kRbRows ? M - m0 : kRbRows;
    const uint32_t stage_tx = (uint32_t)(nt * kRbStageW + kRbTerms * kRbStageX);

    if (threadIdx.x == 0) {
        for (int i = 0; i < kRbStages; i++) { vb_mbar_init(&full[i], 1); vb_mbar_init(&empty[i], 1); }
        vb_mbar_init(accum, 1);
        *abort_flag = 0;
        vb_mbar_init_fence();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(vb_smem_u32(tmem_slot)),
                     "r"((uint32_t)kRbTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *(volatile uint32_t *)tmem_slot;

    if (warp == 4 && lane == 0) {
        /* ---- TMA producer: weights first (they depend on nothing), activation terms after the
         * predecessor kernel has finished ---- */
        auto load_w = [&](int it, int s) {
            unsigned char *sa = stages + (size_t)s * kRbStage;
            for (int t = 0; t < nt; t++) {
                if (ka.a_tiled) tma_load_2d(sa + t * kRbStageW, &mapA, 0, ((t0 + t) * kblocks + kb0 + it) * kTcTileN, &full[s]);
                else tma_load_2d(sa + t * kRbStageW, &mapA, (kb0 + it) * kTcBlockK, (t0 + t) * kTcTileN, &full[s]);
            }
        };
        auto load_x = [&](int it, int s) {
            unsigned char *sx = stages + (size_t)s * kRbStage + kRbTiles * kRbStageW;
#pragma unroll
            for (int j = 0; j < kRbTerms; j++)
                tma_load_2d(sx + j * kRbStageX, &mapB, (kb0 + it) * kTcBlockK, j * rows_pad + m0, &full[s]);
        };
        const int first = n_it < kRbStages ? n_it : kRbStages;
        for (int it = 0; it < first; it++) {
            vb_mbar_arrive_expect_tx(&full[it], stage_tx);
            load_w(it, it);
        }
        issued = first;
        pdl_wait();
        for (int it = 0; it < first; it++) load_x(it, it);
        for (int it = first; it < n_it; it++) {
            const int s = it % kRbStages, use = it / kRbStages;
            if (!vb_mbar_wait(&empty[s], (use & 1u) ^ 1u, abort_flag)) {
                atomicCAS(status, 0, 11);
                *(volatile int *)abort_flag = 1;
                break;
            }
            vb_mbar_arrive_expect_tx(&full[s], stage_tx);
            load_w(it, s);
            load_x(it, s);
            issued = it + 1;
        }
    } else if (warp == 5 && lane == 0) {
        /* ---- MMA issuer ---- */
        const uint32_t idesc = umma_idesc_bf16(kRbRows);
        for (int it = 0; it < n_it; it++) {
            const int s = it % kRbStages, use = it / kRbStages;
            if (!vb_mbar_wait(&full[s], use & 1u, abort_flag)) {
                atomicCAS(status, 0, 12);
                *(volatile int *)abort_flag = 1;
                break;
            }
            tc_fence_after();
            const unsigned char *sa = stages + (size_t)s * kRbStage;
            for (int t = 0; t < nt; t++) {
                const uint64_t adesc = umma_desc_k_sw128(sa + t * kRbStageW);
#pragma unroll
                for (int j = 0; j < kRbTerms; j++) {
                    const uint64_t bdesc = umma_desc_k_sw128(sa + kRbTiles * kRbStageW + j * kRbStageX);
#pragma unroll
                    for (int k = 0; k < kTcBlockK / 16; k++)
                        umma_bf16(tmem + (uint32_t)(t * kRbRows), adesc + 2 * k, bdesc + 2 * k, idesc,
                                  (it | j | k) != 0 ? 1u : 0u);
                }
            }
            umma_commit(&empty[s]);
        }
        umma_commit(accum);
    } else if (warp < 4) {
        /* ---- epilogue: TMEM -> registers -> global ---- */
        pdl_wait();
        if (ka.ssq) {
            for (int m = threadIdx.x; m < Mb; m += 128) {
                float t = 0.0f;
                for (int c = 0; c < ka.ssq_chunks; c++) t += __ldcg(ka.ssq + (m0 + m) * ka.ssq_chunks + c);
                rscale[m] = 1.0f / sqrtf(t / (float)K + ka.eps);
            }
            vb_named_bar(1, 128);
        }
        bool ok = vb_mbar_wait(accum, 0u, abort_flag);
        if (!ok) {
            atomicCAS(status, 0, 13);
            *(volatile int *)abort_flag = 1;
        }
        tc_fence_after();
        if (ok && n_it > 0) {
            /* The accumulators go through shared memory (the pipeline stages are free now: every
             * MMA has completed, so every load has landed and been read) and leave as whole
             * 512-byte row segments, 16 bytes per lane. Storing straight from the TMEM layout -
             * lane = output column, one 4-byte store per activation row - took 23 us per CTA
             * for 128 KB of results: five times the main loop's share. */
            float *stg = (float *)stages;                       /* [tile][128 rows m][128 columns n] */
            for (int t = 0; t < nt; t++) {
#pragma unroll 1
                for (int c0 = 0; c0 < Mb; c0 += 16) {
                    uint32_t r[16];
                    tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(t * kRbRows + c0), r);
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        float v = __uint_as_float(r[i]);
                        if (ka.ssq && c0 + i < Mb) v *= rscale[c0 + i];
                        stg[(t * kRbRows + c0 + i) * kTcTileN + warp * 32 + lane] = v;
                    }
                }
            }
            vb_named_bar(1, 128);
            if (epi == TC_EPI_SWIGLU || epi == TC_EPI_SWIGLU_TERMS) {
                /* a lane turns 8 staged values (4 (gate, up) pairs) into 4 results; the 32 lanes
                 * cover the 128 results of the CTA's two tiles for one activation row */
                const int tt = lane >> 4, n8 = (lane & 15) * 8;
                const int col = (t0 + tt) * (kTcTileN / 2) + (lane & 15) * 4;       /* first result column */
                const size_t ko = (size_t)(N >> 1);
                if (tt < nt && 2 * col + 7 < N) {
                    for (int mb = warp; mb < Mb; mb += 4) {
                        const float4 a = *(const float4 *)(stg + (tt * kRbRows + mb) * kTcTileN + n8);
                        const float4 b = *(const float4 *)(stg + (tt * kRbRows + mb) * kTcTileN + n8 + 4);
                        float res[4];
                        res[0] = (a.x / (1.0f + expf(-a.x))) * a.y;
                        res[1] = (a.z / (1.0f + expf(-a.z))) * a.w;
                        res[2] = (b.x / (1.0f + expf(-b.x))) * b.y;
                        res[3] = (b.z / (1.0f + expf(-b.z))) * b.w;
                        const int m = m0 + mb;
                        if (epi == TC_EPI_SWIGLU) {
                            *(float4 *)(out + (size_t)m * ld_out + col) = make_float4(res[0], res[1], res[2], res[3]);
                        } else {
                            uint16_t q[3][4];
#pragma unroll
                            for (int i = 0; i < 4; i++) vb_split3(res[i], q[0][i], q[1][i], q[2][i]);
                            const size_t o = (size_t)m * ko + col;
#pragma unroll
                            for (int j = 0; j < 3; j++)
                                *(uint2 *)(ka.out_terms + (size_t)j * ka.out_rows_pad * ko + o) =
                                    make_uint2(q[j][0] | ((uint32_t)q[j][1] << 16), q[j][2] | ((uint32_t)q[j][3] << 16));
                        }
                    }
                } else if (tt < nt) {
                    /* ragged edge of the matrix: element by element */
                    for (int mb = warp; mb < Mb; mb += 4) {
                        for (int i = 0; i < 4; i++) {
                            if (2 * (col + i) + 1 >= N) break;
                            const float g = stg[(tt * kRbRows + mb) * kTcTileN + n8 + 2 * i];
                            const float u = stg[(tt * kRbRows + mb) * kTcTileN + n8 + 2 * i + 1];
                            const float res = (g / (1.0f + expf(-g))) * u;
                            const int m = m0 + mb;
                            if (epi == TC_EPI_SWIGLU) out[(size_t)m * ld_out + col + i] = res;
                            else {
                                uint16_t q0, q1, q2;
                                vb_split3(res, q0, q1, q2);
                                const size_t o = (size_t)m * ko + col + i;
                                ka.out_terms[o] = q0;
                                ka.out_terms[(size_t)ka.out_rows_pad * ko + o] = q1;
                                ka.out_terms[(size_t)2 * ka.out_rows_pad * ko + o] = q2;
                            }
                        }
                    }
                }
            } else {
                for (int t = 0; t < nt; t++) {
                    const int n = (t0 + t) * kTcTileN + lane * 4;
                    for (int mb = warp; mb < Mb; mb += 4) {
                        float4 v = *(const float4 *)(stg + (t * kRbRows + mb) * kTcTileN + lane * 4);
                        const size_t o = ((size_t)(epi == TC_EPI_STORE ? 0 : sp) * M + m0 + mb) * ld_out + n;
                        if (n + 3 < N && (ld_out & 3) == 0) {
                            if (epi == TC_EPI_STORE && ka.bias) {
                                const float4 bb = __ldg((const float4 *)(ka.bias + n));
                                v.x += bb.x; v.y += bb.y; v.z += bb.z; v.w += bb.w;
                            }
                            *(float4 *)(out + o) = v;
                        } else {
                            const float e[4] = {v.x, v.y, v.z, v.w};
                            for (int i = 0; i < 4 && n + i < N; i++)
                                out[o + i] = e[i] + (epi == TC_EPI_STORE && ka.bias ? __ldg(ka.bias + n + i) : 0.0f);
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 4 && lane == 0 && *(volatile int *)abort_flag) {
        /* abort path: let copies already in flight land before the shared memory goes away */
        const int first_it = issued > kRbStages ? issued - kRbStages : 0;
        for (int it = first_it; it < issued; it++) {
            const long long t0c = clock64();
            while (!vb_mbar_try_wait(&full[it % kRbStages], (uint32_t)(it / kRbStages) & 1u)) {
                if (clock64() - t0c > VB_WAIT_CYCLES / 8) break;
            }
        }
    }
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)kRbTmemCols)
                     : "memory");
    }
}

static int launch_rows(const TcWeight &w, const TcActs &a, const TcKernelArgs &ka, cudaStream_t st) {
    static bool attr = false;
    if (!attr) {
        if (cudaFuncSetAttribute(vb_tc_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRbSmemBytes) !=
            cudaSuccess) {
            cudaGetLastError();
            return -1;
        }
        attr = true;
    }
    const int tiles = (ka.N + kTcTileN - 1) / kTcTileN, pairs = (tiles + kRbTiles - 1) / kRbTiles;
    const int row_blocks = (ka.M + kRbRows - 1) / kRbRows;
    return launch_pdl(vb_tc_rows_kernel, dim3(pairs * row_blocks * ka.splits), dim3(kTcThreads), (size_t)kRbSmemBytes, st,
                      w.map, a.map_rows, ka) == cudaSuccess
               ? 0
               : -1;
}

int tc_gemm(const TcWeight &w, const TcActs &a, const TcGemm &g, cudaStream_t st) {
    if (!w.ok || !a.ok || w.K != a.K || g.M < 1 || g.M > a.rows_pad) return -1;
    if (g.splits < 1 || g.splits > kTcMaxSplits || g.splits > w.K / kTcBlockK) return -1;
    if (g.epi != TC_EPI_PARTIAL && g.splits != 1) return -1;
    if ((g.epi == TC_EPI_SWIGLU || g.epi == TC_EPI_SWIGLU_TERMS) && (w.N & 1)) return -1;
    if (g.epi == TC_EPI_SWIGLU_TERMS && (!g.out_terms || g.out_rows_pad < g.M)) return -1;
    TcKernelArgs ka;
    ka.a_tiled = w.tiled ? 1 : 0;
    ka.N = w.N; ka.K = w.K; ka.M = g.M; ka.rows_pad = a.rows_pad; ka.ld_out = g.ld_out; ka.splits = g.splits;
    ka.epi = g.epi; ka.out = g.out; ka.bias = g.bias; ka.ssq = g.ssq; ka.ssq_chunks = g.ssq_chunks; ka.eps = g.eps;
    ka.out_terms = g.out_terms; ka.out_rows_pad = g.out_rows_pad; ka.status = g.status;
    {
        const int tiles = (w.N + kTcTileN - 1) / kTcTileN;
        ka.tile0 = g.n_tiles > 0 ? g.tile0 : 0;
        ka.n_tiles_launch = g.n_tiles > 0 ? g.n_tiles : tiles;
        if (ka.tile0 < 0 || ka.tile0 + ka.n_tiles_launch > tiles) return -1;
        if (g.push.n_dst > kTpMaxRanks || (g.push.n_dst > 0 && (!g.push.ticket || !g.push.epoch))) return -1;
    }
    TcTpArgs tpa;
    tpa.push = g.push;
    tpa.wait = g.wait;
    tpa.wait.status = g.status;
    switch (a.rows_pad) {
    case 16: return launch_tc<16, 6>(w, a, ka, tpa, st);
    case 48: return launch_tc<48, 6>(w, a, ka, tpa, st);   /* 8 utterances' acoustic rows: 34 KB stages, six of them */
    case 64: return launch_tc<64, 5>(w, a, ka, tpa, st);
    case 256:
        /* whole-launch calls on one GPU take the row-block kernel; sliced or exchanged launches
         * (tensor parallelism) do not occur at this size */
        if (g.n_tiles == 0 && tpa.push.n_dst == 0 && tpa.wait.n == 0)
            return launch_rows(w, a, ka, st);
        return launch_tc<256, 2>(w, a, ka, tpa, st);
    default:
        if (a.rows_pad > 256 && a.rows_pad % 128 == 0 && g.n_tiles == 0 && tpa.push.n_dst == 0 && tpa.wait.n == 0)
            return launch_rows(w, a, ka, st);
        return -1;
    }
}

/* ---------------------------------------------------------------- prepare */
/* Activation rows -> three BF16 terms. grid = (K / 1024, M), 256 threads x 4 columns.
 *   v = x                                   (plain)
 *   v = residual + sum_p partials[p]        (split-K reduction in fixed order + residual add)
 * optional: x_out = v (the new residual stream); with a gain, the terms hold v*gain and the
 * CTA's sum of v^2 goes to ssq[m][chunk] - the consumer GEMM applies 1/sqrt(mean+eps), so no
 * CTA has to see a whole row and the kernel is a few microseconds instead of a serial pass. */
template <bool TP>
__global__ void vb_tc_prepare_kernel(uint16_t *buf, int rows_pad, int K, const float *x, int ldx,
                                     const float *partials, int n_part, size_t part_stride,
                                     const float *residual, float *x_out, const float *gain, float *ssq,
                                     float *tap, const typename TcWaitSel<TP>::type wait) {
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    if constexpr (TP) {   /* the partials come from every rank */
        if (threadIdx.x == 0) tp_wait(wait);
        __syncthreads();
    }
    const int m = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    float ss = 0.0f;
    if (c < K) {
        float4 v;
        if (partials) {
            /* all partial loads in flight together, then the fixed-order sum */
            float4 t[kTcMaxSplits];
#pragma unroll
            for (int p = 0; p < kTcMaxSplits; p++)
                t[p] = p < n_part ? __ldcg(reinterpret_cast<const float4 *>(partials + (size_t)p * part_stride + (size_t)m * K + c))
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
            v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int p = 0; p < kTcMaxSplits; p++) {
                if (p < n_part) { v.x += t[p].x; v.y += t[p].y; v.z += t[p].z; v.w += t[p].w; }
            }
            if (residual) {
                const float4 r = *reinterpret_cast<const float4 *>(residual + (size_t)m * ldx + c);
                v.x = r.x + v.x; v.y = r.y + v.y; v.z = r.z + v.z; v.w = r.w + v.w;
            }
        } else {
            v = *reinterpret_cast<const float4 *>(x + (size_t)m * ldx + c);
        }
        if (x_out) *reinterpret_cast<float4 *>(x_out + (size_t)m * ldx + c) = v;
        if (tap) *reinterpret_cast<float4 *>(tap + (size_t)m * ldx + c) = v;     /* residual-stream tap for parity checks */
        ss = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
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

int tc_prepare_chunks(int K) { return (K + 1023) / 1024; }

void tc_prepare(const TcActs &acts, const float *x, int ldx, int M, const float *partials, int n_part,
                size_t part_stride, const float *residual, float *x_out, const float *gain, float *ssq,
                cudaStream_t st, const TcWait &wait, float *tap) {
    if (M <= 0) return;
    if (wait.n > 0)
        launch_pdl(vb_tc_prepare_kernel<true>, dim3(tc_prepare_chunks(acts.K), M), dim3(256), 0, st, acts.buf,
                   acts.rows_pad, acts.K, x, ldx, partials, n_part, part_stride, residual, x_out, gain, ssq, tap, wait);
    else
        launch_pdl(vb_tc_prepare_kernel<false>, dim3(tc_prepare_chunks(acts.K), M), dim3(256), 0, st, acts.buf,
                   acts.rows_pad, acts.K, x, ldx, partials, n_part, part_stride, residual, x_out, gain, ssq, tap,
                   TcNoWait());
}

/* y[i] = sum over the split-K partials in fixed order (+ bias[i % N]). */
__global__ void vb_tc_reduce_kernel(float *y, const float *partials, int n_part, size_t stride, size_t count,
                                    const float *bias, int N) {
    pdl_launch_dependents();
    pdl_wait();
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
    launch_pdl(vb_tc_reduce_kernel, dim3((unsigned)((count + 255) / 256)), dim3(256), 0, st, y, partials, n_part, stride, count,
               bias, N);
}

/* ---------------------------------------------------------------- stand-alone probe */
__global__ void vb_tc_fill_kernel(uint16_t *p, size_t n, uint32_t seed) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    /* small BF16 values of both signs: 0x3c00 | 6 hashed mantissa bits, hashed sign */
    uint32_t h = (uint32_t)i * 2654435761u + seed;
    h ^= h >> 15;
    p[i] = (uint16_t)(0x3c00u | (h & 0x3fu) | ((h & 0x40u) << 9));
}

/* One weight matrix [N, K] of generated values, M activation rows, `reps` launches of the GEMM
 * between two events on the default stream. Needs no model: a measurement and profiling aid
 * with a small memory footprint. epi: TC_EPI_PARTIAL (split-K as the frame uses it) or
 * TC_EPI_SWIGLU_TERMS; tiled bit 0: tile-contiguous weight copy as the frame uses it; bit 1: one
 * copy only, so that a matrix smaller than L2 stays resident (how fast is a launch whose weights
 * need no HBM?). */
int tc_probe(int M, int N, int K, int epi, int tiled, int reps, int n_sm, float *ms_out, int *splits_out) {
    if (tc_init() || M < 1 || reps < 1 || (K % kTcBlockK) != 0) return -1;
    const int rp = tc_rows_pad_frame(M);
    if (!rp) return -1;
    /* enough copies of the matrix that successive launches cannot find their weights in L2 */
    const int copies = (tiled & 2) ? 1 : (int)((size_t)512 * 1024 * 1024 / ((size_t)N * K * 2)) + 1;
    tiled &= 1;
    std::vector<uint16_t *> Wc(copies, nullptr);
    std::vector<TcWeight> wc(copies);
    uint16_t *W = nullptr, *terms = nullptr, *out_terms = nullptr;
    float *out = nullptr;
    int *status = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    int rc = -1;
    const size_t wn = (size_t)N * K;
    const int splits = epi == TC_EPI_PARTIAL ? tc_pick_splits(N, K, n_sm) : 1;
    do {
        if (cudaMalloc(&W, wn * 2) != cudaSuccess || cudaMalloc(&terms, tc_acts_bytes(rp, K)) != cudaSuccess ||
            cudaMalloc(&out, sizeof(float) * (size_t)kTcMaxSplits * M * N) != cudaSuccess ||
            cudaMalloc(&out_terms, tc_acts_bytes(rp, N / 2 + 64)) != cudaSuccess ||
            cudaMalloc(&status, sizeof(int)) != cudaSuccess)
            break;
        cudaMemset(status, 0, sizeof(int));
        vb_tc_fill_kernel<<<(unsigned)((wn + 255) / 256), 256>>>(W, wn, 1u);
        const size_t tn = tc_acts_bytes(rp, K) / 2;
        vb_tc_fill_kernel<<<(unsigned)((tn + 255) / 256), 256>>>(terms, tn, 2u);
        bool wok = true;
        for (int c = 0; c < copies && wok; c++) {
            const size_t bytes = tiled ? tc_tiled_bytes(N, K) : wn * 2;
            wok = cudaMalloc(&Wc[c], bytes) == cudaSuccess;
            if (wok && tiled) wok = tc_weight_tiled(&wc[c], W, N, K, Wc[c], 0) == 0;
            else if (wok) wok = cudaMemcpy(Wc[c], W, bytes, cudaMemcpyDeviceToDevice) == cudaSuccess && tc_weight(&wc[c], Wc[c], N, K) == 0;
        }
        if (!wok) break;
        TcActs a;
        if (tc_acts(&a, terms, rp, K)) break;
        TcGemm g;
        g.M = M; g.splits = splits; g.epi = epi; g.out = out; g.ld_out = epi == TC_EPI_PARTIAL ? N : N / 2;
        g.out_terms = out_terms; g.out_rows_pad = rp; g.status = status;
        if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) break;
        bool ok = true;
        for (int i = 0; i < 3 && ok; i++) ok = tc_gemm(wc[i % copies], a, g, 0) == 0;
        cudaEventRecord(e0, 0);
        for (int i = 0; i < reps && ok; i++) ok = tc_gemm(wc[(3 + i) % copies], a, g, 0) == 0;
        cudaEventRecord(e1, 0);
        if (!ok || cudaDeviceSynchronize() != cudaSuccess) break;
        int st = 0;
        cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost);
        if (st) break;
        if (ms_out) cudaEventElapsedTime(ms_out, e0, e1);
        if (splits_out) *splits_out = splits;
        rc = 0;
    } while (0);
    cudaGetLastError();
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    for (uint16_t *p : Wc) cudaFree(p);
    cudaFree(W); cudaFree(terms); cudaFree(out); cudaFree(out_terms); cudaFree(status);
    return rc;
}

} // namespace vb
