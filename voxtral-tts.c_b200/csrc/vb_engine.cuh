/*
 * vb_engine.cuh - launch geometry and shared-memory layout of the persistent
 * frame kernel, shared between the kernel (vb_engine.cu) and its host launcher.
 */
#ifndef VB_ENGINE_CUH
#define VB_ENGINE_CUH

#include "vb_ops.h"

#include <cuda_runtime.h>
#include <stdint.h>

namespace vb {

constexpr int kComputeWarps = 16;                 /* FMA warps; each owns 256-column slices */
constexpr int kEpilogueWarp = kComputeWarps;      /* cross-warp sum, epilogue, global store */
constexpr int kProducerWarp = kComputeWarps + 1;  /* lane 0 issues the bulk copies */
constexpr int kThreads = (kComputeWarps + 2) * 32;
constexpr int kComputeThreads = kComputeWarps * 32;
constexpr int kWorkThreads = kComputeThreads + 32; /* compute + epilogue: named barrier 1 */

constexpr int kSlots = 7;                  /* ring depth */
constexpr int kSlotBytes = 24576;          /* 4 rows of K=3072, 3 of K=4096 */
constexpr int kMaxRowsPerChunk = 4;
constexpr int kMaxM = 8;
constexpr int kMaxV = kMaxRowsPerChunk * kMaxM; /* partial sums per warp per chunk */
constexpr int kSliceCols = 256;            /* columns one warp covers: 32 lanes x 8 bf16 */
constexpr int kMaxSegCols = kComputeWarps * kSliceCols; /* 4096: widest K handled in one pass */
constexpr int kYaccFloats = 2048;          /* cross-pass accumulators (rows x M) */
constexpr int kAttnSubsets = 4;            /* key subsets per head inside a CTA */
constexpr int kHeadDim = 128;

struct SmemLayout {
    alignas(128) unsigned char ring[kSlots][kSlotBytes];
    float part[kSlots][kComputeWarps][kMaxV];
    float yacc[kYaccFloats];
    float attn_o[kAttnSubsets][4][kHeadDim];
    float attn_ml[kAttnSubsets][4][2];
    float qs[4][kHeadDim];
    float cs[kHeadDim];          /* (cos, sin) pairs for the current position */
    float red[kComputeWarps][kMaxM];
    float rinv[kMaxM];
    float xs[64];                /* small per-op vector (latent, 36 wide) */
    uint64_t full[kSlots];
    uint64_t empty[kSlots];
    uint64_t done[kSlots];
    int abort_flag;
    int last_flag;
};

struct EngineArgs {
    const VbOp *ops;
    int n_ops;
    VbDyn *dyn;
    unsigned *bar_counter;   /* grid barrier arrivals, zero between launches */
    unsigned *exit_counter;  /* CTAs that finished; the last one re-zeroes both */
    int *status;             /* VbStatus, sticky until the host clears it */
};

/* Row/column decomposition of one GEMV op for one CTA. Host code uses the same
 * function to validate an op before it is put in a program. */
struct GemvPlan {
    int r0, r1;      /* this CTA's rows */
    int passes;      /* K is cut into `passes` column segments of seg_cols */
    int seg_cols;
    int rows_per_chunk;
    int row_blocks;
    int n_chunks;
};

__host__ __device__ inline GemvPlan gemv_plan(int N, int K, int M, int epi, int cta, int n_cta) {
    GemvPlan p;
    int unit = (epi == VB_EPI_SWIGLU) ? 2 : 1;
    long long U = N / unit;
    p.r0 = (int)(U * cta / n_cta) * unit;
    p.r1 = (int)(U * (cta + 1) / n_cta) * unit;
    p.passes = (K + kMaxSegCols - 1) / kMaxSegCols;
    if (p.passes <= 1) {
        p.passes = 1;
        p.seg_cols = K;
    } else {
        int per = (K + p.passes - 1) / p.passes;
        p.seg_cols = (per + kSliceCols - 1) / kSliceCols * kSliceCols;
        p.passes = (K + p.seg_cols - 1) / p.seg_cols;
    }
    int rc = kSlotBytes / (p.seg_cols * 2);
    if (rc > kMaxRowsPerChunk) rc = kMaxRowsPerChunk;
    if (rc * M > kMaxV) rc = kMaxV / M;
    if (unit == 2) rc &= ~1;
    if (rc < 1) rc = 1;
    p.rows_per_chunk = rc;
    int rows = p.r1 - p.r0;
    p.row_blocks = (rows + rc - 1) / rc;
    p.n_chunks = p.row_blocks * p.passes;
    return p;
}

/* Host-side check that an op can run on this engine. Returns 0 when fine. */
inline int gemv_validate(int N, int K, int M, int epi, int n_cta) {
    if (M < 1 || M > kMaxM) return -1;
    if (K < 8 || (K % 8) != 0) return -2;
    if (epi == VB_EPI_SWIGLU && (N % 2) != 0) return -3;
    GemvPlan p = gemv_plan(N, K, M, epi, 0, n_cta);
    if (p.seg_cols * 2 * p.rows_per_chunk > kSlotBytes) return -4;
    if (p.seg_cols > kMaxSegCols) return -5;
    if (epi == VB_EPI_SWIGLU && (p.rows_per_chunk % 2) != 0) return -6;
    if (p.passes > 1) {
        int unit = (epi == VB_EPI_SWIGLU) ? 2 : 1;
        long long max_rows = ((long long)(N / unit) + n_cta - 1) / n_cta * unit + unit;
        if (max_rows * M > kYaccFloats) return -7;
    }
    return 0;
}

cudaError_t engine_launch(const EngineArgs &args, int n_cta, cudaStream_t stream);
int engine_max_ctas(int device);

} // namespace vb

#endif
