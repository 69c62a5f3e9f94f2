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
constexpr int kPrefetchWarp = kComputeWarps + 2;  /* lane 0 warms L2 ahead of the ring */
constexpr int kThreads = (kComputeWarps + 3) * 32;
constexpr int kComputeThreads = kComputeWarps * 32;
constexpr int kWorkThreads = kComputeThreads + 32; /* compute + epilogue: named barrier 1 */

constexpr int kSlots = 4;                  /* ring depth */
constexpr int kSlotBytes = 49152;          /* 8 rows of K=3072, 6 of K=4096 */
constexpr int kPartSlots = 6;              /* ring of per-chunk partial sums (warps -> epilogue) */
constexpr int kPrefetchChunks = 0;         /* L2 warm-up distance in chunks; 0 = off (measured: no gain, see profiles) */
constexpr int kResFloats = 256;            /* residual values cached per op by the epilogue */
constexpr int kMaxRowsPerChunk = 8;        /* rows a warp reduces together: more rows per barrier round trip */
constexpr int kMaxM = 8;
constexpr int kMaxV = 32;                  /* partial sums per warp per chunk: one per epilogue lane */
/* Rows per chunk for M activation rows: rows x M partial sums must fit the 32 epilogue lanes. */
__host__ __device__ constexpr int rows_cap(int M) { return kMaxV / M < kMaxRowsPerChunk ? kMaxV / M : kMaxRowsPerChunk; }
constexpr int kSliceCols = 256;            /* columns one warp covers: 32 lanes x 8 bf16 */
constexpr int kMaxSegCols = kComputeWarps * kSliceCols; /* 4096: widest K handled in one pass */
constexpr int kYaccFloats = 1024;          /* cross-pass accumulators (rows x M) */
constexpr int kAttnSubsets = 4;            /* key subsets per head inside a CTA */
constexpr int kHeadDim = 128;

struct SmemLayout {
    alignas(128) unsigned char ring[kSlots][kSlotBytes];
    float part[kPartSlots][kComputeWarps][kMaxV];
    float yacc[kYaccFloats];
    float attn_o[kAttnSubsets][4][kHeadDim];
    float attn_ml[kAttnSubsets][4][2];
    float qs[4][kHeadDim];
    float cs[kHeadDim];          /* (cos, sin) pairs for the current position */
    float red[2][kComputeWarps][kMaxM];   /* double-buffered by op parity */
    float resv[kResFloats];
    float rinv[kMaxM];
    float xs[64];                /* small per-op vector (latent, 36 wide) */
    uint64_t full[kSlots];
    uint64_t empty[kSlots];
    uint64_t pdone[kPartSlots];
    uint64_t pfree[kPartSlots];
    unsigned long long issued_bytes;   /* weight bytes the producer has requested so far */
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
    int prefetch_chunks;     /* L2 prefetch distance of the producer, in chunks (0 = off) */
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
    /* balanced split without 64-bit division: the first `rem` CTAs take one unit more */
    const unsigned U = (unsigned)(N / unit), nc = (unsigned)n_cta, q = U / nc, rem = U - q * nc;
    const unsigned c0 = (unsigned)cta, u0 = c0 * q + (c0 < rem ? c0 : rem);
    p.r0 = (int)u0 * unit;
    p.r1 = (int)(u0 + q + (c0 < rem ? 1u : 0u)) * unit;
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
    if (rc > rows_cap(M)) rc = rows_cap(M);
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
