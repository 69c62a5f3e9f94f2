/*
 * vb_tc.cuh - tensor-core (tcgen05 / TMEM / TMA) skinny GEMM for M >= 2 activation
 * rows: host interface.
 *
 *   y[M,N] = x[M,K] . W[N,K]^T     BF16 W, fp32 x and y
 *
 * The weight tile is the 128-row UMMA "A" operand, the activations are the
 * narrow "B" operand (swap-AB), accumulators live in TMEM. fp32 activations are
 * kept exact enough for the reference's fp32 arithmetic by splitting every value
 * into three BF16 terms (x = hi + lo + lo2, 24 mantissa bits) and issuing one MMA
 * per term into the same accumulator; BF16 x BF16 products are exact in fp32.
 */
#ifndef VB_TC_CUH
#define VB_TC_CUH

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

namespace vb {

constexpr int kTcTileN = 128;     /* weight rows per CTA tile = UMMA M */
constexpr int kTcBlockK = 64;     /* K elements per pipeline stage: one 128-byte swizzle row */
constexpr int kTcTerms = 3;       /* BF16 terms per fp32 activation */
constexpr int kTcMaxRows = 16384;  /* activation rows per launch (row-block kernel) */
constexpr int kTcMaxSplits = 8;   /* split-K factor limit (partials are summed in fixed order) */

enum TcEpilogue {
    TC_EPI_PARTIAL = 0,       /* out[split][m][n] = partial sum (fp32) */
    TC_EPI_STORE = 1,         /* splits == 1: out[m][n] = sum (+ bias[n]) */
    TC_EPI_SWIGLU = 2,        /* splits == 1, rows interleaved (gate, up): out[m][n/2] = silu(gate) * up */
    TC_EPI_SWIGLU_TERMS = 3   /* same value, written as three BF16 terms for the next GEMM */
};

/* One weight matrix prepared for the tensor-core path. */
struct TcWeight {
    CUtensorMap map;     /* [N, K] BF16 row-major, box 64 x 128, 128-byte swizzle */
    const uint16_t *W;
    int N, K;
    bool ok;
    bool tiled;          /* W points at the tile-contiguous copy (tc_weight_tiled) */
};

/* Activation rows split into BF16 terms: [terms][rows_pad][K], rows_pad = 16, 64 or 256. */
struct TcActs {
    CUtensorMap map;
    CUtensorMap map_rows;   /* rows_pad == 256 only: box of 128 rows (row-block kernel) */
    uint16_t *buf;
    int rows_pad, K;
    bool ok;
};

/* ---- tensor parallelism: every rank computes a slice of a GEMM's output tiles and stores
 * its results into every rank's copy of the output buffer (peer memory over NVLink); the
 * consumers wait for a per-site sequence number from every rank. ---- */
constexpr int kTpMaxRanks = 8;

/* Producer side: where a GEMM's results also go, and how completion is published: the last
 * CTA of the launch (a local ticket) writes a sequence number, (frame - 1) * visits_per_frame +
 * visit, into a flag word on every destination. (Counting every CTA in with remote atomics
 * instead was measured slower: 4.6-4.9 ms against 4.3 ms per frame at two GPUs.) */
struct TcPush {
    int n_dst = 0;                        /* 0: single GPU, nothing below is used */
    long long dst_off[kTpMaxRanks] = {};  /* byte offset from the local buffer to destination d's copy (0 = local) */
    unsigned *flag[kTpMaxRanks] = {};     /* destination d's flag word for (this buffer, this rank) */
    unsigned *ticket = nullptr;           /* local counter */
    const unsigned *epoch = nullptr;      /* device word: frame number, 1-based */
    int visits_per_frame = 0, visit = 0;  /* this buffer is exchanged visits_per_frame times per frame; 1-based index */
};

/* Consumer side: do not read the exchanged buffer before every rank has published the visit. */
struct TcWait {
    const unsigned *flags = nullptr;      /* [n] local flag words, one per source rank */
    int n = 0;                            /* 0: nothing to wait for */
    const unsigned *epoch = nullptr;
    int visits_per_frame = 0, visit = 0;
    int *status = nullptr;
};

/* Kernels that can wait for exchanged data come in two instantiations; the single-GPU one
 * takes an empty parameter. */
struct TcNoWait {};
template <bool TP> struct TcWaitSel { using type = TcNoWait; };
template <> struct TcWaitSel<true> { using type = TcWait; };

/* One GEMM launch. */
struct TcGemm {
    int M = 0, splits = 1, epi = TC_EPI_STORE;
    float *out = nullptr;
    int ld_out = 0;
    const float *bias = nullptr;
    const float *ssq = nullptr;       /* [M][ssq_chunks] sums of squares of the un-normalised rows:  */
    int ssq_chunks = 0;               /* the result is scaled by 1/sqrt(sum/K + eps) per row          */
    float eps = 0.0f;
    uint16_t *out_terms = nullptr;    /* TC_EPI_SWIGLU_TERMS destination [3][out_rows_pad][N/2] */
    int out_rows_pad = 0;
    int *status = nullptr;            /* device int, set non-zero when a bounded wait runs out */
    int tile0 = 0, n_tiles = 0;       /* output tiles [tile0, tile0 + n_tiles) of the weight matrix; 0 = all */
    TcPush push;
    TcWait wait;                      /* the activation terms (and ssq) are exchanged data */
};

int tc_init();                                     /* resolves cuTensorMapEncodeTiled; 0 when usable */
int tc_weight(TcWeight *w, const uint16_t *d_W, int N, int K);
/* Same, on a tile-contiguous copy of W written to d_tiled (tc_tiled_bytes(N, K) bytes). */
int tc_weight_tiled(TcWeight *w, const uint16_t *d_W, int N, int K, uint16_t *d_tiled, cudaStream_t st);
size_t tc_tiled_bytes(int N, int K);
int tc_acts(TcActs *a, uint16_t *d_buf, int rows_pad, int K);
size_t tc_acts_bytes(int rows_pad, int K);
int tc_rows_pad(int M);                            /* 16, 64, 256; 0 when M is too large */
int tc_rows_pad_frame(int M);                      /* 16, 48, 64, 256: the tile of the frame's GEMMs */
int tc_rows_pad_any(int M);                        /* same, and whole 128-row blocks beyond 256 rows */
int tc_pick_splits(int N, int K, int n_sm);
int tc_prepare_chunks(int K);                      /* column chunks (and ssq entries) per row */

/* Rows -> BF16 terms in `acts`. Source: x[M, ldx], or residual[M, ldx] + the sum of n_part
 * split-K partial buffers ([M, K] each, part_stride floats apart). x_out (optional) receives the
 * fp32 rows. With `gain` the terms hold row*gain and ssq[m][chunk] the chunk's sum of squares
 * (RMSNorm's scalar is applied by the consuming GEMM). */
void tc_prepare(const TcActs &acts, const float *x, int ldx, int M, const float *partials, int n_part,
                size_t part_stride, const float *residual, float *x_out, const float *gain, float *ssq,
                cudaStream_t st, const TcWait &wait = TcWait(), float *tap = nullptr);

int tc_gemm(const TcWeight &w, const TcActs &acts, const TcGemm &g, cudaStream_t st);

void tc_reduce(float *y, const float *partials, int n_part, size_t stride, size_t count, const float *bias, int N,
               cudaStream_t st);

int tc_probe(int M, int N, int K, int epi, int tiled, int reps, int n_sm, float *ms_out, int *splits_out);

/* Launch with the programmatic-stream-serialization attribute: the kernel may begin (weight
 * prefetch, barrier set-up, TMEM allocation) while its predecessor in the stream is still
 * running; whatever depends on the predecessor sits behind griddepcontrol.wait in the kernel.
 * VB200_NO_PDL=1 turns the attribute off. */
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args... args) {
    static const bool no_pdl = getenv("VB200_NO_PDL") != nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = no_pdl ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

} // namespace vb

#endif
