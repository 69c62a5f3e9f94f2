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

namespace vb {

constexpr int kTcTileN = 128;     /* weight rows per CTA tile = UMMA M */
constexpr int kTcBlockK = 64;     /* K elements per pipeline stage: one 128-byte swizzle row */
constexpr int kTcTerms = 3;       /* BF16 terms per fp32 activation */
constexpr int kTcMaxSplits = 8;   /* split-K factor limit (partials are summed in fixed order) */

enum TcEpilogue {
    TC_EPI_PARTIAL = 0,  /* out[split][m][n] = partial sum (fp32) */
    TC_EPI_STORE = 1,    /* splits == 1: out[m][n] = sum (+ bias[n]) */
    TC_EPI_SWIGLU = 2    /* splits == 1, rows interleaved (gate, up): out[m][n/2] = silu(gate) * up */
};

/* One weight matrix prepared for the tensor-core path. */
struct TcWeight {
    CUtensorMap map;     /* [N, K] BF16 row-major, box 64 x 128, 128-byte swizzle */
    const uint16_t *W;
    int N, K;
    bool ok;
};

/* Activation rows split into BF16 terms: [terms][rows_pad][K], rows_pad = 16, 64 or 256. */
struct TcActs {
    CUtensorMap map;
    uint16_t *buf;
    int rows_pad, K;
    bool ok;
};

int tc_init();                                     /* resolves cuTensorMapEncodeTiled; 0 when usable */
int tc_weight(TcWeight *w, const uint16_t *d_W, int N, int K);
int tc_acts(TcActs *a, uint16_t *d_buf, int rows_pad, int K);
size_t tc_acts_bytes(int rows_pad, int K);
int tc_rows_pad(int M);                            /* 16, 64, 256; 0 when M is too large */
int tc_pick_splits(int N, int K, int n_sm);

/* x[M,K] fp32 (optionally: sum of `n_part` partial buffers + residual, optionally RMS-normalised
 * with `gain`) -> BF16 terms in `acts`; optionally also stores the summed fp32 rows to x_out. */
void tc_prepare(const TcActs &acts, const float *x, int ldx, int M, const float *partials, int n_part,
                size_t part_stride, const float *residual, float *x_out, const float *gain, float eps,
                cudaStream_t st);

/* Launches the GEMM. out layout by epilogue (see TcEpilogue). status: device int, set non-zero
 * when a bounded wait runs out. */
int tc_gemm(const TcWeight &w, const TcActs &acts, int M, float *out, int ld_out, int splits, int epi,
            const float *bias, int *d_status, cudaStream_t st);

void tc_reduce(float *y, const float *partials, int n_part, size_t stride, size_t count, const float *bias, int N,
               cudaStream_t st);

} // namespace vb

#endif
