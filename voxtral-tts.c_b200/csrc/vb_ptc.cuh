/*
 * vb_ptc.cuh - persistent tensor-core kernel: one launch runs a list of ops, weight
 * tiles keep streaming across op boundaries. Host interface.
 */
#ifndef VB_PTC_CUH
#define VB_PTC_CUH

#include <cuda_runtime.h>
#include <stdint.h>

namespace vb {

constexpr int kPTileBytes = 16384;     /* one weight tile: 128 rows x 64 BF16 columns, swizzled image */
constexpr int kPMaxRows = 10;          /* activation rows an op can take (3 BF16 terms each, <= 32 B-operand rows) */

enum POpType { P_GEMM = 1 };
enum PEpilogue {
    P_EPI_FIXUP = 0,   /* split-K partials; the last CTA of a tile sums them: y = (res +) sum */
    P_EPI_SWIGLU = 1   /* splits == 1, rows interleaved (gate, up): y[n/2] = silu(gate) * up */
};

/* One op of the program (device memory). */
struct POp {
    int type, M, N, K;
    int tiles, splits, epi, nb;   /* nb: B-operand rows = 3*M rounded up to 16 */
    const uint16_t *W;            /* swizzled tile images, tile-major then k-block */
    const float *x;               /* activations [M][ldx] fp32 */
    int ldx;
    const float *gain;            /* [K] or null: terms hold x*gain */
    const float *ssq;             /* [M][ssq_n] sums of squares of x or null: result * 1/sqrt(sum/K + eps) */
    int ssq_n;
    float eps;
    float *part;                  /* [splits][M][N] */
    float *y;                     /* [M][ldy] */
    int ldy;
    const float *res;             /* [M][ldy] or null; may alias y */
    float *ssq_out;               /* [M][tiles] or null */
    unsigned *tickets;            /* [tiles] */
    int dep, dep_count;           /* op that must have completed dep_count units before x is read (-1: none) */
};

size_t ptc_image_bytes(int N, int K);
/* Row-major BF16 [N, K] -> swizzled tile images at d_img. */
int ptc_make_image(uint16_t *d_img, const uint16_t *d_W, int N, int K, cudaStream_t st);
/* Fills the derived fields of a GEMM op (tiles, splits, nb). */
int ptc_gemm_op(POp *op, int M, int N, int K, int epi, int n_sm);
int ptc_units(const POp &op);     /* completion units the op produces */

struct PtcLaunch {
    const POp *d_ops;
    int n_ops;
    unsigned *d_done;             /* [n_ops] completion counters, monotonic across launches */
    unsigned epoch;               /* launch number, 1-based: op i is complete at epoch * units(i) */
    int *d_status;
    long long *d_timeline = nullptr;   /* optional [n_ops][8] ns timestamps from CTA 0 (debug aid) */
};
int ptc_launch(const PtcLaunch &l, int n_cta, cudaStream_t st);
int ptc_max_ctas();
int ptc_linear(float *d_y, const float *d_x, const uint16_t *d_W, int M, int K, int N, int swiglu, int reps,
               float *ms_out);

} // namespace vb

#endif
