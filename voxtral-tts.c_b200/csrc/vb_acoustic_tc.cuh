/*
 * vb_acoustic_tc.cuh - the tensor-core acoustic path's buffers, shared between the
 * single-utterance frame (vb_acoustic_tc.cu) and the batched frame (vb_batch.cu).
 */
#ifndef VB_ACOUSTIC_TC_CUH
#define VB_ACOUSTIC_TC_CUH

#include <vector>

#include "vb_model.cuh"
#include "vb_tc.cuh"

namespace vb {

/* Element strides from one utterance of a batch to the next. */
struct AcStrides {
    int lat = 0, vel = 0, codes = 0;
    size_t noise = 0, codes_all = 0;
};

/* Activation buffers of the Euler loop for B utterances: 6 token rows each. */
struct AcBuffers {
    int B = 0, rows = 0, rows_pad = 0;
    TcActs aD, aQ, aH;             /* BF16 terms feeding the GEMMs (K = 3072, 4096, 9216) */
    uint16_t *bD = nullptr, *bQ = nullptr, *bH = nullptr;
    float *part = nullptr;         /* split-K partials [splits][rows][N] */
    float *ssq = nullptr;          /* per-row, per-chunk sums of squares (deferred RMSNorm scale) */
    float *X6 = nullptr;           /* residual stream [rows][3072] */
    /* supplied by the owner, strided per utterance by `sd` */
    float *lat = nullptr, *vel = nullptr, *ltok = nullptr;
    int *codes = nullptr;
    VbDyn *dyn = nullptr;
    int *status = nullptr;
    AcStrides sd;
};

/* Allocates bD/bQ/bH/part/ssq (and X6 when it is null) for B utterances; pointers are
 * appended to `owner` for the caller to free. */
int acoustic_buffers_alloc(AcBuffers *b, int B, std::vector<void *> *owner);

/* Enqueues 7 Euler steps + FSQ for every utterance of `b` on the library's stream. */
int acoustic_tc_enqueue_on(const AcBuffers &b, const float *noise_all, int *codes_all, int frame_cap, bool advance,
                           bool ignore_end);

} // namespace vb

#endif
