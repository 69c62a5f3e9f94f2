/*
 * vb_stream.cuh - the persistent streaming decoder-step kernel: op list, work split and
 * launch interface (kernel in vb_stream.cu).
 *
 * One cooperative launch (one CTA per SM) runs the whole decoder step of a frame
 * (tts_llm_forward, voxtral_tts_llm.c:171-271) plus the two M = 1 heads that follow it
 * (semantic logits + argmax, llm token: voxtral_tts_acoustic.c:283-309, :204). Every
 * matrix is stored a second time in "slab" order: CTA c owns a fixed, contiguous range
 * of output rows of every matrix, and its rows are laid out k-block by k-block
 * ([K/64][rows][64] BF16, the eight 16-byte chunks of a row XOR-swizzled by the row index so that
 * ldmatrix reads them without bank conflicts), so that the bytes a CTA needs for an op form ONE contiguous
 * range that a producer thread copies into a shared-memory ring with plain 1-D bulk
 * copies (cp.async.bulk), without ever waiting for the op's input: the HBM stream keeps
 * running across op boundaries while the other warps synchronise.
 */
#ifndef VB_STREAM_CUH
#define VB_STREAM_CUH

#include <cuda_runtime.h>
#include <stdint.h>

#include "vb_ops.h"

namespace vb {

constexpr int kSConsumerWarps = 12;
constexpr int kSConsumerThreads = kSConsumerWarps * 32;
constexpr int kSThreads = kSConsumerThreads + 32;      /* + the producer warp */
constexpr int kSSlotBytes = 16384;                     /* one ring slot: whole k-blocks of the CTA's rows */
constexpr int kSSlots = 10;
constexpr int kSBlockK = 64;                           /* columns per k-block: 128 bytes per row */
constexpr int kSMaxRows = kSSlotBytes / (kSBlockK * 2);/* 128 rows per CTA per op: one k-block fits a slot */
constexpr int kSMaxRowTiles = kSMaxRows / 16;          /* 16-row MMA tiles per CTA per op */
constexpr int kSMaxK = 9216;
constexpr int kSHeadDim = 128;
constexpr int kSPrefetchBytes = 0;            /* default L2 prefetch distance per CTA */

enum SOpType {
    S_OP_GEMV = 1,      /* y[N] = epi(W[N,K] . pro(x[K])) */
    S_OP_ATTN = 2,      /* RoPE + cache append + GQA decode attention for one new token */
    S_OP_EMBED = 3,     /* decoder input from the previous frame's 37 codes */
    S_OP_ARGMAX = 4,    /* masked first-maximum over the semantic logits */
    S_OP_WAIT = 5,      /* wait (bounded) until a global word reaches a value */
    S_OP_ATTN_MERGE = 6 /* merges the key slices of S_OP_ATTN */
};

enum SEpi { S_EPI_STORE = 0, S_EPI_ADD = 1, S_EPI_SWIGLU = 2 };

enum SFlags {
    S_F_NOSYNC = 1,       /* no grid barrier after this op */
    S_F_SKIP_FRAME0 = 2,  /* S_OP_EMBED: frame 0 of a run keeps the row the host supplied */
    /* Tagged vectors: every element is 8 bytes, {fp32 value, 32-bit tag}, written with one
     * 64-bit store. The tag names the op (and the launch) that produced the element, so a reader
     * needs no barrier: it loads the element and looks at the tag, and loads again if the
     * producer has not got there yet. Exchange and readiness check are one trip to L2. */
    S_F_X_TAGGED = 4,     /* x (S_OP_GEMV, S_OP_ATTN) is tagged and carries tag x_tag */
    S_F_Y_TAGGED = 8,     /* y is written tagged with y_tag */
    S_F_RES_TAGGED = 16   /* res is a tagged vector (read by the thread that wrote it: no check) */
};

typedef unsigned long long stag_t;   /* one tagged element */

struct SOp {
    int type, N, K, epi;
    int flags, i0, i1, i2;
    const uint16_t *W;      /* slab layout (stream_slab_bytes(N, K) bytes) */
    const float *x;         /* [K] */
    const float *gain;      /* non-null: RMSNorm prologue, x * gain with the row scale applied to the sums */
    float *y;               /* [N] ([N/2] for S_EPI_SWIGLU) */
    const float *res;       /* S_EPI_ADD: y = res + W.x (may alias y) */
    const float *bias;      /* [N] or null */
    float *tap;             /* optional copy of y */
    float *xn_out;          /* optional: CTA 0 stores the normalised input row rmsnorm(x) * gain */
    const void *p0;
    const void *p1;
    void *p2;
    void *p3;
    float eps, f0, f1, f2;
    int x_tag, y_tag;       /* 1 .. 255, unique per producing op within a launch */
    int pad0, pad1;
};

/* How one GEMV op is cut for one CTA. Rows are dealt out in units (1 row, or a
 * (gate, up) pair); the first `rem` CTAs take one unit more. A ring slot holds `kbs` whole
 * k-blocks of the CTA's rows; slot s belongs to consumer warp s for the whole launch (one
 * waiter per mbarrier, which therefore sees every phase of it in order), and the owner walks
 * all T 16-row tiles of every k-block in its slot. */
struct SPlan {
    int r0, n_rows;     /* this CTA's rows */
    int kblocks;        /* K / 64 */
    int kbs;            /* k-blocks per ring slot */
    int n_chunks;       /* ring slots this op takes */
    int T;              /* 16-row tiles: ceil(n_rows / 16) */
};

__host__ __device__ inline SPlan stream_plan(int N, int K, int epi, int cta, int n_cta) {
    SPlan p;
    const int unit = epi == S_EPI_SWIGLU ? 2 : 1;
    const unsigned U = (unsigned)(N / unit), nc = (unsigned)n_cta, q = U / nc, rem = U - q * nc;
    const unsigned c0 = (unsigned)cta, u0 = c0 * q + (c0 < rem ? c0 : rem);
    p.r0 = (int)u0 * unit;
    p.n_rows = (int)(q + (c0 < rem ? 1u : 0u)) * unit;
    p.kblocks = K / kSBlockK;
    p.kbs = p.n_rows > 0 ? kSSlotBytes / (p.n_rows * kSBlockK * 2) : 0;
    if (p.kbs > p.kblocks) p.kbs = p.kblocks;
    p.n_chunks = p.kbs > 0 ? (p.kblocks + p.kbs - 1) / p.kbs : 0;
    p.T = (p.n_rows + 15) / 16;
    return p;
}

/* 0 when the op can run on n_cta CTAs. */
inline int stream_validate(int N, int K, int epi, int n_cta) {
    if (N <= 0 || K <= 0 || (K % kSBlockK) != 0 || K > kSMaxK) return -1;
    if (epi == S_EPI_SWIGLU && (N & 1)) return -2;
    const SPlan p = stream_plan(N, K, epi, 0, n_cta);   /* CTA 0 has the most rows */
    if (p.n_rows > kSMaxRows) return -3;
    return 0;
}

inline size_t stream_slab_bytes(int N, int K) { return (size_t)N * K * 2; }

/* Re-lays a row-major [N, K] BF16 matrix out in slab order for n_cta CTAs. */
int stream_make_slabs(uint16_t *d_dst, const uint16_t *d_src, int N, int K, int epi, int n_cta, cudaStream_t st);

/* What the producer thread needs to know about a GEMV op, in program order. */
struct SWeights {
    const uint16_t *W;
    int N, K, epi, pad;
};

struct SArgs {
    const SOp *ops;
    int n_ops;
    const SWeights *wl;         /* the GEMV ops' weights, in the order the ops appear */
    int n_wl;
    VbDyn *dyn;
    unsigned *bar_counter;      /* grid barrier arrivals; zero between launches */
    unsigned *exit_counter;     /* CTAs that finished; the last one re-zeroes both */
    unsigned *seq;              /* launches so far: makes the tags of this launch differ from the last one's */
    int *status;                /* 0, or the code of the wait that ran out */
    long long wait_cycles;      /* limit of every wait inside the kernel */
};

/* Status codes of this kernel (distinct from the other kernels' codes). */
enum SStatus {
    S_ERR_GRID_BARRIER = 41, S_ERR_FULL_WAIT = 42, S_ERR_EMPTY_WAIT = 43, S_ERR_BAD_OP = 44,
    S_ERR_POS_RANGE = 45, S_ERR_DRAIN = 46, S_ERR_FLAG_WAIT = 47, S_ERR_DATA_WAIT = 48
};

/* CTAs of a launch on `device` (one per SM), or 0 when the kernel does not fit. */
int stream_max_ctas(int device);
cudaError_t stream_launch(const SArgs &args, int n_cta, cudaStream_t st);
int stream_probe(int N, int K, int n_ops, int sync, int reps, float *ms_out, double *bytes_per_launch);

} // namespace vb

#endif
