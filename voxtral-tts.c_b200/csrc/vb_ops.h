/*
 * vb_ops.h - the op list ("program") a persistent frame kernel executes.
 *
 * One launch of the engine kernel walks an array of VbOp in device memory.
 * Every CTA executes every op on its share of the work; a grid-wide barrier
 * separates dependent ops. Weight matrices named by GEMV ops are streamed
 * through a shared-memory ring by a producer thread that runs ahead of the
 * barriers, so HBM stays busy while the rest of the CTA waits.
 */
#ifndef VB_OPS_H
#define VB_OPS_H

#include <stdint.h>

enum VbOpType {
    VB_OP_GEMV = 1,        /* y[M,N] = epi(W[N,K] . pro(x[M,K])) */
    VB_OP_ATTN_DECODE = 2, /* RoPE + cache append + GQA attention for one new token */
    VB_OP_ATTN_AC = 3,     /* unmasked 3-token attention, batched sequences */
    VB_OP_NORM = 4,        /* y[M,K] = rmsnorm(x[M,K]) * norm_w */
    VB_OP_AC_TOKENS = 5,   /* Euler update + build the six acoustic input rows */
    VB_OP_ARGMAX = 6,      /* masked first-maximum over semantic logits */
    VB_OP_FSQ = 7,         /* last Euler update + quantise the latent to codes */
    VB_OP_EMBED = 8,       /* next decoder input from 37 codes (sum of BF16 rows) */
    VB_OP_ADVANCE = 9      /* end of a device-resident frame: pos++, frame++, END check */
};

enum VbEpilogue {
    VB_EPI_STORE = 0,  /* y = Wx (+bias) */
    VB_EPI_ADD = 1,    /* y = res + Wx */
    VB_EPI_SWIGLU = 2  /* rows interleaved (gate,up): y[n/2] = silu(gate)*up */
};

enum VbOpFlags {
    VB_F_NOSYNC = 1,   /* no grid barrier after this op (next op is independent) */
    VB_F_LAST_TOKEN = 2
};

/* Per-launch scalars, read from device memory so one program serves all frames. */
struct VbDyn {
    int pos;           /* cache row of the token being decoded */
    int kv_max;        /* rows per layer in the cache */
    int frame;         /* frames completed in a device-resident run (indexes noise / code arrays) */
    int done;          /* set once an END code was produced: later launches of the run return at once */
};

struct VbOp {
    int type, M, N, K;
    int epi, ldx, ldy, flags;
    const uint16_t *W;    /* BF16 [N,K] row-major */
    const float *x;       /* [M, ldx] */
    float *y;             /* [M, ldy] */
    const float *res;     /* VB_EPI_ADD source, may alias y */
    const float *norm_w;  /* non-null: RMSNorm prologue with this gain */
    const float *bias;    /* [N] or null */
    float *tap;           /* optional copy of the epilogue result [M, ldy] */
    const void *p0;       /* op-specific pointers */
    const void *p1;
    void *p2;
    void *p3;
    float eps, f0, f1, f2;
    int i0, i1, i2, i3;
};

/* Status word values written by the kernel on a failed bounded wait. */
enum VbStatus {
    VB_OK = 0,
    VB_ERR_GRID_BARRIER = 1,
    VB_ERR_FULL_WAIT = 2,
    VB_ERR_EMPTY_WAIT = 3,
    VB_ERR_DONE_WAIT = 4,
    VB_ERR_BAD_OP = 5,
    VB_ERR_POS_RANGE = 6,
    VB_ERR_DRAIN = 7
};

#endif
