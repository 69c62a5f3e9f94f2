/*
 * vb_ptc.cu - persistent tensor-core kernel (sm_100a).
 *
 * The frame's GEMMs are HBM-bound streams of weight tiles separated by small dependent
 * steps. As separate launches every GEMM pays a ramp and a tail during which no weight
 * byte moves. Here one cooperative launch (one CTA per SM) walks a list of ops; the producer
 * thread streams the weight tiles of ALL ops, in program order, through a shared-memory ring
 * and is never held up by a dependency (weights depend on nothing), so tiles of the next op
 * are already in flight while the CTA finishes the current one.
 *
 *   y[M,N] = x[M,K] . W[N,K]^T   (tts_linear_nobias_bf16, voxtral_tts_kernels.c:187-198),
 *   BF16 W, fp32 x and y, M <= 10 rows.
 *
 * Per CTA: warp 4 lane 0 producer (1-D bulk copies of 16 KB pre-swizzled tile images,
 * no multicast), warps 6-7 build the B operand: they wait for the op's dependency, read the
 * fp32 activations of the next 64 columns, multiply by the RMSNorm gain, split each value
 * into three BF16 terms (hi + lo + lo2; exact products in fp32) and write them as rows
 * 3m..3m+2 of a swizzled K-major tile; warp 5 lane 0 issues tcgen05.mma (128 weight rows x
 * 16 or 32 B rows, accumulator in TMEM); warps 0-3 read the accumulator back, add the three
 * term columns, apply 1/sqrt(mean(x^2)+eps), and finish the op: SwiGLU, or split-K partials
 * with the last CTA of a tile (a ticket, no spin) summing them in split order, adding the
 * residual and writing the sums of squares the next RMSNorm needs. Ops are ordered by
 * completion counters in global memory (release increment, acquire poll by one thread):
 * no grid-wide barrier. Every wait is bounded; on expiry a status word is set, every role
 * falls through, copies in flight are drained and the TMEM columns are released.
 */
#include "vb_ptc.cuh"
#include "vb_umma.cuh"

#include <stdio.h>
#include <stdlib.h>
#include <vector>

namespace vb {

constexpr int kPSlots = 10;        /* weight ring: 160 KB in flight per SM */
constexpr int kPBSlots = 4;        /* activation ring */
constexpr int kPBBytes = 4096;     /* 32 rows x 64 BF16 */
constexpr int kPThreads = 320;      /* 4 epilogue warps, producer, MMA issuer, 4 B-operand warps */
constexpr int kPBThreads = 128;
constexpr int kPTmemCols = 32;
constexpr int kPXFloats = 10240;   /* 40 KB staging for activations: 160 k-blocks of one row, 16 of ten rows */

enum PStatus {
    P_ERR_PRODUCER = 21, P_ERR_MMA_A = 22, P_ERR_MMA_B = 23, P_ERR_MMA_ACC = 24, P_ERR_EPILOGUE = 25,
    P_ERR_BPREP = 26, P_ERR_DEPENDENCY = 27, P_ERR_BAD_OP = 28
};

struct PSmem {
    unsigned char a[kPSlots][kPTileBytes];
    unsigned char b[kPBSlots][kPBBytes];
    uint64_t a_full[kPSlots], a_empty[kPSlots], b_full[kPBSlots], b_empty[kPBSlots];
    uint64_t acc_full, acc_empty;
    uint32_t tmem;
    int abort_flag, last_flag;
    float rscale[16];
    float red[4][16];
    float xs[kPXFloats];          /* activations of the current chunk of k-blocks, x*gain, fp32 */
};

struct PArgs {
    const POp *ops;
    int n_ops;
    unsigned *done;
    unsigned epoch;
    int *status;
    long long *timeline;     /* optional [n_ops][8] timestamps (ns) written by CTA 0: where an op's time goes */
};

VB_DEVINL long long p_now() {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
VB_DEVINL void p_stamp(const PArgs &a, int oi, int k) {
    if (a.timeline && blockIdx.x == 0) a.timeline[oi * 8 + k] = p_now();
}

VB_DEVINL void p_raise(PSmem *s, const PArgs &a, int code) {
    atomicCAS(a.status, 0, code);
    *(volatile int *)&s->abort_flag = 1;
}
VB_DEVINL bool p_aborted(PSmem *s) { return *(volatile int *)&s->abort_flag != 0; }

VB_DEVINL void p_item(const POp &op, int item, int &tile, int &sp, int &kb0, int &kb1) {
    tile = item / op.splits;
    sp = item - tile * op.splits;
    const int kblocks = op.K >> 6;
    kb0 = (int)((long long)kblocks * sp / op.splits);
    kb1 = (int)((long long)kblocks * (sp + 1) / op.splits);
}

/* ---- producer: weight tiles of every op, in order, as far ahead as the ring allows ---- */
__device__ void p_producer(PSmem *s, const PArgs &a) {
    uint32_t cnt = 0;
    for (int oi = 0; oi < a.n_ops; oi++) {
        const POp &op = a.ops[oi];
        if (op.type != P_GEMM) continue;
        const int n_items = op.tiles * op.splits, kblocks = op.K >> 6;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            int tile, sp, kb0, kb1;
            p_item(op, item, tile, sp, kb0, kb1);
            const unsigned char *src = (const unsigned char *)op.W + ((size_t)tile * kblocks + kb0) * kPTileBytes;
            for (int kb = kb0; kb < kb1; kb++, cnt++, src += kPTileBytes) {
                const uint32_t slot = cnt % kPSlots, use = cnt / kPSlots;
                if (!vb_mbar_wait(&s->a_empty[slot], (use & 1u) ^ 1u, &s->abort_flag)) {
                    p_raise(s, a, P_ERR_PRODUCER);
                    return;
                }
                vb_mbar_arrive_expect_tx(&s->a_full[slot], (uint32_t)kPTileBytes);
                vb_bulk_g2s(s->a[slot], src, (uint32_t)kPTileBytes, &s->a_full[slot]);
            }
        }
    }
}

/* Waits until op `dep` has completed `count` units in this launch (one polling thread). */
VB_DEVINL bool p_wait_dep(PSmem *s, const PArgs &a, int dep, int count) {
    const unsigned target = a.epoch * (unsigned)count;
    const long long t0 = clock64();
    while ((int)(vb_ld_acquire_gpu(a.done + dep) - target) < 0) {
        if (p_aborted(s)) return false;
        if (clock64() - t0 > VB_WAIT_CYCLES) { p_raise(s, a, P_ERR_DEPENDENCY); return false; }
    }
    return true;
}

/* ---- B operand: activations -> three BF16 terms per value, swizzled K-major tile ---- */
__device__ void p_bprep(PSmem *s, const PArgs &a, int t) {
    uint32_t bcnt = 0;
    const int half = t >> 6, tc = t & 63;       /* two halves fill alternate k-blocks */
    for (int oi = 0; oi < a.n_ops; oi++) {
        const POp &op = a.ops[oi];
        if (op.type != P_GEMM) continue;
        if (t == 0) p_stamp(a, oi, 0);
        if (op.dep >= 0) {
            if (t == 0) p_wait_dep(s, a, op.dep, op.dep_count);
            vb_named_bar(3, kPBThreads);
            if (p_aborted(s)) return;
        }
        if (t == 0) p_stamp(a, oi, 1);
        const int M = op.M, n_items = op.tiles * op.splits;
        const int chunk_kb = kPXFloats / (64 * M);      /* k-blocks whose activations fit the staging buffer */
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            int tile, sp, kb0, kb1;
            p_item(op, item, tile, sp, kb0, kb1);
            for (int kc = kb0; kc < kb1; kc += chunk_kb) {
                const int kce = kc + chunk_kb < kb1 ? kc + chunk_kb : kb1;
                const int ncol = (kce - kc) * 64;
                /* stage x*gain for these columns: every load of the chunk is in flight at once */
                vb_named_bar(3, kPBThreads);            /* the previous chunk has been consumed */
                for (int m = 0; m < M; m++) {
                    const float *xr = op.x + (size_t)m * op.ldx + kc * 64;
                    for (int c0 = t; c0 < ncol; c0 += kPBThreads * 12) {
                        float xv[12], gv[12];
#pragma unroll
                        for (int i = 0; i < 12; i++) {
                            const int c = c0 + kPBThreads * i;
                            xv[i] = c < ncol ? __ldcg(xr + c) : 0.0f;
                            gv[i] = (c < ncol && op.gain) ? __ldg(op.gain + kc * 64 + c) : 1.0f;
                        }
#pragma unroll
                        for (int i = 0; i < 12; i++) {
                            const int c = c0 + kPBThreads * i;
                            if (c < ncol) s->xs[m * ncol + c] = xv[i] * gv[i];
                        }
                    }
                }
                vb_named_bar(3, kPBThreads);
                if (t == 0) p_stamp(a, oi, 2);
                for (int kb = kc + half; kb < kce; kb += 2) {
                    const uint32_t n = bcnt + (uint32_t)(kb - kc);
                    const uint32_t slot = n % kPBSlots, use = n / kPBSlots;
                    if (!vb_mbar_wait(&s->b_empty[slot], (use & 1u) ^ 1u, &s->abort_flag)) {
                        p_raise(s, a, P_ERR_BPREP);
                        return;
                    }
                    unsigned char *B = s->b[slot];
                    const int c = (kb - kc) * 64 + tc;
#pragma unroll
                    for (int m = 0; m < kPMaxRows; m++) {
                        if (m < M) {
                            uint16_t tk[3];
                            vb_split3(s->xs[m * ncol + c], tk[0], tk[1], tk[2]);
#pragma unroll
                            for (int q = 0; q < 3; q++) {
                                uint32_t o = (uint32_t)(3 * m + q) * 128u + (uint32_t)tc * 2u;
                                o ^= ((o >> 7) & 7u) << 4;     /* 128-byte swizzle: 16-byte chunk ^= row % 8 */
                                *reinterpret_cast<uint16_t *>(B + o) = tk[q];
                            }
                        }
                    }
                    /* the tensor core reads shared memory through the async proxy */
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    vb_mbar_arrive(&s->b_full[slot]);
                }
                bcnt += (uint32_t)(kce - kc);
            }
            if (t == 0) p_stamp(a, oi, 3);
        }
    }
}

/* ---- MMA issue ---- */
__device__ void p_mma(PSmem *s, const PArgs &a, uint32_t tmem) {
    uint32_t cnt = 0, bcnt = 0, ic = 0;
    for (int oi = 0; oi < a.n_ops; oi++) {
        const POp &op = a.ops[oi];
        if (op.type != P_GEMM) continue;
        const uint32_t idesc = umma_idesc_bf16(op.nb);
        const int n_items = op.tiles * op.splits;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ic++) {
            int tile, sp, kb0, kb1;
            p_item(op, item, tile, sp, kb0, kb1);
            if (!vb_mbar_wait(&s->acc_empty, (ic & 1u) ^ 1u, &s->abort_flag)) {
                p_raise(s, a, P_ERR_MMA_ACC);
                return;
            }
            tc_fence_after();
            for (int kb = kb0; kb < kb1; kb++, cnt++, bcnt++) {
                const uint32_t slot = cnt % kPSlots, use = cnt / kPSlots;
                const uint32_t bslot = bcnt % kPBSlots, buse = bcnt / kPBSlots;
                if (!vb_mbar_wait(&s->a_full[slot], use & 1u, &s->abort_flag)) {
                    p_raise(s, a, P_ERR_MMA_A);
                    return;
                }
                if (!vb_mbar_wait(&s->b_full[bslot], buse & 1u, &s->abort_flag)) {
                    p_raise(s, a, P_ERR_MMA_B);
                    return;
                }
                tc_fence_after();
                if (kb == kb0) p_stamp(a, oi, 4);
                const uint64_t adesc = umma_desc_k_sw128(s->a[slot]);
                const uint64_t bdesc = umma_desc_k_sw128(s->b[bslot]);
#pragma unroll
                for (int k = 0; k < 4; k++)
                    umma_bf16(tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                umma_commit(&s->a_empty[slot]);
                umma_commit(&s->b_empty[bslot]);
            }
            umma_commit(&s->acc_full);
            p_stamp(a, oi, 5);
        }
    }
}

/* ---- epilogue: TMEM -> registers -> op-specific finish ---- */
__device__ void p_epilogue(PSmem *s, const PArgs &a, uint32_t tmem, int tid) {
    const int warp = tid >> 5, lane = tid & 31;
    uint32_t ic = 0;
    for (int oi = 0; oi < a.n_ops; oi++) {
        const POp &op = a.ops[oi];
        if (op.type != P_GEMM) continue;
        const int M = op.M, N = op.N, n_items = op.tiles * op.splits;
        if (op.ssq && (int)blockIdx.x < n_items) {
            /* The activations went in as x*gain; 1/sqrt(mean(x^2)+eps) is applied to the
             * accumulators (tts_rms_norm, voxtral_tts_kernels.c:333-349). Warp 0 fetches the sums
             * of squares while the MMAs run: it waits for the op's dependency itself. */
            if (warp == 0) {
                bool ok = true;
                if (op.dep >= 0 && lane == 0) ok = p_wait_dep(s, a, op.dep, op.dep_count);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                for (int m = 0; m < M && ok; m++) {
                    float t = 0.0f;
                    for (int c = lane; c < op.ssq_n; c += 32) t += __ldcg(op.ssq + m * op.ssq_n + c);
                    t = vb_warp_sum(t);
                    if (lane == 0) s->rscale[m] = 1.0f / sqrtf(t / (float)op.K + op.eps);
                }
            }
            vb_named_bar(1, 128);
        }
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ic++) {
            int tile, sp, kb0, kb1;
            p_item(op, item, tile, sp, kb0, kb1);
            const int row = tile * 128 + tid;
            if (!vb_mbar_wait(&s->acc_full, ic & 1u, &s->abort_flag)) {
                p_raise(s, a, P_ERR_EPILOGUE);
                return;
            }
            tc_fence_after();
            if (tid == 0) p_stamp(a, oi, 6);
            uint32_t r0[16], r1[16];
            tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16), r0);
            if (op.nb > 16) tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + 16u, r1);
            else {
#pragma unroll
                for (int i = 0; i < 16; i++) r1[i] = 0u;
            }
            tc_fence_before();
            vb_mbar_arrive(&s->acc_empty);
            float v[kPMaxRows];
#pragma unroll
            for (int m = 0; m < kPMaxRows; m++) {
                /* B rows 3m, 3m+1, 3m+2 = the hi, lo, lo2 products of activation row m */
                const float d0 = __uint_as_float(3 * m < 16 ? r0[(3 * m) & 15] : r1[(3 * m) & 15]);
                const float d1 = __uint_as_float(3 * m + 1 < 16 ? r0[(3 * m + 1) & 15] : r1[(3 * m + 1) & 15]);
                const float d2 = __uint_as_float(3 * m + 2 < 16 ? r0[(3 * m + 2) & 15] : r1[(3 * m + 2) & 15]);
                v[m] = (d0 + d1) + d2;
                if (op.ssq && m < M) v[m] *= s->rscale[m];
            }
            if (op.epi == P_EPI_SWIGLU) {
#pragma unroll
                for (int m = 0; m < kPMaxRows; m++) {
                    if (m < M) {
                        const float other = __shfl_xor_sync(0xffffffffu, v[m], 1);
                        if ((lane & 1) == 0 && row < N)
                            op.y[(size_t)m * op.ldy + (row >> 1)] = (v[m] / (1.0f + expf(-v[m]))) * other;
                    }
                }
                /* bar.sync orders the CTA's stores before thread 0's release increment */
                vb_named_bar(1, 128);
                if (tid == 0) { vb_atomic_add_release_gpu(a.done + oi, 1u); p_stamp(a, oi, 7); }
                continue;
            }
            /* split-K partials, then the last CTA of this tile finishes it */
            if (row < N) {
#pragma unroll
                for (int m = 0; m < kPMaxRows; m++)
                    if (m < M) op.part[((size_t)sp * M + m) * N + row] = v[m];
            }
            vb_named_bar(1, 128);
            if (tid == 0) {
                int last = 0;
                if (!p_aborted(s)) {
                    const unsigned t = vb_atomic_add_acq_rel_gpu(&op.tickets[tile], 1u);
                    last = (t == (unsigned)(op.splits - 1));
                    if (last) op.tickets[tile] = 0u;
                }
                s->last_flag = last;
            }
            vb_named_bar(1, 128);
            if (tid == 0) p_stamp(a, oi, 7);
            if (!s->last_flag) continue;
            for (int m = 0; m < M; m++) {
                float pv[8];
#pragma unroll
                for (int p = 0; p < 8; p++)
                    pv[p] = (p < op.splits && row < N) ? __ldcg(op.part + ((size_t)p * M + m) * N + row) : 0.0f;
                /* the residual's load is in flight together with the partials' */
                const float rv = (op.res && row < N) ? __ldcg(op.res + (size_t)m * op.ldy + row) : 0.0f;
                float acc = 0.0f;
#pragma unroll
                for (int p = 0; p < 8; p++) acc += pv[p];     /* split order; unused splits add 0 */
                if (row < N) {
                    if (op.res) acc = rv + acc;
                    op.y[(size_t)m * op.ldy + row] = acc;
                } else {
                    acc = 0.0f;
                }
                if (op.ssq_out) {
                    const float ss = vb_warp_sum(acc * acc);
                    if (lane == 0) s->red[warp][m] = ss;
                }
            }
            if (op.ssq_out) {
                vb_named_bar(1, 128);
                if (tid < M)
                    op.ssq_out[tid * op.tiles + tile] = ((s->red[0][tid] + s->red[1][tid]) + s->red[2][tid]) + s->red[3][tid];
            }
            vb_named_bar(1, 128);
            if (tid == 0) vb_atomic_add_release_gpu(a.done + oi, 1u);
        }
    }
}

__global__ void __launch_bounds__(kPThreads, 1) vb_ptc_kernel(PArgs a) {
    extern __shared__ unsigned char p_smem_raw[];
    PSmem *s = reinterpret_cast<PSmem *>(((uintptr_t)p_smem_raw + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < kPSlots; i++) { vb_mbar_init(&s->a_full[i], 1); vb_mbar_init(&s->a_empty[i], 1); }
        for (int i = 0; i < kPBSlots; i++) { vb_mbar_init(&s->b_full[i], 64); vb_mbar_init(&s->b_empty[i], 1); }
        vb_mbar_init(&s->acc_full, 1);
        vb_mbar_init(&s->acc_empty, 128);
        s->abort_flag = 0;
        s->last_flag = 0;
        vb_mbar_init_fence();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(vb_smem_u32(&s->tmem)),
                     "r"((uint32_t)kPTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *(volatile uint32_t *)&s->tmem;

    if (warp == 4) {
        if (lane == 0) p_producer(s, a);
    } else if (warp == 5) {
        if (lane == 0) p_mma(s, a, tmem);
    } else if (warp >= 6) {
        p_bprep(s, a, tid - 192);
    } else {
        p_epilogue(s, a, tmem, tid);
    }

    tc_fence_before();
    __syncthreads();
    /* abort path: let copies already in flight land before the shared memory goes away */
    if (warp == 4 && lane == 0 && p_aborted(s)) {
        for (int i = 0; i < kPSlots; i++) {
            const long long t0 = clock64();
            while (!vb_mbar_try_wait(&s->a_full[i], 0u) && !vb_mbar_try_wait(&s->a_full[i], 1u)) {
                if (clock64() - t0 > VB_WAIT_CYCLES / 8) break;
            }
        }
    }
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)kPTmemCols)
                     : "memory");
    }
}

/* ------------------------------------------------------------------ host */
/* dst: for every tile and k-block the 16 KB image the tensor core expects in shared memory
 * (K-major rows of 128 bytes, 16-byte chunk index XOR row % 8), so that one linear bulk copy
 * fills a ring slot. Rows past N are zero. */
__global__ void vb_ptc_image_kernel(uint4 *dst, const uint4 *src, int N, int K) {
    const int kblocks = K >> 6;
    const size_t n_vec = (size_t)((N + 127) / 128) * kblocks * 1024;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_vec) return;
    const int p = (int)(i & 7);                /* chunk position inside the 128-byte row */
    const int r = (int)((i >> 3) & 127);       /* row inside the tile */
    const size_t blk = i >> 10;
    const int kb = (int)(blk % kblocks), t = (int)(blk / kblocks);
    const int j = p ^ (r & 7);                 /* the source chunk that lands at position p */
    const int row = t * 128 + r;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (row < N) val = src[((size_t)row * K + (size_t)kb * 64) / 8 + j];
    dst[i] = val;
}

size_t ptc_image_bytes(int N, int K) { return (size_t)((N + 127) / 128) * 128 * K * 2; }

int ptc_make_image(uint16_t *d_img, const uint16_t *d_W, int N, int K, cudaStream_t st) {
    if (N <= 0 || K <= 0 || (K & 63) || ((uintptr_t)d_img & 15) || ((uintptr_t)d_W & 15)) return -1;
    const size_t n_vec = ptc_image_bytes(N, K) / 16;
    vb_ptc_image_kernel<<<(unsigned)((n_vec + 255) / 256), 256, 0, st>>>((uint4 *)d_img, (const uint4 *)d_W, N, K);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int ptc_gemm_op(POp *op, int M, int N, int K, int epi, int n_sm) {
    if (M < 1 || M > kPMaxRows || N < 1 || K < 64 || (K & 63)) return -1;
    if (epi == P_EPI_SWIGLU && (N & 1)) return -1;
    op->type = P_GEMM; op->M = M; op->N = N; op->K = K; op->epi = epi;
    op->tiles = (N + 127) / 128;
    op->splits = epi == P_EPI_FIXUP ? tc_pick_splits(N, K, n_sm) : 1;
    op->nb = 3 * M <= 16 ? 16 : 32;
    return 0;
}

int ptc_units(const POp &op) { return op.tiles; }

static size_t ptc_smem_bytes() { return sizeof(PSmem) + 1024; }

int ptc_max_ctas() {
    static int cached = -1;
    if (cached >= 0) return cached;
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaFuncSetAttribute(vb_ptc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ptc_smem_bytes()) !=
        cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, vb_ptc_kernel, kPThreads, ptc_smem_bytes()) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cached = per_sm > 0 ? sms : 0;     /* one CTA per SM */
    return cached;
}

int ptc_launch(const PtcLaunch &l, int n_cta, cudaStream_t st) {
    const int max_cta = ptc_max_ctas();
    if (max_cta <= 0 || n_cta < 1 || !l.d_ops || l.n_ops < 1) return -1;
    if (n_cta > max_cta) n_cta = max_cta;
    PArgs a;
    a.ops = l.d_ops; a.n_ops = l.n_ops; a.done = l.d_done; a.epoch = l.epoch; a.status = l.d_status;
    a.timeline = l.d_timeline;
    void *params[] = {&a};
    /* cooperative: every CTA must be resident, ops wait on one another's completion counters */
    return cudaLaunchCooperativeKernel((const void *)vb_ptc_kernel, dim3(n_cta), dim3(kPThreads), params,
                                       ptc_smem_bytes(), st) == cudaSuccess
               ? 0
               : -1;
}

/* y[M,N] = x[M,K] . W[N,K]^T (or the SwiGLU of interleaved rows -> [M, N/2]) on device
 * buffers through a one-op program: a self-contained check and timing aid. */
int ptc_linear(float *d_y, const float *d_x, const uint16_t *d_W, int M, int K, int N, int swiglu, int reps,
               float *ms_out) {
    int dev = 0, n_sm = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    POp op = {};
    if (ptc_gemm_op(&op, M, N, K, swiglu ? P_EPI_SWIGLU : P_EPI_FIXUP, n_sm)) return -1;
    uint16_t *img = nullptr;
    float *part = nullptr;
    unsigned *tickets = nullptr, *done = nullptr;
    int *status = nullptr;
    POp *d_op = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    int rc = -1;
    do {
        if (cudaMalloc(&img, ptc_image_bytes(N, K)) != cudaSuccess ||
            cudaMalloc(&part, sizeof(float) * 8 * (size_t)M * N) != cudaSuccess ||
            cudaMalloc(&tickets, sizeof(unsigned) * op.tiles) != cudaSuccess ||
            cudaMalloc(&done, sizeof(unsigned) * 4) != cudaSuccess || cudaMalloc(&status, sizeof(int)) != cudaSuccess ||
            cudaMalloc(&d_op, sizeof(POp)) != cudaSuccess)
            break;
        cudaMemset(tickets, 0, sizeof(unsigned) * op.tiles);
        cudaMemset(done, 0, sizeof(unsigned) * 4);
        cudaMemset(status, 0, sizeof(int));
        if (ptc_make_image(img, d_W, N, K, 0)) break;
        op.W = img; op.x = d_x; op.ldx = K; op.part = part; op.y = d_y; op.ldy = swiglu ? N / 2 : N;
        op.tickets = tickets; op.dep = -1;
        if (cudaMemcpy(d_op, &op, sizeof(POp), cudaMemcpyHostToDevice) != cudaSuccess) break;
        if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) break;
        PtcLaunch l;
        l.d_ops = d_op; l.n_ops = 1; l.d_done = done; l.d_status = status;
        bool ok = true;
        unsigned epoch = 0;
        l.epoch = ++epoch;
        ok = ptc_launch(l, n_sm, 0) == 0;
        cudaEventRecord(e0, 0);
        for (int i = 0; i < reps && ok; i++) {
            l.epoch = ++epoch;
            ok = ptc_launch(l, n_sm, 0) == 0;
        }
        cudaEventRecord(e1, 0);
        if (!ok || cudaDeviceSynchronize() != cudaSuccess) break;
        int st = 0;
        cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost);
        if (st) {
            fprintf(stderr, "voxtral_b200: persistent GEMM kernel gave up with status %d\n", st);
            break;
        }
        if (ms_out) cudaEventElapsedTime(ms_out, e0, e1);
        rc = 0;
    } while (0);
    cudaGetLastError();
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(img); cudaFree(part); cudaFree(tickets); cudaFree(done); cudaFree(status); cudaFree(d_op);
    return rc;
}

} // namespace vb
