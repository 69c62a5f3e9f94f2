/*
 * vb_engine.cu - the persistent frame kernel (sm_100a).
 *
 * One cooperative launch, one CTA per SM, executes a whole program of ops
 * (vb_ops.h): the 26-layer decoder step, the flow-matching acoustic frame, or a
 * single op for the reference-compatible ABI entry points.
 *
 * Warp roles inside a CTA:
 *   warps 0..15  compute. In a GEMV each warp owns one 256-column slice of the
 *                current column segment; its 8 activations per row of x live in
 *                registers, weights come from the shared-memory ring as 128-bit
 *                loads, products accumulate in fp32 (BF16 -> fp32 is an exact
 *                shift, as in voxtral_tts_kernels.c:49-53,177-182).
 *   warp 16      epilogue. Adds the 16 per-warp partials of a chunk in fixed
 *                order (deterministic), applies bias / residual / SwiGLU
 *                (voxtral_tts_llm.c:245-263) and stores to global memory. The
 *                partials travel through their own small ring, so a ring slot
 *                goes back to the producer as soon as its weights are in
 *                registers.
 *   warp 17      producer. Lane 0 walks the whole program ahead of everyone and
 *                keeps the ring full with 1-D bulk (TMA) copies of weight rows,
 *                and further ahead pulls the coming chunks into L2
 *                (cp.async.bulk.prefetch.L2); it never waits at a grid barrier,
 *                so HBM keeps streaming the next op's weights while the other
 *                warps synchronise.
 *
 * Every wait (mbarrier, grid barrier) is bounded; on expiry a status code is
 * stored, the CTA's abort flag is raised and all roles fall through to the exit
 * path, where the producer waits (bounded) for its copies in flight.
 */
#include "vb_engine.cuh"
#include "vb_common.cuh"

#include <cooperative_groups.h>

namespace vb {

struct Ctx {
    SmemLayout *s;
    EngineArgs a;
    int tid, warp, lane;
    unsigned chunk_counter;   /* chunks consumed/produced so far by this role */
    unsigned barrier_epoch;   /* grid barriers passed */
};

VB_DEVINL bool aborted(const Ctx &c) { return *(volatile int *)&c.s->abort_flag != 0; }

VB_DEVINL void raise_abort(Ctx &c, int code) {
    atomicCAS(c.a.status, 0, code);
    *(volatile int *)&c.s->abort_flag = 1;
}

/* ------------------------------------------------------------------ */
/* grid barrier for the 17 working warps (compute + epilogue)          */
/* ------------------------------------------------------------------ */
__device__ void grid_sync(Ctx &c) {
    c.barrier_epoch++;
    vb_named_bar(1, kWorkThreads);
    if (c.tid == 0 && !aborted(c)) {
        __threadfence();
        vb_atomic_add_release_gpu(c.a.bar_counter, 1u);
        const unsigned target = c.barrier_epoch * gridDim.x;
        long long t0 = clock64();
        while (vb_ld_acquire_gpu(c.a.bar_counter) < target) {
            if (vb_ld_relaxed_gpu_s32(c.a.status) != 0) { *(volatile int *)&c.s->abort_flag = 1; break; }
            if (clock64() - t0 > VB_WAIT_CYCLES) { raise_abort(c, VB_ERR_GRID_BARRIER); break; }
        }
        __threadfence();
    }
    vb_named_bar(1, kWorkThreads);
}

/* ------------------------------------------------------------------ */
/* GEMV: producer side                                                 */
/* ------------------------------------------------------------------ */
/* One thread feeds the ring. Everything that can be hoisted out of the per-chunk
 * path is: a chunk costs a bounded wait, one expect_tx and one bulk copy (or one
 * per row when K is cut into column passes). `issued_bytes` in shared memory tells
 * the prefetch warp how far the loads have got. */
__device__ void produce_all(Ctx &c) {
    SmemLayout *s = c.s;
    unsigned long long issued = 0;
    for (int oi = 0; oi < c.a.n_ops; oi++) {
        const VbOp &op = c.a.ops[oi];
        if (op.type != VB_OP_GEMV) continue;
        const GemvPlan p = gemv_plan(op.N, op.K, op.M, op.epi, blockIdx.x, gridDim.x);
        if (p.n_chunks == 0) continue;
        const size_t K = (size_t)op.K;
        const int rpc = p.rows_per_chunk;
        for (int pass = 0; pass < p.passes; pass++) {
            const int k0 = pass * p.seg_cols;
            const uint32_t row_bytes = (uint32_t)min(p.seg_cols, op.K - k0) * 2u;
            const uint16_t *src = op.W + (size_t)p.r0 * K + k0;
            int rows_left = p.r1 - p.r0;
            for (int rb = 0; rb < p.row_blocks; rb++, src += (size_t)rpc * K, rows_left -= rpc) {
                const int rc = min(rpc, rows_left);
                const unsigned slot = c.chunk_counter % kSlots;
                const unsigned use = c.chunk_counter / kSlots;
                c.chunk_counter++;
                if (!vb_mbar_wait(&s->empty[slot], (use & 1u) ^ 1u, &s->abort_flag)) {
                    if (!aborted(c)) raise_abort(c, VB_ERR_EMPTY_WAIT);
                    return;
                }
                unsigned char *dst = s->ring[slot];
                const uint32_t bytes = row_bytes * (uint32_t)rc;
                vb_mbar_arrive_expect_tx(&s->full[slot], bytes);
                if (p.passes == 1) {
                    vb_bulk_g2s(dst, src, bytes, &s->full[slot]);
                } else {
                    for (int i = 0; i < rc; i++)
                        vb_bulk_g2s(dst + (size_t)i * p.seg_cols * 2, src + (size_t)i * K, row_bytes, &s->full[slot]);
                }
                issued += bytes;
                *(volatile unsigned long long *)&s->issued_bytes = issued;
            }
        }
    }
    *(volatile unsigned long long *)&s->issued_bytes = ~0ull; /* done: nothing left to run ahead of */
}

/* L2 warm-up ahead of the ring. A second thread walks the same weights in the same
 * order, as plain byte ranges (a CTA's rows of one matrix are contiguous), and keeps
 * `lead` bytes ahead of the loads with cp.async.bulk.prefetch.L2. The ring alone
 * holds about 4 us of HBM traffic; the prefetched window keeps HBM streaming through
 * the longer stalls at op boundaries (grid barrier, prologue, attention). */
__device__ void prefetch_all(Ctx &c) {
    SmemLayout *s = c.s;
    const unsigned long long lead = (unsigned long long)c.a.prefetch_chunks * kSlotBytes;
    if (lead == 0) return;
    unsigned long long ahead = 0;
    for (int oi = 0; oi < c.a.n_ops; oi++) {
        const VbOp &op = c.a.ops[oi];
        if (op.type != VB_OP_GEMV) continue;
        const GemvPlan p = gemv_plan(op.N, op.K, op.M, op.epi, blockIdx.x, gridDim.x);
        if (p.n_chunks == 0) continue;
        const unsigned char *ptr = (const unsigned char *)(op.W + (size_t)p.r0 * op.K);
        size_t left = (size_t)(p.r1 - p.r0) * op.K * 2;
        while (left > 0) {
            long long t0 = clock64();
            while (true) {
                const unsigned long long done = *(volatile unsigned long long *)&s->issued_bytes;
                if (done == ~0ull || aborted(c)) return;
                if (ahead < done + lead) break;
                if (clock64() - t0 > VB_WAIT_CYCLES) return; /* only a hint: give up quietly */
                __nanosleep(64);
            }
            const uint32_t n = (uint32_t)(left < (size_t)kSlotBytes ? left : (size_t)kSlotBytes);
            vb_prefetch_l2(ptr, n);
            ptr += n;
            left -= n;
            ahead += n;
        }
    }
}

/* ------------------------------------------------------------------ */
/* GEMV: compute warps                                                 */
/* ------------------------------------------------------------------ */
template <int M>
__device__ void gemv_compute(Ctx &c, const VbOp &op, int op_index) {
    SmemLayout *s = c.s;
    const GemvPlan p = gemv_plan(op.N, op.K, M, op.epi, blockIdx.x, gridDim.x);
    const int K = op.K;
    float(*red)[kMaxM] = s->red[op_index & 1];
    const bool norm_from_regs = op.norm_w && p.passes == 1;

    /* RMSNorm prologue (voxtral_tts_kernels.c:333-349) when K needs several column
     * passes: the sum of squares is taken over the whole row first. With a single
     * pass the CTA's warps together hold the whole row in registers and the sum
     * comes from there (below), saving one trip to L2. */
    if (op.norm_w && !norm_from_regs) {
        float ss[M];
#pragma unroll
        for (int m = 0; m < M; m++) ss[m] = 0.0f;
        for (int i = c.tid * 4; i < K; i += kComputeThreads * 4) {
#pragma unroll
            for (int m = 0; m < M; m++) {
                float4 v = vb_ldcg4(op.x + (size_t)m * op.ldx + i);
                ss[m] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        }
#pragma unroll
        for (int m = 0; m < M; m++) {
            float t = vb_warp_sum(ss[m]);
            if (c.lane == 0) red[c.warp][m] = t;
        }
        vb_named_bar(2, kComputeThreads);
    }

    for (int pass = 0; pass < p.passes; pass++) {
        const int k0 = pass * p.seg_cols;
        const int klen = min(p.seg_cols, K - k0);
        const int col = c.warp * kSliceCols + c.lane * 8;   /* within the segment */
        const bool active = col < klen;

        float xr[M][8];
        float g[8];
        if (active) {
#pragma unroll
            for (int m = 0; m < M; m++) {
                const float *px = op.x + (size_t)m * op.ldx + k0 + col;
                float4 a = vb_ldcg4(px), b = vb_ldcg4(px + 4);
                xr[m][0] = a.x; xr[m][1] = a.y; xr[m][2] = a.z; xr[m][3] = a.w;
                xr[m][4] = b.x; xr[m][5] = b.y; xr[m][6] = b.z; xr[m][7] = b.w;
            }
            if (op.norm_w) {
                const float4 ga = __ldg(reinterpret_cast<const float4 *>(op.norm_w + k0 + col));
                const float4 gb = __ldg(reinterpret_cast<const float4 *>(op.norm_w + k0 + col + 4));
                g[0] = ga.x; g[1] = ga.y; g[2] = ga.z; g[3] = ga.w;
                g[4] = gb.x; g[5] = gb.y; g[6] = gb.z; g[7] = gb.w;
            }
        } else {
#pragma unroll
            for (int m = 0; m < M; m++)
#pragma unroll
                for (int j = 0; j < 8; j++) xr[m][j] = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; j++) g[j] = 0.0f;
        }
        if (norm_from_regs) {
#pragma unroll
            for (int m = 0; m < M; m++) {
                float t = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; j++) t = fmaf(xr[m][j], xr[m][j], t);
                t = vb_warp_sum(t);
                if (c.lane == 0) red[c.warp][m] = t;
            }
            vb_named_bar(2, kComputeThreads);
        }
        if (op.norm_w) {
#pragma unroll
            for (int m = 0; m < M; m++) {
                float t = 0.0f;
#pragma unroll
                for (int w = 0; w < kComputeWarps; w++) t += red[w][m];
                const float ri = 1.0f / sqrtf(t / (float)K + op.eps);
#pragma unroll
                for (int j = 0; j < 8; j++) xr[m][j] = xr[m][j] * ri * g[j];
            }
        }

        const int pitch = p.seg_cols * 2; /* bytes between rows inside a slot */
        for (int rb = 0; rb < p.row_blocks; rb++) {
            const int row = p.r0 + rb * p.rows_per_chunk;
            const int rc = min(p.rows_per_chunk, p.r1 - row);
            const unsigned chunk = c.chunk_counter++;
            const unsigned slot = chunk % kSlots, use = chunk / kSlots;
            const unsigned pslot = chunk % kPartSlots, puse = chunk / kPartSlots;
            if (!vb_mbar_wait(&s->full[slot], use & 1u, &s->abort_flag)) {
                if (!aborted(c)) raise_abort(c, VB_ERR_FULL_WAIT);
                return;
            }
            constexpr int RPC = rows_cap(M);
            float acc[RPC * M];
#pragma unroll
            for (int v = 0; v < RPC * M; v++) acc[v] = 0.0f;
            if (active) {
                const unsigned char *base = s->ring[slot] + (size_t)col * 2;
                /* rows past the end of a ragged last chunk re-read its last row; their
                 * sums are ignored by the epilogue, and the loads stay unconditional */
                uint4 wv[RPC];
#pragma unroll
                for (int i = 0; i < RPC; i++)
                    wv[i] = *reinterpret_cast<const uint4 *>(base + (size_t)min(i, rc - 1) * pitch);
#pragma unroll
                for (int i = 0; i < RPC; i++) {
                    float wf[8];
                    wf[0] = vb_bf16_lo(wv[i].x); wf[1] = vb_bf16_hi(wv[i].x);
                    wf[2] = vb_bf16_lo(wv[i].y); wf[3] = vb_bf16_hi(wv[i].y);
                    wf[4] = vb_bf16_lo(wv[i].z); wf[5] = vb_bf16_hi(wv[i].z);
                    wf[6] = vb_bf16_lo(wv[i].w); wf[7] = vb_bf16_hi(wv[i].w);
#pragma unroll
                    for (int m = 0; m < M; m++) {
                        float a = 0.0f;
#pragma unroll
                        for (int j = 0; j < 8; j++) a = fmaf(wf[j], xr[m][j], a);
                        acc[i * M + m] = a;
                    }
                }
            }
            /* the weights are in registers: hand the ring slot back to the producer */
            __syncwarp();
            if (c.lane == 0) vb_mbar_arrive(&s->empty[slot]);

            const int idx = vb_warp_multi_sum<RPC * M>(acc, c.lane);
            if (!vb_mbar_wait(&s->pfree[pslot], (puse & 1u) ^ 1u, &s->abort_flag)) {
                if (!aborted(c)) raise_abort(c, VB_ERR_DONE_WAIT);
                return;
            }
            if (idx < RPC * M) s->part[pslot][c.warp][idx] = acc[0];
            __syncwarp();
            if (c.lane == 0) vb_mbar_arrive(&s->pdone[pslot]);
        }
    }
}

/* ------------------------------------------------------------------ */
/* GEMV: epilogue warp                                                 */
/* ------------------------------------------------------------------ */
template <int M>
__device__ void gemv_epilogue(Ctx &c, const VbOp &op) {
    SmemLayout *s = c.s;
    const GemvPlan p = gemv_plan(op.N, op.K, M, op.epi, blockIdx.x, gridDim.x);
    const int v = c.lane;
    const int i = v / M, m = v % M;
    /* op fields in registers: the waits below are compiler barriers for memory */
    const int epi = op.epi, ldy = op.ldy, K = op.K;
    float *const y = op.y;
    float *const tap = op.tap;
    const float *const bias = op.bias;
    const float *const res = op.res;

    /* Residual values of this CTA's rows, fetched once up front instead of one L2
     * round trip per chunk on the epilogue's critical path. */
    const int n_rows = p.r1 - p.r0;
    const bool res_cached = epi == VB_EPI_ADD && n_rows * M <= kResFloats;
    if (res_cached) {
        for (int e = c.lane; e < n_rows * M; e += 32)
            s->resv[e] = vb_ldcg(res + (size_t)(e % M) * ldy + p.r0 + e / M);
        __syncwarp();
    }

    for (int pass = 0; pass < p.passes; pass++) {
        const int klen = min(p.seg_cols, K - pass * p.seg_cols);
        const int n_slices = min(kComputeWarps, (klen + kSliceCols - 1) / kSliceCols);
        for (int rb = 0; rb < p.row_blocks; rb++) {
            const int row0 = p.r0 + rb * p.rows_per_chunk;
            const int rc = min(p.rows_per_chunk, p.r1 - row0);
            const unsigned chunk = c.chunk_counter++;
            const unsigned pslot = chunk % kPartSlots, puse = chunk / kPartSlots;
            if (!vb_mbar_wait(&s->pdone[pslot], puse & 1u, &s->abort_flag)) {
                if (!aborted(c)) raise_abort(c, VB_ERR_DONE_WAIT);
                return;
            }
            const bool mine = (v < rows_cap(M) * M) && (i < rc);
            float val = 0.0f;
            if (mine) {
                for (int w = 0; w < n_slices; w++) val += s->part[pslot][w][v];
            }
            __syncwarp();
            if (c.lane == 0) vb_mbar_arrive(&s->pfree[pslot]);

            const int yi = (rb * p.rows_per_chunk + i) * M + m;
            if (p.passes > 1) {
                if (mine) {
                    if (pass > 0) val += s->yacc[yi];
                    if (pass < p.passes - 1) s->yacc[yi] = val;
                }
                if (pass < p.passes - 1) continue;
            }

            const int row = row0 + i;
            if (epi == VB_EPI_SWIGLU) {
                /* gate rows are even, up rows odd; the up value sits M lanes higher */
                const float upv = __shfl_down_sync(0xffffffffu, val, M);
                if (mine && (i & 1) == 0) {
                    const float g = val / (1.0f + expf(-val));
                    const float r = g * upv;
                    const size_t o = (size_t)m * ldy + (row >> 1);
                    y[o] = r;
                    if (tap) tap[o] = r;
                }
            } else if (mine) {
                const size_t o = (size_t)m * ldy + row;
                float r = val;
                if (bias) r += __ldg(bias + row);
                if (epi == VB_EPI_ADD) r = (res_cached ? s->resv[yi] : vb_ldcg(res + o)) + r;
                y[o] = r;
                if (tap) tap[o] = r;
            }
        }
    }
}

template <int M>
__device__ void gemv_work(Ctx &c, const VbOp &op, int op_index) {
    if (c.warp < kComputeWarps) gemv_compute<M>(c, op, op_index);
    else gemv_epilogue<M>(c, op);
}

/* ------------------------------------------------------------------ */
/* decode attention: RoPE, cache append, GQA attention (one new token) */
/* ------------------------------------------------------------------ */
/* op.x = qkv row [q | k | v]; op.y = attention output; op.p2/op.p3 = this
 * layer's K and V cache [kv_max, kv_dim]; op.p0 = float scratch for split
 * partials; op.p1 = per-KV-head tickets. i0 = query heads, i1 = KV heads,
 * f0 = softmax scale, f1 = RoPE theta. Restates voxtral_tts_llm.c:221-238 with
 * tts_apply_rope / tts_causal_attention (voxtral_tts_kernels.c:403-465,602-634):
 * interleaved pairs, score scaled after the dot product, running max from -1e30.
 * Keys are split over CTAs and over four warp subsets and merged with the usual
 * log-sum-exp weights in a fixed order. */
__device__ void op_attn_decode(Ctx &c, const VbOp &op) {
    SmemLayout *s = c.s;
    const int pos = c.a.dyn->pos;
    const int kv_max = c.a.dyn->kv_max;
    if (pos < 0 || pos >= kv_max) {
        if (c.tid == 0) raise_abort(c, VB_ERR_POS_RANGE);
        return;
    }
    const int H = op.i0, G = op.i1;
    const int group = H / G;                  /* 4 */
    const int kv_dim = G * kHeadDim;
    const int q_dim = H * kHeadDim;
    const int nk = pos + 1;
    int S = (nk + 31) / 32;
    const int max_s = (int)gridDim.x / G;
    if (S > max_s) S = max_s;
    if (S < 1) S = 1;
    const int item = blockIdx.x;
    if (item >= G * S) return;
    const int g = item / S, sp = item % S;
    const int j0 = (int)((long long)nk * sp / S), j1 = (int)((long long)nk * (sp + 1) / S);
    float *Kc = (float *)op.p2, *Vc = (float *)op.p3;
    const float *q = op.x, *kn = op.x + q_dim, *vn = op.x + q_dim + kv_dim;

    if (c.tid < kHeadDim / 2) {
        const float freq = 1.0f / powf(op.f1, (float)(2 * c.tid) / (float)kHeadDim);
        const float ang = (float)pos * freq;
        s->cs[2 * c.tid] = cosf(ang);
        s->cs[2 * c.tid + 1] = sinf(ang);
    }
    vb_named_bar(2, kComputeThreads);
    const int half = kHeadDim / 2;
    if (c.tid < group * half) {
        const int hh = c.tid / half, d = c.tid % half;
        const float *src = q + (size_t)(g * group + hh) * kHeadDim;
        const float a = vb_ldcg(src + 2 * d), b = vb_ldcg(src + 2 * d + 1);
        const float cv = s->cs[2 * d], sv = s->cs[2 * d + 1];
        s->qs[hh][2 * d] = a * cv - b * sv;
        s->qs[hh][2 * d + 1] = a * sv + b * cv;
    } else if (sp == S - 1 && c.tid < group * half + half) {
        const int d = c.tid - group * half;
        const float a = vb_ldcg(kn + g * kHeadDim + 2 * d), b = vb_ldcg(kn + g * kHeadDim + 2 * d + 1);
        const float cv = s->cs[2 * d], sv = s->cs[2 * d + 1];
        float *dst = Kc + (size_t)pos * kv_dim + g * kHeadDim;
        dst[2 * d] = a * cv - b * sv;
        dst[2 * d + 1] = a * sv + b * cv;
        __threadfence();
    } else if (sp == S - 1 && c.tid >= 384 && c.tid < 384 + kHeadDim) {
        const int d = c.tid - 384;
        Vc[(size_t)pos * kv_dim + g * kHeadDim + d] = vb_ldcg(vn + g * kHeadDim + d);
        __threadfence();
    }
    vb_named_bar(2, kComputeThreads);

    const int hh = c.warp & 3, ss = c.warp >> 2;
    const float4 q4 = *reinterpret_cast<const float4 *>(&s->qs[hh][4 * c.lane]);
    float mx = -1e30f, den = 0.0f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = j0 + ss; j < j1; j += kAttnSubsets) {
        const float4 kv = vb_ldcg4(Kc + (size_t)j * kv_dim + g * kHeadDim + 4 * c.lane);
        const float4 vv = vb_ldcg4(Vc + (size_t)j * kv_dim + g * kHeadDim + 4 * c.lane);
        float d = q4.x * kv.x + q4.y * kv.y + q4.z * kv.z + q4.w * kv.w;
        d = vb_warp_sum(d) * op.f0;
        if (d > mx) {
            const float corr = expf(mx - d);
            den = den * corr + 1.0f;
            o.x = o.x * corr + vv.x; o.y = o.y * corr + vv.y;
            o.z = o.z * corr + vv.z; o.w = o.w * corr + vv.w;
            mx = d;
        } else {
            const float w = expf(d - mx);
            den += w;
            o.x += w * vv.x; o.y += w * vv.y; o.z += w * vv.z; o.w += w * vv.w;
        }
    }
    *reinterpret_cast<float4 *>(&s->attn_o[ss][hh][4 * c.lane]) = o;
    if (c.lane == 0) { s->attn_ml[ss][hh][0] = mx; s->attn_ml[ss][hh][1] = den; }
    vb_named_bar(2, kComputeThreads);

    /* merge the four key subsets: thread = (head, dim) */
    const int th = c.tid / kHeadDim, td = c.tid % kHeadDim;
    float M0 = -1e30f;
#pragma unroll
    for (int u = 0; u < kAttnSubsets; u++) M0 = fmaxf(M0, s->attn_ml[u][th][0]);
    float L = 0.0f, O = 0.0f;
#pragma unroll
    for (int u = 0; u < kAttnSubsets; u++) {
        const float w = (s->attn_ml[u][th][1] > 0.0f) ? expf(s->attn_ml[u][th][0] - M0) : 0.0f;
        L += s->attn_ml[u][th][1] * w;
        O += s->attn_o[u][th][td] * w;
    }
    float *out = op.y + (size_t)(g * group + th) * kHeadDim + td;
    if (S == 1) {
        *out = (L > 0.0f) ? O * (1.0f / L) : 0.0f;
        return;
    }
    /* several CTAs share this KV head: publish the partial, last arrival merges */
    float *po = (float *)op.p0;                /* [G][max_s][group][kHeadDim + 2] */
    const int stride = kHeadDim + 2;
    float *mine = po + ((size_t)(g * max_s + sp) * group + th) * stride;
    mine[td] = O;
    if (td == 0) { mine[kHeadDim] = M0; mine[kHeadDim + 1] = L; }
    __threadfence();
    vb_named_bar(2, kComputeThreads);
    unsigned *tickets = (unsigned *)op.p1;
    if (c.tid == 0) {
        const unsigned t = atomicAdd(&tickets[g], 1u);
        s->last_flag = (t == (unsigned)(S - 1));
        if (s->last_flag) tickets[g] = 0u;
    }
    vb_named_bar(2, kComputeThreads);
    if (!s->last_flag) return;
    __threadfence();
    float Mg = -1e30f;
    for (int u = 0; u < S; u++)
        Mg = fmaxf(Mg, vb_ldcg(po + ((size_t)(g * max_s + u) * group + th) * stride + kHeadDim));
    float Lg = 0.0f, Og = 0.0f;
    for (int u = 0; u < S; u++) {
        const float *pu = po + ((size_t)(g * max_s + u) * group + th) * stride;
        const float lu = vb_ldcg(pu + kHeadDim + 1);
        const float w = (lu > 0.0f) ? expf(vb_ldcg(pu + kHeadDim) - Mg) : 0.0f;
        Lg += lu * w;
        Og += vb_ldcg(pu + td) * w;
    }
    *out = (Lg > 0.0f) ? Og * (1.0f / Lg) : 0.0f;
}

/* ------------------------------------------------------------------ */
/* acoustic attention: sequences of 3 tokens, no mask, no RoPE         */
/* ------------------------------------------------------------------ */
/* op.x = qkv [M, ldx] with M = 3 * n_seq; op.y = out [M, ldy]. One warp per
 * (sequence, head, query); keys visited in order with the reference's running
 * maximum (voxtral_tts_kernels.c:487-522). */
__device__ void op_attn_ac(Ctx &c, const VbOp &op) {
    const int H = op.i0, G = op.i1, group = H / G;
    const int q_dim = H * kHeadDim, kv_dim = G * kHeadDim;
    const int T = 3;
    const int n_tasks = op.M * H; /* rows x heads */
    for (int t = blockIdx.x + gridDim.x * c.warp; t < n_tasks; t += gridDim.x * kComputeWarps) {
        const int row = t / H, h = t % H;
        const int seq0 = (row / T) * T;
        const int kvh = h / group;
        const float4 q4 = vb_ldcg4(op.x + (size_t)row * op.ldx + h * kHeadDim + 4 * c.lane);
        float mx = -1e30f, den = 0.0f;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < T; j++) {
            const float *kr = op.x + (size_t)(seq0 + j) * op.ldx + q_dim + kvh * kHeadDim + 4 * c.lane;
            const float4 kv = vb_ldcg4(kr);
            const float4 vv = vb_ldcg4(kr + kv_dim);
            float d = q4.x * kv.x + q4.y * kv.y + q4.z * kv.z + q4.w * kv.w;
            d = vb_warp_sum(d) * op.f0;
            if (d > mx) {
                const float corr = expf(mx - d);
                den = den * corr + 1.0f;
                o.x = o.x * corr + vv.x; o.y = o.y * corr + vv.y;
                o.z = o.z * corr + vv.z; o.w = o.w * corr + vv.w;
                mx = d;
            } else {
                const float w = expf(d - mx);
                den += w;
                o.x += w * vv.x; o.y += w * vv.y; o.z += w * vv.z; o.w += w * vv.w;
            }
        }
        const float inv = (den > 0.0f) ? 1.0f / den : 0.0f;
        float4 r = make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv);
        *reinterpret_cast<float4 *>(op.y + (size_t)row * op.ldy + h * kHeadDim + 4 * c.lane) = r;
    }
}

/* ------------------------------------------------------------------ */
/* small ops                                                           */
/* ------------------------------------------------------------------ */

/* y[m,:] = rmsnorm(x[m,:]) * gain, CTA 0 only (final decoder norm,
 * voxtral_tts_llm.c:267). */
__device__ void op_norm(Ctx &c, const VbOp &op) {
    if (blockIdx.x != 0) return;
    SmemLayout *s = c.s;
    for (int m = 0; m < op.M; m++) {
        const float *x = op.x + (size_t)m * op.ldx;
        float ss = 0.0f;
        for (int i = c.tid; i < op.K; i += kComputeThreads) { const float v = vb_ldcg(x + i); ss += v * v; }
        ss = vb_warp_sum(ss);
        if (c.lane == 0) s->red[0][c.warp][0] = ss;
        vb_named_bar(2, kComputeThreads);
        float t = 0.0f;
        for (int w = 0; w < kComputeWarps; w++) t += s->red[0][w][0];
        const float inv = 1.0f / sqrtf(t / (float)op.K + op.eps);
        for (int i = c.tid; i < op.K; i += kComputeThreads)
            op.y[(size_t)m * op.ldy + i] = vb_ldcg(x + i) * inv * __ldg(op.norm_w + i);
        vb_named_bar(2, kComputeThreads);
    }
}

/* One Euler step with classifier-free guidance (voxtral_tts_acoustic.c:350-354),
 * written without fused multiply-adds so that it rounds like the host code. */
VB_DEVINL float euler_update(float x, float vc, float vu, float alpha, float dt) {
    const float v = __fadd_rn(__fmul_rn(alpha, vc), __fmul_rn(__fsub_rn(1.0f, alpha), vu));
    return __fadd_rn(x, __fmul_rn(v, dt));
}

/* Builds the six input rows of an acoustic pass for Euler step i0
 * (voxtral_tts_acoustic.c:198-212, both guidance branches at once):
 *   rows 0,3: input_proj(x_t)      rows 1,4: time_proj(temb(t_i)) (precomputed)
 *   row  2  : llm_proj(h)          row  5  : llm_proj(0) = 0
 * For i0 > 0 the latent is first advanced with the previous step's velocities.
 * op.W = input_proj [dim, A]; op.x = latents [steps+1][A]; op.p0 = velocities
 * [2][A] (cond, uncond); op.p1 = time tokens [steps][dim]; op.p2 = llm token
 * [dim]; op.y = rows [6, ldy]; f0 = alpha, f1 = dt of the previous step. */
__device__ void op_ac_tokens(Ctx &c, const VbOp &op) {
    SmemLayout *s = c.s;
    const int A = op.K, dim = op.N, step = op.i0;
    float *lat = (float *)op.x;
    if (c.tid < A) {
        float xv;
        if (step == 0) {
            if (op.p3) {
                /* device-resident run: this frame's noise comes from the uploaded array */
                xv = vb_ldcg((const float *)op.p3 + (size_t)c.a.dyn->frame * A + c.tid);
                if (blockIdx.x == 0) lat[c.tid] = xv;
            } else {
                xv = vb_ldcg(lat + c.tid);
            }
        } else {
            const float *vel = (const float *)op.p0;
            xv = euler_update(vb_ldcg(lat + (size_t)(step - 1) * A + c.tid), vb_ldcg(vel + c.tid),
                              vb_ldcg(vel + A + c.tid), op.f0, op.f1);
            if (blockIdx.x == 0) lat[(size_t)step * A + c.tid] = xv;
        }
        s->xs[c.tid] = xv;
    }
    vb_named_bar(2, kComputeThreads);
    const int n0 = (int)((long long)dim * blockIdx.x / gridDim.x);
    const int n1 = (int)((long long)dim * (blockIdx.x + 1) / gridDim.x);
    const bool single = op.i1 != 0; /* one row only: the caller supplies rows 1 and 2 */
    const float *ttok = single ? nullptr : (const float *)op.p1 + (size_t)step * dim;
    const float *ltok = (const float *)op.p2;
    for (int n = n0 + c.tid; n < n1; n += kComputeThreads) {
        const uint16_t *wr = op.W + (size_t)n * A;
        float acc = 0.0f;
        for (int k = 0; k < A; k++)
            acc = __fadd_rn(acc, __fmul_rn(__uint_as_float((uint32_t)__ldg(wr + k) << 16), s->xs[k]));
        op.y[n] = acc;
        if (single) continue;
        const float tt = __ldg(ttok + n);
        op.y[(size_t)3 * op.ldy + n] = acc;
        op.y[(size_t)1 * op.ldy + n] = tt;
        op.y[(size_t)4 * op.ldy + n] = tt;
        op.y[(size_t)2 * op.ldy + n] = vb_ldcg(ltok + n);
        op.y[(size_t)5 * op.ldy + n] = 0.0f;
    }
}

/* Masked greedy argmax over the semantic logits (voxtral_tts_acoustic.c:290-309):
 * index 0 and indices >= i0 are excluded, the first strict maximum wins.
 * op.x = logits [N]; op.p2 = int codes[]; CTA 0 only. */
__device__ void op_argmax(Ctx &c, const VbOp &op) {
    if (blockIdx.x != 0) return;
    SmemLayout *s = c.s;
    float best = -1e30f;
    int bi = 0; /* index 0 carries the masked value -1e30, exactly as the reference starts */
    for (int i = c.tid; i < op.N; i += kComputeThreads) {
        const float v = (i == 0 || i >= op.i0) ? -1e30f : vb_ldcg(op.x + i);
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (c.lane == 0) { s->red[0][c.warp][0] = best; s->red[0][c.warp][1] = __int_as_float(bi); }
    vb_named_bar(2, kComputeThreads);
    if (c.tid == 0) {
        for (int w = 0; w < kComputeWarps; w++) {
            const float ov = s->red[0][w][0];
            const int oi = __float_as_int(s->red[0][w][1]);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        ((int *)op.p2)[0] = bi;
    }
}

/* Last Euler update, then finite-scalar quantisation of the latent
 * (voxtral_tts_acoustic.c:358-372); an END semantic code (1) forces the acoustic
 * codes to 2 (:312-320). op.x = latents; op.p0 = velocities; op.p2 = codes;
 * i0 = steps taken, i1 = levels. CTA 0 only. */
__device__ void op_fsq(Ctx &c, const VbOp &op) {
    if (blockIdx.x != 0) return;
    const int A = op.K, steps = op.i0, levels = op.i1;
    float *lat = (float *)op.x;
    int *codes = (int *)op.p2;
    if (c.tid < A) {
        const float *vel = (const float *)op.p0;
        float xv = euler_update(vb_ldcg(lat + (size_t)(steps - 1) * A + c.tid), vb_ldcg(vel + c.tid),
                                vb_ldcg(vel + A + c.tid), op.f0, op.f1);
        lat[(size_t)steps * A + c.tid] = xv;
        if (xv > 1.0f) xv = 1.0f;
        if (xv < -1.0f) xv = -1.0f;
        const float scaled = __fmul_rn(__fdiv_rn(__fadd_rn(xv, 1.0f), 2.0f), (float)(levels - 1));
        int code = (int)__fadd_rn(scaled, 0.5f);
        if (code < 0) code = 0;
        if (code >= levels) code = levels - 1;
        const int sem = __ldcg(codes);
        const int out = (sem == 1) ? 2 : code + 2;
        codes[1 + c.tid] = out;
        if (op.p3) { /* device-resident run: keep every frame's codes */
            int *log = (int *)op.p3 + (size_t)c.a.dyn->frame * (A + 1);
            log[1 + c.tid] = out;
            if (c.tid == 0) log[0] = sem;
        }
    }
}

/* End of one frame of a device-resident run (the loop of voxtral_tts.c:301-321
 * without the host): the next frame decodes at the next cache row and reads the
 * next noise row; an END code (or a full cache) stops the run. op.p0 = codes;
 * i0 = frames the noise / code arrays hold; i1 != 0: END does not stop the run
 * (fixed-length timing runs). CTA 0 only. */
__device__ void op_advance(Ctx &c, const VbOp &op) {
    if (blockIdx.x != 0 || c.tid != 0) return;
    VbDyn *d = c.a.dyn;
    const int sem = __ldcg((const int *)op.p0);
    const int frame = d->frame + 1, pos = d->pos + 1;
    d->frame = frame;
    d->pos = pos;
    if (sem == 1 && !op.i1) d->done = 2;                       /* END code */
    else if (frame >= op.i0 || pos >= d->kv_max) d->done = 1;  /* arrays or cache exhausted */
}

/* Next decoder input from the 37 codes: sum of BF16 table rows in codebook order
 * (voxtral_tts_voice.c:292-315, offsets :275-283). op.W = table; op.p0 = codes;
 * op.y = out [dim]; i0 = codebooks, i1 = rows of codebook 0, i2 = rows of the
 * others. */
__device__ void op_embed(Ctx &c, const VbOp &op) {
    const int dim = op.N;
    const int *codes = (const int *)op.p0;
    const int n0 = (int)((long long)dim * blockIdx.x / gridDim.x);
    const int n1 = (int)((long long)dim * (blockIdx.x + 1) / gridDim.x);
    for (int n = n0 + c.tid; n < n1; n += kComputeThreads) {
        float acc = 0.0f;
        int base = 0;
        for (int cb = 0; cb < op.i0; cb++) {
            const int row = base + __ldcg(codes + cb);
            acc += __uint_as_float((uint32_t)__ldg(op.W + (size_t)row * dim + n) << 16);
            base += (cb == 0) ? op.i1 : op.i2;
        }
        op.y[n] = acc;
    }
}

/* ------------------------------------------------------------------ */
/* the kernel                                                          */
/* ------------------------------------------------------------------ */
__global__ void __launch_bounds__(kThreads, 1) vb_engine_kernel(EngineArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    SmemLayout *s = reinterpret_cast<SmemLayout *>(smem_raw);
    Ctx c;
    c.s = s; c.a = a;
    c.tid = threadIdx.x; c.warp = threadIdx.x >> 5; c.lane = threadIdx.x & 31;
    c.chunk_counter = 0; c.barrier_epoch = 0;

    /* A device-resident run that has produced END: its remaining queued launches do
     * nothing. The flag was written by an earlier launch, so the whole grid agrees. */
    if (a.dyn->done) return;

    if (c.tid == 0) {
        for (int i = 0; i < kSlots; i++) {
            vb_mbar_init(&s->full[i], 1);
            vb_mbar_init(&s->empty[i], kComputeWarps);
        }
        for (int i = 0; i < kPartSlots; i++) {
            vb_mbar_init(&s->pdone[i], kComputeWarps);
            vb_mbar_init(&s->pfree[i], 1);
        }
        s->abort_flag = 0;
        s->issued_bytes = 0;
        s->last_flag = 0;
        vb_mbar_init_fence();
    }
    __syncthreads();

    if (c.warp == kProducerWarp) {
        if (c.lane == 0) produce_all(c);
    } else if (c.warp == kPrefetchWarp) {
        if (c.lane == 0) prefetch_all(c);
    } else {
        for (int oi = 0; oi < a.n_ops && !aborted(c); oi++) {
            const VbOp &op = a.ops[oi];
            switch (op.type) {
            case VB_OP_GEMV:
                switch (op.M) {
                case 1: gemv_work<1>(c, op, oi); break;
                case 2: gemv_work<2>(c, op, oi); break;
                case 3: gemv_work<3>(c, op, oi); break;
                case 4: gemv_work<4>(c, op, oi); break;
                case 5: gemv_work<5>(c, op, oi); break;
                case 6: gemv_work<6>(c, op, oi); break;
                case 7: gemv_work<7>(c, op, oi); break;
                case 8: gemv_work<8>(c, op, oi); break;
                default: if (c.tid == 0) raise_abort(c, VB_ERR_BAD_OP); break;
                }
                break;
            case VB_OP_ATTN_DECODE: if (c.warp < kComputeWarps) op_attn_decode(c, op); break;
            case VB_OP_ATTN_AC:     if (c.warp < kComputeWarps) op_attn_ac(c, op); break;
            case VB_OP_NORM:        if (c.warp < kComputeWarps) op_norm(c, op); break;
            case VB_OP_AC_TOKENS:   if (c.warp < kComputeWarps) op_ac_tokens(c, op); break;
            case VB_OP_ARGMAX:      if (c.warp < kComputeWarps) op_argmax(c, op); break;
            case VB_OP_FSQ:         if (c.warp < kComputeWarps) op_fsq(c, op); break;
            case VB_OP_EMBED:       if (c.warp < kComputeWarps) op_embed(c, op); break;
            case VB_OP_ADVANCE:     if (c.warp < kComputeWarps) op_advance(c, op); break;
            default: if (c.tid == 0) raise_abort(c, VB_ERR_BAD_OP); break;
            }
            if (!(op.flags & VB_F_NOSYNC) && oi + 1 < a.n_ops) grid_sync(c);
        }
    }

    __syncthreads();
    /* Abort path only: the producer may have copies in flight into this CTA's
     * shared memory; wait for them (bounded) before the CTA retires. */
    if (c.warp == kProducerWarp && c.lane == 0 && aborted(c)) {
        const unsigned issued = c.chunk_counter;
        const unsigned first = issued > (unsigned)kSlots ? issued - kSlots : 0u;
        for (unsigned k = first; k < issued; k++) {
            long long t0 = clock64();
            while (!vb_mbar_try_wait(&s->full[k % kSlots], (k / kSlots) & 1u)) {
                if (clock64() - t0 > VB_WAIT_CYCLES) { atomicCAS(a.status, 0, VB_ERR_DRAIN); break; }
            }
        }
    }
    /* The last CTA out re-zeroes the barrier counters for the next launch. */
    if (c.tid == 0) {
        __threadfence();
        const unsigned t = atomicAdd(a.exit_counter, 1u);
        if (t == gridDim.x - 1) {
            *a.bar_counter = 0u;
            *a.exit_counter = 0u;
            __threadfence();
        }
    }
}

cudaError_t engine_launch(const EngineArgs &args, int n_cta, cudaStream_t stream) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(vb_engine_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)sizeof(SmemLayout));
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    EngineArgs a = args;
    void *params[] = {&a};
    return cudaLaunchCooperativeKernel((const void *)vb_engine_kernel, dim3(n_cta), dim3(kThreads), params,
                                       sizeof(SmemLayout), stream);
}

int engine_max_ctas(int device) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return 0;
    int per_sm = 0;
    cudaFuncSetAttribute(vb_engine_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SmemLayout));
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, vb_engine_kernel, kThreads, sizeof(SmemLayout)) !=
        cudaSuccess)
        return 0;
    return per_sm > 0 ? prop.multiProcessorCount : 0;
}

} // namespace vb
