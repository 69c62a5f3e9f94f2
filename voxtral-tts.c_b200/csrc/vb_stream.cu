/*
 * vb_stream.cu - the persistent streaming decoder-step kernel (sm_100a).
 *
 * What it computes: one call of tts_llm_forward (voxtral_tts_llm.c:171-271) - per layer
 * RMSNorm + QKV, RoPE + cache append + GQA attention, O + residual, RMSNorm + gate/up with
 * SwiGLU, down + residual - followed by the semantic head with its masked argmax and the
 * llm token of the acoustic stage (voxtral_tts_acoustic.c:283-309, :204). All of it is
 * M = 1 work: 6.1 GB of BF16 weights read exactly once, so the kernel is built around one
 * thing, keeping HBM busy from the first byte to the last.
 *
 * Roles inside a CTA (one CTA per SM, cooperative launch):
 *   warp 12, lane 0   producer. Walks the list of weight matrices ahead of everyone and copies
 *                     this CTA's slab of every matrix, 16 KB at a time, into an 11-slot ring
 *                     with 1-D bulk copies (cp.async.bulk, completion on an mbarrier, no
 *                     multicast). It never waits for an op's input, only for a free slot:
 *                     while the other warps sit at a grid barrier the ring fills up with the
 *                     next matrix.
 *   warps 0..11       consumers. Warp s owns ring slot s (warps 10 and 11 own none): it waits
 *                     for the slot alone and hands it back alone. The weights never pass
 *                     through the CUDA cores: ldmatrix moves a 16 x 16 tile from the slot into
 *                     registers and one mma.sync (m16n8k16, BF16 in, fp32 out) multiplies it
 *                     by the input row, which is held as three BF16 terms (three B columns).
 *                     Partial sums stay in registers for the whole op; the three columns and
 *                     the warps are summed once per op, in fixed order (bit-reproducible).
 * RMSNorm is folded in: the input row is staged as x * gain, the sum of squares is taken on
 * the side, and 1/sqrt(mean + eps) multiplies the finished sums (voxtral_tts_kernels.c:333-349).
 *
 * Every wait (mbarrier, grid barrier, flag) is bounded by SArgs.wait_cycles; on expiry a
 * status code is stored and the CTA raises its abort flag. Threads that have given up keep
 * taking part in the CTA barriers of the op they are in, the whole CTA leaves the op loop at
 * the next grid barrier, the other CTAs follow when they see the status word, and the
 * producer waits (bounded) for its copies in flight before the CTA retires.
 */
#include "vb_stream.cuh"
#include "vb_common.cuh"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <vector>

namespace vb {

struct SSmem {
    alignas(128) unsigned char ring[kSSlots][kSSlotBytes];
    /* the staged input row as three BF16 terms in B-fragment order (see s_gemv); the attention
     * op uses the same bytes */
    alignas(16) uint16_t xs[3][kSMaxK];
    float part[kSConsumerWarps][kSMaxRows];     /* per-warp partial sums of the CTA's rows */
    float red[kSConsumerWarps];
    alignas(16) SOp opbuf[2];                   /* the current and the next op descriptor */
    uint64_t full[kSSlots];
    uint64_t empty[kSSlots];
    int abort_flag;     /* raised by any thread of the CTA, at any time */
    int abort_seen;     /* the abort flag as sampled inside the last grid barrier: the same for every consumer thread */
};

static_assert(sizeof(SSmem) <= 232448, "over the 227 KB a CTA may use");
static_assert(sizeof(SOp) % 16 == 0, "op descriptors are copied in 16-byte pieces");
static_assert(kSSlots <= kSConsumerWarps, "every ring slot needs an owner warp");
static_assert(kSConsumerThreads == 3 * kSHeadDim, "the attention op gives one pair of q, k or v values to every thread");

struct SCtx {
    SSmem *s;
    SArgs a;
    int tid, warp, lane;
    unsigned chunk_counter;
    unsigned barrier_epoch;
    unsigned tag_base;      /* launch sequence number << 8 */
};

VB_DEVINL bool s_aborted(const SCtx &c) { return *(volatile int *)&c.s->abort_flag != 0; }

VB_DEVINL void s_raise(SCtx &c, int code) {
    atomicCAS(c.a.status, 0, code);
    *(volatile int *)&c.s->abort_flag = 1;
}

/* Bounded mbarrier wait. try_wait suspends the thread for a while by itself; between tries the
 * thread sleeps a little more so that waiting warps leave the issue slots to the working ones. */
VB_DEVINL bool s_mbar_wait(SCtx &c, uint64_t *bar, uint32_t parity) {
    if (vb_mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (vb_mbar_try_wait(bar, parity)) return true;
        if (s_aborted(c)) return false;
        if (clock64() - t0 > c.a.wait_cycles) return false;
        __nanosleep(32);
    }
}

/* ---- tagged vectors ---- */
VB_DEVINL void s_st_tagged(stag_t *p, float v, unsigned tag) {
    const stag_t w = ((stag_t)tag << 32) | (stag_t)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
VB_DEVINL stag_t s_ld_tagged(const stag_t *p) {
    stag_t w;
    asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
VB_DEVINL void s_ld_tagged2(const stag_t *p, stag_t &a, stag_t &b) {
    asm volatile("ld.relaxed.gpu.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
VB_DEVINL float s_tag_value(stag_t w) { return __uint_as_float((unsigned)(w & 0xffffffffull)); }
VB_DEVINL unsigned s_tag_of(stag_t w) { return (unsigned)(w >> 32); }

/* Polls one element until it carries `tag`. Bounded; on expiry (or when another CTA has given
 * up) the CTA's abort flag is raised and whatever was read last is returned. */
__device__ stag_t s_poll_tagged(SCtx &c, const stag_t *p, unsigned tag) {
    const long long t0 = clock64();
    int spins = 0;
    while (true) {
        const stag_t w = s_ld_tagged(p);
        if (s_tag_of(w) == tag) return w;
        if (s_aborted(c)) return w;
        if ((++spins & 63) == 0) {
            if (vb_ld_relaxed_gpu_s32(c.a.status) != 0) { *(volatile int *)&c.s->abort_flag = 1; return w; }
            if (clock64() - t0 > c.a.wait_cycles) { s_raise(c, S_ERR_DATA_WAIT); return w; }
        }
    }
}

/* Grid barrier of the consumer warps. Returns true when the kernel is giving up; the answer is
 * sampled by one thread between the two CTA barriers, so every consumer thread of the CTA gets
 * the same one and the threads leave the op loop together (a thread that has given up still
 * takes part in every CTA barrier on its way: nobody is left waiting at a bar.sync). */
__device__ bool s_grid_sync(SCtx &c) {
    c.barrier_epoch++;
    vb_named_bar(1, kSConsumerThreads);
    if (c.tid == 0) {
        if (!s_aborted(c)) {
            /* release: everything this CTA wrote before the CTA barrier above is visible to
             * whoever acquires the counter; no return value, so the arrival costs no round trip */
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(c.a.bar_counter) : "memory");
            const unsigned target = c.barrier_epoch * gridDim.x;
            const long long t0 = clock64();
            /* relaxed polls (no fence per try), one acquire fence once the count is there */
            while ((unsigned)vb_ld_relaxed_gpu_s32((const int *)c.a.bar_counter) < target) {
                if (vb_ld_relaxed_gpu_s32(c.a.status) != 0) { *(volatile int *)&c.s->abort_flag = 1; break; }
                if (clock64() - t0 > c.a.wait_cycles) { s_raise(c, S_ERR_GRID_BARRIER); break; }
            }
            asm volatile("fence.acq_rel.gpu;" ::: "memory");
        }
        c.s->abort_seen = s_aborted(c) ? 1 : 0;
    }
    vb_named_bar(1, kSConsumerThreads);
    return *(volatile int *)&c.s->abort_seen != 0;
}

/* ------------------------------------------------------------------ producer */
/* One thread. The weight list is read one entry ahead, so an op switch costs no memory round
 * trip: the only thing this thread ever waits for is a free ring slot.
 */
__device__ void s_produce(SCtx &c) {
    SSmem *s = c.s;
    if (c.a.n_wl <= 0) return;
    SWeights cur = c.a.wl[0];
    for (int i = 0; i < c.a.n_wl; i++) {
        const SWeights nxt = c.a.wl[i + 1 < c.a.n_wl ? i + 1 : i];
        const SPlan p = stream_plan(cur.N, cur.K, cur.epi, blockIdx.x, gridDim.x);
        const unsigned char *src = (const unsigned char *)cur.W + (size_t)p.r0 * cur.K * 2;
        const uint32_t kb_bytes = (uint32_t)p.n_rows * (kSBlockK * 2);
        for (int ch = 0; ch < p.n_chunks; ch++) {
            const int nkb = min(p.kbs, p.kblocks - ch * p.kbs);
            const uint32_t bytes = (uint32_t)nkb * kb_bytes;
            const unsigned slot = c.chunk_counter % kSSlots, use = c.chunk_counter / kSSlots;
            if (!s_mbar_wait(c, &s->empty[slot], (use & 1u) ^ 1u)) {
                if (!s_aborted(c)) s_raise(c, S_ERR_EMPTY_WAIT);
                return;
            }
            c.chunk_counter++;
            vb_mbar_arrive_expect_tx(&s->full[slot], bytes);
            vb_bulk_g2s(s->ring[slot], src, bytes, &s->full[slot]);
            src += bytes;
        }
        cur = nxt;
    }
}

/* ------------------------------------------------------------------ GEMV */
/* The weight side of a GEMV op for one warp: every ring slot this warp owns, through the tensor
 * cores, into per-warp partial sums of the CTA's rows (SSmem::part).
 *
 * Tensor cores as the reduction engine: one mma.sync m16n8k16 multiplies a 16-row x 16-column
 * weight tile (A, fetched with ldmatrix from the swizzled slab rows) by the three term columns of
 * the input (B: column t = term t, the other five columns zero) and adds into a 16 x 8 fp32
 * fragment. Two instructions per 512 weight bytes instead of the twenty a CUDA-core dot product
 * needs: the SM drains a full ring in a fraction of the time HBM needs to fill it.
 * TMAX = row tiles the instantiation handles (2, 4 or 8). The eight accumulator fragments a lane
 * holds are used as TMAX tiles x (8 / TMAX) independent sets taken in turn by the k-steps, so that
 * a CTA with few rows does not serialise on the latency of one accumulator chain. */
template <int TMAX>
__device__ void s_gemv_slots(SCtx &c, const SPlan &p) {
    SSmem *s = c.s;
    constexpr int NSETS = 8 / TMAX;
    const int warp = c.warp, lane = c.lane;
    const int gid = lane >> 2, tig = lane & 3;
    const int T = p.T;
    const int kb_bytes = p.n_rows * (kSBlockK * 2);
    float acc[NSETS][TMAX][4];
#pragma unroll
    for (int a = 0; a < NSETS; a++)
#pragma unroll
        for (int t = 0; t < TMAX; t++) { acc[a][t][0] = acc[a][t][1] = acc[a][t][2] = acc[a][t][3] = 0.0f; }
    /* ldmatrix: lane l addresses row (l & 7) + 8 * ((l >> 3) & 1) of the tile, chunk 2 * ks + (l >> 4) */
    const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8, lm_half = lane >> 4;
    const uint16_t *xt = gid < 3 ? &s->xs[gid][0] : nullptr;      /* this lane's term (B column), if any */

    /* Ring slot s belongs to warp s: it alone waits for the slot's fills (and so sees every
     * phase of that mbarrier in order) and hands the slot back. */
    for (int ch = 0; ch < p.n_chunks; ch++) {
        const unsigned g = c.chunk_counter++;
        const unsigned slot = g % kSSlots, use = g / kSSlots;
        if (slot != (unsigned)warp) continue;
        if (!s_mbar_wait(c, &s->full[slot], use & 1u)) {
            if (!s_aborted(c)) s_raise(c, S_ERR_FULL_WAIT);
            break;      /* carry on to the CTA barriers; the results no longer matter */
        }
        const int kb0 = ch * p.kbs, kb1 = min(kb0 + p.kbs, p.kblocks);
        uint32_t kb_addr = vb_smem_u32(s->ring[slot]);
        for (int kb = kb0; kb < kb1; kb++, kb_addr += kb_bytes) {
            uint32_t bf[4][2];
            if (xt) {
                const uint4 lo = *reinterpret_cast<const uint4 *>(xt + ((kb * 4 + tig) * 4) * 4);
                const uint4 hi = *reinterpret_cast<const uint4 *>(xt + ((kb * 4 + tig) * 4 + 2) * 4);
                bf[0][0] = lo.x; bf[0][1] = lo.y; bf[1][0] = lo.z; bf[1][1] = lo.w;
                bf[2][0] = hi.x; bf[2][1] = hi.y; bf[3][0] = hi.z; bf[3][1] = hi.w;
            } else {
#pragma unroll
                for (int ks = 0; ks < 4; ks++) bf[ks][0] = bf[ks][1] = 0u;
            }
#pragma unroll
            for (int t = 0; t < TMAX; t++) {
                if (t < T) {
                    const int row = t * 16 + lm_row;
                    const uint32_t row_addr = kb_addr + row * 128;
                    uint32_t a[4][4];
#pragma unroll
                    for (int ks = 0; ks < 4; ks++) {
                        const uint32_t addr = row_addr + (((2 * ks + lm_half) ^ (row & 7)) << 4);
                        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(a[ks][0]), "=r"(a[ks][1]), "=r"(a[ks][2]), "=r"(a[ks][3])
                                     : "r"(addr));
                    }
#pragma unroll
                    for (int ks = 0; ks < 4; ks++) {
                        float *d = acc[ks % NSETS][t];
                        asm volatile(
                            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                            : "r"(a[ks][0]), "r"(a[ks][1]), "r"(a[ks][2]), "r"(a[ks][3]), "r"(bf[ks][0]), "r"(bf[ks][1]));
                    }
                }
            }
        }
        /* the slot's bytes have been read */
        __syncwarp();
        if (lane == 0) vb_mbar_arrive(&s->empty[slot]);
    }

    /* once per op: the accumulator sets in order, then the three term columns of a row (hi + lo
     * in quad lane 0, lo2 in quad lane 1); the warps are summed by the caller, in fixed order */
#pragma unroll
    for (int t = 0; t < TMAX; t++) {
        if (t < T) {
            float v[4] = {acc[0][t][0], acc[0][t][1], acc[0][t][2], acc[0][t][3]};
#pragma unroll
            for (int a = 1; a < NSETS; a++) { v[0] += acc[a][t][0]; v[1] += acc[a][t][1]; v[2] += acc[a][t][2]; v[3] += acc[a][t][3]; }
            const float n0 = __shfl_down_sync(0xffffffffu, v[0], 1);
            const float n2 = __shfl_down_sync(0xffffffffu, v[2], 1);
            if (tig == 0) {
                s->part[warp][t * 16 + gid] = (v[0] + v[1]) + n0;
                s->part[warp][t * 16 + gid + 8] = (v[2] + v[3]) + n2;
            }
        }
    }
}

__device__ void s_gemv(SCtx &c, const SOp &op) {
    SSmem *s = c.s;
    const int K = op.K, epi = op.epi;
    const SPlan p = stream_plan(op.N, K, epi, blockIdx.x, gridDim.x);
    const int tid = c.tid, warp = c.warp, lane = c.lane;
    float *const y = op.y;
    float *const tap = op.tap;
    const float *const bias = op.bias;
    const float *const gain = op.gain;
    const float *const x = op.x;
    const float eps = op.eps;
    float *const xn_out = op.xn_out;

    const int flags = op.flags;
    const unsigned x_tag = c.tag_base | (unsigned)op.x_tag, y_tag = c.tag_base | (unsigned)op.y_tag;

    /* this thread's residual value, requested before anything else needs L2. A tagged residual
     * was written by this very thread in an earlier op (same rows, same thread), so it needs no
     * check. */
    float resv = 0.0f;
    if (epi == S_EPI_ADD && tid < p.n_rows) {
        if (flags & S_F_RES_TAGGED) resv = s_tag_value(s_ld_tagged((const stag_t *)op.res + p.r0 + tid));
        else resv = __ldcg(op.res + p.r0 + tid);
    }

    /* Stage the input row as three BF16 terms, x * gain = hi + lo + lo2 (24 mantissa bits;
     * BF16 x BF16 products are exact in fp32, so the tensor core multiplies what the reference
     * multiplies and only the summation order differs). Inside a k-block the terms are stored in
     * the order the MMA's B fragment wants them: [quad q][k-step][4] with the four values of
     * (q, k-step) = columns 2q, 2q+1, 2q+8, 2q+9 of that 16-column step, so a lane fetches the
     * fragments of two k-steps with one 16-byte load. */
    float ss = 0.0f;
    auto stage2 = [&](int k, float va, float vb) {       /* columns k (even) and k + 1 */
        ss += va * va + vb * vb;
        if (gain) {
            const float2 g = __ldg(reinterpret_cast<const float2 *>(gain + k));
            va *= g.x; vb *= g.y;
        }
        const int kb = k >> 6, ks = (k >> 4) & 3, w16 = k & 15;
        const int pos = ((kb * 4 + ((w16 & 7) >> 1)) * 4 + ks) * 4 + ((w16 >> 3) << 1);
        uint16_t a0, a1, a2, b0, b1, b2;
        vb_split3(va, a0, a1, a2);
        vb_split3(vb, b0, b1, b2);
        *reinterpret_cast<uint32_t *>(&s->xs[0][pos]) = a0 | ((uint32_t)b0 << 16);
        *reinterpret_cast<uint32_t *>(&s->xs[1][pos]) = a1 | ((uint32_t)b1 << 16);
        *reinterpret_cast<uint32_t *>(&s->xs[2][pos]) = a2 | ((uint32_t)b2 << 16);
    };
    if (flags & S_F_X_TAGGED) {
        /* Exchange and readiness in one trip: all of this thread's 16-byte loads (two tagged
         * elements each) go out together; an element whose tag is not there yet is polled. */
        const stag_t *xt = (const stag_t *)x;
        constexpr int kBatch = 6;       /* 16-byte loads in flight per thread */
        for (int i0 = tid; i0 < K / 2; i0 += kBatch * kSConsumerThreads) {
            stag_t wa[kBatch], wb[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; u++) {
                const int i = i0 + u * kSConsumerThreads;
                if (i < K / 2) s_ld_tagged2(xt + 2 * i, wa[u], wb[u]);
            }
#pragma unroll
            for (int u = 0; u < kBatch; u++) {
                const int i = i0 + u * kSConsumerThreads;
                if (i < K / 2) {
                    if (s_tag_of(wa[u]) != x_tag) wa[u] = s_poll_tagged(c, xt + 2 * i, x_tag);
                    if (s_tag_of(wb[u]) != x_tag) wb[u] = s_poll_tagged(c, xt + 2 * i + 1, x_tag);
                    stage2(2 * i, s_tag_value(wa[u]), s_tag_value(wb[u]));
                }
            }
        }
    } else {
        for (int i = tid; i < K / 4; i += kSConsumerThreads) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(x) + i);
            stage2(4 * i, v.x, v.y);
            stage2(4 * i + 2, v.z, v.w);
        }
    }
    if (gain) {
        ss = vb_warp_sum(ss);
        if (lane == 0) s->red[warp] = ss;
    }
    vb_named_bar(2, kSConsumerThreads);
    float rscale = 1.0f;
    if (gain) {
        float t = 0.0f;
#pragma unroll
        for (int w = 0; w < kSConsumerWarps; w++) t += s->red[w];
        rscale = 1.0f / sqrtf(t / (float)K + eps);
        if (xn_out && blockIdx.x == 0) {
            for (int k = tid; k < K; k += kSConsumerThreads) {
                const float xv = (flags & S_F_X_TAGGED) ? s_tag_value(s_ld_tagged((const stag_t *)x + k)) : __ldcg(x + k);
                xn_out[k] = xv * rscale * __ldg(gain + k);
            }
        }
    }

    /* the weights: ring slots -> tensor cores -> per-warp partial sums in shared memory */
    if (p.T <= 2) s_gemv_slots<2>(c, p);
    else if (p.T <= 4) s_gemv_slots<4>(c, p);
    else s_gemv_slots<8>(c, p);
    vb_named_bar(2, kSConsumerThreads);
    if (warp * 32 < p.n_rows) {
        const int t = tid;
        const bool valid = t < p.n_rows;
        float sum = 0.0f;
        if (valid) {
#pragma unroll
            for (int w = 0; w < kSSlots; w++) sum += s->part[w][t];
        }
        sum *= rscale;
        if (epi == S_EPI_SWIGLU) {
            /* rows interleaved (gate, up): the up value sits one lane higher */
            const float up = __shfl_down_sync(0xffffffffu, sum, 1);
            if (valid && (t & 1) == 0) {
                const float r = (sum / (1.0f + expf(-sum))) * up;
                const int o = (p.r0 + t) >> 1;
                if (flags & S_F_Y_TAGGED) s_st_tagged((stag_t *)y + o, r, y_tag);
                else y[o] = r;
                if (tap) tap[o] = r;
            }
        } else if (valid) {
            float r = sum;
            if (bias) r += __ldg(bias + p.r0 + t);
            if (epi == S_EPI_ADD) r = resv + r;
            if (flags & S_F_Y_TAGGED) s_st_tagged((stag_t *)y + p.r0 + t, r, y_tag);
            else y[p.r0 + t] = r;
            if (tap) tap[p.r0 + t] = r;
        }
    }
}

/* ------------------------------------------------------------------ decode attention */
/* Two ops. S_OP_ATTN: CTA (g, sp) serves the four query heads of KV head g on slice sp of the
 * keys (S = ceil(keys / 32) slices, at most 16: 128 of the grid's CTAs work and every K/V row is
 * fetched once per group, not once per head). S_OP_ATTN_MERGE: CTA h merges the S slices of
 * query head h with log-sum-exp weights in slice order. With one slice the first op writes the
 * result itself and the second has nothing to do.
 *
 * op.x = [q | k | v] of the new token (6144 elements); op.y = attention output (4096);
 * op.p2 / op.p3 = this layer's K and V cache [kv_max, 1024]; op.p0 = the slices' partial
 * results, tagged, [G][16][4][128 + 2]; i0 = query heads, i1 = KV heads, i2 = the tag of the
 * final output; f0 = softmax scale, f1 = RoPE theta. Restates voxtral_tts_llm.c:221-238 with
 * tts_apply_rope and tts_causal_attention (voxtral_tts_kernels.c:403-465, 602-634): interleaved
 * pairs, the score is scaled after the dot product, the running maximum starts at -1e30. Inside
 * a CTA warp w serves head w & 3 on every third key of the slice, eight keys per pass so that
 * their sixteen loads are in flight together, with the reference's running-maximum update. The
 * new token's key and value are used from shared memory; the CTA of the last slice also appends
 * them to the cache. */
constexpr int kSAttnSplits = 16;
constexpr int kSAttnSubsets = kSConsumerWarps / 4;

struct SAttnSmem {
    alignas(16) float q[4][kSHeadDim];
    alignas(16) float kn[kSHeadDim];
    alignas(16) float vn[kSHeadDim];
    alignas(16) float wo[kSConsumerWarps][kSHeadDim];
    float wml[kSConsumerWarps][2];
    float cm[kSAttnSplits], cl[kSAttnSplits];
};
static_assert(sizeof(SAttnSmem) <= sizeof(uint16_t) * 3 * kSMaxK, "attention scratch must fit the row buffer");

VB_DEVINL int s_attn_slices(int nk, int grid, int G) {
    int max_s = grid / G;
    if (max_s > kSAttnSplits) max_s = kSAttnSplits;
    if (max_s < 1) max_s = 1;
    int S = (nk + 31) / 32;
    return S > max_s ? max_s : S;
}

__device__ void s_attn(SCtx &c, const SOp &op) {
    SAttnSmem *s = reinterpret_cast<SAttnSmem *>(&c.s->xs[0][0]);
    const int tid = c.tid, warp = c.warp, lane = c.lane;
    const int pos = c.a.dyn->pos, kv_max = c.a.dyn->kv_max;
    if (pos < 0 || pos >= kv_max) {
        if (tid == 0) s_raise(c, S_ERR_POS_RANGE);
        return;
    }
    const int H = op.i0, G = op.i1, group = H / G;      /* 32, 8, 4 */
    const int nk = pos + 1;
    const int S = s_attn_slices(nk, (int)gridDim.x, G);
    const int item = blockIdx.x;
    if (item >= G * S) return;
    const int g = item / S, sp = item % S;
    const int j0 = (int)((long long)nk * sp / S), j1 = (int)((long long)nk * (sp + 1) / S);
    const int kv_dim = G * kSHeadDim, q_dim = H * kSHeadDim;
    const float scale = op.f0;
    const float *Kc = (const float *)op.p2 + g * kSHeadDim, *Vc = (const float *)op.p3 + g * kSHeadDim;
    const bool writer = sp == S - 1;        /* its slice ends with the new token */
    constexpr int half = kSHeadDim / 2;
    const bool tagged = (op.flags & S_F_X_TAGGED) != 0;
    const unsigned x_tag = c.tag_base | (unsigned)op.x_tag;

    /* one pair of raw values per thread (q: 4 heads x 64 pairs, k: 64 pairs, v: 64 pairs), then
     * the rotation of q and k */
    {
        size_t e;
        if (tid < group * half) e = (size_t)(g * group + tid / half) * kSHeadDim + 2 * (tid % half);
        else if (tid < group * half + half) e = (size_t)q_dim + g * kSHeadDim + 2 * (tid - group * half);
        else e = (size_t)q_dim + kv_dim + g * kSHeadDim + 2 * (tid - group * half - half);
        float ra, rb;
        if (tagged) {
            const stag_t *xt = (const stag_t *)op.x;
            stag_t wa, wb;
            s_ld_tagged2(xt + e, wa, wb);
            if (s_tag_of(wa) != x_tag) wa = s_poll_tagged(c, xt + e, x_tag);
            if (s_tag_of(wb) != x_tag) wb = s_poll_tagged(c, xt + e + 1, x_tag);
            ra = s_tag_value(wa); rb = s_tag_value(wb);
        } else {
            ra = __ldcg(op.x + e); rb = __ldcg(op.x + e + 1);
        }
        if (tid < group * half + half) {
            const int d = tid < group * half ? tid % half : tid - group * half;
            const float freq = 1.0f / powf(op.f1, (float)(2 * d) / (float)kSHeadDim);
            const float ang = (float)pos * freq;
            const float cv = cosf(ang), sv = sinf(ang);
            const float o0 = ra * cv - rb * sv, o1 = ra * sv + rb * cv;
            if (tid < group * half) { s->q[tid / half][2 * d] = o0; s->q[tid / half][2 * d + 1] = o1; }
            else {
                s->kn[2 * d] = o0; s->kn[2 * d + 1] = o1;
                if (writer) {
                    float *dst = (float *)op.p2 + (size_t)pos * kv_dim + g * kSHeadDim;
                    dst[2 * d] = o0; dst[2 * d + 1] = o1;
                }
            }
        } else {
            const int d = 2 * (tid - group * half - half);
            s->vn[d] = ra; s->vn[d + 1] = rb;
            if (writer) {
                float *dst = (float *)op.p3 + (size_t)pos * kv_dim + g * kSHeadDim;
                dst[d] = ra; dst[d + 1] = rb;
            }
        }
    }
    vb_named_bar(2, kSConsumerThreads);

    const int hh = warp & 3, ss = warp >> 2;
    const float4 q4 = *reinterpret_cast<const float4 *>(&s->q[hh][4 * lane]);
    float mx = -1e30f, den = 0.0f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    constexpr int kKeysPerPass = 8;
    for (int jb = j0 + ss; jb < j1; jb += kKeysPerPass * kSAttnSubsets) {
        float4 kq[kKeysPerPass], vq[kKeysPerPass];
#pragma unroll
        for (int u = 0; u < kKeysPerPass; u++) {
            const int j = jb + u * kSAttnSubsets;
            if (j < j1 && j < pos) {
                kq[u] = vb_ldcg4(Kc + (size_t)j * kv_dim + 4 * lane);
                vq[u] = vb_ldcg4(Vc + (size_t)j * kv_dim + 4 * lane);
            } else if (j == pos) {
                kq[u] = *reinterpret_cast<const float4 *>(&s->kn[4 * lane]);
                vq[u] = *reinterpret_cast<const float4 *>(&s->vn[4 * lane]);
            } else {
                kq[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                vq[u] = kq[u];
            }
        }
        float dq[kKeysPerPass];
#pragma unroll
        for (int u = 0; u < kKeysPerPass; u++)
            dq[u] = q4.x * kq[u].x + q4.y * kq[u].y + q4.z * kq[u].z + q4.w * kq[u].w;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
            for (int u = 0; u < kKeysPerPass; u++) dq[u] += __shfl_xor_sync(0xffffffffu, dq[u], off);
        }
#pragma unroll
        for (int u = 0; u < kKeysPerPass; u++) {
            if (jb + u * kSAttnSubsets >= j1) break;
            const float d = dq[u] * scale;
            const float4 vv = vq[u];
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
    }
    *reinterpret_cast<float4 *>(&s->wo[warp][4 * lane]) = o;
    if (lane == 0) { s->wml[warp][0] = mx; s->wml[warp][1] = den; }
    vb_named_bar(2, kSConsumerThreads);

    /* merge the key subsets of each head: element = (head, dim) */
    const unsigned out_tag = c.tag_base | (unsigned)(S == 1 ? op.i2 : op.y_tag);
    for (int e = tid; e < group * kSHeadDim; e += kSConsumerThreads) {
        const int th = e / kSHeadDim, td = e % kSHeadDim;
        float M0 = -1e30f;
#pragma unroll
        for (int u = 0; u < kSAttnSubsets; u++) M0 = fmaxf(M0, s->wml[u * 4 + th][0]);
        float L = 0.0f, O = 0.0f;
#pragma unroll
        for (int u = 0; u < kSAttnSubsets; u++) {
            const float lw = s->wml[u * 4 + th][1];
            const float w = lw > 0.0f ? expf(s->wml[u * 4 + th][0] - M0) : 0.0f;
            L += lw * w;
            O += s->wo[u * 4 + th][td] * w;
        }
        if (S == 1) {
            const float r = L > 0.0f ? O * (1.0f / L) : 0.0f;
            const size_t oi = (size_t)(g * group + th) * kSHeadDim + td;
            if (op.flags & S_F_Y_TAGGED) s_st_tagged((stag_t *)op.y + oi, r, out_tag);
            else op.y[oi] = r;
        } else {
            stag_t *mine = (stag_t *)op.p0 + ((size_t)(g * kSAttnSplits + sp) * group + th) * (kSHeadDim + 2);
            s_st_tagged(mine + td, O, out_tag);
            if (td == 0) { s_st_tagged(mine + kSHeadDim, M0, out_tag); s_st_tagged(mine + kSHeadDim + 1, L, out_tag); }
        }
    }
}

/* op.p0 = the slices' partial results (written by the S_OP_ATTN op before, tag x_tag);
 * op.y = attention output, written with y_tag; i0, i1 as above. One CTA per query head. */
__device__ void s_attn_merge(SCtx &c, const SOp &op) {
    SAttnSmem *s = reinterpret_cast<SAttnSmem *>(&c.s->xs[0][0]);
    const int tid = c.tid;
    const int pos = c.a.dyn->pos, kv_max = c.a.dyn->kv_max;
    if (pos < 0 || pos >= kv_max) return;       /* reported by the op before */
    const int H = op.i0, G = op.i1, group = H / G;
    const int S = s_attn_slices(pos + 1, (int)gridDim.x, G);
    const int h = blockIdx.x;
    if (S == 1 || h >= H) return;
    const int g = h / group, th = h % group;
    const unsigned x_tag = c.tag_base | (unsigned)op.x_tag;
    const stag_t *base = (const stag_t *)op.p0 + ((size_t)(g * kSAttnSplits) * group + th) * (kSHeadDim + 2);
    const size_t slice_stride = (size_t)group * (kSHeadDim + 2);
    if (tid < 2 * S) {
        const int u = tid >> 1;
        const stag_t w = s_poll_tagged(c, base + u * slice_stride + kSHeadDim + (tid & 1), x_tag);
        if (tid & 1) s->cl[u] = s_tag_value(w);
        else s->cm[u] = s_tag_value(w);
    }
    float ov[kSAttnSplits];
    if (tid < kSHeadDim) {
#pragma unroll
        for (int u = 0; u < kSAttnSplits; u++)
            ov[u] = u < S ? s_tag_value(s_poll_tagged(c, base + u * slice_stride + tid, x_tag)) : 0.0f;
    }
    vb_named_bar(2, kSConsumerThreads);
    if (tid < kSHeadDim) {
        float Mg = -1e30f;
        for (int u = 0; u < S; u++) Mg = fmaxf(Mg, s->cm[u]);
        float Lg = 0.0f, Og = 0.0f;
#pragma unroll
        for (int u = 0; u < kSAttnSplits; u++) {
            if (u < S) {
                const float lu = s->cl[u];
                const float w = lu > 0.0f ? expf(s->cm[u] - Mg) : 0.0f;
                Lg += lu * w;
                Og += ov[u] * w;
            }
        }
        const float r = Lg > 0.0f ? Og * (1.0f / Lg) : 0.0f;
        const size_t oi = (size_t)h * kSHeadDim + tid;
        if (op.flags & S_F_Y_TAGGED) s_st_tagged((stag_t *)op.y + oi, r, c.tag_base | (unsigned)op.y_tag);
        else op.y[oi] = r;
    }
}

/* ------------------------------------------------------------------ small ops */
/* Decoder input of the next frame: the sum of the 37 code rows of the audio table in codebook
 * order (voxtral_tts_voice.c:292-315, offsets :275-283). op.W = table [rows, N] row-major;
 * op.p0 = codes; op.y = out [N]; i0 = codebooks, i1 = rows of codebook 0, i2 = rows of the
 * others. The N columns are dealt out over the CTAs. */
__device__ void s_embed(SCtx &c, const SOp &op) {
    if ((op.flags & S_F_SKIP_FRAME0) && c.a.dyn->frame == 0) return;
    const int dim = op.N;
    const int *codes = (const int *)op.p0;
    const int n0 = (int)((long long)dim * blockIdx.x / gridDim.x);
    const int n1 = (int)((long long)dim * (blockIdx.x + 1) / gridDim.x);
    constexpr int kMaxCodes = 40;
    const int ncb = op.i0 < kMaxCodes ? op.i0 : kMaxCodes;
    for (int n = n0 + c.tid; n < n1; n += kSConsumerThreads) {
        int rowi[kMaxCodes];
        uint16_t val[kMaxCodes];
#pragma unroll
        for (int cb = 0; cb < kMaxCodes; cb++) rowi[cb] = cb < ncb ? __ldcg(codes + cb) : 0;
#pragma unroll
        for (int cb = 0; cb < kMaxCodes; cb++) {
            const int base = cb == 0 ? 0 : op.i1 + (cb - 1) * op.i2;
            val[cb] = cb < ncb ? __ldg(op.W + (size_t)(base + rowi[cb]) * dim + n) : (uint16_t)0;
        }
        float acc = 0.0f;
#pragma unroll
        for (int cb = 0; cb < kMaxCodes; cb++)
            if (cb < ncb) acc += __uint_as_float((uint32_t)val[cb] << 16);
        op.y[n] = acc;
    }
}

/* Masked greedy argmax over the semantic logits (voxtral_tts_acoustic.c:290-309): index 0 and
 * indices >= i0 are excluded, the first strict maximum wins. op.x = logits [N]; op.p2 = int
 * destination. CTA 0 only. */
__device__ void s_argmax(SCtx &c, const SOp &op) {
    if (blockIdx.x != 0) return;
    SSmem *s = c.s;
    float best = -1e30f;
    int bi = 0;     /* index 0 carries the masked value -1e30, exactly as the reference starts */
    for (int i = c.tid; i < op.N; i += kSConsumerThreads) {
        const float v = (i == 0 || i >= op.i0) ? -1e30f : __ldcg(op.x + i);
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (c.lane == 0) { s->part[c.warp][0] = best; s->part[c.warp][1] = __int_as_float(bi); }
    vb_named_bar(2, kSConsumerThreads);
    if (c.tid == 0) {
        for (int w = 0; w < kSConsumerWarps; w++) {
            const float ov = s->part[w][0];
            const int oi = __float_as_int(s->part[w][1]);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        ((int *)op.p2)[0] = bi;
    }
}

/* Waits until the word at op.p0 reaches i0 (something outside this kernel publishes it).
 * One thread of CTA 0 polls; its limit is i1 microseconds when i1 > 0, else the kernel's. When
 * the limit passes it records S_ERR_FLAG_WAIT and every CTA leaves through the abort path at
 * its next barrier. */
__device__ void s_wait_flag(SCtx &c, const SOp &op) {
    if (blockIdx.x != 0 || c.tid != 0) return;
    const unsigned *flag = (const unsigned *)op.p0;
    const long long limit = op.i1 > 0 ? (long long)op.i1 * 2000 : c.a.wait_cycles;
    const long long t0 = clock64();
    while (vb_ld_acquire_gpu(flag) < (unsigned)op.i0) {
        if (clock64() - t0 > limit) { s_raise(c, S_ERR_FLAG_WAIT); break; }
    }
}

/* ------------------------------------------------------------------ the kernel */
VB_DEVINL void s_cp_async16(void *smem_dst, const void *gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(vb_smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
VB_DEVINL void s_cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__global__ void __launch_bounds__(kSThreads, 1) vb_stream_kernel(SArgs a) {
    extern __shared__ __align__(128) unsigned char s_smem_raw[];
    SSmem *s = reinterpret_cast<SSmem *>(s_smem_raw);
    SCtx c;
    c.s = s; c.a = a;
    c.tid = threadIdx.x; c.warp = threadIdx.x >> 5; c.lane = threadIdx.x & 31;
    c.chunk_counter = 0; c.barrier_epoch = 0;

    /* a device-resident run that has ended: its remaining queued launches do nothing (the flag
     * was written by an earlier launch, so the whole grid agrees) */
    if (a.dyn->done) return;
    c.tag_base = *(volatile const unsigned *)a.seq << 8;     /* written by the previous launch's last CTA */

    constexpr int kOpVecs = (int)(sizeof(SOp) / 16);
    if (c.tid == 0) {
        for (int i = 0; i < kSSlots; i++) {
            vb_mbar_init(&s->full[i], 1);
            vb_mbar_init(&s->empty[i], 1);
        }
        s->abort_flag = 0;
        s->abort_seen = 0;
        vb_mbar_init_fence();
    }
    if (c.tid < kOpVecs && a.n_ops > 0)
        reinterpret_cast<uint4 *>(&s->opbuf[0])[c.tid] = __ldg(reinterpret_cast<const uint4 *>(a.ops) + c.tid);
    __syncthreads();

    if (c.warp == kSConsumerWarps) {
        if (c.lane == 0) s_produce(c);
    } else {
        for (int oi = 0; oi < a.n_ops; oi++) {
            /* Descriptors reach shared memory one op ahead (asynchronous copies issued by a few
             * threads during the previous op), so no op starts with a round trip to L2 for its
             * own parameters. The CTA barrier makes op oi's copy visible to every thread and
             * tells the copying threads that nobody reads op oi-1's buffer any more. */
            if (c.tid < kOpVecs) s_cp_async_wait_all();
            /* the same barrier tells every thread whether any thread of the CTA has given up
             * (ops that exchange tagged data have no grid barrier between them to learn it at) */
            {
                int any;
                asm volatile(
                    "{\n\t.reg .pred p, q;\n\t"
                    "setp.ne.b32 p, %1, 0;\n\t"
                    "barrier.cta.red.or.pred q, 3, %2, p;\n\t"
                    "selp.b32 %0, 1, 0, q;\n\t}"
                    : "=r"(any)
                    : "r"(s_aborted(c) ? 1 : 0), "r"(kSConsumerThreads)
                    : "memory");
                if (any) break;
            }
            if (c.tid < kOpVecs && oi + 1 < a.n_ops)
                s_cp_async16(reinterpret_cast<uint4 *>(&s->opbuf[(oi + 1) & 1]) + c.tid,
                             reinterpret_cast<const uint4 *>(a.ops + oi + 1) + c.tid);
            const SOp &op = s->opbuf[oi & 1];
            const int flags = op.flags;
            switch (op.type) {
            case S_OP_GEMV:   s_gemv(c, op); break;
            case S_OP_ATTN:   s_attn(c, op); break;
            case S_OP_ATTN_MERGE: s_attn_merge(c, op); break;
            case S_OP_EMBED:  s_embed(c, op); break;
            case S_OP_ARGMAX: s_argmax(c, op); break;
            case S_OP_WAIT:   s_wait_flag(c, op); break;
            default: if (c.tid == 0) s_raise(c, S_ERR_BAD_OP); break;
            }
            if (!(flags & S_F_NOSYNC) && oi + 1 < a.n_ops && s_grid_sync(c)) break;
        }
        if (c.tid < kOpVecs) s_cp_async_wait_all();
    }

    __syncthreads();
    /* abort path only: copies may still be in flight into this CTA's shared memory */
    if (c.warp == kSConsumerWarps && c.lane == 0 && s_aborted(c)) {
        const unsigned issued = c.chunk_counter;
        const unsigned first = issued > (unsigned)kSSlots ? issued - kSSlots : 0u;
        for (unsigned k = first; k < issued; k++) {
            const long long t0 = clock64();
            while (!vb_mbar_try_wait(&s->full[k % kSSlots], (k / kSSlots) & 1u)) {
                if (clock64() - t0 > a.wait_cycles) { atomicCAS(a.status, 0, (int)S_ERR_DRAIN); break; }
            }
        }
    }
    /* the last CTA out re-zeroes the barrier counters for the next launch */
    if (c.tid == 0) {
        __threadfence();
        const unsigned t = atomicAdd(a.exit_counter, 1u);
        if (t == gridDim.x - 1) {
            *a.bar_counter = 0u;
            *a.exit_counter = 0u;
            *a.seq = (c.tag_base >> 8) + 1u;        /* the next launch's tags differ from this one's */
            __threadfence();
        }
    }
}

/* ------------------------------------------------------------------ host */
/* dst (slab order) from src (row-major), one 16-byte vector per thread. */
__global__ void vb_stream_slab_kernel(uint4 *dst, const uint4 *src, int N, int K, int unit, int n_cta) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t vec_per_row = (size_t)K / 8;
    if (i >= (size_t)N * vec_per_row) return;
    const unsigned vr = (unsigned)(i / vec_per_row);            /* a row of the slab's owner */
    const unsigned U = (unsigned)(N / unit), nc = (unsigned)n_cta, q = U / nc, rem = U - q * nc;
    const unsigned vu = vr / (unsigned)unit;
    unsigned cta;
    if (vu < rem * (q + 1)) cta = vu / (q + 1);
    else cta = rem + (q ? (vu - rem * (q + 1)) / q : 0u);
    const unsigned u0 = cta * q + (cta < rem ? cta : rem);
    const unsigned r0 = u0 * (unsigned)unit, n_rows = (q + (cta < rem ? 1u : 0u)) * (unsigned)unit;
    const size_t li = i - (size_t)r0 * vec_per_row;              /* vector index inside the slab */
    const unsigned kb = (unsigned)(li / ((size_t)n_rows * 8)), within = (unsigned)(li % ((size_t)n_rows * 8));
    const unsigned r = within / 8, v = within % 8;
    /* physical 16-byte chunk v of slab row r holds the row's chunk v ^ (r & 7) */
    dst[i] = src[((size_t)(r0 + r) * K + (size_t)kb * kSBlockK) / 8 + (v ^ (r & 7))];
}

int stream_make_slabs(uint16_t *d_dst, const uint16_t *d_src, int N, int K, int epi, int n_cta, cudaStream_t st) {
    if (stream_validate(N, K, epi, n_cta)) return -1;
    if (((uintptr_t)d_dst | (uintptr_t)d_src) & 15) return -1;
    const int unit = epi == S_EPI_SWIGLU ? 2 : 1;
    const size_t n_vec = (size_t)N * K / 8;
    vb_stream_slab_kernel<<<(unsigned)((n_vec + 255) / 256), 256, 0, st>>>((uint4 *)d_dst, (const uint4 *)d_src, N, K,
                                                                           unit, n_cta);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

static bool g_stream_attr = false;

static int stream_attr() {
    if (g_stream_attr) return 0;
    if (cudaFuncSetAttribute(vb_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SSmem)) !=
        cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    g_stream_attr = true;
    return 0;
}

int stream_max_ctas(int device) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return 0;
    if (stream_attr()) return 0;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, vb_stream_kernel, kSThreads, sizeof(SSmem)) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return per_sm > 0 ? prop.multiProcessorCount : 0;
}

cudaError_t stream_launch(const SArgs &args, int n_cta, cudaStream_t st) {
    if (stream_attr()) return cudaErrorInvalidValue;
    SArgs a = args;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_cta); cfg.blockDim = dim3(kSThreads);
    cfg.dynamicSmemBytes = sizeof(SSmem); cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, vb_stream_kernel, a);
}

/* ---------------------------------------------------------------- stand-alone probe */
__global__ void vb_stream_fill_kernel(uint16_t *p, size_t n, uint32_t seed) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint32_t h = (uint32_t)i * 2654435761u + seed;
    h ^= h >> 15;
    p[i] = (uint16_t)(0x3c00u | (h & 0x3fu) | ((h & 0x40u) << 9));   /* small BF16 values of both signs */
}

/* The kernel alone, without a model: `n_ops` GEMV ops on generated [N, K] matrices (enough
 * copies that no op finds its weights in L2), `reps` launches between two events on the default
 * stream. sync = 1: a grid barrier after every op (as in a decoder step); 0: none. A measurement
 * and profiling aid with a small memory footprint. */
int stream_probe(int N, int K, int n_ops, int sync, int reps, float *ms_out, double *bytes_per_launch) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    const int n_cta = stream_max_ctas(dev);
    if (n_cta <= 0 || n_ops < 1 || n_ops > 128 || reps < 1 || stream_validate(N, K, S_EPI_STORE, n_cta)) return -1;
    const size_t wn = (size_t)N * K;
    int copies = (int)((size_t)400 * 1024 * 1024 / (wn * 2)) + 1;
    if (copies > n_ops) copies = n_ops;
    std::vector<uint16_t *> W(copies, nullptr);
    float *x = nullptr, *y = nullptr;
    unsigned *words = nullptr;
    SOp *d_ops = nullptr;
    SWeights *d_wl = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    int rc = -1;
    do {
        bool ok = true;
        for (int c = 0; c < copies && ok; c++) {
            ok = cudaMalloc(&W[c], wn * 2) == cudaSuccess;
            if (ok) vb_stream_fill_kernel<<<(unsigned)((wn + 255) / 256), 256>>>(W[c], wn, 1u + c);
        }
        if (!ok || cudaMalloc(&x, sizeof(float) * K) != cudaSuccess || cudaMalloc(&y, sizeof(float) * N) != cudaSuccess ||
            cudaMalloc(&words, sizeof(unsigned) * 64) != cudaSuccess || cudaMalloc(&d_ops, sizeof(SOp) * n_ops) != cudaSuccess)
            break;
        cudaMemset(x, 0, sizeof(float) * K);
        cudaMemset(words, 0, sizeof(unsigned) * 64);
        std::vector<SOp> ops(n_ops);
        for (int i = 0; i < n_ops; i++) {
            SOp &o = ops[i];
            memset(&o, 0, sizeof(o));
            o.type = S_OP_GEMV; o.N = N; o.K = K; o.epi = S_EPI_STORE; o.W = W[i % copies]; o.x = x; o.y = y;
            o.flags = sync ? 0 : S_F_NOSYNC;
        }
        std::vector<SWeights> wl(n_ops);
        for (int i = 0; i < n_ops; i++) wl[i] = SWeights{ops[i].W, N, K, S_EPI_STORE, 0};
        if (cudaMalloc(&d_wl, sizeof(SWeights) * n_ops) != cudaSuccess ||
            cudaMemcpy(d_wl, wl.data(), sizeof(SWeights) * n_ops, cudaMemcpyHostToDevice) != cudaSuccess ||
            cudaMemcpy(d_ops, ops.data(), sizeof(SOp) * n_ops, cudaMemcpyHostToDevice) != cudaSuccess)
            break;
        SArgs a;
        a.ops = d_ops; a.n_ops = n_ops; a.dyn = (VbDyn *)(words + 52);
        a.wl = d_wl; a.n_wl = n_ops;
        a.bar_counter = words; a.exit_counter = words + 16; a.status = (int *)(words + 32); a.seq = words + 40;
        a.wait_cycles = 2000000000LL;
        if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) break;
        for (int i = 0; i < 2 && ok; i++) ok = stream_launch(a, n_cta, 0) == cudaSuccess;
        cudaEventRecord(e0, 0);
        for (int i = 0; i < reps && ok; i++) ok = stream_launch(a, n_cta, 0) == cudaSuccess;
        cudaEventRecord(e1, 0);
        if (!ok || cudaDeviceSynchronize() != cudaSuccess) break;
        int st = 0;
        cudaMemcpy(&st, words + 32, sizeof(int), cudaMemcpyDeviceToHost);
        if (st) break;
        if (ms_out) cudaEventElapsedTime(ms_out, e0, e1);
        if (bytes_per_launch) *bytes_per_launch = 2.0 * (double)wn * n_ops;
        rc = 0;
    } while (0);
    cudaGetLastError();
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    for (uint16_t *p : W) cudaFree(p);
    cudaFree(x); cudaFree(y); cudaFree(words); cudaFree(d_ops); cudaFree(d_wl);
    return rc;
}

} // namespace vb
