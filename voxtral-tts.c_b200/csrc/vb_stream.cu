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
 *   warps 0..11       consumers. Warp s owns ring slot s: it waits for the slot alone and
 *                     hands it back alone (warp 11 owns none). The slab order makes a warp
 *                     load 512 contiguous bytes (4 rows x 8 chunks of 8 BF16): lane = (row r,
 *                     chunk c). A lane keeps its 8 activations of the k-block in registers and
 *                     one accumulator per row step, so nothing is reduced per slot: the 8
 *                     lanes of a row and the warps are summed once per op, in fixed order
 *                     (bit-reproducible; BF16 -> fp32 is an exact shift and all products are
 *                     fp32, as in voxtral_tts_kernels.c:152-185).
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
    /* the staged input row (permuted, see s_gemv); the attention op uses the same bytes */
    alignas(16) float xs[kSMaxK];
    float part[kSConsumerWarps][kSMaxRows];     /* per-warp partial sums of the CTA's rows */
    float red[kSConsumerWarps];
    alignas(16) SOp opbuf[2];                   /* the current and the next op descriptor */
    uint64_t full[kSSlots];
    uint64_t empty[kSSlots];
    int abort_flag;     /* raised by any thread of the CTA, at any time */
    int abort_seen;     /* the abort flag as sampled inside the last grid barrier: the same for every consumer thread */
};

/* Attention scratch, overlaid on SSmem::xs. */
struct SAttnSmem {
    alignas(16) float q[kSHeadDim];
    alignas(16) float kn[kSHeadDim];
    alignas(16) float vn[kSHeadDim];
    float cs[kSHeadDim];
    alignas(16) float wo[kSConsumerWarps][kSHeadDim];
    float wml[kSConsumerWarps][2];
};
static_assert(sizeof(SAttnSmem) <= sizeof(float) * kSMaxK, "attention scratch must fit the row buffer");
static_assert(sizeof(SSmem) <= 232448, "over the 227 KB a CTA may use");
static_assert(sizeof(SOp) % 16 == 0, "op descriptors are copied in 16-byte pieces");
static_assert(kSSlots <= kSConsumerWarps, "every ring slot needs an owner warp");
static_assert(kSConsumerThreads >= 2 * kSHeadDim, "the attention op rotates q and k and copies v with one thread each");

struct SCtx {
    SSmem *s;
    SArgs a;
    int tid, warp, lane;
    unsigned chunk_counter;
    unsigned barrier_epoch;
    int tl_op;
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
 *
 * Second level: a cursor runs `pf_bytes` ahead of the ring through the same byte sequence and
 * asks L2 for it (cp.async.bulk.prefetch.L2). The ring alone holds 4 us of this SM's share of
 * HBM; the dependent chain between two ops (epilogue, grid barrier, staging of the next input)
 * is about as long, so without the second level HBM idles at every op boundary. With it HBM
 * keeps filling L2 through the stall, and the ring then refills from L2, faster than HBM could. */
struct SCursor {
    const SWeights *wl;
    int n, i;
    const unsigned char *ptr;
    size_t left;
};

__device__ void s_cursor_open(SCursor &k, int i) {
    k.i = i;
    k.left = 0;
    k.ptr = nullptr;
    if (i >= k.n) return;
    const SWeights w = k.wl[i];
    const SPlan p = stream_plan(w.N, w.K, w.epi, blockIdx.x, gridDim.x);
    k.ptr = (const unsigned char *)w.W + (size_t)p.r0 * w.K * 2;
    k.left = (size_t)p.n_rows * w.K * 2;
}

/* Prefetches the next `bytes` of the sequence (crossing into following matrices as needed). */
__device__ void s_cursor_prefetch(SCursor &k, size_t bytes) {
    while (bytes > 0 && k.i < k.n) {
        if (k.left == 0) { s_cursor_open(k, k.i + 1); continue; }
        const uint32_t n = (uint32_t)(k.left < bytes ? k.left : bytes);
        vb_prefetch_l2(k.ptr, n);
        k.ptr += n;
        k.left -= n;
        bytes -= n;
    }
}

__device__ void s_produce(SCtx &c) {
    SSmem *s = c.s;
    if (c.a.n_wl <= 0) return;
    SCursor pf;
    pf.wl = c.a.wl; pf.n = c.a.pf_bytes > 0 ? c.a.n_wl : 0;
    s_cursor_open(pf, 0);
    /* the ring's own first fill needs no prefetch: start the cursor one ring ahead */
    {
        size_t skip = (size_t)kSSlots * kSSlotBytes;
        while (skip > 0 && pf.i < pf.n) {
            if (pf.left == 0) { s_cursor_open(pf, pf.i + 1); continue; }
            const size_t n = pf.left < skip ? pf.left : skip;
            pf.ptr += n; pf.left -= n; skip -= n;
        }
        for (int b = 0; b < c.a.pf_bytes; b += kSSlotBytes) s_cursor_prefetch(pf, kSSlotBytes);
    }
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
            s_cursor_prefetch(pf, bytes);       /* the cursor keeps its distance */
        }
        cur = nxt;
    }
}

#define S_TL(k) do { if (c.a.timeline && blockIdx.x == 0 && c.tid == 0) c.a.timeline[c.tl_op * 8 + (k)] = clock64(); } while (0)

/* ------------------------------------------------------------------ GEMV */
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

    S_TL(0);
    /* this thread's residual value, requested before anything else needs L2 */
    float resv = 0.0f;
    if (epi == S_EPI_ADD && tid < p.n_rows) resv = __ldcg(op.res + p.r0 + tid);

    /* Stage the input row. Inside a k-block of 64 columns, column chunk cc (8 floats) is
     * stored as two 16-byte halves at [cc*4] and [32 + cc*4]: the 8 lanes of a row then read
     * 128 contiguous bytes per load (no bank conflicts), the 4 row groups broadcast. */
    float ss = 0.0f;
    for (int i = tid; i < K / 4; i += kSConsumerThreads) {
        float4 v = __ldcg(reinterpret_cast<const float4 *>(x) + i);
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        if (gain) {
            const float4 g = __ldg(reinterpret_cast<const float4 *>(gain) + i);
            v.x *= g.x; v.y *= g.y; v.z *= g.z; v.w *= g.w;
        }
        const int k = 4 * i, kb = k >> 6, e = k & 63;
        *reinterpret_cast<float4 *>(&s->xs[kb * 64 + ((e >> 2) & 1) * 32 + (e >> 3) * 4]) = v;
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
            for (int k = tid; k < K; k += kSConsumerThreads) xn_out[k] = __ldcg(x + k) * rscale * __ldg(gain + k);
        }
    }

    S_TL(1);
    const int c8 = lane & 7, rg = lane >> 3;
    const int J = p.J;
    const int kb_bytes = p.n_rows * (kSBlockK * 2);
    float acc[kSMaxRowSteps];
#pragma unroll
    for (int j = 0; j < kSMaxRowSteps; j++) acc[j] = 0.0f;

    /* Ring slot s belongs to warp s: it alone waits for the slot's fills (and so sees every
     * phase of that mbarrier in order) and hands the slot back. The owner walks every row step
     * of every k-block in the slot. */
    for (int ch = 0; ch < p.n_chunks; ch++) {
        const unsigned g = c.chunk_counter++;
        const unsigned slot = g % kSSlots, use = g / kSSlots;
        if (slot != (unsigned)warp) continue;
        if (!s_mbar_wait(c, &s->full[slot], use & 1u)) {
            if (!s_aborted(c)) s_raise(c, S_ERR_FULL_WAIT);
            break;      /* carry on to the CTA barriers below; the results no longer matter */
        }
        S_TL(6);
        const int kb0 = ch * p.kbs, kb1 = min(kb0 + p.kbs, p.kblocks);
        const unsigned char *base = s->ring[slot] + lane * 16;
        for (int kb = (c.a.dbg & 1) ? kb1 : kb0; kb < kb1; kb++, base += kb_bytes) {
            const float4 xa = *reinterpret_cast<const float4 *>(&s->xs[kb * 64 + c8 * 4]);
            const float4 xb = *reinterpret_cast<const float4 *>(&s->xs[kb * 64 + 32 + c8 * 4]);
            /* Row steps in groups of eight: the eight 16-byte loads of a group are issued
             * together and feed eight independent accumulator chains. A row past the CTA's last
             * one (the group is padded, and the last row step may be ragged) loads zeros. */
#pragma unroll
            for (int g8 = 0; g8 < kSMaxRowSteps / 8; g8++) {
                if (g8 * 8 < J) {
                    uint4 w[8];
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const int j = g8 * 8 + u;
                        w[u] = make_uint4(0u, 0u, 0u, 0u);
                        if (4 * j + rg < p.n_rows) w[u] = *reinterpret_cast<const uint4 *>(base + j * 512);
                    }
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        float a = acc[g8 * 8 + u];
                        a = fmaf(vb_bf16_lo(w[u].x), xa.x, a); a = fmaf(vb_bf16_hi(w[u].x), xa.y, a);
                        a = fmaf(vb_bf16_lo(w[u].y), xa.z, a); a = fmaf(vb_bf16_hi(w[u].y), xa.w, a);
                        a = fmaf(vb_bf16_lo(w[u].z), xb.x, a); a = fmaf(vb_bf16_hi(w[u].z), xb.y, a);
                        a = fmaf(vb_bf16_lo(w[u].w), xb.z, a); a = fmaf(vb_bf16_hi(w[u].w), xb.w, a);
                        acc[g8 * 8 + u] = a;
                    }
                }
            }
        }
        /* the slot's bytes are in registers */
        __syncwarp();
        if (lane == 0) vb_mbar_arrive(&s->empty[slot]);
    }

    S_TL(2);
    /* once per op: the 8 column chunks of a row (lanes), then the warps, in fixed order */
#pragma unroll
    for (int g8 = 0; g8 < kSMaxRowSteps / 8; g8++) {
        if (g8 * 8 < J) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; u++) v[u] = acc[g8 * 8 + u];
#pragma unroll
            for (int off = 1; off < 8; off <<= 1) {
#pragma unroll
                for (int u = 0; u < 8; u++) v[u] += __shfl_xor_sync(0xffffffffu, v[u], off);
            }
            if (c8 == 0) {
#pragma unroll
                for (int u = 0; u < 8; u++) s->part[warp][(g8 * 8 + u) * 4 + rg] = v[u];
            }
        }
    }
    vb_named_bar(2, kSConsumerThreads);
    S_TL(3);
    if (warp * 32 < p.n_rows) {
        const int t = tid;
        const bool valid = t < p.n_rows;
        float sum = 0.0f;
        if (valid) {
#pragma unroll
            for (int w = 0; w < kSConsumerWarps; w++) sum += s->part[w][t];
        }
        sum *= rscale;
        if (epi == S_EPI_SWIGLU) {
            /* rows interleaved (gate, up): the up value sits one lane higher */
            const float up = __shfl_down_sync(0xffffffffu, sum, 1);
            if (valid && (t & 1) == 0) {
                const float r = (sum / (1.0f + expf(-sum))) * up;
                const int o = (p.r0 + t) >> 1;
                y[o] = r;
                if (tap) tap[o] = r;
            }
        } else if (valid) {
            float r = sum;
            if (bias) r += __ldg(bias + p.r0 + t);
            if (epi == S_EPI_ADD) r = resv + r;
            y[p.r0 + t] = r;
            if (tap) tap[p.r0 + t] = r;
        }
    }
}

/* ------------------------------------------------------------------ decode attention */
/* op.x = [q | k | v] of the new token (6144 floats); op.y = attention output (4096);
 * op.p2 / op.p3 = this layer's K and V cache [kv_max, 1024]; i0 = query heads, i1 = KV heads;
 * f0 = softmax scale, f1 = RoPE theta. Restates voxtral_tts_llm.c:221-238 with tts_apply_rope
 * and tts_causal_attention (voxtral_tts_kernels.c:403-465, 602-634): interleaved pairs, the
 * score is scaled after the dot product, the running maximum starts at -1e30.
 * One CTA per query head (32 of the grid's CTAs work, no exchange between CTAs): warp w takes
 * the keys w, w + 12, ... with the reference's running-maximum update, eight keys per pass so
 * that their sixteen loads are in flight together; the warps are merged with log-sum-exp
 * weights in warp order. The new token's key and value are used from shared memory; the first
 * query head of each group also appends them to the cache. */
__device__ void s_attn(SCtx &c, const SOp &op) {
    SAttnSmem *s = reinterpret_cast<SAttnSmem *>(c.s->xs);
    const int tid = c.tid, warp = c.warp, lane = c.lane;
    const int pos = c.a.dyn->pos, kv_max = c.a.dyn->kv_max;
    if (pos < 0 || pos >= kv_max) {
        if (tid == 0) s_raise(c, S_ERR_POS_RANGE);
        return;
    }
    const int H = op.i0, G = op.i1, group = H / G;      /* 32, 8, 4 */
    const int h = blockIdx.x;
    if (h >= H) return;
    const int g = h / group;
    const int kv_dim = G * kSHeadDim, q_dim = H * kSHeadDim;
    const float scale = op.f0;
    const float *Kc = (const float *)op.p2 + g * kSHeadDim, *Vc = (const float *)op.p3 + g * kSHeadDim;
    const float *qg = op.x + (size_t)h * kSHeadDim, *kg = op.x + q_dim + g * kSHeadDim,
                *vg = op.x + q_dim + kv_dim + g * kSHeadDim;
    const bool writer = (h % group) == 0;
    constexpr int half = kSHeadDim / 2;

    /* raw values first (three loads in flight per thread group), then the rotation */
    float ra = 0.0f, rb = 0.0f;
    if (tid < half) { ra = __ldcg(qg + 2 * tid); rb = __ldcg(qg + 2 * tid + 1); }
    else if (tid < 2 * half) { ra = __ldcg(kg + 2 * (tid - half)); rb = __ldcg(kg + 2 * (tid - half) + 1); }
    else if (tid < 2 * half + kSHeadDim) { ra = __ldcg(vg + (tid - 2 * half)); }
    if (tid < 2 * half) {
        const int d = tid < half ? tid : tid - half;
        const float freq = 1.0f / powf(op.f1, (float)(2 * d) / (float)kSHeadDim);
        const float ang = (float)pos * freq;
        const float cv = cosf(ang), sv = sinf(ang);
        const float o0 = ra * cv - rb * sv, o1 = ra * sv + rb * cv;
        if (tid < half) { s->q[2 * d] = o0; s->q[2 * d + 1] = o1; }
        else {
            s->kn[2 * d] = o0; s->kn[2 * d + 1] = o1;
            if (writer) {
                float *dst = (float *)op.p2 + (size_t)pos * kv_dim + g * kSHeadDim;
                dst[2 * d] = o0; dst[2 * d + 1] = o1;
            }
        }
    } else if (tid < 2 * half + kSHeadDim) {
        const int d = tid - 2 * half;
        s->vn[d] = ra;
        if (writer) ((float *)op.p3)[(size_t)pos * kv_dim + g * kSHeadDim + d] = ra;
    }
    vb_named_bar(2, kSConsumerThreads);

    const float4 q4 = *reinterpret_cast<const float4 *>(&s->q[4 * lane]);
    float mx = -1e30f, den = 0.0f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    constexpr int kKeysPerPass = 8;
    for (int jb = warp; jb <= pos; jb += kKeysPerPass * kSConsumerWarps) {
        float4 kq[kKeysPerPass], vq[kKeysPerPass];
#pragma unroll
        for (int u = 0; u < kKeysPerPass; u++) {
            const int j = jb + u * kSConsumerWarps;
            if (j < pos) {
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
            if (jb + u * kSConsumerWarps > pos) break;
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
    if (tid < kSHeadDim) {
        float M0 = -1e30f;
#pragma unroll
        for (int w = 0; w < kSConsumerWarps; w++) M0 = fmaxf(M0, s->wml[w][0]);
        float L = 0.0f, O = 0.0f;
#pragma unroll
        for (int w = 0; w < kSConsumerWarps; w++) {
            const float lw = s->wml[w][1];
            const float e = lw > 0.0f ? expf(s->wml[w][0] - M0) : 0.0f;
            L += lw * e;
            O += s->wo[w][tid] * e;
        }
        op.y[(size_t)h * kSHeadDim + tid] = L > 0.0f ? O * (1.0f / L) : 0.0f;
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
    c.chunk_counter = 0; c.barrier_epoch = 0; c.tl_op = 0;

    /* a device-resident run that has ended: its remaining queued launches do nothing (the flag
     * was written by an earlier launch, so the whole grid agrees) */
    if (a.dyn->done) return;

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
            vb_named_bar(3, kSConsumerThreads);
            if (c.tid < kOpVecs && oi + 1 < a.n_ops)
                s_cp_async16(reinterpret_cast<uint4 *>(&s->opbuf[(oi + 1) & 1]) + c.tid,
                             reinterpret_cast<const uint4 *>(a.ops + oi + 1) + c.tid);
            const SOp &op = s->opbuf[oi & 1];
            const int flags = op.flags;
            switch (op.type) {
            case S_OP_GEMV:   s_gemv(c, op); break;
            case S_OP_ATTN:   s_attn(c, op); break;
            case S_OP_EMBED:  s_embed(c, op); break;
            case S_OP_ARGMAX: s_argmax(c, op); break;
            case S_OP_WAIT:   s_wait_flag(c, op); break;
            default: if (c.tid == 0) s_raise(c, S_ERR_BAD_OP); break;
            }
            S_TL(4);
            const bool stop = !(flags & S_F_NOSYNC) && oi + 1 < a.n_ops && s_grid_sync(c);
            S_TL(5);
            c.tl_op++;
            if (stop) break;
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
    dst[i] = src[((size_t)(r0 + r) * K + (size_t)kb * kSBlockK) / 8 + v];
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
int stream_probe(int N, int K, int n_ops, int sync, int reps, int dbg, float *ms_out, double *bytes_per_launch) {
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
        a.bar_counter = words; a.exit_counter = words + 16; a.status = (int *)(words + 32);
        a.wait_cycles = 2000000000LL; a.dbg = dbg; a.timeline = nullptr;
        a.pf_bytes = getenv("VB200_STREAM_PF") ? atoi(getenv("VB200_STREAM_PF")) : kSPrefetchBytes;
        if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) break;
        for (int i = 0; i < 2 && ok; i++) ok = stream_launch(a, n_cta, 0) == cudaSuccess;
        cudaEventRecord(e0, 0);
        for (int i = 0; i < reps && ok; i++) ok = stream_launch(a, n_cta, 0) == cudaSuccess;
        cudaEventRecord(e1, 0);
        if (!ok || cudaDeviceSynchronize() != cudaSuccess) break;
        int st = 0;
        cudaMemcpy(&st, words + 32, sizeof(int), cudaMemcpyDeviceToHost);
        if (st) break;
        if (getenv("VB200_STREAM_TL")) {
            long long *tl = nullptr;
            if (cudaMalloc(&tl, sizeof(long long) * 8 * n_ops) == cudaSuccess) {
                cudaMemset(tl, 0, sizeof(long long) * 8 * n_ops);
                a.timeline = tl;
                stream_launch(a, n_cta, 0);
                cudaDeviceSynchronize();
                std::vector<long long> h(8 * n_ops);
                cudaMemcpy(h.data(), tl, sizeof(long long) * 8 * n_ops, cudaMemcpyDeviceToHost);
                for (int i = 0; i < n_ops; i++) {
                    fprintf(stderr, "op %2d:", i);
                    for (int k = 0; k < 7; k++) fprintf(stderr, " %8.2f", (double)(h[8 * i + k] - h[0]) / 1965.0);
                    fprintf(stderr, "\n");
                }
                cudaFree(tl);
                a.timeline = nullptr;
            }
        }
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
