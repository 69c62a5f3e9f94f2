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
 *   warp 16, lane 0   producer. Walks the op list ahead of everyone and copies this CTA's
 *                     slab of every matrix, 16 KB at a time, into an 11-slot ring with 1-D
 *                     bulk copies (cp.async.bulk, completion on an mbarrier, no multicast).
 *                     It never waits for an op's input, only for a free slot: while the
 *                     other warps sit at a grid barrier the ring fills up with the next
 *                     matrix.
 *   warps 0..15       consumers. The slab order makes a warp load 512 contiguous bytes
 *                     (4 rows x 8 chunks of 8 BF16): lane = (row r, chunk c). A lane keeps
 *                     its 8 activations of the k-block in registers and one accumulator per
 *                     row step, so nothing is reduced per chunk: the 8 lanes of a row and
 *                     the warps that share a row range are summed once per op, in fixed
 *                     order (bit-reproducible; BF16 -> fp32 is an exact shift and all
 *                     products are fp32, as in voxtral_tts_kernels.c:152-185).
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

namespace vb {

struct SSmem {
    alignas(128) unsigned char ring[kSSlots][kSSlotBytes];
    /* the staged input row (permuted, see s_gemv); the attention op uses the same bytes */
    alignas(16) float xs[kSMaxK];
    float part[kSConsumerWarps][kSMaxRowSteps * 4];
    float red[kSConsumerWarps];
    uint64_t full[kSSlots];
    uint64_t empty[kSSlots];
    int abort_flag;     /* raised by any thread of the CTA, at any time */
    int abort_seen;     /* the abort flag as sampled inside the last grid barrier: the same for every consumer thread */
    int last_flag;
};

/* Attention scratch, overlaid on SSmem::xs. */
struct SAttnSmem {
    alignas(16) float qs[4][kSHeadDim];
    alignas(16) float attn_o[kSAttnSubsets][4][kSHeadDim];
    float attn_ml[kSAttnSubsets][4][2];
    float cs[kSHeadDim];
    float cmb_m[kSKeySplitsMax * 4], cmb_l[kSKeySplitsMax * 4];
};
static_assert(sizeof(SAttnSmem) <= sizeof(float) * kSMaxK, "attention scratch must fit the row buffer");
static_assert(sizeof(SSmem) <= 232448, "over the 227 KB a CTA may use");

struct SCtx {
    SSmem *s;
    SArgs a;
    int tid, warp, lane;
    unsigned chunk_counter;
    unsigned barrier_epoch;
};

VB_DEVINL bool s_aborted(const SCtx &c) { return *(volatile int *)&c.s->abort_flag != 0; }

VB_DEVINL void s_raise(SCtx &c, int code) {
    atomicCAS(c.a.status, 0, code);
    *(volatile int *)&c.s->abort_flag = 1;
}

VB_DEVINL bool s_mbar_wait(SCtx &c, uint64_t *bar, uint32_t parity) {
    if (vb_mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (vb_mbar_try_wait(bar, parity)) return true;
        if (s_aborted(c)) return false;
        if (clock64() - t0 > c.a.wait_cycles) return false;
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
            __threadfence();
            vb_atomic_add_release_gpu(c.a.bar_counter, 1u);
            const unsigned target = c.barrier_epoch * gridDim.x;
            const long long t0 = clock64();
            while (vb_ld_acquire_gpu(c.a.bar_counter) < target) {
                if (vb_ld_relaxed_gpu_s32(c.a.status) != 0) { *(volatile int *)&c.s->abort_flag = 1; break; }
                if (clock64() - t0 > c.a.wait_cycles) { s_raise(c, S_ERR_GRID_BARRIER); break; }
            }
            __threadfence();
        }
        c.s->abort_seen = s_aborted(c) ? 1 : 0;
    }
    vb_named_bar(1, kSConsumerThreads);
    return *(volatile int *)&c.s->abort_seen != 0;
}

/* ------------------------------------------------------------------ producer */
__device__ void s_produce(SCtx &c) {
    SSmem *s = c.s;
    for (int oi = 0; oi < c.a.n_ops; oi++) {
        const SOp &op = c.a.ops[oi];
        if (op.type != S_OP_GEMV) continue;
        const SPlan p = stream_plan(op.N, op.K, op.epi, blockIdx.x, gridDim.x);
        if (p.n_chunks == 0) continue;
        const unsigned char *src = (const unsigned char *)op.W + (size_t)p.r0 * op.K * 2;
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
    }
}

/* ------------------------------------------------------------------ GEMV */
__device__ void s_gemv(SCtx &c, const SOp &op) {
    SSmem *s = c.s;
    const int N = op.N, K = op.K, epi = op.epi;
    (void)N;
    const SPlan p = stream_plan(op.N, K, epi, blockIdx.x, gridDim.x);
    const int tid = c.tid, warp = c.warp, lane = c.lane;
    float *const y = op.y;
    float *const tap = op.tap;
    const float *const bias = op.bias;
    const float *const gain = op.gain;

    /* this thread's residual value, requested before anything else needs L2 */
    float resv = 0.0f;
    if (epi == S_EPI_ADD && tid < p.n_rows) resv = __ldcg(op.res + p.r0 + tid);

    /* Stage the input row. Inside a k-block of 64 columns, column chunk cc (8 floats) is
     * stored as two 16-byte halves at [cc*4] and [32 + cc*4]: the 8 lanes of a row then read
     * 128 contiguous bytes per load (no bank conflicts), the 4 row groups broadcast. */
    float ss = 0.0f;
    for (int i = tid; i < K / 4; i += kSConsumerThreads) {
        float4 v = __ldcg(reinterpret_cast<const float4 *>(op.x) + i);
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
        rscale = 1.0f / sqrtf(t / (float)K + op.eps);
        if (op.xn_out && blockIdx.x == 0) {
            for (int k = tid; k < K; k += kSConsumerThreads)
                op.xn_out[k] = __ldcg(op.x + k) * rscale * __ldg(gain + k);
        }
    }

    const int c8 = lane & 7, rg = lane >> 3;
    const int R = p.R, jr = p.jr;
    const int rr = warp & (R - 1), kmod = kSConsumerWarps / R, kres = warp / R;
    const int kb_bytes = p.n_rows * (kSBlockK * 2);
    const int row0 = rr * jr * 4 + rg;          /* this lane's row in row step 0 */
    float acc[kSMaxRowSteps];
#pragma unroll
    for (int j = 0; j < kSMaxRowSteps; j++) acc[j] = 0.0f;

    for (int ch = 0; ch < p.n_chunks; ch++) {
        const unsigned slot = c.chunk_counter % kSSlots, use = c.chunk_counter / kSSlots;
        c.chunk_counter++;
        if (!s_mbar_wait(c, &s->full[slot], use & 1u)) {
            if (!s_aborted(c)) s_raise(c, S_ERR_FULL_WAIT);
            break;      /* carry on to the CTA barriers below; the results no longer matter */
        }
        const int kb0 = ch * p.kbs, kb1 = min(kb0 + p.kbs, p.kblocks);
        int kb = kb0 + ((kres - (kb0 % kmod)) + kmod) % kmod;
        for (; kb < kb1; kb += kmod) {
            const float4 xa = *reinterpret_cast<const float4 *>(&s->xs[kb * 64 + c8 * 4]);
            const float4 xb = *reinterpret_cast<const float4 *>(&s->xs[kb * 64 + 32 + c8 * 4]);
            const unsigned char *base = s->ring[slot] + (size_t)(kb - kb0) * kb_bytes + rr * jr * 512 + lane * 16;
#pragma unroll
            for (int j = 0; j < kSMaxRowSteps; j++) {
                if (j < jr && row0 + 4 * j < p.n_rows) {
                    const uint4 w = *reinterpret_cast<const uint4 *>(base + j * 512);
                    float a = acc[j];
                    a = fmaf(vb_bf16_lo(w.x), xa.x, a); a = fmaf(vb_bf16_hi(w.x), xa.y, a);
                    a = fmaf(vb_bf16_lo(w.y), xa.z, a); a = fmaf(vb_bf16_hi(w.y), xa.w, a);
                    a = fmaf(vb_bf16_lo(w.z), xb.x, a); a = fmaf(vb_bf16_hi(w.z), xb.y, a);
                    a = fmaf(vb_bf16_lo(w.w), xb.z, a); a = fmaf(vb_bf16_hi(w.w), xb.w, a);
                    acc[j] = a;
                }
            }
        }
        /* the slot's bytes this warp needs are in registers */
        __syncwarp();
        if (lane == 0) vb_mbar_arrive(&s->empty[slot]);
    }

    /* once per op: the 8 column chunks of a row (lanes), then the warps of a row range */
#pragma unroll
    for (int j = 0; j < kSMaxRowSteps; j++) {
        float v = acc[j];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        if (c8 == 0) s->part[warp][j * 4 + rg] = v;
    }
    vb_named_bar(2, kSConsumerThreads);
    if (warp * 32 < p.n_rows) {
        const int t = tid;
        const bool valid = t < p.n_rows;
        float sum = 0.0f;
        if (valid) {
            const int js = t >> 2, rt = js / jr, j = js - rt * jr, rl = j * 4 + (t & 3);
            for (int w = rt; w < kSConsumerWarps; w += R) sum += s->part[w][rl];
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
 * op.p2 / op.p3 = this layer's K and V cache [kv_max, 1024]; op.p0 = float scratch for the
 * key-split partials; op.p1 = one ticket per KV head; i0 = query heads, i1 = KV heads;
 * f0 = softmax scale, f1 = RoPE theta. Restates voxtral_tts_llm.c:221-238 with tts_apply_rope
 * and tts_causal_attention (voxtral_tts_kernels.c:403-465, 602-634): interleaved pairs,
 * the score is scaled after the dot product, the running maximum starts at -1e30. A CTA
 * serves the four query heads of one KV head on one slice of the keys; four warp subsets
 * split the slice; slices are merged with log-sum-exp weights in slice order by the last
 * CTA of the KV head to finish (a ticket, no spin). */
__device__ void s_attn(SCtx &c, const SOp &op) {
    SAttnSmem *s = reinterpret_cast<SAttnSmem *>(c.s->xs);
    const int tid = c.tid, warp = c.warp, lane = c.lane;
    const int pos = c.a.dyn->pos, kv_max = c.a.dyn->kv_max;
    if (pos < 0 || pos >= kv_max) {
        if (tid == 0) s_raise(c, S_ERR_POS_RANGE);
        return;
    }
    const int H = op.i0, G = op.i1, group = H / G;      /* 32, 8, 4 */
    const int kv_dim = G * kSHeadDim, q_dim = H * kSHeadDim;
    const int nk = pos + 1;
    int max_s = (int)gridDim.x / G;
    if (max_s > kSKeySplitsMax) max_s = kSKeySplitsMax;
    if (max_s < 1) max_s = 1;
    int S = (nk + 31) / 32;
    if (S > max_s) S = max_s;
    const int item = blockIdx.x;
    if (item >= G * S) return;
    const int g = item / S, sp = item % S;
    const int j0 = (int)((long long)nk * sp / S), j1 = (int)((long long)nk * (sp + 1) / S);
    float *Kc = (float *)op.p2, *Vc = (float *)op.p3;
    const float *q = op.x, *kn = op.x + q_dim, *vn = op.x + q_dim + kv_dim;
    const bool writer = sp == S - 1;    /* its key range ends with the new token */

    if (tid < kSHeadDim / 2) {
        const float freq = 1.0f / powf(op.f1, (float)(2 * tid) / (float)kSHeadDim);
        const float ang = (float)pos * freq;
        s->cs[2 * tid] = cosf(ang);
        s->cs[2 * tid + 1] = sinf(ang);
    }
    vb_named_bar(2, kSConsumerThreads);
    const int half = kSHeadDim / 2;
    if (tid < group * half) {
        const int hh = tid / half, d = tid % half;
        const float *src = q + (size_t)(g * group + hh) * kSHeadDim;
        const float a = __ldcg(src + 2 * d), b = __ldcg(src + 2 * d + 1);
        const float cv = s->cs[2 * d], sv = s->cs[2 * d + 1];
        s->qs[hh][2 * d] = a * cv - b * sv;
        s->qs[hh][2 * d + 1] = a * sv + b * cv;
    } else if (writer && tid < group * half + half) {
        const int d = tid - group * half;
        const float a = __ldcg(kn + g * kSHeadDim + 2 * d), b = __ldcg(kn + g * kSHeadDim + 2 * d + 1);
        const float cv = s->cs[2 * d], sv = s->cs[2 * d + 1];
        float *dst = Kc + (size_t)pos * kv_dim + g * kSHeadDim;
        dst[2 * d] = a * cv - b * sv;
        dst[2 * d + 1] = a * sv + b * cv;
        __threadfence();
    } else if (writer && tid >= 384 && tid < 384 + kSHeadDim) {
        const int d = tid - 384;
        Vc[(size_t)pos * kv_dim + g * kSHeadDim + d] = __ldcg(vn + g * kSHeadDim + d);
        __threadfence();
    }
    vb_named_bar(2, kSConsumerThreads);

    const int hh = warp & 3, ss = warp >> 2;
    const float4 q4 = *reinterpret_cast<const float4 *>(&s->qs[hh][4 * lane]);
    float mx = -1e30f, den = 0.0f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    /* four keys per pass: their eight loads are in flight together, the running-maximum update
     * then takes them in key order as the reference does */
    constexpr int kKeysPerPass = 4;
    for (int jb = j0 + ss; jb < j1; jb += kKeysPerPass * kSAttnSubsets) {
        float4 kq[kKeysPerPass], vq[kKeysPerPass];
#pragma unroll
        for (int u = 0; u < kKeysPerPass; u++) {
            const int j = jb + u * kSAttnSubsets;
            if (j < j1) {
                kq[u] = vb_ldcg4(Kc + (size_t)j * kv_dim + g * kSHeadDim + 4 * lane);
                vq[u] = vb_ldcg4(Vc + (size_t)j * kv_dim + g * kSHeadDim + 4 * lane);
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
            const float d = dq[u] * op.f0;
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
    *reinterpret_cast<float4 *>(&s->attn_o[ss][hh][4 * lane]) = o;
    if (lane == 0) { s->attn_ml[ss][hh][0] = mx; s->attn_ml[ss][hh][1] = den; }
    vb_named_bar(2, kSConsumerThreads);

    /* merge the four key subsets: thread = (head, dim) */
    const int th = tid / kSHeadDim, td = tid % kSHeadDim;
    float M0 = -1e30f;
#pragma unroll
    for (int u = 0; u < kSAttnSubsets; u++) M0 = fmaxf(M0, s->attn_ml[u][th][0]);
    float L = 0.0f, O = 0.0f;
#pragma unroll
    for (int u = 0; u < kSAttnSubsets; u++) {
        const float w = (s->attn_ml[u][th][1] > 0.0f) ? expf(s->attn_ml[u][th][0] - M0) : 0.0f;
        L += s->attn_ml[u][th][1] * w;
        O += s->attn_o[u][th][td] * w;
    }
    float *out = op.y + (size_t)(g * group + th) * kSHeadDim + td;
    if (S == 1) {
        *out = (L > 0.0f) ? O * (1.0f / L) : 0.0f;
        return;
    }
    /* several CTAs share this KV head: publish the slice, the last arrival merges */
    const int stride = kSHeadDim + 2;
    float *po = (float *)op.p0 + (size_t)g * kSKeySplitsMax * group * stride;   /* [slice][head][128 + 2] */
    float *mine = po + ((size_t)sp * group + th) * stride;
    mine[td] = O;
    if (td == 0) { mine[kSHeadDim] = M0; mine[kSHeadDim + 1] = L; }
    __threadfence();
    vb_named_bar(2, kSConsumerThreads);
    unsigned *tickets = (unsigned *)op.p1;
    if (tid == 0) {
        const unsigned t = atomicAdd(&tickets[g], 1u);
        c.s->last_flag = (t == (unsigned)(S - 1));
        if (c.s->last_flag) tickets[g] = 0u;
    }
    vb_named_bar(2, kSConsumerThreads);
    if (!c.s->last_flag) return;
    __threadfence();
    if (tid < S * group) {
        const float *pu = po + (size_t)tid * stride;     /* (slice, head) = tid / group, tid % group */
        s->cmb_m[tid] = __ldcg(pu + kSHeadDim);
        s->cmb_l[tid] = __ldcg(pu + kSHeadDim + 1);
    }
    float ov[kSKeySplitsMax];
#pragma unroll
    for (int u = 0; u < kSKeySplitsMax; u++)
        ov[u] = u < S ? __ldcg(po + ((size_t)u * group + th) * stride + td) : 0.0f;
    vb_named_bar(2, kSConsumerThreads);
    float Mg = -1e30f;
    for (int u = 0; u < S; u++) Mg = fmaxf(Mg, s->cmb_m[u * group + th]);
    float Lg = 0.0f, Og = 0.0f;
#pragma unroll
    for (int u = 0; u < kSKeySplitsMax; u++) {
        if (u < S) {
            const float lu = s->cmb_l[u * group + th];
            const float w = (lu > 0.0f) ? expf(s->cmb_m[u * group + th] - Mg) : 0.0f;
            Lg += lu * w;
            Og += ov[u] * w;
        }
    }
    *out = (Lg > 0.0f) ? Og * (1.0f / Lg) : 0.0f;
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

    if (c.tid == 0) {
        for (int i = 0; i < kSSlots; i++) {
            vb_mbar_init(&s->full[i], 1);
            vb_mbar_init(&s->empty[i], kSConsumerWarps);
        }
        s->abort_flag = 0;
        s->abort_seen = 0;
        s->last_flag = 0;
        vb_mbar_init_fence();
    }
    __syncthreads();

    if (c.warp == kSConsumerWarps) {
        if (c.lane == 0) s_produce(c);
    } else {
        for (int oi = 0; oi < a.n_ops; oi++) {
            const SOp &op = a.ops[oi];
            switch (op.type) {
            case S_OP_GEMV:   s_gemv(c, op); break;
            case S_OP_ATTN:   s_attn(c, op); break;
            case S_OP_EMBED:  s_embed(c, op); break;
            case S_OP_ARGMAX: s_argmax(c, op); break;
            case S_OP_WAIT:   s_wait_flag(c, op); break;
            default: if (c.tid == 0) s_raise(c, S_ERR_BAD_OP); break;
            }
            if (!(op.flags & S_F_NOSYNC) && oi + 1 < a.n_ops && s_grid_sync(c)) break;
        }
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

} // namespace vb
