/*
 * vb_common.cuh - sm_100a PTX wrappers shared by the kernels: mbarriers, 1-D bulk
 * (TMA) copies into shared memory, scoped atomics for the grid barrier, and
 * bounded waits. Every wait in this library has a deadline; a wait that runs out
 * records a status code and lets the kernel return instead of hanging the GPU.
 */
#ifndef VB_COMMON_CUH
#define VB_COMMON_CUH

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define VB_DEVINL __device__ __forceinline__

/* ~1 s at 1.9 GHz: far beyond any legitimate wait in a millisecond-scale kernel. */
#define VB_WAIT_CYCLES (2000000000LL)

VB_DEVINL uint32_t vb_smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

VB_DEVINL void vb_mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(vb_smem_u32(bar)), "r"(count));
}

VB_DEVINL void vb_mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

VB_DEVINL void vb_mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(vb_smem_u32(bar)) : "memory");
}

VB_DEVINL void vb_mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(vb_smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

VB_DEVINL bool vb_mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(vb_smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

/* Waits for the phase with the given parity to complete. Returns false when the
 * deadline passes or another thread of the CTA has already given up. */
VB_DEVINL bool vb_mbar_wait(uint64_t *bar, uint32_t parity, volatile int *cta_abort) {
    if (vb_mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    while (true) {
        if (vb_mbar_try_wait(bar, parity)) return true;
        if (*cta_abort) return false;
        if (clock64() - t0 > VB_WAIT_CYCLES) return false;
    }
}

/* 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.
 * Both addresses 16-byte aligned, size a multiple of 16. No multicast. */
VB_DEVINL void vb_bulk_g2s(void *smem_dst, const void *gmem_src, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            vb_smem_u32(smem_dst)),
        "l"(gmem_src), "r"(bytes), "r"(vb_smem_u32(bar))
        : "memory");
}

/* Pulls a global range into L2 without a destination (16-byte aligned, size a
 * multiple of 16). */
VB_DEVINL void vb_prefetch_l2(const void *gmem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gmem_src), "r"(bytes) : "memory");
}

VB_DEVINL void vb_named_bar(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

VB_DEVINL unsigned vb_atomic_add_release_gpu(unsigned *p, unsigned v) {
    unsigned old;
    asm volatile("atom.add.release.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}

VB_DEVINL unsigned vb_atomic_add_acq_rel_gpu(unsigned *p, unsigned v) {
    unsigned old;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}

VB_DEVINL unsigned vb_ld_acquire_gpu(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

/* System scope: words that another GPU writes or reads over NVLink (tensor-parallel flags). */
VB_DEVINL unsigned vb_ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
VB_DEVINL void vb_st_release_sys(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

VB_DEVINL int vb_ld_relaxed_gpu_s32(const int *p) {
    int v;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

/* Activations are produced by other SMs earlier in the same launch: read them
 * from L2, never through a possibly stale L1 line or the read-only path. */
VB_DEVINL float vb_ldcg(const float *p) { return __ldcg(p); }
VB_DEVINL float4 vb_ldcg4(const float *p) { return __ldcg(reinterpret_cast<const float4 *>(p)); }

VB_DEVINL float vb_bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
VB_DEVINL float vb_bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }

VB_DEVINL float vb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

/* Sums V per-lane values over the 32 lanes with the halving butterfly: at each
 * step a lane keeps half of its values and hands the other half to its partner,
 * so the total is about V + 5 shuffles instead of 5 * V. On return v[0] holds the
 * complete sum of value `index` (returned); lanes whose index is >= V hold
 * nothing useful. */
template <int V>
VB_DEVINL int vb_warp_multi_sum(float (&v)[V], int lane) {
    int base = 0;
    int count = V;    /* slots per lane, padding included (same on every lane) */
    int real = V;     /* how many of this lane's slots carry actual values */
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        if (count > 1) {
            const int half = (count + 1) >> 1;
            const bool up = (lane & o) != 0;
#pragma unroll
            for (int i = 0; i < (V + 1) / 2; i++) {
                if (i < half) {
                    float hi = (i + half < count) ? v[i + half] : 0.0f;
                    float send = up ? v[i] : hi;
                    float keep = up ? hi : v[i];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                }
            }
            if (up) { base += half; real = real > half ? real - half : 0; }
            else real = real < half ? real : half;
            count = half;
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
        }
    }
    /* a lane that ended on a padding slot (odd counts on the way) owns no value */
    return real > 0 ? base : V;
}

/* Programmatic dependent launch: launch_dependents lets the next kernel of the stream begin
 * its prologue; wait blocks until the previous kernel has completed and its writes are visible
 * (a no-op for kernels launched without the attribute). */
VB_DEVINL void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
VB_DEVINL void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

/* v = t0 + t1 + t2 with three BF16 terms (8 + 8 + 8 mantissa bits): what the tensor-core
 * path feeds instead of an fp32 activation. */
VB_DEVINL void vb_split3(float v, uint16_t &t0, uint16_t &t1, uint16_t &t2) {
    const __nv_bfloat16 h0 = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(h0);
    const __nv_bfloat16 h1 = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(h1);
    const __nv_bfloat16 h2 = __float2bfloat16_rn(r2);
    t0 = __bfloat16_as_ushort(h0);
    t1 = __bfloat16_as_ushort(h1);
    t2 = __bfloat16_as_ushort(h2);
}

#endif
