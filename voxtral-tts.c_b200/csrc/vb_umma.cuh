/*
 * vb_umma.cuh - sm_100a tensor-core PTX wrappers shared by the GEMM kernels: TMA tile
 * loads, UMMA shared-memory and instruction descriptors, tcgen05.mma / commit / ld, fences.
 */
#ifndef VB_UMMA_CUH
#define VB_UMMA_CUH

#include <cuda.h>

#include "vb_common.cuh"
#include "vb_tc.cuh"

namespace vb {

VB_DEVINL void tma_load_2d(void *smem_dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            vb_smem_u32(smem_dst)),
        "l"(map), "r"(vb_smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

/* K-major operand tile with 128-byte swizzle: rows 128 B apart, 8-row groups 1024 B apart
 * (stride byte offset), descriptor version 1 (sm_100), layout type 2 (SWIZZLE_128B). */
VB_DEVINL uint64_t umma_desc_k_sw128(const void *smem_tile) {
    const uint32_t addr = vb_smem_u32(smem_tile);
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;                 /* leading byte offset: unused for swizzled K-major */
    d |= (uint64_t)(1024 >> 4) << 32;       /* stride byte offset */
    d |= (uint64_t)1 << 46;                 /* descriptor version */
    d |= (uint64_t)2 << 61;                 /* SWIZZLE_128B */
    return d;
}

/* kind::f16, BF16 x BF16 -> fp32, both operands K-major, M = 128, N = nb. */
VB_DEVINL uint32_t umma_idesc_bf16(int nb) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(nb >> 3) << 17) | ((uint32_t)(kTcTileN >> 4) << 24);
}

VB_DEVINL void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

VB_DEVINL void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     vb_smem_u32(bar))
                 : "memory");
}

VB_DEVINL void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

/* Tensor-parallel consumer wait (one thread): every source rank has published this visit of
 * the buffer. Bounded; false (and a status code) when it runs out. */
VB_DEVINL bool tp_wait(const TcWait &w) {
    if (w.n <= 0) return true;
    const unsigned frame = *(volatile const unsigned *)w.epoch;
    const unsigned target = (frame - 1u) * (unsigned)w.visits_per_frame + (unsigned)w.visit;
    const long long t0 = clock64();
    for (int i = 0; i < w.n; i++) {
        while ((int)(vb_ld_acquire_sys(w.flags + i) - target) < 0) {
            if (clock64() - t0 > VB_WAIT_CYCLES) {
                if (w.status) atomicCAS(w.status, 0, 31);
                return false;
            }
        }
    }
    return true;
}

/* Tensor-parallel producer side, called by one thread of a CTA after the CTA's stores and a
 * CTA-wide barrier: make them visible system-wide and take a ticket; the last CTA of the launch
 * publishes the visit's sequence number on every rank. */
VB_DEVINL void tp_publish(const TcPush &p, unsigned n_ctas) {
    __threadfence_system();
    const unsigned t = atomicAdd(p.ticket, 1u);
    if (t != n_ctas - 1u) return;
    *p.ticket = 0u;
    __threadfence_system();
    const unsigned seq = (*(volatile const unsigned *)p.epoch - 1u) * (unsigned)p.visits_per_frame + (unsigned)p.visit;
    for (int d = 0; d < p.n_dst; d++) vb_st_release_sys(p.flag[d], seq);
}

VB_DEVINL void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
VB_DEVINL void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }


} // namespace vb

#endif
