/*
 * vb_noalloc.cu - a linear (y = x . W^T) entry point that never allocates.
 *
 * Who needs it: code that is not allowed to take memory from the CUDA allocator at
 * the moment it wants a matrix product - a plugin running inside a host application
 * that owns all of the device memory and hands out fixed buffers, a real-time audio
 * callback where cudaMalloc's implicit device synchronisation is unacceptable, or a
 * caller that must not disturb an allocator another library is tracking. The
 * regular entry point (tts_cuda_linear_bf16) needs tts_cuda_init first, which
 * allocates the K/V cache and all working buffers; this one needs nothing.
 *
 * How: the frame kernel needs a little global memory besides its operands - the op
 * descriptors it executes, its grid-barrier counters, a status word and the
 * per-launch scalars. Here those live in a file-scope device array of fixed size
 * that every GPU loading this library carries until the process exits.
 */
#include "../../include/voxtral_b200_ext.h"
#include "vb_engine.cuh"
#include "vb_simple.cuh"

#include <stdio.h>
#include <string.h>

namespace {

constexpr int kMaxOps = 64;                   /* row blocks of 8 -> at most 512 activation rows */
constexpr int kMaxDevices = 64;

struct StaticScratch {
    VbOp ops[kMaxOps];
    VbDyn dyn;
    unsigned bar_counter[4];
    unsigned exit_counter[4];
    int status[4];
};

/* The scratch itself. In host code this name is only a handle for the runtime; the
 * address the kernel needs comes from cudaGetSymbolAddress, per device. */
static __device__ __align__(256) unsigned char g_static_scratch[sizeof(StaticScratch)];

struct PerDevice {
    bool ready = false;
    StaticScratch *scratch = nullptr;   /* device address of g_static_scratch on that GPU */
    int n_cta = 0;
};
PerDevice g_dev[kMaxDevices];

/* First use on a device, with that device current: resolve the array's device
 * address, size the grid, zero the words that must start at zero. */
int setup_device(int dev) {
    PerDevice &d = g_dev[dev];
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) {
        fprintf(stderr, "voxtral_b200: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
        return -1;
    }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess || prop.major != 10) {
        fprintf(stderr, "voxtral_b200: device %d is not sm_100\n", dev);
        return -1;
    }
    d.n_cta = vb::engine_max_ctas(dev);
    if (d.n_cta <= 0) return -1;
    d.scratch = (StaticScratch *)p;
    if (cudaMemset(p, 0, sizeof(StaticScratch)) != cudaSuccess) return -1;
    d.ready = true;
    return 0;
}

} // namespace

extern "C" int vb200_linear_bf16_static(float *d_y, const float *d_x, const uint16_t *d_W, int seq_len,
                                        int in_dim, int out_dim) {
    if (seq_len < 0 || in_dim <= 0 || out_dim <= 0) return -1;
    if (seq_len == 0) return 0;
    if (seq_len > kMaxOps * vb::kMaxM) {
        fprintf(stderr, "voxtral_b200: vb200_linear_bf16_static takes at most %d rows per call (got %d)\n",
                kMaxOps * vb::kMaxM, seq_len);
        return -2;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
    if (!g_dev[dev].ready && setup_device(dev) != 0) return -1;
    PerDevice &d = g_dev[dev];

    const bool aligned = (((uintptr_t)d_x | (uintptr_t)d_W) & 15) == 0;
    /* validated for the widest row block the ops below use: the cross-pass accumulators of a
     * K > 4096 matrix hold rows-per-CTA x M floats */
    const int m_max = seq_len < vb::kMaxM ? seq_len : vb::kMaxM;
    if (!aligned || (seq_len > 1 && (in_dim & 3)) ||
        vb::gemv_validate(out_dim, in_dim, m_max, VB_EPI_STORE, d.n_cta) != 0) {
        /* shapes the streaming kernel does not take: the plain kernel needs no scratch at all */
        vb::linear_generic(d_y, d_x, d_W, nullptr, seq_len, in_dim, out_dim, 0);
        return cudaGetLastError() == cudaSuccess ? 0 : -1;
    }

    VbOp ops[kMaxOps];
    int n = 0;
    for (int r = 0; r < seq_len; r += vb::kMaxM, n++) {
        VbOp &o = ops[n];
        memset(&o, 0, sizeof(o));
        o.type = VB_OP_GEMV;
        o.M = seq_len - r < vb::kMaxM ? seq_len - r : vb::kMaxM;
        o.N = out_dim; o.K = in_dim; o.epi = VB_EPI_STORE;
        o.W = d_W;
        o.x = d_x + (size_t)r * in_dim; o.ldx = in_dim;
        o.y = d_y + (size_t)r * out_dim; o.ldy = out_dim;
        o.flags = VB_F_NOSYNC;               /* row blocks are independent */
    }
    /* Stream 0 orders this copy after the previous call's kernel, which still reads the slots. */
    if (cudaMemcpyAsync(d.scratch->ops, ops, sizeof(VbOp) * n, cudaMemcpyHostToDevice, 0) != cudaSuccess) return -1;
    vb::EngineArgs a;
    a.ops = d.scratch->ops; a.n_ops = n; a.dyn = &d.scratch->dyn;
    a.bar_counter = d.scratch->bar_counter; a.exit_counter = d.scratch->exit_counter;
    a.status = d.scratch->status; a.prefetch_chunks = 0;
    const cudaError_t e = vb::engine_launch(a, d.n_cta, 0);
    if (e != cudaSuccess) {
        fprintf(stderr, "voxtral_b200: launch failed: %s\n", cudaGetErrorString(e));
        return -1;
    }
    return 0;
}

extern "C" int vb200_linear_bf16_static_status(void) {
    int dev = 0, st = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices || !g_dev[dev].ready) return -1;
    if (cudaMemcpy(&st, g_dev[dev].scratch->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (st != 0) {
        /* a bounded wait ran out inside the kernel: start the next call from clean counters */
        cudaMemset(g_dev[dev].scratch->bar_counter, 0, sizeof(unsigned) * 8 + sizeof(int) * 4);
    }
    return st;
}
