/*
 * voxtral_b200_probe.h - measurement and inspection aids of libvoxtral_b200.so.
 *
 * None of these is part of the synthesis path and none has a counterpart in
 * mudler/voxtral-tts.c: they time kernels in isolation (the benchmark's roofline leg uses
 * them) or expose host-side planning arithmetic to the CPU tests.
 */
#ifndef VOXTRAL_B200_PROBE_H
#define VOXTRAL_B200_PROBE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Measurement aid: the decoder's 104 layer GEMMs (every decoder weight byte once) launched
 * back to back `iters` times between two CUDA events, on the single-utterance buffers
 * (which = 0) or on the open batch (which = 1). Returns the elapsed ms, the weight bytes of
 * one sweep and its launch count. */
int vb200_gemm_sweep(int which, int iters, float *ms, double *bytes_per_sweep, int *launches_per_sweep);
/* Measurement aid without a model: a generated [N, K] BF16 matrix, M activation rows, `reps`
 * launches of the tensor-core GEMM between two CUDA events on the default stream (split-K
 * partial epilogue, or the SwiGLU epilogue when swiglu != 0; tiled bit 0: tile-contiguous weight
 * copy as the frame uses; bit 1: a single copy, which stays in L2 when it fits, instead of
 * rotating through 512 MB of copies). Returns elapsed ms and the split-K factor chosen. */
int vb200_tc_gemm_probe(int M, int N, int K, int swiglu, int tiled, int reps, float *ms, int *splits);
/* Measurement aid: the streaming decoder-step kernel (26 layers, semantic head, llm token,
 * argmax: one launch that reads every decoder weight byte once) launched `iters` times back to
 * back at cache row `pos` between two CUDA events. Returns the elapsed ms and the algorithmic
 * bytes of one launch (weights + the cache rows attention reads). Needs all weights uploaded. */
int vb200_stream_step_ms(int pos, int iters, float *ms, double *bytes_per_launch);
/* Measurement aid without a model: the streaming kernel on `n_ops` GEMV ops over generated
 * [N, K] BF16 matrices (rotating copies, so no op finds its weights in L2), with (sync = 1) or
 * without a grid barrier after every op; `reps` launches between two CUDA events on the default
 * stream. Returns elapsed ms and the weight bytes of one launch. */
int vb200_stream_probe(int N, int K, int n_ops, int sync, int reps, float *ms, double *bytes_per_launch);
/* Failure-path self test that is safe on a shared GPU: launches the streaming kernel on an op
 * that waits for a flag nothing ever sets, with a wait limit of limit_us microseconds. The
 * kernel gives up by itself, records its status and returns; nothing faults and nothing is
 * killed. Returns the status word the kernel left (47 = the flag wait ran out, as it should),
 * or -1 when the launch could not be made. */
int vb200_selftest_wait_expiry(int limit_us);
/* How the frame kernel splits a [N,K] matrix product with M activation rows
 * over `n_cta` CTAs (host logic, usable without a GPU). out[0..6] = first row,
 * end row, column passes, columns per pass, rows per chunk, row blocks, chunks of
 * CTA `cta`; the return value is 0 when the shape is runnable, negative if not. */
int vb200_debug_gemv_plan(int N, int K, int M, int swiglu, int cta, int n_cta, int *out);

#ifdef __cplusplus
}
#endif
#endif
