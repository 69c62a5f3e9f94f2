/* vb_simple.cuh - host launchers of the stand-alone kernels in vb_simple.cu. */
#ifndef VB_SIMPLE_CUH
#define VB_SIMPLE_CUH

#include <cuda_runtime.h>
#include <stdint.h>

namespace vb {

void rms_norm(float *out, const float *x, const float *w, int rows, int dim, float eps, cudaStream_t st);
void silu_mul(float *gate, const float *up, int n, cudaStream_t st);
void add_inplace(float *a, const float *b, int n, cudaStream_t st);
void rope_table(float *cs, int start, int seq, int head_dim, float theta, cudaStream_t st);
void rope_apply(float *x, const float *cs, int seq, int heads, int head_dim, int ld, cudaStream_t st);
void embed_token(float *out, const uint16_t *table, int id, int dim, cudaStream_t st);
void embed_rows(float *out, const uint16_t *table, const int *ids, int n, int dim, cudaStream_t st);
int attention_rows(float *out, const float *Q, const float *K, const float *V, int seq_q, int seq_k,
                   int n_heads, int n_kv_heads, int head_dim, float scale, int q_offset, int causal,
                   int ldq, int ldk, int ldo, cudaStream_t st);
void linear_generic(float *y, const float *x, const uint16_t *W, const float *bias, int M, int K, int N,
                    cudaStream_t st);
void interleave_rows(uint16_t *dst, const uint16_t *a, const uint16_t *b, int rows, int cols, cudaStream_t st);

} // namespace vb

#endif
