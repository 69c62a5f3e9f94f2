/*
 * vb_prefill.cu - multi-token prefill of the decoder on the GPU
 * (tts_llm_prefill, voxtral_tts_llm.c:277-373): all prompt rows go through the
 * 26 layers, K and V of every row land in the cache, hidden states are dropped.
 *
 * The linears run as batches of row blocks through the streaming engine (fp32
 * activations, exact BF16 weights, fp32 accumulation - the arithmetic of the
 * reference); RoPE, the cache write and the causal attention use the
 * stand-alone kernels.
 */
#include "vb_model.cuh"
#include "vb_simple.cuh"

#include <math.h>
#include <stdio.h>
#include <string.h>

namespace vb {

static const int D = VB200_DIM, QD = VB200_Q_DIM, KVD = VB200_KV_DIM, HID = VB200_HIDDEN;
static const int QKV = QD + 2 * KVD;

/* Runs `op` once per block of up to 8 rows; blocks are independent, so a launch
 * carries up to 64 of them without grid barriers in between. */
static int run_row_blocks(VbOp proto, int M, int x_ld, int y_ld, bool res_is_y) {
    std::vector<VbOp> ops;
    const float *x0 = proto.x;
    float *y0 = proto.y;
    for (int r = 0; r < M; r += kMaxM) {
        VbOp o = proto;
        o.M = (M - r < kMaxM) ? M - r : kMaxM;
        o.x = x0 + (size_t)r * x_ld;
        o.y = y0 + (size_t)r * y_ld;
        if (res_is_y) o.res = o.y;
        o.flags |= VB_F_NOSYNC;
        ops.push_back(o);
        if (ops.size() == 64) {
            if (run_ops(ops)) return -1;
            ops.clear();
        }
    }
    if (!ops.empty() && run_ops(ops)) return -1;
    return 0;
}

int prefill(const float *embeds, int seq_len, int start_pos) {
    Model &m = model();
    if (!m.inited || !m.llm_ready) return -1;
    if (seq_len <= 0) return 0;
    if (start_pos < 0 || start_pos + seq_len > m.kv_max) {
        fprintf(stderr, "voxtral_b200: prefill of %d rows at %d exceeds the %d-row cache\n", seq_len, start_pos,
                m.kv_max);
        return -1;
    }
    const int M = seq_len;
    float *x = nullptr, *qkv = nullptr, *attn = nullptr, *h = nullptr, *cs = nullptr;
    int rc = 0;
    if (cudaMalloc(&x, (size_t)M * D * 4) != cudaSuccess) rc = -1;
    if (!rc && cudaMalloc(&qkv, (size_t)M * QKV * 4) != cudaSuccess) rc = -1;
    if (!rc && cudaMalloc(&attn, (size_t)M * QD * 4) != cudaSuccess) rc = -1;
    if (!rc && cudaMalloc(&h, (size_t)M * HID * 4) != cudaSuccess) rc = -1;
    if (!rc && cudaMalloc(&cs, (size_t)M * VB200_HEAD_DIM * 4) != cudaSuccess) rc = -1;
    const float scale = 1.0f / sqrtf((float)VB200_HEAD_DIM);
    if (!rc && cudaMemcpyAsync(x, embeds, (size_t)M * D * 4, cudaMemcpyDefault, m.st) != cudaSuccess) rc = -1;
    if (!rc) rope_table(cs, start_pos, M, VB200_HEAD_DIM, VB200_ROPE_THETA, m.st);

    for (int l = 0; l < VB200_DEC_LAYERS && !rc; l++) {
        const LayerDev &L = m.dec[l];
        float *ck = m.kv_k + ((size_t)l * m.kv_max + start_pos) * KVD;
        float *cv = m.kv_v + ((size_t)l * m.kv_max + start_pos) * KVD;

        VbOp o;
        memset(&o, 0, sizeof(o));
        o.type = VB_OP_GEMV; o.N = QKV; o.K = D; o.W = L.wqkv; o.x = x; o.ldx = D; o.y = qkv; o.ldy = QKV;
        o.epi = VB_EPI_STORE; o.norm_w = L.attn_norm; o.eps = VB200_NORM_EPS;
        rc = run_row_blocks(o, M, D, QKV, false);
        if (rc) break;

        rope_apply(qkv, cs, M, VB200_HEADS, VB200_HEAD_DIM, QKV, m.st);
        rope_apply(qkv + QD, cs, M, VB200_KV_HEADS, VB200_HEAD_DIM, QKV, m.st);
        if (cudaMemcpy2DAsync(ck, (size_t)KVD * 4, qkv + QD, (size_t)QKV * 4, (size_t)KVD * 4, M,
                              cudaMemcpyDeviceToDevice, m.st) != cudaSuccess ||
            cudaMemcpy2DAsync(cv, (size_t)KVD * 4, qkv + QD + KVD, (size_t)QKV * 4, (size_t)KVD * 4, M,
                              cudaMemcpyDeviceToDevice, m.st) != cudaSuccess) {
            rc = -1;
            break;
        }
        const float *k0 = m.kv_k + (size_t)l * m.kv_max * KVD;
        const float *v0 = m.kv_v + (size_t)l * m.kv_max * KVD;
        if (attention_rows(attn, qkv, k0, v0, M, start_pos + M, VB200_HEADS, VB200_KV_HEADS, VB200_HEAD_DIM,
                           scale, start_pos, 1, QKV, KVD, QD, m.st)) {
            rc = -1;
            break;
        }

        memset(&o, 0, sizeof(o));
        o.type = VB_OP_GEMV; o.N = D; o.K = QD; o.W = L.wo; o.x = attn; o.ldx = QD; o.y = x; o.ldy = D;
        o.epi = VB_EPI_ADD; o.eps = VB200_NORM_EPS;
        rc = run_row_blocks(o, M, QD, D, true);
        if (rc) break;

        memset(&o, 0, sizeof(o));
        o.type = VB_OP_GEMV; o.N = 2 * HID; o.K = D; o.W = L.w13; o.x = x; o.ldx = D; o.y = h; o.ldy = HID;
        o.epi = VB_EPI_SWIGLU; o.norm_w = L.ffn_norm; o.eps = VB200_NORM_EPS;
        rc = run_row_blocks(o, M, D, HID, false);
        if (rc) break;

        memset(&o, 0, sizeof(o));
        o.type = VB_OP_GEMV; o.N = D; o.K = HID; o.W = L.w2; o.x = h; o.ldx = HID; o.y = x; o.ldy = D;
        o.epi = VB_EPI_ADD; o.eps = VB200_NORM_EPS;
        rc = run_row_blocks(o, M, HID, D, true);
    }
    if (cudaStreamSynchronize(m.st) != cudaSuccess) rc = -1;
    cudaFree(x); cudaFree(qkv); cudaFree(attn); cudaFree(h); cudaFree(cs);
    if (!rc) {
        int status = 0;
        cudaMemcpy(&status, &m.d_out->status, sizeof(int), cudaMemcpyDeviceToHost);
        m.last_status = status;
        if (status) rc = -1;
    }
    return rc;
}

} // namespace vb
