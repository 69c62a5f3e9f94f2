"""GPU parity of the single-op entry points (voxtral_tts_cuda.h:105-154) against the CPU
oracle, through the C ABI. Shapes, seeds-by-name and tolerances follow the reference's own
harness (test_kernels.c:122-430) and add ragged / odd shapes."""
import numpy as np
import pytest

from gpu_common import close_like_reference_harness, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng(engine):
    return engine


@pytest.fixture(scope="module")
def model(synth_model):
    return synth_model


def test_add_inplace_bit_exact(pkg, eng):
    a = pkg.synth_f32(3072, 1000, "a", 0.0, 0.1)
    b = pkg.synth_f32(3072, 1001, "b", 0.0, 0.1)
    da, db = pkg.DeviceBuffer(a), pkg.DeviceBuffer(b)
    eng.L.tts_cuda_add_inplace(da.ptr, db.ptr, 3072)
    assert np.array_equal(da.get(3072), a + b)          # rtol 0 / atol 0 in test_kernels.c:372
    da.free(); db.free()


def test_silu_mul(pkg, eng, oracle):
    g = pkg.synth_f32(9216, 800, "g", 0.0, 0.1)
    u = pkg.synth_f32(9216, 900, "u", 0.0, 0.1)
    dg, du = pkg.DeviceBuffer(g), pkg.DeviceBuffer(u)
    eng.L.tts_cuda_silu_mul(dg.ptr, du.ptr, 9216)
    assert close_like_reference_harness(oracle.silu_mul(g, u), dg.get(9216), 1e-5, 1e-7)
    dg.free(); du.free()


@pytest.mark.parametrize("rows,dim", [(1, 3072), (3, 3072), (5, 1000), (2, 8)])
def test_rms_norm(pkg, eng, oracle, rows, dim):
    x = pkg.synth_f32((rows, dim), 42, "x", 0.0, 0.1)
    w = np.abs(pkg.synth_f32(dim, 123, "w", 0.0, 0.1)) + 0.01
    dx, dw, do = pkg.DeviceBuffer(x), pkg.DeviceBuffer(w), pkg.DeviceBuffer(nbytes=x.nbytes)
    eng.L.tts_cuda_rms_norm(do.ptr, dx.ptr, dw.ptr, rows, dim, 1e-5)
    assert close_like_reference_harness(oracle.rms_norm(x, w), do.get((rows, dim)), 1e-4, 1e-6)
    for d in (dx, dw, do):
        d.free()


# (M, K, N): decode and acoustic shapes, the reference's test shape, ragged and tiny ones,
# K > 4096 (several column passes), K not a multiple of 8 (generic kernel), M > 8 (row blocks)
LINEAR_SHAPES = [
    (1, 3072, 4096), (1, 3072, 6144), (1, 4096, 3072), (1, 9216, 3072), (1, 3072, 8320), (1, 3072, 36),
    (6, 3072, 6144), (6, 4096, 3072), (6, 9216, 3072), (2, 3072, 36), (3, 3072, 1024), (7, 3072, 3072),
    (8, 512, 96), (5, 264, 10), (1, 8, 3), (4, 5000, 33), (1, 36, 3072), (3, 100, 7), (19, 512, 96),
    (1, 12288, 40),
    # the row counts of the other tensor-core tiles: 48 (eight utterances' acoustic rows, 64-row
    # tile), 100 and 256 (prefill, 256-row tile), and 257+ (two row blocks)
    (48, 3072, 6144), (48, 9216, 3072), (100, 3072, 1024), (256, 3072, 6144), (256, 4096, 3072),
    (256, 9216, 3072), (300, 3072, 256), (700, 1024, 3072), (1000, 3072, 500),
    # K > 4096 with many rows per CTA on the streaming engine (cross-pass accumulators)
    (8, 9224, 4000),
]


@pytest.mark.parametrize("M,K,N", LINEAR_SHAPES)
def test_linear_device_pointers(pkg, eng, oracle, M, K, N):
    x = pkg.synth_f32((M, K), 1100, f"x{M}.{K}", 0.0, 0.1)
    W = pkg.synth_bf16((N, K), 1200, f"W{N}.{K}")
    dx, dW, dy = pkg.DeviceBuffer(x), pkg.DeviceBuffer(W), pkg.DeviceBuffer(nbytes=M * N * 4)
    eng.L.tts_cuda_memset(dy.ptr, 0xFF, M * N * 4)
    eng.L.tts_cuda_linear_bf16(dy.ptr, dx.ptr, None, M, K, N, dW.ptr)
    y = dy.get((M, N))
    ref = oracle.linear(x, W)
    assert eng.L.vb200_last_status() == 0
    # M >= 2 runs on the tensor cores: fp32 rows as three BF16 terms, TMEM accumulation order
    assert rel_l2(y, ref) < (2e-6 if M == 1 else 2e-5), rel_l2(y, ref)
    assert close_like_reference_harness(ref, y, 1e-3, 1e-4)   # test_kernels.c:416
    for d in (dx, dW, dy):
        d.free()


def test_linear_host_pointers_and_weight_upload(pkg, eng, oracle):
    """x, y in host memory and W uploaded for the call (W_gpu == NULL), voxtral_tts_cuda.cu:374-431."""
    x = pkg.synth_f32((2, 512), 5, "hx", 0.0, 0.1)
    W = pkg.synth_bf16((96, 512), 5, "hW")
    y = np.zeros((2, 96), dtype=np.float32)
    from ctypes import c_void_p
    eng.L.tts_cuda_linear_bf16(y.ctypes.data_as(c_void_p), x.ctypes.data_as(c_void_p),
                               W.ctypes.data_as(c_void_p), 2, 512, 96, None)
    assert rel_l2(y, oracle.linear(x, W)) < 2e-5


def test_linear_empty(pkg, eng):
    d = pkg.DeviceBuffer(nbytes=64)
    eng.L.tts_cuda_linear_bf16(d.ptr, d.ptr, None, 0, 512, 96, d.ptr)   # no rows: nothing happens
    eng.L.tts_cuda_sync()
    assert eng.L.vb200_last_status() == 0
    d.free()


@pytest.mark.parametrize("seq_k", [1, 3, 10, 50, 100, 225, 468])
def test_causal_attention_decode(pkg, eng, oracle, seq_k):
    scale = float(1.0 / np.sqrt(128.0))
    q = pkg.synth_f32(4096, 100 + seq_k, "q", 0.0, 0.1)
    k = pkg.synth_f32((seq_k, 1024), 200 + seq_k, "k", 0.0, 0.1)
    v = pkg.synth_f32((seq_k, 1024), 300 + seq_k, "v", 0.0, 0.1)
    dq, dk, dv, do = pkg.DeviceBuffer(q), pkg.DeviceBuffer(k), pkg.DeviceBuffer(v), pkg.DeviceBuffer(nbytes=4096 * 4)
    eng.L.tts_cuda_memset(do.ptr, 0, 4096 * 4)
    eng.L.tts_cuda_causal_attention_decode(do.ptr, dq.ptr, dk.ptr, dv.ptr, seq_k, 32, 8, 128, scale, 1024)
    ref = oracle.attention_causal(q, k, v, 32, 8, 128, scale, seq_k - 1)[0]
    assert close_like_reference_harness(ref, do.get(4096), 1e-3, 1e-5)
    for d in (dq, dk, dv, do):
        d.free()


def test_bidirectional_attention(pkg, eng, oracle):
    scale = float(1.0 / np.sqrt(128.0))
    q = pkg.synth_f32((3, 4096), 500, "q", 0.0, 0.1)
    k = pkg.synth_f32((3, 1024), 600, "k", 0.0, 0.1)
    v = pkg.synth_f32((3, 1024), 700, "v", 0.0, 0.1)
    dq, dk, dv, do = pkg.DeviceBuffer(q), pkg.DeviceBuffer(k), pkg.DeviceBuffer(v), pkg.DeviceBuffer(nbytes=q.nbytes)
    eng.L.tts_cuda_bidirectional_attention(do.ptr, dq.ptr, dk.ptr, dv.ptr, 3, 32, 8, 128, scale)
    ref = oracle.attention_full(q, k, v, 32, 8, 128, scale)
    assert close_like_reference_harness(ref, do.get((3, 4096)), 1e-3, 1e-5)
    for d in (dq, dk, dv, do):
        d.free()


@pytest.mark.parametrize("seq,start", [(7, 0), (5, 9), (1, 0)])
def test_causal_attention_prefill(pkg, eng, oracle, seq, start):
    scale = float(1.0 / np.sqrt(128.0))
    q = pkg.synth_f32((seq, 4096), 1, "pq", 0.0, 0.1)
    k = pkg.synth_f32((start + seq, 1024), 2, "pk", 0.0, 0.1)
    v = pkg.synth_f32((start + seq, 1024), 3, "pv", 0.0, 0.1)
    dq, dk, dv, do = pkg.DeviceBuffer(q), pkg.DeviceBuffer(k), pkg.DeviceBuffer(v), pkg.DeviceBuffer(nbytes=q.nbytes)
    eng.L.tts_cuda_causal_attention_prefill(do.ptr, dq.ptr, dk.ptr, dv.ptr, seq, start, 32, 8, 128, scale)
    ref = oracle.attention_causal(q, k, v, 32, 8, 128, scale, start)
    assert close_like_reference_harness(ref, do.get((seq, 4096)), 1e-3, 1e-5)
    for d in (dq, dk, dv, do):
        d.free()


def test_rope_table_and_apply(pkg, eng, oracle):
    seq, start = 4, 464
    cs_ref = oracle.rope_table(list(range(start, start + seq)))
    dcs = pkg.DeviceBuffer(nbytes=cs_ref.nbytes)
    eng.L.tts_cuda_compute_rope_freqs(dcs.ptr, start, seq, 128, 1e6)
    cs = dcs.get(cs_ref.shape)
    assert np.abs(cs - cs_ref).max() < 2e-6       # libm vs CUDA cos/sin at angles up to ~470 rad
    x = pkg.synth_f32((seq, 1024), 9, "rx")
    dx = pkg.DeviceBuffer(x)
    eng.L.tts_cuda_apply_rope(dx.ptr, dcs.ptr, seq, 8, 128)
    assert rel_l2(dx.get((seq, 1024)), oracle.rope_apply(x, cs_ref, 8)) < 2e-6
    dcs.free(); dx.free()


def test_embed_token(pkg, eng):
    table = pkg.synth_bf16((50, 3072), 4, "tbl")
    dt, do = pkg.DeviceBuffer(table), pkg.DeviceBuffer(nbytes=3072 * 4)
    eng.L.tts_cuda_embed_token(do.ptr, dt.ptr, 37, 3072)
    assert np.array_equal(do.get(3072), (table[37].astype(np.uint32) << 16).view(np.float32))
    dt.free(); do.free()
