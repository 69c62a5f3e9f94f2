"""GPU parity of the persistent tensor-core kernel's GEMM op (vb200_ptc_linear) against the CPU
oracle's tts_linear_nobias_bf16 restatement: split-K with the in-kernel last-CTA sum, and the
SwiGLU epilogue on interleaved gate/up rows."""
import ctypes as C

import numpy as np
import pytest

from gpu_common import rel_l2

pytestmark = pytest.mark.gpu


def _run(pkg, engine, M, K, N, swiglu, seed):
    x = pkg.synth_f32((M, K), seed, "ptc.x")
    W = pkg.synth_bf16((N, K), seed + 1, "ptc.W")
    dx, dW = pkg.DeviceBuffer(x), pkg.DeviceBuffer(W)
    n_out = N // 2 if swiglu else N
    dy = pkg.DeviceBuffer(nbytes=M * n_out * 4)
    ms = C.c_float(0.0)
    rc = engine.L.vb200_ptc_linear(dy.ptr, dx.ptr, dW.ptr, M, K, N, 1 if swiglu else 0, 2, C.byref(ms))
    assert rc == 0, rc
    y = dy.get((M, n_out))
    Wf = (W.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    ref = x.astype(np.float64) @ Wf.T
    if swiglu:
        g, u = ref[:, 0::2], ref[:, 1::2]
        ref = g / (1.0 + np.exp(-g)) * u
    return y, ref


@pytest.mark.parametrize("M,K,N", [(1, 3072, 6144), (1, 4096, 3072), (1, 9216, 3072), (6, 3072, 6144),
                                   (6, 9216, 3072), (3, 3072, 8320), (10, 3072, 3072), (1, 64, 128), (2, 192, 200)])
def test_split_k_gemm_matches_fp64(pkg, engine, M, K, N):
    y, ref = _run(pkg, engine, M, K, N, False, 300 + M)
    assert rel_l2(y, ref) < 2e-6, rel_l2(y, ref)


@pytest.mark.parametrize("M", [1, 6])
def test_swiglu_epilogue(pkg, engine, M):
    y, ref = _run(pkg, engine, M, 3072, 18432, True, 320 + M)
    assert rel_l2(y, ref) < 2e-5, rel_l2(y, ref)
