"""The allocation-free linear entry point (vb200_linear_bf16_static) against the regular one.

Some users of this library cannot call cudaMalloc when they need a matrix product: a plugin
inside a host application that pre-allocates the whole device heap, an audio callback that
must not hit the allocator's implicit synchronisation. For them the library keeps the frame
kernel's bookkeeping memory in a fixed device array instead of allocated buffers. This test
calls that entry point through the C ABI twice in a row - the second call finds the array as
the first one left it - and compares with tts_cuda_linear_bf16 on the same device operands.

Collected last on purpose (file name), so a run that stops at the first failure has already
run everything else; it also passes alone in a fresh process.
"""
import numpy as np
import pytest

from gpu_common import rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K,N", [(1, 3072, 4096), (19, 512, 96), (6, 9216, 3072), (3, 100, 7)])
def test_static_scratch_linear_matches_regular_entry_point(pkg, M, K, N):
    eng = pkg.Engine(kv_cache_max=64)          # the regular entry point needs the context; idempotent
    L = eng.L
    x = pkg.synth_f32((M, K), 5, f"na.x{M}.{K}", 0.0, 0.1)
    W = pkg.synth_bf16((N, K), 5, f"na.W{N}.{K}")
    dx, dW = pkg.DeviceBuffer(x), pkg.DeviceBuffer(W)
    d_ref, d_new = pkg.DeviceBuffer(nbytes=M * N * 4), pkg.DeviceBuffer(nbytes=M * N * 4)
    L.tts_cuda_linear_bf16(d_ref.ptr, dx.ptr, None, M, K, N, dW.ptr)
    ref = d_ref.get((M, N))
    for call in range(2):
        L.tts_cuda_memset(d_new.ptr, 0xFF, M * N * 4)
        assert L.vb200_linear_bf16_static(d_new.ptr, dx.ptr, dW.ptr, M, K, N) == 0
        got = d_new.get((M, N))                # synchronises
        assert L.vb200_linear_bf16_static_status() == 0
        # the regular entry point runs M >= 2 on the tensor cores, this one on the streaming kernel
        assert rel_l2(got, ref) < 2e-5, (call, rel_l2(got, ref))
    for d in (dx, dW, d_ref, d_new):
        d.free()


def test_static_scratch_linear_rejects_too_many_rows(pkg):
    eng = pkg.Engine(kv_cache_max=64)
    d = pkg.DeviceBuffer(nbytes=64)
    assert eng.L.vb200_linear_bf16_static(d.ptr, d.ptr, d.ptr, 513, 512, 96) == -2
    assert eng.L.vb200_linear_bf16_static(d.ptr, d.ptr, d.ptr, 0, 512, 96) == 0
    d.free()


_FRESH_PROCESS = r"""
import ctypes as C, os, sys
import numpy as np
sys.path.insert(0, os.path.join(ROOT, "tests"))
from conftest import load_package
pkg = load_package()
L = pkg.lib()
assert L.tts_cuda_available() == 0                      # tts_cuda_init was never called in this process
rt = C.CDLL("libcudart.so.12")
def free_bytes():
    f, t = C.c_size_t(0), C.c_size_t(0)
    assert rt.cudaMemGetInfo(C.byref(f), C.byref(t)) == 0
    return f.value
M, K, N = 6, 3072, 1024
x = pkg.synth_f32((M, K), 5, "na2.x", 0.0, 0.1)
W = pkg.synth_bf16((N, K), 5, "na2.W")
dx, dW, dy = pkg.DeviceBuffer(x), pkg.DeviceBuffer(W), pkg.DeviceBuffer(nbytes=M * N * 4)
ref = x.astype(np.float64) @ (W.astype(np.uint32) << 16).view(np.float32).astype(np.float64).T
free = []
for call in range(3):
    L.tts_cuda_memset(dy.ptr, 0xFF, M * N * 4)
    assert L.vb200_linear_bf16_static(dy.ptr, dx.ptr, dW.ptr, M, K, N) == 0
    got = dy.get((M, N))
    assert L.vb200_linear_bf16_static_status() == 0
    err = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert err < 2e-5, err
    free.append(free_bytes())
assert L.tts_cuda_available() == 0
# the first call may create the CUDA context and load the module; from then on nothing is allocated
assert free[1] == free[2], free
print("OK", free)
"""


def test_static_scratch_linear_alone_in_a_fresh_process_allocates_nothing():
    """The two properties the entry point promises, in a process of its own: it works without
    tts_cuda_init (operands from tts_cuda_alloc), and the device's free memory does not change
    across the second and later calls."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", f"ROOT = {root!r}\n" + _FRESH_PROCESS], capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0 and "OK" in r.stdout, (r.stdout[-2000:], r.stderr[-2000:])
