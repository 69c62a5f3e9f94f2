"""The drop-in boundary, executed: the reference's own GPU test harness (test_kernels.c, compiled
unchanged from the reference checkout and linked against libvoxtral_b200.so by
oracle/build_oracle.py) must pass all of its CPU-vs-GPU comparisons (test_kernels.c:436-479:
add, silu*mul, rms_norm, gemm, six causal-attention lengths, bidirectional attention)."""
import os
import re
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_kernel_harness_passes_against_this_library():
    exe = os.path.join(ROOT, "oracle", "_ref", "test_kernels_b200")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/test_kernels_b200 not built (needs the reference checkout at build time)")
    env = dict(os.environ)
    libdir = os.path.join(ROOT, "voxtral-tts.c_b200", "lib")
    env["LD_LIBRARY_PATH"] = libdir + os.pathsep + env.get("LD_LIBRARY_PATH", "")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600, env=env)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-3000:]
    m = re.search(r"(\d+)\s*/\s*(\d+)\s+(?:tests\s+)?passed", out)
    assert m, out[-3000:]
    assert m.group(1) == m.group(2) and int(m.group(2)) >= 11, out[-3000:]
    assert "FAIL" not in out, out[-3000:]
