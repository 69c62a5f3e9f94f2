"""Helpers shared by the GPU parity tests."""
import numpy as np


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def close_like_reference_harness(ref, test, rtol, atol):
    """The acceptance rule of the reference's test_kernels.c:79-116: no element may
    exceed both tolerances, and max-rel <= rtol or max-abs <= atol overall."""
    ref = np.asarray(ref, dtype=np.float32).ravel()
    test = np.asarray(test, dtype=np.float32).ravel()
    diff = np.abs(ref - test)
    rel = diff / np.maximum(np.abs(ref), 1e-8)
    bad = int(np.sum((rel > rtol) & (diff > atol)))
    return bad == 0 and (rel.max(initial=0.0) <= rtol or diff.max(initial=0.0) <= atol)
