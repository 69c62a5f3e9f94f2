#!/usr/bin/env python3
"""Build libvoxtral_b200.so in-tree with nvcc for sm_100a.

    python voxtral-tts.c_b200/build.py [--force] [--verbose-ptxas]

The shared library lands next to this file (lib/libvoxtral_b200.so). It is built
for sm_100a only (-gencode arch=compute_100a,code=sm_100a); nvcc cross-compiles
without a GPU.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "libvoxtral_b200.so")
OBJDIR = os.path.join(LIBDIR, "obj")

CU_SOURCES = ["vb_engine.cu", "vb_simple.cu", "vb_model.cu", "vb_prefill.cu", "vb_abi.cu", "vb_noalloc.cu",
              "vb_tc.cu", "vb_acoustic_tc.cu", "vb_batch.cu", "vb_stream.cu", "vb_codec.cu"]
CPP_SOURCES = ["vb_synth.cpp"]
NVCC = os.environ.get("NVCC", "nvcc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall"]


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    inc = os.path.join(os.path.dirname(HERE), "include")
    hs += [os.path.join(inc, f) for f in os.listdir(inc) if f.endswith(".h")]
    return hs


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd):
    print("+", " ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def build(force=False, verbose_ptxas=False):
    os.makedirs(OBJDIR, exist_ok=True)
    headers = _headers()
    objs = []
    for src in CU_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJDIR, src + ".o")
        if force or _stale(o, [s] + headers):
            extra = ["-Xptxas", "-v"] if verbose_ptxas else []
            _run([NVCC, *NVCC_FLAGS, *extra, "-c", s, "-o", o])
        objs.append(o)
    for src in CPP_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJDIR, src + ".o")
        if force or _stale(o, [s] + headers):
            _run(["g++", "-O3", "-std=c++17", "-fPIC", "-fopenmp", "-ffp-contract=off", "-Wall", "-c", s, "-o", o])
        objs.append(o)
    # the synthetic-tensor generator also as a small library of its own: code that must not map
    # the CUDA library (the CPU reference arm of the benchmark) loads only this one
    synth_lib = os.path.join(LIBDIR, "libvb_synth.so")
    synth_obj = os.path.join(OBJDIR, "vb_synth.cpp.o")
    if force or _stale(synth_lib, [synth_obj]):
        tmp = synth_lib + ".tmp"
        _run(["g++", "-shared", "-o", tmp, synth_obj, "-fopenmp"])
        os.replace(tmp, synth_lib)
    if force or _stale(LIB, objs):
        # link under a temporary name and rename: a reader never sees a half-written library
        tmp = LIB + ".tmp"
        _run([NVCC, "-shared", "-o", tmp, *objs, "-Xcompiler", "-fopenmp", "-lcudart", "-lgomp"])
        os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose_ptxas="--verbose-ptxas" in sys.argv)
    print(LIB)
