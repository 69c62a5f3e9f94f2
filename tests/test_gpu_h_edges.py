"""GPU edge cases of the frame-level entry points: the last cache row, a full cache inside a
device-resident run, refused positions and sizes, and that a refused call leaves the library
usable."""
import ctypes as C
import os

import numpy as np
import pytest

from gpu_common import rel_l2

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu


def _prompt(pkg, synth_model, rows, seed):
    voice = pkg.synth_f32((rows - 2, 3072), seed, "edge.voice", 0.0, 0.5)
    return np.concatenate([voice, synth_model.token_rows([1001 + seed, 2002 + seed])], axis=0)


def _noise(oracle, seed, frames):
    n, _ = oracle.randn(oracle.seed(seed), 36 * frames)
    return n.reshape(frames, 36)


def test_frame_on_the_last_cache_row(pkg, engine, oracle, synth_model):
    last = engine.kv_max - 1
    p = _prompt(pkg, synth_model, 6, 1)
    engine.prefill(p, last - 6)                     # rows last-6 .. last-1; earlier rows hold older data
    e = synth_model.token_rows([24])[0]
    noise = _noise(oracle, 11, 1)[0]
    codes, hidden = engine.frame(e, noise, last)
    h2 = engine.llm_forward(e, last)                # the streaming kernel on the same row
    assert rel_l2(hidden, h2) < 1e-4
    c2, _ = engine.acoustic_frame(h2, noise)
    assert codes[0] == c2[0]


def test_position_outside_cache_is_refused_and_recoverable(pkg, engine, oracle, synth_model):
    e = synth_model.token_rows([24])[0]
    noise = _noise(oracle, 12, 1)[0]
    codes = np.zeros(37, dtype=np.int32)
    for bad in (-1, engine.kv_max, engine.kv_max + 7):
        assert engine.L.vb200_frame(e.ctypes.data, noise.ctypes.data, bad, None, codes.ctypes.data) == -1
    p = _prompt(pkg, synth_model, 5, 2)
    engine.prefill(p, 0)
    c, h = engine.frame(e, noise, 5)                # still works
    assert c.shape == (37,) and np.isfinite(h).all()


def test_device_loop_stops_when_the_cache_is_full(pkg, engine, oracle, synth_model):
    start = engine.kv_max - 2
    p = _prompt(pkg, synth_model, 8, 3)
    engine.prefill(p, start - 8)
    e = synth_model.token_rows([24])[0]
    noise = _noise(oracle, 13, 5)
    codes, hit_end, _ = engine.utterance(e, start, noise)
    assert codes.shape[0] == 2 and not hit_end      # rows kv_max-2 and kv_max-1, then full
    # same two frames one by one
    c0, _ = engine.frame(e, noise[0], start)
    assert np.array_equal(c0, codes[0])


def test_single_frame_run(pkg, engine, oracle, synth_model):
    p = _prompt(pkg, synth_model, 7, 4)
    engine.prefill(p, 0)
    e = synth_model.token_rows([24])[0]
    noise = _noise(oracle, 14, 1)
    codes, hit_end, ms = engine.utterance(e, 7, noise)
    c0, _ = engine.frame(e, noise[0], 7)
    assert codes.shape == (1, 37) and np.array_equal(codes[0], c0) and ms > 0


def test_batch_refuses_bad_sizes(pkg, engine, synth_model):
    L = engine.L
    assert L.vb200_batch_open(2, 16, 4) == 0
    rows = pkg.synth_f32((17, 3072), 5, "edge.rows", 0.0, 0.5)
    assert L.vb200_batch_prefill(0, rows.ctypes.data, 17) == -1      # more rows than the slab holds
    assert L.vb200_batch_prefill(0, rows.ctypes.data, 0) == -1
    fe = np.zeros((2, 3072), dtype=np.float32)
    noise = np.zeros((2, 4, 36), dtype=np.float32)
    bad = np.array([3, 16], dtype=np.int32)                           # second start row outside the slab
    assert L.vb200_batch_begin(fe.ctypes.data, bad.ctypes.data, noise.ctypes.data) == -1
    L.vb200_batch_close()
    assert L.vb200_batch_hidden(fe.ctypes.data) == -1                 # nothing open


def test_long_device_loop_equals_frame_by_frame(pkg, engine, oracle, synth_model):
    """64 graph replays with state kept on the device == 64 single-frame calls with the host
    carrying position and re-embedding (same kernels, so the codes must be identical)."""
    frames = 64
    p = _prompt(pkg, synth_model, 40, 7)
    e0 = synth_model.token_rows([24])[0]
    noise = _noise(oracle, 21, frames)
    engine.L.vb200_set_option(b"ignore_end", 1)
    try:
        engine.prefill(p, 0)
        codes, hit_end, _ = engine.utterance(e0, 40, noise)
        assert codes.shape == (frames, 37) and not hit_end
        engine.prefill(p, 0)
        table = synth_model.audio_table()
        e = e0
        for f in range(frames):
            c, _ = engine.frame(e, noise[f], 40 + f)
            assert np.array_equal(c, codes[f]), f
            e = oracle.audio_embed(table, c)
    finally:
        engine.L.vb200_set_option(b"ignore_end", 0)


def test_context_can_be_torn_down_and_brought_up_again():
    """tts_cuda_free followed by tts_cuda_init in one process (a host that reloads its model): every
    cached copy and buffer of the first context is forgotten, and the second context decodes the same
    frame. Runs in a child process so that the suite's own context is not disturbed."""
    import subprocess
    import sys
    code = r"""
import os, sys
import numpy as np
sys.path.insert(0, os.path.join(%r, "tests"))
from conftest import load_package
pkg = load_package()
model = pkg.SynthModel(seed=77, dec_layers=2)
out = []
for round_ in range(2):
    eng = pkg.Engine(kv_cache_max=128)
    eng.upload(model, decoder=True, acoustic=True, audio_table=True)
    rows = pkg.synth_f32((70, 3072), 9, "reinit.rows", 0.0, 0.5)
    eng.prefill(rows, 0)
    noise = pkg.randn(123, 36)[0]
    codes, hidden = eng.frame(model.token_rows([24])[0], noise, rows.shape[0])
    out.append((codes.copy(), hidden.copy()))
    eng.close()
assert np.array_equal(out[0][0], out[1][0]) and np.array_equal(out[0][1], out[1][1])
print("reinit ok")
""" % ROOT
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "reinit ok" in r.stdout, (r.stdout[-1500:], r.stderr[-1500:])
