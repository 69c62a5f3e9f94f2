"""GPU parity of the whole frame in one launch (decoder step + acoustic frame) and of chained
frames with the re-embedding on the device, against the golden fixture of the reference CPU
build (three frames: decode -> acoustic -> re-embed, voxtral_tts.c:301-318)."""
import os

import numpy as np
import pytest

from cases import frames_inputs
from gpu_common import rel_l2

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _start(pkg, engine):
    first, kvk, kvv, seed, n = frames_inputs(pkg)
    for l in range(26):
        engine.kv_write(l, 0, kvk[l], kvv[l])
    return first, kvk.shape[1], seed, n


def test_three_frames_host_reembedding(pkg, engine, oracle, synth_model):
    g = np.load(os.path.join(GOLD, "frames3.npz"))
    e, pos, seed, n = _start(pkg, engine)
    st = oracle.seed(seed)
    for f in range(n):
        noise, st_next = oracle.randn(st, 36)
        codes, hidden = engine.frame(e, noise, pos + f)
        assert rel_l2(hidden, g["hidden"][f]) < 2e-3
        assert np.array_equal(codes, g["codes"][f])
        if codes[0] != 1:
            st = st_next                       # END frames draw no noise (voxtral_tts_acoustic.c:312-320)
        e = oracle.audio_embed(synth_model.audio_table(), codes)
    assert st == int(g["rng_after"])


def test_three_frames_device_reembedding(pkg, engine, oracle):
    g = np.load(os.path.join(GOLD, "frames3.npz"))
    e, pos, seed, n = _start(pkg, engine)
    st = oracle.seed(seed)
    for f in range(n):
        noise, st = oracle.randn(st, 36)
        codes, hidden = engine.frame(e if f == 0 else None, noise, pos + f)
        assert rel_l2(hidden, g["hidden"][f]) < 2e-3
        assert np.array_equal(codes, g["codes"][f])


def test_frame_equals_separate_calls(pkg, engine, oracle):
    e, pos, seed, _ = _start(pkg, engine)
    noise, _ = oracle.randn(oracle.seed(seed), 36)
    codes, hidden = engine.frame(e, noise, pos)
    h2 = engine.llm_forward(e, pos)
    c2, _ = engine.acoustic_frame(h2, noise)
    # the frame runs the decoder step on the tensor-core GEMM, the separate call on the streaming
    # kernel: same arithmetic, different summation order
    assert rel_l2(hidden, h2) < 1e-4 and np.array_equal(codes, c2)


def test_device_resident_loop_matches_golden(pkg, engine, oracle):
    """The frame loop kept on the device (noise uploaded up front, re-embedding, position and
    frame counter in device memory) produces the reference's codes for the three golden frames."""
    g = np.load(os.path.join(GOLD, "frames3.npz"))
    e, pos, seed, n = _start(pkg, engine)
    noise, _ = oracle.randn(oracle.seed(seed), 36 * n)
    codes, hit_end, ms = engine.utterance(e, pos, noise.reshape(n, 36))
    assert not hit_end and codes.shape == (n, 37)
    assert np.array_equal(codes, g["codes"])
    assert ms > 0.0
    # the single-call entry points still work afterwards
    c1, _ = engine.frame(e, noise[:36], pos)
    assert np.array_equal(c1, g["codes"][0])


def test_device_resident_loop_stops_at_end(pkg, engine, oracle, synth_model):
    name = "acoustic_transformer.semantic_codebook_output.bias"
    e, pos, seed, n = _start(pkg, engine)
    noise, _ = oracle.randn(oracle.seed(seed), 36 * 4)
    try:
        bias = np.zeros(8320, dtype=np.float32)
        bias[1] = 1e6
        synth_model.t[name] = bias
        engine.upload(synth_model, decoder=False, acoustic=True)
        codes, hit_end, _ = engine.utterance(e, pos, noise.reshape(4, 36))
        assert hit_end and codes.shape[0] == 1 and codes[0, 0] == 1 and np.all(codes[0, 1:] == 2)
    finally:
        del synth_model.t[name]
        engine.upload(synth_model, decoder=False, acoustic=True)
