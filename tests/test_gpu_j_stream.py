"""GPU parity of the frame path's decoder step, on both kernels that can run it - the GEMM launches
of the frame graph (default) and the persistent streaming kernel (option "decoder_kernel" = 1) -
against the CPU oracle and the golden fixtures of the reference CPU build: per-layer residual
stream (voxtral_tts_llm.c:245,263) within 2e-3 relative L2, the greedy semantic code identical, at
cache lengths that cover every key-split count of the decode attention and the lengths the
benchmark runs at. Plus the streaming kernel's failure path: a wait that runs out."""
import os

import numpy as np
import pytest

from cases import config1_inputs
from gpu_common import rel_l2

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
LAYER_TOL = 2e-3


def _fill_cache(engine, kvk, kvv):
    for l in range(26):
        engine.kv_write(l, 0, kvk[l], kvv[l])


@pytest.fixture(params=["graph", "stream"])
def path(engine, request):
    """Selects the kernel that runs the decoder step of vb200_frame / vb200_utterance_*."""
    want = 1 if request.param == "stream" else 0
    assert engine.L.vb200_set_option(b"decoder_kernel", want) == 0
    assert engine.L.vb200_frame_on_stream_kernel() == want
    assert engine.L.vb200_frame_on_tensor_cores() == 1      # the acoustic half is the GEMM graph either way
    yield request.param
    engine.L.vb200_set_option(b"decoder_kernel", 0)


@pytest.fixture
def stream(engine):
    assert engine.L.vb200_set_option(b"decoder_kernel", 1) == 0
    yield
    engine.L.vb200_set_option(b"decoder_kernel", 0)


def test_per_layer_taps_on_the_frame_path(pkg, engine, oracle, synth_model, path):
    """One decoder step at cache length 64 (the first benchmark configuration) through
    vb200_frame with the residual tap on: all 52 taps, the hidden row, the new cache row and the
    semantic code."""
    g = np.load(os.path.join(GOLD, "config1_decode.npz"))
    embed, kvk, kvv = config1_inputs(pkg)
    _fill_cache(engine, kvk, kvv)
    st = oracle.seed(3)
    noise, _ = oracle.randn(st, 36)
    engine.tap(True)
    try:
        assert engine.L.vb200_frame_on_stream_kernel() == (1 if path == "stream" else 0)
        codes, hidden = engine.frame(embed, noise, 64)
        tap = engine.tap_read()
    finally:
        engine.tap(False)
    k = np.zeros((26, 128, 1024), dtype=np.float32)
    v = np.zeros_like(k)
    k[:, :64] = kvk
    v[:, :64] = kvv
    h_ref, tap_ref = oracle.llm_forward(oracle.decoder(synth_model), k, v, 64, embed, tap=True)
    worst = max(rel_l2(tap[l, j], tap_ref[l, j]) for l in range(26) for j in range(2))
    assert worst < LAYER_TOL, worst
    assert rel_l2(hidden, h_ref) < LAYER_TOL
    assert rel_l2(hidden, g["hidden"]) < LAYER_TOL          # the reference CPU build's own output
    assert rel_l2(tap[-1], g["tap_last"]) < LAYER_TOL
    assert np.allclose(np.linalg.norm(tap.astype(np.float64), axis=-1), g["tap_norms"], rtol=LAYER_TOL)
    for l in (0, 13, 25):
        kr, vr = engine.kv_read(l, 64, 1)
        assert rel_l2(kr[0], g["k_row64"][l]) < LAYER_TOL and rel_l2(vr[0], g["v_row64"][l]) < LAYER_TOL
    ref_codes, _, _, _ = oracle.acoustic_forward(oracle.acoustic(synth_model), st, h_ref)
    assert codes[0] == ref_codes[0]
    assert np.array_equal(codes, ref_codes)
    # the tap must not change the result, and the kernel is bit-reproducible
    codes2, hidden2 = engine.frame(embed, noise, 64)
    assert np.array_equal(hidden, hidden2) and np.array_equal(codes, codes2)


@pytest.mark.parametrize("pos", [0, 1, 31, 32, 33, 200, 256, 281, 467, 511])
def test_frame_against_oracle_at_cache_lengths(pkg, engine, oracle, synth_model, path, pos):
    """Key-split counts 1 ... 16+ of the decode attention, the cache lengths the benchmark runs at
    (256 ... 467) and the last row of the cache."""
    kvk = pkg.synth_f32((26, max(pos, 1), 1024), 21, f"s.kvk{pos}")
    kvv = pkg.synth_f32((26, max(pos, 1), 1024), 22, f"s.kvv{pos}")
    embed = pkg.synth_f32(3072, 23, f"s.e{pos}")
    k = np.zeros((26, 512, 1024), dtype=np.float32)
    v = np.zeros_like(k)
    if pos:
        k[:, :pos] = kvk
        v[:, :pos] = kvv
        _fill_cache(engine, kvk, kvv)
    st = oracle.seed(100 + pos)
    noise, _ = oracle.randn(st, 36)
    codes, hidden = engine.frame(embed, noise, pos)
    h_ref = oracle.llm_forward(oracle.decoder(synth_model), k, v, pos, embed)
    assert rel_l2(hidden, h_ref) < LAYER_TOL, rel_l2(hidden, h_ref)
    ref_codes, _, _, _ = oracle.acoustic_forward(oracle.acoustic(synth_model), st, h_ref)
    assert codes[0] == ref_codes[0]
    assert int(np.sum(codes != ref_codes)) <= 1      # an FSQ rounding boundary may fall either way
    kr, vr = engine.kv_read(25, pos, 1)
    assert rel_l2(kr[0], k[25, pos]) < LAYER_TOL and rel_l2(vr[0], v[25, pos]) < LAYER_TOL


def test_streaming_step_timer_reads_every_weight_once(engine, stream):
    import ctypes as C
    ms, nbytes = C.c_float(0.0), C.c_double(0.0)
    assert engine.L.vb200_stream_step_ms(64, 3, C.byref(ms), C.byref(nbytes)) == 0
    assert ms.value > 0.0
    assert 6.0e9 < nbytes.value < 6.3e9


def test_a_wait_that_runs_out_is_reported_and_survivable(pkg, engine, oracle, synth_model, stream):
    """A flag nothing ever sets, a 2 ms limit: the kernel records status 47, returns by itself,
    and the next ordinary frame works."""
    assert engine.L.vb200_selftest_wait_expiry(2000) == 47
    embed, kvk, kvv = config1_inputs(pkg)
    _fill_cache(engine, kvk, kvv)
    noise, _ = oracle.randn(oracle.seed(3), 36)
    codes, hidden = engine.frame(embed, noise, 64)
    g = np.load(os.path.join(GOLD, "config1_decode.npz"))
    assert rel_l2(hidden, g["hidden"]) < LAYER_TOL


def test_streaming_device_loop_matches_the_graph_path(pkg, engine, oracle, synth_model):
    """32 frames of the device-resident loop on each decoder-step kernel: the semantic codes agree
    and at least 31 frames agree in all 37 codes up to the first frame where a latent on an FSQ
    rounding boundary falls the other way (summation order differs between the two kernels)."""
    first = synth_model.token_rows([24])[0]
    prompt = pkg.synth_f32((40, 3072), 78, "sl.prompt", 0.0, 0.5)
    noise, _ = oracle.randn(oracle.seed(9), 36 * 32)
    noise = noise.reshape(32, 36)
    engine.L.vb200_set_option(b"ignore_end", 1)
    out = {}
    try:
        for name, opt in (("graph", 0), ("stream", 1)):
            engine.L.vb200_set_option(b"decoder_kernel", opt)
            engine.prefill(prompt, 0)
            out[name], hit_end, _ = engine.utterance(first, 40, noise)
            assert out[name].shape == (32, 37) and not hit_end
    finally:
        engine.L.vb200_set_option(b"decoder_kernel", 0)
        engine.L.vb200_set_option(b"ignore_end", 0)
    agree = [bool(np.array_equal(out["graph"][f], out["stream"][f])) for f in range(32)]
    first_slip = agree.index(False) if False in agree else 32
    assert first_slip >= 8, agree
    if first_slip < 32:
        assert out["graph"][first_slip, 0] == out["stream"][first_slip, 0]
        assert int(np.sum(out["graph"][first_slip] != out["stream"][first_slip])) <= 1


def test_ignore_end_option_takes_effect_between_runs_of_equal_length(pkg, engine, oracle, synth_model):
    """The option is an argument of captured launches: flipping it must reach a device-resident
    run of the same length as the one captured before."""
    name = "acoustic_transformer.semantic_codebook_output.bias"
    first = synth_model.token_rows([24])[0]
    prompt = pkg.synth_f32((6, 3072), 77, "ie.prompt", 0.0, 0.5)
    noise, _ = oracle.randn(oracle.seed(8), 36 * 4)
    noise = noise.reshape(4, 36)
    try:
        bias = np.zeros(8320, dtype=np.float32)
        bias[1] = 1e6                                   # every frame's semantic code is END
        synth_model.t[name] = bias
        engine.upload(synth_model, decoder=False, acoustic=True)
        engine.L.vb200_set_option(b"ignore_end", 1)
        for _ in range(3):                              # direct, captured, replayed
            engine.prefill(prompt, 0)
            codes, hit_end, _ = engine.utterance(first, 6, noise)
            assert codes.shape[0] == 4 and not hit_end and np.all(codes[:, 0] == 1)
        engine.L.vb200_set_option(b"ignore_end", 0)
        engine.prefill(prompt, 0)
        codes, hit_end, _ = engine.utterance(first, 6, noise)
        assert hit_end and codes.shape[0] == 1
    finally:
        engine.L.vb200_set_option(b"ignore_end", 0)
        del synth_model.t[name]
        engine.upload(synth_model, decoder=False, acoustic=True)
