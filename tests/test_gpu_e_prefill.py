"""GPU parity of the multi-token prefill (tts_cuda_llm_prefill): cache rows against the CPU
oracle on a short prompt, and size-independent properties at benchmark configuration 3's full size
(256 rows: 224 voice-embedding rows ~N(0,0.5) followed by 32 token rows)."""
import numpy as np
import pytest

from gpu_common import rel_l2

pytestmark = pytest.mark.gpu


def _prompt(pkg, synth_model, n_voice, n_text, seed=31):
    voice = pkg.synth_f32((n_voice, 3072), seed, "pf.voice", 0.0, 0.5)
    ids = 1000 + (pkg.synth_bf16(n_text, seed, "pf.ids").astype(np.int64) * 2 % (131072 - 1000))
    return np.concatenate([voice, synth_model.token_rows(ids)], axis=0)


def test_short_prompt_cache_rows(pkg, engine, oracle, synth_model):
    rows = _prompt(pkg, synth_model, 14, 5)
    M = rows.shape[0]
    engine.prefill(rows, 0)
    k = np.zeros((26, 32, 1024), dtype=np.float32)
    v = np.zeros_like(k)
    oracle.llm_prefill(oracle.decoder(synth_model), k, v, 0, rows)
    for l in range(26):
        kg, vg = engine.kv_read(l, 0, M)
        assert rel_l2(kg, k[l, :M]) < 2e-3 and rel_l2(vg, v[l, :M]) < 2e-3, l


def test_prefill_then_decode_matches_oracle(pkg, engine, oracle, synth_model):
    rows = _prompt(pkg, synth_model, 9, 3, seed=32)
    M = rows.shape[0]
    engine.prefill(rows, 0)
    nxt = pkg.synth_f32(3072, 33, "pf.next", 0.0, 0.02)
    h = engine.llm_forward(nxt, M)
    dec = oracle.decoder(synth_model)
    k = np.zeros((26, 32, 1024), dtype=np.float32)
    v = np.zeros_like(k)
    oracle.llm_prefill(dec, k, v, 0, rows)
    assert rel_l2(h, oracle.llm_forward(dec, k, v, M, nxt)) < 2e-3


def test_full_size_chunking_and_stepwise_agree(pkg, engine, synth_model):
    """256 rows at once == 100 + 156 rows in two calls == the last 3 rows decoded one by one."""
    rows = _prompt(pkg, synth_model, 224, 32, seed=34)
    engine.prefill(rows, 0)
    whole = [engine.kv_read(l, 0, 256) for l in (0, 12, 25)]
    engine.prefill(rows[:100], 0)
    engine.prefill(rows[100:], 100)
    for (k1, v1), l in zip(whole, (0, 12, 25)):
        k2, v2 = engine.kv_read(l, 0, 256)
        assert rel_l2(k2, k1) < 1e-4 and rel_l2(v2, v1) < 1e-4
    engine.prefill(rows[:253], 0)
    for i in range(253, 256):
        engine.llm_forward(rows[i], i)
    for (k1, v1), l in zip(whole, (0, 12, 25)):
        k2, v2 = engine.kv_read(l, 0, 256)
        assert rel_l2(k2, k1) < 1e-4 and rel_l2(v2, v1) < 1e-4


def test_prefill_out_of_range_is_refused(pkg, engine):
    rows = np.zeros((8, 3072), dtype=np.float32)
    engine.L.tts_cuda_llm_prefill(rows.ctypes.data, 8, 510)
    assert engine.L.vb200_last_status() == 0


def test_full_size_prompt_against_the_reference_build(pkg, engine, synth_model):
    """Benchmark configuration 3 at its size: 256 rows through tts_cuda_llm_prefill, cache rows of
    layers 0, 12 and 25 against the fixture written by the reference's own OpenBLAS build
    (tts_llm_prefill, voxtral_tts_llm.c:277-373)."""
    import os
    from cases import GOLDEN_LAYERS, GOLDEN_ROWS, config3_prompt
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "config3_prefill.npz"))
    rows = config3_prompt(pkg, synth_model)
    engine.prefill(rows, 0)
    for i, l in enumerate(GOLDEN_LAYERS):
        k, v = engine.kv_read(l, 0, 256)
        for j, r in enumerate(GOLDEN_ROWS):
            assert rel_l2(k[r], g["k_rows"][i, j]) < 2e-3 and rel_l2(v[r], g["v_rows"][i, j]) < 2e-3, (l, r)
        assert np.allclose(np.linalg.norm(k.astype(np.float64), axis=-1), g["k_norms"][i], rtol=2e-3), l
        assert np.allclose(np.linalg.norm(v.astype(np.float64), axis=-1), g["v_norms"][i], rtol=2e-3), l


def test_full_size_prompt_then_frames_against_the_reference_build(pkg, engine, oracle, synth_model):
    """Benchmark configuration 4, first 16 frames: the 256-row prompt prefilled on the GPU, then
    frames at cache rows 256.. . Each frame is checked against the reference build's fixture with
    the reference's own codes fed back (so one rounding-boundary slip cannot cascade): hidden row
    within 2e-3, semantic code identical, at least 15 of 16 frames identical in all 37 codes. The
    free-running device loop must reproduce the fixture up to its first such slip, if any."""
    import os
    from cases import CONFIG4_FRAMES, CONFIG4_SEED, config3_prompt, config4_first_embed
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "config4_slice.npz"))
    rows = config3_prompt(pkg, synth_model)
    n = CONFIG4_FRAMES
    noise, st_after = oracle.randn(oracle.seed(CONFIG4_SEED), 36 * n)   # no END among the fixture's frames
    noise = noise.reshape(n, 36)
    assert not np.any(g["codes"][:, 0] == 1) and st_after == int(g["rng_after"])
    engine.prefill(rows, 0)
    e = config4_first_embed(synth_model)
    table = synth_model.audio_table()
    same = 0
    for f in range(n):
        codes, hidden = engine.frame(e, noise[f], 256 + f)
        assert rel_l2(hidden, g["hidden"][f]) < 2e-3, f
        assert codes[0] == g["codes"][f, 0], f
        assert int(np.sum(codes != g["codes"][f])) <= 1, f
        same += int(np.array_equal(codes, g["codes"][f]))
        e = oracle.audio_embed(table, g["codes"][f])
    assert same >= n - 1, same
    # free-running on the device
    engine.prefill(rows, 0)
    loop, hit_end, _ = engine.utterance(config4_first_embed(synth_model), 256, noise)
    assert loop.shape == (n, 37) and not hit_end
    agree = [bool(np.array_equal(loop[f], g["codes"][f])) for f in range(n)]
    first_slip = agree.index(False) if False in agree else n
    assert first_slip >= min(n, 8), agree
    if first_slip < n:
        assert loop[first_slip, 0] == g["codes"][first_slip, 0]
        assert int(np.sum(loop[first_slip] != g["codes"][first_slip])) <= 1
