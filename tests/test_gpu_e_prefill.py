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
