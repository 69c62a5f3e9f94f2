"""GPU prompt construction (vb200_prefill_prompt): the prompt the reference's orchestrator
assembles on the host (voxtral_tts.c:230-272: [BOS] [BEGIN_AUDIO] voice rows [/INST] text [INST]
[BEGIN_AUDIO], token rows through tts_embed_token_bf16, voice rows BF16 -> fp32 as tts_voice_embed
does, voxtral_tts_voice.c:228-248) built on the device from ids and BF16 rows. The cache rows must be
exactly those of tts_cuda_llm_prefill on the host-built fp32 prompt, and match the CPU oracle."""
import numpy as np
import pytest

from gpu_common import rel_l2

pytestmark = pytest.mark.gpu


def _host_prompt(synth_model, text_ids, voice_bf16):
    voice = (voice_bf16.astype(np.uint32) << 16).view(np.float32)
    rows = [synth_model.token_rows([1, 25]), voice, synth_model.token_rows([36]),
            synth_model.token_rows(list(text_ids)) if len(text_ids) else np.zeros((0, 3072), np.float32),
            synth_model.token_rows([35, 25])]
    return np.concatenate(rows, axis=0).astype(np.float32)


@pytest.fixture(scope="module")
def engine_with_tokens(engine, synth_model):
    engine.upload(synth_model, decoder=True, acoustic=False, token_table=True)
    return engine


@pytest.mark.parametrize("n_voice,n_text", [(7, 4), (0, 3), (5, 0), (224, 27)])
def test_device_prompt_equals_host_prompt(pkg, engine_with_tokens, synth_model, n_voice, n_text):
    eng = engine_with_tokens
    voice = pkg.synth_bf16((n_voice, 3072), 61, f"pr.voice{n_voice}", 0.5)
    ids = (1000 + (pkg.synth_bf16(max(n_text, 1), 62, f"pr.ids{n_text}").astype(np.int64) * 2 % (131072 - 1000)))[:n_text]
    rows = _host_prompt(synth_model, ids, voice)
    n = eng.prefill_prompt(ids, voice, 0)
    assert n == rows.shape[0] == n_voice + n_text + 5
    got = [eng.kv_read(l, 0, n) for l in (0, 13, 25)]
    eng.prefill(rows, 0)
    for (k1, v1), l in zip(got, (0, 13, 25)):
        k2, v2 = eng.kv_read(l, 0, n)
        assert np.array_equal(k1, k2) and np.array_equal(v1, v2), l     # same rows in, same kernels: same bits


def test_device_prompt_against_the_oracle(pkg, engine_with_tokens, oracle, synth_model):
    eng = engine_with_tokens
    voice = pkg.synth_bf16((6, 3072), 63, "pr.voice.o", 0.5)
    ids = np.array([4321, 99999, 1000], dtype=np.int32)
    n = eng.prefill_prompt(ids, voice, 0)
    rows = _host_prompt(synth_model, ids, voice)
    k = np.zeros((26, 32, 1024), dtype=np.float32)
    v = np.zeros_like(k)
    oracle.llm_prefill(oracle.decoder(synth_model), k, v, 0, rows)
    for l in range(26):
        kg, vg = eng.kv_read(l, 0, n)
        assert rel_l2(kg, k[l, :n]) < 2e-3 and rel_l2(vg, v[l, :n]) < 2e-3, l


def test_device_prompt_refuses_bad_arguments(pkg, engine_with_tokens):
    L = engine_with_tokens.L
    voice = pkg.synth_bf16((4, 3072), 64, "pr.voice.b", 0.5)
    bad = np.array([131072], dtype=np.int32)
    assert L.vb200_prefill_prompt(bad.ctypes.data, 1, voice.ctypes.data, 4, 0) == -1          # id outside the table
    ok = np.array([5], dtype=np.int32)
    assert L.vb200_prefill_prompt(ok.ctypes.data, 1, voice.ctypes.data, 4, 510) == -1         # does not fit the cache
    assert L.vb200_prefill_prompt(None, 2, voice.ctypes.data, 4, 0) == -1
    assert L.vb200_last_status() == 0
