"""One utterance through the library end to end, the way the reference's tts_generate strings its
stages together (voxtral_tts.c:230-334): token ids + BF16 voice rows -> prompt built and prefilled on
the device (vb200_prefill_prompt) -> device-resident frame loop (vb200_utterance_*) -> codec decoder
(vb200_codec_decode) -> waveform. Checked stage by stage against the CPU side: the oracle's prefill /
decoder step / acoustic frame / re-embedding loop on the host-built prompt for the codes, the
reference's own codec for the waveform."""
import numpy as np
import pytest

from cases import CODEC_SEED
from gpu_common import rel_l2

pytestmark = pytest.mark.gpu
FRAMES = 4


def test_ids_to_waveform(pkg, engine, oracle, synth_model):
    import oracle_bind
    ref = oracle_bind.load_ref("blas") or oracle_bind.load_ref("noblas")
    if ref is None or not hasattr(ref.L, "refh_codec_decode"):
        pytest.skip("the reference's codec is not built (oracle/_ref)")
    eng = engine
    eng.upload(synth_model, decoder=True, acoustic=False, token_table=True)
    codec = pkg.SynthCodec(seed=CODEC_SEED)
    eng.codec_upload(codec)

    voice = pkg.synth_bf16((9, 3072), 71, "pipe.voice", 0.5)
    ids = np.array([2345, 77777, 1001, 50000], dtype=np.int32)
    n = eng.prefill_prompt(ids, voice, 0)
    assert n == 9 + 4 + 5
    first = synth_model.token_rows([24])[0]                    # embed(AUDIO), voxtral_tts.c:295
    seed = oracle.seed(2024)
    noise = oracle.randn(seed, 36 * FRAMES)[0].reshape(FRAMES, 36)
    codes, hit_end, _ = eng.utterance(first, n, noise)
    assert codes.shape == (FRAMES, 37) and not hit_end
    pcm, _ = eng.codec_decode(codes)
    assert pcm.shape == (FRAMES * 1920,)

    # the CPU side: the same stages in the reference's order
    rows = np.concatenate([synth_model.token_rows([1, 25]), (voice.astype(np.uint32) << 16).view(np.float32),
                           synth_model.token_rows([36]), synth_model.token_rows(list(ids)),
                           synth_model.token_rows([35, 25])], axis=0).astype(np.float32)
    dec, ac = oracle.decoder(synth_model), oracle.acoustic(synth_model)
    k = np.zeros((26, 32, 1024), dtype=np.float32)
    v = np.zeros_like(k)
    oracle.llm_prefill(dec, k, v, 0, rows)
    table = synth_model.audio_table()
    e, st, want = first, seed, []
    for f in range(FRAMES):
        h = oracle.llm_forward(dec, k, v, n + f, e)
        c, _, _, st = oracle.acoustic_forward(ac, st, h)
        want.append(c)
        e = oracle.audio_embed(table, c)
    want = np.stack(want)
    assert np.array_equal(codes[:, 0], want[:, 0])             # semantic codes: a greedy argmax
    # a latent on an FSQ rounding boundary may fall either way under another summation order; the
    # frames after such a slip see a different input row, so the comparison stops there
    for f in range(FRAMES):
        if not np.array_equal(codes[f], want[f]):
            assert int(np.sum(codes[f] != want[f])) <= 1, f
            break
    else:
        want_pcm = ref.codec_decode(codec.struct(), want)
        assert rel_l2(pcm, want_pcm) < 1e-3
    # whatever the codes: the GPU codec reproduces the reference codec on the codes the GPU produced
    assert rel_l2(pcm, ref.codec_decode(codec.struct(), codes)) < 1e-3
