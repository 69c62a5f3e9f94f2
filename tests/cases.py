"""Seeded inputs of the parity cases, shared by the golden generator and the tests.

They follow the benchmark configurations: config 1 = one decoder step with a cache
pre-filled with 64 positions of N(0,1); config 2 = one acoustic frame on a
N(0,1) hidden state; config 3 = a 256-row prompt (224 voice-embedding rows ~N(0,0.5), then 32
token rows with ids in [1000, 131072)); config 4 = that prompt followed by generated frames."""
import numpy as np

MODEL_SEED = 1234
INPUT_SEED = 7


def config1_inputs(pkg):
    embed = pkg.synth_f32(3072, INPUT_SEED, "cfg1.embed")
    kvk = pkg.synth_f32((26, 64, 1024), INPUT_SEED, "cfg1.kv_k")
    kvv = pkg.synth_f32((26, 64, 1024), INPUT_SEED, "cfg1.kv_v")
    return embed, kvk, kvv


def config2_inputs(pkg):
    return pkg.synth_f32(3072, INPUT_SEED, "cfg2.hidden"), 42


def frames_inputs(pkg):
    first = pkg.synth_f32(3072, INPUT_SEED, "frames.embed", 0.0, 0.02)
    kvk = pkg.synth_f32((26, 5, 1024), INPUT_SEED, "frames.kv_k")
    kvv = pkg.synth_f32((26, 5, 1024), INPUT_SEED, "frames.kv_v")
    return first, kvk, kvv, 99, 3


def primitive_inputs(pkg):
    s = INPUT_SEED
    return {
        "x1": pkg.synth_f32(512, s, "prim.x1"),
        "x3": pkg.synth_f32((3, 512), s, "prim.x3"),
        "W": pkg.synth_bf16((96, 512), s, "prim.W"),
        "bias": pkg.synth_f32(96, s, "prim.bias"),
        "gain": pkg.synth_f32(512, s, "prim.gain", 1.0, 0.1),
        "q": pkg.synth_f32(32 * 128, s, "prim.q", 0.0, 0.1),
        "q3": pkg.synth_f32((3, 32 * 128), s, "prim.q3", 0.0, 0.1),
        "k": pkg.synth_f32((225, 8 * 128), s, "prim.k", 0.0, 0.1),
        "v": pkg.synth_f32((225, 8 * 128), s, "prim.v", 0.0, 0.1),
        "rope_x": pkg.synth_f32((4, 8 * 128), s, "prim.rope_x"),
        "gate": pkg.synth_f32(1024, s, "prim.gate"),
        "up": pkg.synth_f32(1024, s, "prim.up"),
    }


CONFIG4_SEED = 4242
CONFIG4_FRAMES = 16
GOLDEN_LAYERS = (0, 12, 25)
GOLDEN_ROWS = (0, 100, 255)


def config3_prompt(pkg, model):
    voice = pkg.synth_f32((224, 3072), INPUT_SEED, "cfg3.voice", 0.0, 0.5)
    ids = 1000 + (pkg.synth_bf16(32, INPUT_SEED, "cfg3.ids").astype(np.int64) * 2 % (131072 - 1000))
    return np.concatenate([voice, model.token_rows(ids)], axis=0)


def config4_first_embed(model):
    return model.token_rows([24])[0]          # embed(AUDIO), voxtral_tts.c:295


# ---- codec decoder (voxtral_tts_codec.c:389-510) ----
CODEC_SEED = 77
CODEC_GOLDEN_FRAMES = 5


def codec_codes(n_frames, seed=5):
    """[n_frames, 37] codes as the acoustic stage emits them: semantic 2 .. 8193, acoustic
    2 .. 22 (FSQ level + 2). Frame 0 also carries values below the special-token offset and
    above the code books (the decoder clamps them, voxtral_tts_codec.c:283-296) when there is
    more than one frame."""
    import numpy as np
    rng = np.random.default_rng(seed + 1000 * n_frames)
    codes = np.concatenate([rng.integers(2, 8194, size=(n_frames, 1)), rng.integers(2, 23, size=(n_frames, 36))],
                           axis=1).astype(np.int32)
    if n_frames > 1:
        codes[0, 0] = 0
        codes[0, 1] = 1
        codes[0, 2] = 30
        codes[1, 0] = 9000
    return codes
