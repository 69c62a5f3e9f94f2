"""GPU parity of the codec decoder (vb200_codec_upload / vb200_codec_decode) against the
reference's own tts_codec_decode (voxtral_tts_codec.c:389-510) compiled unchanged, and against the
committed fixture made from it. Tolerance: 1e-3 relative L2 on the waveform (the transformer
linears multiply BF16 weights with hi + lo BF16 activation terms, 4e-6 per GEMM; the rest is fp32
summation order; measured ~1e-5)."""
import ctypes as C
import os

import numpy as np
import pytest

from cases import CODEC_GOLDEN_FRAMES, CODEC_SEED, codec_codes
from gpu_common import rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-3
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "codec_frames.npz")


@pytest.fixture(scope="module")
def codec(pkg):
    return pkg.SynthCodec(seed=CODEC_SEED)


@pytest.fixture(scope="module")
def codec_engine(engine, codec):
    engine.codec_upload(codec)
    return engine


@pytest.fixture(scope="module")
def ref_codec():
    import oracle_bind
    for kind in ("blas", "noblas"):
        r = oracle_bind.load_ref(kind)
        if r is not None and hasattr(r.L, "refh_codec_decode"):
            return r
    pytest.skip("the reference's codec is not built (oracle/_ref)")


def test_golden_waveform(codec_engine):
    want = np.load(GOLDEN)["pcm"]
    got, ms = codec_engine.codec_decode(codec_codes(CODEC_GOLDEN_FRAMES))
    assert got.shape == want.shape == (CODEC_GOLDEN_FRAMES * 1920,)
    assert ms > 0.0
    assert rel_l2(got, want) < TOL


@pytest.mark.parametrize("n_frames", [1, 2, 3, 17, 33, 40, 100])
def test_against_the_reference_decoder(codec_engine, codec, ref_codec, n_frames):
    """1 frame (every convolution sees its reflect padding only), 17 (136 rows in the last stage:
    two row blocks), 33 (264 rows: past the 256-row term buffer), 100 (800 rows)."""
    if n_frames > 40 and ref_codec.kind != "blas":
        pytest.skip("the portable reference build needs minutes for this size")
    codes = codec_codes(n_frames)
    want = ref_codec.codec_decode(codec.struct(), codes)
    got, _ = codec_engine.codec_decode(codes)
    assert got.shape == want.shape
    assert rel_l2(got, want) < TOL, n_frames
    assert np.max(np.abs(got - want)) < 5e-3 * max(1.0, float(np.max(np.abs(want))))


def test_optional_tensors_absent(pkg, engine, ref_codec, codec):
    """No QK norm, no layer scale, no convolution bias: the NULL branches of
    voxtral_tts_codec.c:333-337,350-357 and voxtral_tts_kernels.c:241."""
    bare = pkg.SynthCodec(seed=CODEC_SEED + 1, qk_norm=False, layer_scale=False, conv_bias=False)
    try:
        engine.codec_upload(bare)
        codes = codec_codes(6)
        want = ref_codec.codec_decode(bare.struct(), codes)
        got, _ = engine.codec_decode(codes)
        assert rel_l2(got, want) < TOL
    finally:
        engine.codec_upload(codec)


def test_refuses_weights_bf16_cannot_hold(pkg, engine, codec):
    """The transformer matrices are kept as BF16: a value that would be rounded is refused."""
    w = codec.struct()
    name = "codec.layers.3.wo"
    keep = codec.t[name]
    bad = keep.copy()
    bad[5, 7] = np.float32(0.0123456789)
    try:
        codec.t[name] = bad
        assert engine.L.vb200_codec_upload(C.byref(codec.struct())) == -1
        out = np.empty(1920, dtype=np.float32)
        n = C.c_int(0)
        codes = codec_codes(1)
        assert engine.L.vb200_codec_decode(codes.ctypes.data_as(C.c_void_p), 1, out.ctypes.data_as(C.c_void_p), 1920,
                                           C.byref(n)) == -1       # nothing uploaded now
    finally:
        codec.t[name] = keep
        engine.codec_upload(codec)
    del w


def test_rejects_bad_arguments(codec_engine):
    L = codec_engine.L
    codes = codec_codes(2)
    out = np.empty(2 * 1920, dtype=np.float32)
    n = C.c_int(0)
    cp, op = codes.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p)
    assert L.vb200_codec_decode(cp, 0, op, out.size, C.byref(n)) == -1
    assert L.vb200_codec_decode(None, 2, op, out.size, C.byref(n)) == -1
    assert L.vb200_codec_decode(cp, 2, op, out.size - 1, C.byref(n)) == -1      # too small
    assert L.vb200_codec_decode(cp, 2, op, out.size, C.byref(n)) == 0 and n.value == out.size


def test_frames_decode_independently_of_the_batch_they_come_in(codec_engine):
    """The decoder is causal: the first frames of a long decode equal a short decode of them,
    up to the window the later stages look back over (none looks ahead)."""
    codes = codec_codes(24)
    long, _ = codec_engine.codec_decode(codes)
    short, _ = codec_engine.codec_decode(codes[:9])
    # the output convolution (kernel 7, reflect padding only on the left) never reads ahead
    assert rel_l2(long[:9 * 1920], short) < 1e-5


def test_long_utterances_go_block_by_block(codec_engine):
    """Blocks of 64 frames with 32 frames of re-decoded left context reproduce the one-piece decode
    (the decoder's look-back is under 17 frames)."""
    codes = codec_codes(200)
    whole, _ = codec_engine.codec_decode(codes)
    try:
        assert codec_engine.L.vb200_set_option(b"codec_block_frames", 64) == 0
        parts, _ = codec_engine.codec_decode(codes)
    finally:
        assert codec_engine.L.vb200_set_option(b"codec_block_frames", 2048) == 0
    assert parts.shape == whole.shape
    # not bit-identical: the split-K counts of the convolution GEMMs follow the row count
    # (measured 3e-6, the level of the hi + lo operand split)
    assert rel_l2(parts, whole) < 2e-5
    assert codec_engine.L.vb200_set_option(b"codec_block_frames", 10) == -1
