"""Pins the CPU oracle (oracle/vox_oracle.c).

1. Against the committed golden fixtures, which were produced by the reference's
   own CPU sources (tests/golden/make_golden.py). Bit-exact: the port keeps the
   reference's operation order.
2. Against the reference libraries themselves (oracle/_ref) when they are
   present, including the OpenBLAS build, whose M>1 sums are ordered differently
   (tolerance 1e-4 relative L2).
3. Against the known-answer checks the reference's own test file makes
   (test_kernels.c:122-430 compares CPU and GPU on these shapes; here the CPU
   restatement is compared with the reference CPU build on the same shapes).
"""
import os

import numpy as np
import pytest

from cases import MODEL_SEED, config1_inputs, config2_inputs, frames_inputs, primitive_inputs

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


@pytest.fixture(scope="module")
def model(pkg):
    return pkg.SynthModel(seed=MODEL_SEED)


def test_primitives_match_golden(pkg, oracle):
    g = np.load(os.path.join(GOLD, "primitives.npz"))
    P = primitive_inputs(pkg)
    assert np.array_equal(oracle.linear(P["x1"], P["W"]), g["linear_m1"])
    assert np.array_equal(oracle.linear(P["x3"], P["W"], P["bias"]), g["linear_m3_bias"])
    assert np.array_equal(oracle.rms_norm(P["x3"], P["gain"]), g["rms_norm"])
    scale = float(1.0 / np.sqrt(128.0))
    for sk in (1, 3, 50, 225):
        o = oracle.attention_causal(P["q"], P["k"][:sk], P["v"][:sk], 32, 8, 128, scale, sk - 1)
        assert np.array_equal(o[0], g[f"causal_attn_{sk}"]), sk
    o = oracle.attention_full(P["q3"], P["k"][:3], P["v"][:3], 32, 8, 128, scale)
    assert np.array_equal(o, g["bidir_attn"])
    cs = oracle.rope_table([0, 1, 77, 467])
    assert np.array_equal(cs, g["rope_table"])
    assert np.array_equal(oracle.rope_apply(P["rope_x"], cs, 8), g["rope_apply"])
    assert np.array_equal(oracle.silu_mul(P["gate"], P["up"]), g["silu_mul"])
    rn, st = oracle.randn(oracle.seed(0), 8)
    assert np.array_equal(rn, g["randn_seed0"]) and st == int(g["randn_seed0_state"])


def test_rng_known_properties(oracle):
    # seed 0 maps to the fixed default (voxtral_tts_kernels.c:640-642)
    assert oracle.seed(0) == 0x12345678ABCDEF01
    assert oracle.seed(5) == 5
    a, s1 = oracle.randn(5, 36)
    b, s2 = oracle.randn(5, 36)
    assert np.array_equal(a, b) and s1 == s2
    big, _ = oracle.randn(1, 20000)
    assert abs(big.mean()) < 0.03 and abs(big.std() - 1.0) < 0.03


def test_config1_decode_matches_golden(pkg, oracle, model):
    g = np.load(os.path.join(GOLD, "config1_decode.npz"))
    embed, kvk, kvv = config1_inputs(pkg)
    k = np.zeros((26, 128, 1024), dtype=np.float32)
    v = np.zeros_like(k)
    k[:, :64] = kvk
    v[:, :64] = kvv
    hidden, tap = oracle.llm_forward(oracle.decoder(model), k, v, 64, embed, tap=True)
    assert np.array_equal(hidden, g["hidden"])
    assert np.array_equal(tap[-1], g["tap_last"])
    assert np.array_equal(tap[:, :, :8], g["tap_first8"])
    assert np.array_equal(k[:, 64], g["k_row64"]) and np.array_equal(v[:, 64], g["v_row64"])


def test_config2_acoustic_matches_golden(pkg, oracle, model):
    g = np.load(os.path.join(GOLD, "config2_acoustic.npz"))
    hidden, seed = config2_inputs(pkg)
    ac = oracle.acoustic(model)
    codes, logits, xf, st = oracle.acoustic_forward(ac, oracle.seed(seed), hidden)
    assert np.array_equal(codes, g["codes"])
    assert st == int(g["rng_after"])
    assert 1 <= codes[0] <= 8193 and np.all(codes[1:] >= 2) and np.all(codes[1:] <= 22)
    assert logits[0] == np.float32(-1e30) and np.all(logits[8194:] == np.float32(-1e30))
    assert np.array_equal(oracle.predict_velocity(ac, g["noise"], hidden, 0.0), g["vel_t0_cond"])
    assert np.array_equal(oracle.predict_velocity(ac, g["noise"], np.zeros_like(hidden), 3.0 / 7.0),
                          g["vel_t3_uncond"])


def test_chained_frames_match_golden(pkg, oracle, model):
    g = np.load(os.path.join(GOLD, "frames3.npz"))
    first, kvk, kvv, seed, n = frames_inputs(pkg)
    k = np.zeros((26, 128, 1024), dtype=np.float32)
    v = np.zeros_like(k)
    k[:, :kvk.shape[1]] = kvk
    v[:, :kvv.shape[1]] = kvv
    dec, ac = oracle.decoder(model), oracle.acoustic(model)
    st = oracle.seed(seed)
    e = first
    pos = kvk.shape[1]
    for f in range(n):
        h = oracle.llm_forward(dec, k, v, pos + f, e)
        codes, _, _, st = oracle.acoustic_forward(ac, st, h)
        assert np.array_equal(h, g["hidden"][f]) and np.array_equal(codes, g["codes"][f])
        e = oracle.audio_embed(model.audio_table(), codes)
    assert np.array_equal(e, g["next_embed"]) and st == int(g["rng_after"])


def test_end_code_draws_no_noise(pkg, oracle, model):
    """A bias that forces semantic code 1 (END): acoustic codes are all 2 and the RNG
    state is untouched (voxtral_tts_acoustic.c:312-320)."""
    hidden, seed = config2_inputs(pkg)
    ac = oracle.acoustic(model)
    bias = np.zeros(8320, dtype=np.float32)
    bias[1] = 1e6
    ac.semantic_bias = bias.ctypes.data_as(type(ac.semantic_bias))
    st0 = oracle.seed(seed)
    codes, _, _, st = oracle.acoustic_forward(ac, st0, hidden)
    assert codes[0] == 1 and np.all(codes[1:] == 2) and st == st0


def test_prefill_equals_stepwise_decode(pkg, oracle, model):
    """Prefill of n rows leaves the cache that n single steps leave (two-layer model to keep it fast)."""
    dec = oracle.decoder(model, n_layers=2)
    rows = pkg.synth_f32((5, 3072), 3, "pf.rows", 0.0, 0.5)
    k1 = np.zeros((2, 16, 1024), dtype=np.float32)
    v1 = np.zeros_like(k1)
    oracle.llm_prefill(dec, k1, v1, 0, rows)
    k2 = np.zeros_like(k1)
    v2 = np.zeros_like(k1)
    for i in range(5):
        oracle.llm_forward(dec, k2, v2, i, rows[i])
    assert np.array_equal(k1, k2) and np.array_equal(v1, v2)


# ---- against the reference libraries themselves (present only with the checkout) ----

def test_port_vs_reference_decode_bit_exact(pkg, oracle, model, ref_noblas):
    embed, kvk, kvv = config1_inputs(pkg)
    ref_noblas.open(model, kv_max=128)
    k, v = ref_noblas.kv()
    k[:, :64] = kvk
    v[:, :64] = kvv
    ref_noblas.set_kv_len(64)
    h_ref, tap_ref = ref_noblas.llm_forward(embed, tap=True)
    ko = np.zeros((26, 128, 1024), dtype=np.float32)
    vo = np.zeros_like(ko)
    ko[:, :64] = kvk
    vo[:, :64] = kvv
    h, tap = oracle.llm_forward(oracle.decoder(model), ko, vo, 64, embed, tap=True)
    assert np.array_equal(h, h_ref) and np.array_equal(tap, tap_ref)
    assert ref_noblas.kv_len() == 65
    ref_noblas.close()


def test_port_vs_reference_blas_prefill(pkg, oracle, model, ref_blas):
    """M>1 goes through cblas_sgemm in the reference's default build; sums are ordered
    differently, so the comparison is by relative L2 (1e-4), per layer."""
    rows = pkg.synth_f32((6, 3072), 3, "pf.rows6", 0.0, 0.5)
    ref_blas.open(model, kv_max=16)
    tap_ref = ref_blas.llm_prefill(rows, tap=True)
    kr, vr = ref_blas.kv()
    ko = np.zeros((26, 16, 1024), dtype=np.float32)
    vo = np.zeros_like(ko)
    tap = oracle.llm_prefill(oracle.decoder(model), ko, vo, 0, rows, tap=True)
    for l in range(26):
        assert rel_l2(tap[l, 1], tap_ref[l, 1]) < 1e-4, l
    assert rel_l2(ko[:, :6], kr[:, :6]) < 1e-4 and rel_l2(vo[:, :6], vr[:, :6]) < 1e-4
    assert ref_blas.kv_len() == 6
    ref_blas.close()


def test_reference_test_kernels_shapes(pkg, oracle, ref_noblas):
    """The shapes, seeds-by-name and tolerances of the reference's own harness
    (test_kernels.c: rms_norm 1x3072 1e-4/1e-6; gemm 1x3072 @ 4096x3072 1e-3/1e-4;
    causal attention seq_k in {1,3,10,50,100,225} 1e-3/1e-5; bidirectional seq 3)."""
    x = pkg.synth_f32(3072, 11, "tk.x", 0.0, 0.1)
    w = np.abs(pkg.synth_f32(3072, 11, "tk.w", 0.0, 0.1)) + 0.01
    o_ref = np.empty(3072, dtype=np.float32)
    from oracle_bind import _p
    ref_noblas.L.tts_rms_norm(_p(o_ref), _p(x), _p(w), 1, 3072, 1e-5)
    assert np.array_equal(oracle.rms_norm(x, w)[0], o_ref)
    W = pkg.synth_bf16((4096, 3072), 11, "tk.W")
    assert np.array_equal(oracle.linear(x, W), ref_noblas.linear(x, W))
    scale = float(1.0 / np.sqrt(128.0))
    for sk in (1, 3, 10, 50, 100, 225):
        q = pkg.synth_f32(4096, 100 + sk, "tk.q", 0.0, 0.1)
        k = pkg.synth_f32((sk, 1024), 200 + sk, "tk.k", 0.0, 0.1)
        v = pkg.synth_f32((sk, 1024), 300 + sk, "tk.v", 0.0, 0.1)
        o_ref = np.zeros(4096, dtype=np.float32)
        ref_noblas.L.tts_causal_attention(_p(o_ref), _p(q), _p(k), _p(v), 1, sk, 32, 8, 128, scale, 0, sk - 1)
        assert np.array_equal(oracle.attention_causal(q, k, v, 32, 8, 128, scale, sk - 1)[0], o_ref), sk


def test_codec_fixture_is_the_reference_decoder_output(ref_noblas):
    """tests/golden/codec_frames.npz (what the GPU codec tests compare with when oracle/_ref is absent)
    is reproduced by the reference's tts_codec_decode (voxtral_tts_codec.c:389-510) on the seeded
    synthetic codec weights."""
    import os
    from cases import CODEC_GOLDEN_FRAMES, CODEC_SEED, codec_codes
    from conftest import load_package
    if not hasattr(ref_noblas.L, "refh_codec_decode"):
        pytest.skip("oracle/_ref was built without the codec")
    pkg = load_package()
    want = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "codec_frames.npz"))["pcm"]
    got = ref_noblas.codec_decode(pkg.SynthCodec(seed=CODEC_SEED).struct(), codec_codes(CODEC_GOLDEN_FRAMES))
    assert got.shape == want.shape
    assert np.array_equal(got, want)
