"""GPU parity of the decoder step (tts_cuda_llm_forward) against the CPU oracle and the golden
fixtures of the reference CPU build: benchmark configuration 1 (cache pre-filled with 64 positions).
Tolerance of the hot path: every layer's residual stream within 2e-3 relative L2."""
import os

import numpy as np
import pytest

from cases import MODEL_SEED, config1_inputs
from gpu_common import rel_l2

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
LAYER_TOL = 2e-3


@pytest.fixture(scope="module")
def eng(engine):
    return engine


@pytest.fixture(scope="module")
def model(synth_model):
    return synth_model


def _fill_cache(eng, kvk, kvv):
    for l in range(26):
        eng.kv_write(l, 0, kvk[l], kvv[l])


def test_config1_per_layer_and_hidden(pkg, eng, oracle, model):
    g = np.load(os.path.join(GOLD, "config1_decode.npz"))
    embed, kvk, kvv = config1_inputs(pkg)
    _fill_cache(eng, kvk, kvv)
    eng.tap(True)
    hidden = eng.llm_forward(embed, 64)
    tap = eng.tap_read()
    eng.tap(False)

    k = np.zeros((26, 128, 1024), dtype=np.float32)
    v = np.zeros_like(k)
    k[:, :64] = kvk
    v[:, :64] = kvv
    h_ref, tap_ref = oracle.llm_forward(oracle.decoder(model), k, v, 64, embed, tap=True)
    worst = max(rel_l2(tap[l, j], tap_ref[l, j]) for l in range(26) for j in range(2))
    assert worst < LAYER_TOL, worst
    assert rel_l2(hidden, h_ref) < LAYER_TOL
    # golden fixture of the reference CPU build
    assert rel_l2(hidden, g["hidden"]) < LAYER_TOL
    assert rel_l2(tap[-1], g["tap_last"]) < LAYER_TOL
    norms = np.linalg.norm(tap.astype(np.float64), axis=-1)
    assert np.allclose(norms, g["tap_norms"], rtol=LAYER_TOL)
    # the new K/V row
    for l in (0, 13, 25):
        kr, vr = eng.kv_read(l, 64, 1)
        assert rel_l2(kr[0], g["k_row64"][l]) < LAYER_TOL and rel_l2(vr[0], g["v_row64"][l]) < LAYER_TOL
    # the tap must not change the result
    assert np.array_equal(hidden, eng.llm_forward(embed, 64))


def test_repeatable_bit_for_bit(pkg, eng):
    embed, kvk, kvv = config1_inputs(pkg)
    _fill_cache(eng, kvk, kvv)
    a = eng.llm_forward(embed, 64)
    b = eng.llm_forward(embed, 64)
    assert np.array_equal(a, b)      # fixed summation order: no atomics on the data path


@pytest.mark.parametrize("pos", [0, 1, 31, 32, 33, 200, 467, 511])
def test_positions_and_key_splits(pkg, eng, oracle, model, pos):
    """Cache lengths around the 32-key split boundaries, the first and the last row."""
    kvk = pkg.synth_f32((26, max(pos, 1), 1024), 21, f"kvk{pos}")
    kvv = pkg.synth_f32((26, max(pos, 1), 1024), 22, f"kvv{pos}")
    embed = pkg.synth_f32(3072, 23, f"e{pos}")
    k = np.zeros((26, 512, 1024), dtype=np.float32)
    v = np.zeros_like(k)
    if pos:
        k[:, :pos] = kvk
        v[:, :pos] = kvv
        _fill_cache(eng, kvk, kvv)
    h = eng.llm_forward(embed, pos)
    h_ref = oracle.llm_forward(oracle.decoder(model), k, v, pos, embed)
    assert rel_l2(h, h_ref) < LAYER_TOL, rel_l2(h, h_ref)


def test_position_outside_cache_is_refused(pkg, eng):
    embed, _, _ = config1_inputs(pkg)
    out = np.zeros(3072, dtype=np.float32)
    from ctypes import c_void_p
    eng.L.tts_cuda_llm_forward(out.ctypes.data_as(c_void_p), embed.ctypes.data_as(c_void_p), 512)
    assert not out.any()             # reported on stderr, nothing written, no launch
    assert eng.L.vb200_last_status() == 0
