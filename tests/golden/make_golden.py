#!/usr/bin/env python3
"""Generate the golden fixtures in this directory from the reference's own CPU
code (oracle/_ref/libvoxref_noblas.so, built from the reference checkout by
oracle/build_oracle.py). Run it where the reference checkout is present:

    python tests/golden/make_golden.py

Inputs are the seeded synthetic tensors of the package (SynthModel, synth_f32),
so the fixtures hold outputs only:
  config1_decode.npz   one decoder step at cache length 64
  config2_acoustic.npz one acoustic frame, RNG seed 42
  frames3.npz          three chained frames: decode -> acoustic -> re-embed
  primitives.npz       the kernel-level functions on small seeded inputs
With --full (minutes of CPU; uses the OpenBLAS build, as the reference's `make blas` does):
  config3_prefill.npz  cache rows after a 256-row prompt: three rows of three layers in full,
                       and the norm of every row of those layers
  config4_slice.npz    that prompt followed by 16 generated frames: codes, hidden rows, RNG state
With --codec (seconds):
  codec_frames.npz     the codec decoder's waveform for a few frames of seeded codes (SynthCodec)
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from conftest import load_package  # noqa: E402
import oracle_bind as ob  # noqa: E402
from cases import (CONFIG4_FRAMES, CONFIG4_SEED, GOLDEN_LAYERS, GOLDEN_ROWS, MODEL_SEED, config1_inputs,  # noqa: E402
                   config2_inputs, config3_prompt, config4_first_embed, frames_inputs, primitive_inputs)


def full_size(pkg, model):
    """Configurations 3 and 4 at their full size on the reference's OpenBLAS build."""
    ref = ob.load_ref("blas")
    if ref is None:
        raise SystemExit("oracle/_ref/libvoxref_blas.so missing: run oracle/build_oracle.py with the reference present")
    rows = config3_prompt(pkg, model)
    M = rows.shape[0]
    ref.open(model, kv_max=M + CONFIG4_FRAMES + 8)
    ref.llm_prefill(rows)
    assert ref.kv_len() == M
    k, v = ref.kv()
    L, R = list(GOLDEN_LAYERS), list(GOLDEN_ROWS)
    np.savez_compressed(os.path.join(HERE, "config3_prefill.npz"),
                        k_rows=k[L][:, R].copy(), v_rows=v[L][:, R].copy(),
                        k_norms=np.linalg.norm(k[L, :M].astype(np.float64), axis=-1).astype(np.float32),
                        v_norms=np.linalg.norm(v[L, :M].astype(np.float64), axis=-1).astype(np.float32))
    ref.seed(CONFIG4_SEED)
    e = config4_first_embed(model)
    codes, hidden = [], []
    for _ in range(CONFIG4_FRAMES):
        h = ref.llm_forward(e)
        c = ref.acoustic_forward(h)
        codes.append(c)
        hidden.append(h)
        e = ref.audio_embed(c)
    np.savez_compressed(os.path.join(HERE, "config4_slice.npz"), codes=np.stack(codes), hidden=np.stack(hidden),
                        rng_after=np.uint64(ref.rng_state()))
    ref.close()
    print("full-size fixtures written to", HERE)


def codec(pkg):
    """The reference's tts_codec_decode on the seeded synthetic codec weights."""
    from cases import CODEC_GOLDEN_FRAMES, CODEC_SEED, codec_codes
    ref = ob.load_ref("noblas")
    if ref is None or not hasattr(ref.L, "refh_codec_decode"):
        raise SystemExit("oracle/_ref/libvoxref_noblas.so (with the codec) missing: run oracle/build_oracle.py")
    w = pkg.SynthCodec(seed=CODEC_SEED)
    pcm = ref.codec_decode(w.struct(), codec_codes(CODEC_GOLDEN_FRAMES))
    np.savez_compressed(os.path.join(HERE, "codec_frames.npz"), pcm=pcm)
    print("codec fixture written:", pcm.shape)


def main():
    pkg = load_package()
    if "--codec" in sys.argv:
        return codec(pkg)
    if "--full" in sys.argv:
        return full_size(pkg, pkg.SynthModel(seed=MODEL_SEED))
    ref = ob.load_ref("noblas")
    if ref is None:
        raise SystemExit("oracle/_ref/libvoxref_noblas.so missing: run oracle/build_oracle.py with the reference present")
    model = pkg.SynthModel(seed=MODEL_SEED)
    ref.open(model, kv_max=128)

    # config 1
    embed, kvk, kvv = config1_inputs(pkg)
    k, v = ref.kv()
    k[:, :64] = kvk
    v[:, :64] = kvv
    ref.set_kv_len(64)
    hidden, tap = ref.llm_forward(embed, tap=True)
    k, v = ref.kv()
    np.savez_compressed(os.path.join(HERE, "config1_decode.npz"), hidden=hidden,
                        tap_norms=np.linalg.norm(tap.astype(np.float64), axis=-1).astype(np.float32),
                        tap_first8=tap[:, :, :8].copy(), tap_last=tap[-1].copy(),
                        k_row64=k[:, 64].copy(), v_row64=v[:, 64].copy())

    # config 2
    h2, seed = config2_inputs(pkg)
    ref.seed(seed)
    codes = ref.acoustic_forward(h2)
    st = ref.rng_state()
    noise, _ = ref.randn(ob.Oracle().seed(seed), 36)
    vel0 = ref.predict_velocity(noise, h2, 0.0)
    velu = ref.predict_velocity(noise, np.zeros_like(h2), 3.0 / 7.0)
    np.savez_compressed(os.path.join(HERE, "config2_acoustic.npz"), codes=codes, rng_after=np.uint64(st),
                        noise=noise, vel_t0_cond=vel0, vel_t3_uncond=velu)

    # chained frames
    first_embed, kvk3, kvv3, seed3, n_frames = frames_inputs(pkg)
    ref.open(model, kv_max=128)
    k, v = ref.kv()
    k[:, :kvk3.shape[1]] = kvk3
    v[:, :kvv3.shape[1]] = kvv3
    ref.set_kv_len(kvk3.shape[1])
    ref.seed(seed3)
    e = first_embed
    all_codes, all_hidden = [], []
    for _ in range(n_frames):
        h = ref.llm_forward(e)
        c = ref.acoustic_forward(h)
        all_codes.append(c)
        all_hidden.append(h)
        e = ref.audio_embed(c)
    np.savez_compressed(os.path.join(HERE, "frames3.npz"), codes=np.stack(all_codes), hidden=np.stack(all_hidden),
                        next_embed=e, rng_after=np.uint64(ref.rng_state()))

    # primitives
    P = primitive_inputs(pkg)
    out = {}
    out["linear_m1"] = ref.linear(P["x1"], P["W"])
    out["linear_m3_bias"] = ref.linear(P["x3"], P["W"], P["bias"])
    L = ref.L
    o = np.empty_like(P["x3"])
    L.tts_rms_norm(ob._p(o), ob._p(P["x3"]), ob._p(P["gain"]), 3, P["x3"].shape[1], 1e-5)
    out["rms_norm"] = o
    for sk in (1, 3, 50, 225):
        q, kk, vv = P["q"], P["k"][:sk], P["v"][:sk]
        o = np.zeros(32 * 128, dtype=np.float32)
        L.tts_causal_attention(ob._p(o), ob._p(q), ob._p(np.ascontiguousarray(kk)), ob._p(np.ascontiguousarray(vv)),
                               1, sk, 32, 8, 128, 1.0 / np.sqrt(128.0), 0, sk - 1)
        out[f"causal_attn_{sk}"] = o
    o = np.zeros((3, 32 * 128), dtype=np.float32)
    L.tts_bidirectional_attention(ob._p(o), ob._p(P["q3"]), ob._p(np.ascontiguousarray(P["k"][:3])),
                                  ob._p(np.ascontiguousarray(P["v"][:3])), 3, 32, 8, 128, 1.0 / np.sqrt(128.0))
    out["bidir_attn"] = o
    pos = np.array([0, 1, 77, 467], dtype=np.int32)
    cs = np.empty((4, 64, 2), dtype=np.float32)
    L.tts_compute_rope_freqs(ob._p(cs), ob._p(pos), 4, 128, 1e6)
    out["rope_table"] = cs
    xr = P["rope_x"].copy()
    L.tts_apply_rope(ob._p(xr), ob._p(cs), 4, 8, 128)
    out["rope_apply"] = xr
    g = P["gate"].copy()
    L.tts_silu(ob._p(g), g.size)
    L.tts_mul_inplace(ob._p(g), ob._p(P["up"]), g.size)
    out["silu_mul"] = g
    rn, st = ref.randn(ob.Oracle().seed(0), 8)
    out["randn_seed0"] = rn
    out["randn_seed0_state"] = np.uint64(st)
    np.savez_compressed(os.path.join(HERE, "primitives.npz"), **out)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
