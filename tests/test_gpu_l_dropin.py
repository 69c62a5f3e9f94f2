"""The stage entry points of the drop-in, executed: tts_llm_load, tts_llm_kv_cache_alloc,
tts_acoustic_load, tts_cuda_init + weight upload, tts_llm_prefill, tts_llm_forward,
tts_acoustic_forward and tts_audio_embed_forward of voxtral-tts.c_b200/dropin/ are driven by
oracle/dropin_harness.c exactly as the reference's orchestrator drives its own stage files
(voxtral_tts.c:22-107, :279-321) on a synthetic safetensors checkpoint, and compared with the
same harness linked against the reference's own voxtral_tts_llm.c / voxtral_tts_acoustic.c on the
CPU: codes and RNG state frame by frame, including a frame that ends the utterance."""
import os
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")


def _run(exe, args, timeout):
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = os.path.join(ROOT, "voxtral-tts.c_b200", "lib") + os.pathsep + env.get("LD_LIBRARY_PATH", "")
    r = subprocess.run([exe] + [str(a) for a in args], capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0, (exe, r.stdout[-2000:], r.stderr[-2000:])
    frames, done = [], None
    for line in r.stdout.splitlines():
        w = line.split()
        if w and w[0] == "frame":
            frames.append((int(w[3]), np.array([int(x) for x in w[5:]], dtype=np.int32)))
        elif w and w[0] == "done":
            done = {"frames": int(w[2]), "rng": int(w[4]), "kv_len": int(w[6])}
    assert done is not None and len(frames) == done["frames"], r.stdout[-2000:]
    return frames, done


def test_stage_entry_points_match_the_reference_stages(pkg, synth_model, oracle, tmp_path_factory):
    cand, chk = os.path.join(REF_DIR, "dropin_run_b200"), os.path.join(REF_DIR, "dropin_run_ref")
    if not (os.path.exists(cand) and os.path.exists(chk)):
        pytest.skip("oracle/_ref/dropin_run_* not built (needs the reference checkout at build time)")
    d = tmp_path_factory.mktemp("dropin")
    ckpt, prompt_file = str(d / "consolidated.safetensors"), str(d / "prompt.f32")
    try:
        synth_model.write_safetensors(ckpt)
        voice = pkg.synth_f32((9, 3072), 51, "dropin.voice", 0.0, 0.5)
        prompt = np.concatenate([voice, synth_model.token_rows([36, 1234, 35])], axis=0).astype(np.float32)
        prompt.tofile(prompt_file)
        n, seed, frames, kv_max = prompt.shape[0], 777, 8, 64
        want, wdone = _run(chk, [ckpt, prompt_file, n, seed, frames, kv_max, 0], 1200)
        got, gdone = _run(cand, [ckpt, prompt_file, n, seed, frames, kv_max, 0], 600)
        assert wdone["frames"] == frames and gdone == wdone           # frames, RNG state, cache length
        same = 0
        for f in range(frames):
            assert got[f][0] == want[f][0], f                         # RNG state after the frame
            assert got[f][1][0] == want[f][1][0], f                   # semantic code
            same += int(np.array_equal(got[f][1], want[f][1]))
            if not np.array_equal(got[f][1], want[f][1]):
                # a latent on an FSQ rounding boundary: one code may differ, and the frames after it
                # see a different input row
                assert int(np.sum(got[f][1] != want[f][1])) <= 1, f
                break
        else:
            assert same == frames
        # END: the frame is reported with codes 1, 2, 2, ... and draws nothing from the RNG
        want_e, wdone_e = _run(chk, [ckpt, prompt_file, n, seed, frames, kv_max, 1], 1200)
        got_e, gdone_e = _run(cand, [ckpt, prompt_file, n, seed, frames, kv_max, 1], 600)
        assert wdone_e["frames"] == 1 and gdone_e == wdone_e
        assert got_e[0][1][0] == 1 and np.all(got_e[0][1][1:] == 2) and np.array_equal(got_e[0][1], want_e[0][1])
        assert gdone_e["rng"] == oracle.seed(seed)                    # untouched
    finally:
        for p in (ckpt, prompt_file):
            if os.path.exists(p):
                os.remove(p)


def test_codec_stage_matches_the_reference_codec(pkg, tmp_path_factory):
    """tts_codec_load + tts_codec_decode of dropin/voxtral_tts_codec_b200.c against the reference's own
    voxtral_tts_codec.c, both run by oracle/codec_harness.c on the same synthetic safetensors file
    (weight-normed and plain convolutions, the cluster-usage clamp, BF16 matrices)."""
    from cases import CODEC_SEED, codec_codes
    cand, chk = os.path.join(REF_DIR, "codec_run_b200"), os.path.join(REF_DIR, "codec_run_ref")
    if not (os.path.exists(cand) and os.path.exists(chk)):
        pytest.skip("oracle/_ref/codec_run_* not built (needs the reference checkout at build time)")
    d = tmp_path_factory.mktemp("codec")
    ckpt, codes_file = str(d / "codec.safetensors"), str(d / "codes.i32")
    outs = [str(d / "ref.f32"), str(d / "b200.f32")]
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = os.path.join(ROOT, "voxtral-tts.c_b200", "lib") + os.pathsep + env.get("LD_LIBRARY_PATH", "")
    try:
        pkg.SynthCodec(seed=CODEC_SEED + 2).write_safetensors(ckpt)
        n_frames = 12
        codec_codes(n_frames).tofile(codes_file)
        for exe, out in ((chk, outs[0]), (cand, outs[1])):
            r = subprocess.run([exe, ckpt, codes_file, str(n_frames), out], capture_output=True, text=True, timeout=900,
                               env=env)
            assert r.returncode == 0 and f"samples {n_frames * 1920}" in r.stdout, (exe, r.stdout[-1000:], r.stderr[-1000:])
        want, got = np.fromfile(outs[0], dtype=np.float32), np.fromfile(outs[1], dtype=np.float32)
        assert want.shape == got.shape == (n_frames * 1920,)
        err = np.linalg.norm(got.astype(np.float64) - want) / np.linalg.norm(want.astype(np.float64))
        assert err < 1e-3, err
    finally:
        for p in [ckpt, codes_file] + outs:
            if os.path.exists(p):
                os.remove(p)
