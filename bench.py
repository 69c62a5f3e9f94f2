#!/usr/bin/env python3
"""Benchmark of the per-frame hot path: frames/s of (decoder step + acoustic frame).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (configuration 4 of the benchmark description, "full autoregressive utterance"): a 256-row prompt is
prefilled, then frames are generated one after another; one step = one audio frame = one
26-layer decoder step at a growing cache (256, 257, ...) + one acoustic frame (semantic
argmax, 7 Euler steps x 2 guidance branches, FSQ) + re-embedding of the 37 codes. Weights are
seeded random-init tensors of the real shapes (no checkpoint offline); an END code is treated
as an ordinary code so that the frame count is fixed.

value : frames/s with the whole loop resident on the device (inputs in HBM, no host traffic
        inside the timed region), timed with CUDA events on the launching stream.
e2e   : the same metric through the host-facing C-ABI call (vb200_frame: host embedding and
        noise in, host hidden state and codes out, every frame) with the re-embedding on the
        host, as the reference's frame loop does (voxtral_tts.c:301-318).
N > 1 : independent utterances, one per GPU (weak scaling, no data-path collective); the line also
        carries `tp`, the same utterance decoded by all N GPUs together (tensor-parallel decoder).

Further keys of the line: roofline (the GEMM kernel timed live, and the whole frame), cpu_baseline
(the reference's CPU code on a bounded sample, with per-configuration timings), gpu_reference (the
reference's own CUDA backend on the same GPU, in a child process), batched (8 utterances per GPU in
lock step), streaming_decoder (the decoder step on the persistent streaming kernel), upload (weight
upload seconds and bytes), codec (the codec decoder on the utterance's codes), utterance (prefill
and first-frame latency), clocks. `--micro gemv|gemm|stream|prefill|codec` runs one kernel or stage on
its own (small cases for profiling).

--impl reference times the reference's own CPU code for the same frames (oracle/_ref, the
unmodified reference sources built with OpenBLAS; or the CPU restatement if that library is
absent) on the host cores; it never touches a GPU.
"""
import argparse
import ctypes as C
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG_DIR = os.path.join(ROOT, "voxtral-tts.c_b200")

PROMPT_ROWS = 256
W_LAYER = 232_783_872                      # BF16 bytes of one transformer layer's seven matrices
LLM_WEIGHT_BYTES = 26 * W_LAYER
LLM_NORM_BYTES = 651_264
KV_WRITE_BYTES = 212_992
ACOUSTIC_BYTES = 4_962_152_448             # semantic head + llm_proj once + 7 x (3 layers + small heads)
REEMBED_BYTES = 37 * 3072 * 2


def load_package():
    name = "voxtral_tts_c_b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(PKG_DIR, "__init__.py"),
                                                  submodule_search_locations=[PKG_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def utterance_seeds(rank):
    """Each rank generates its own utterance (prompt and noise seeds): independent units, no
    data-path collective."""
    return {"prompt": 100 + rank, "noise": 1000 + rank}


def aggregate(local_ms, frames_per_rank, dist=None, device="cuda", shared=False):
    """Whole-job frames/s: every rank ran frames_per_rank frames in local_ms of device time; the
    job took the slowest rank's time. shared: all ranks worked on the SAME frames (tensor
    parallelism), so they count once. Returns (frames_per_s, max_ms)."""
    import torch
    t = torch.tensor([float(local_ms)], dtype=torch.float64, device=device)
    world = 1
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        world = dist.get_world_size()
    max_ms = float(t.item())
    return (1 if shared else world) * frames_per_rank / (max_ms / 1000.0), max_ms


def frame_bytes(pos):
    """Algorithmic HBM bytes of one frame decoded at cache row `pos` (keys = pos + 1)."""
    return (LLM_WEIGHT_BYTES + LLM_NORM_BYTES + 26 * (pos + 1) * 8192 + KV_WRITE_BYTES + ACOUSTIC_BYTES
            + REEMBED_BYTES)


def prompt_rows(pkg, model, seed):
    """224 voice-embedding rows ~N(0,0.5) then 32 token rows with ids in [1000, 131072)."""
    voice = pkg.synth_f32((224, pkg.DIM), seed, "bench.voice", 0.0, 0.5)
    ids = 1000 + (pkg.synth_bf16(32, seed, "bench.ids").astype(np.int64) * 2 % (pkg.VOCAB - 1000))
    return np.concatenate([voice, model.token_rows(ids)], axis=0)


def noise_rows(seed, n):
    """n x 36 normals from the reference's generator (the library's bit-exact restatement of
    tts_randn_fill, voxtral_tts_kernels.c:640-669), state = seed."""
    vals, _ = load_package().randn(seed, n * 36)
    return vals.reshape(n, 36)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while a timed region runs. The sampler is started
    well before the region (nvidia-smi needs up to a second to come up on an 8-GPU node, longer
    than a short timed region); begin() / end() mark the region and only samples that arrived
    inside it count. If the region was too short to catch one, the samples taken while the GPU
    was under the same load just before and after it (warm-up, host-ABI frames) are used and the
    result says so. It is stopped right after the region: its polling slows host-side launches
    (a 256-row prefill measured 27 ms with it running, 12.7 ms without)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None
        self.t0 = self.t1 = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def begin(self):
        self.t0 = time.time()

    def end(self):
        self.t1 = time.time()

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

        def summarise(rows):
            sm, mx, reasons = [], [], set()
            for _, r in rows:
                if len(r) < 8:
                    continue
                try:
                    sm.append(float(r[0]))
                    mx.append(float(r[1]))
                except ValueError:
                    continue
                for name, val in zip(names, r[4:8]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            return sm, mx, reasons

        t0 = self.t0 if self.t0 is not None else 0.0
        t1 = self.t1 if self.t1 is not None else float("inf")
        inside = [x for x in self.rows if t0 <= x[0] <= t1 + 0.05]
        sm, mx, reasons = summarise(inside)
        window = "timed region"
        if not sm:
            near = [x for x in self.rows if t0 - 2.0 <= x[0] <= t1 + 2.0]
            sm, mx, reasons = summarise(near)
            window = "the 2 s before the timed region (warm-up frames, same load; the region itself was shorter than a sample interval)"
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons), "window": window}


def measured_hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


# ----------------------------------------------------------------------------------------------
# reference CPU arm and cpu_baseline
# ----------------------------------------------------------------------------------------------
def set_host_threads():
    """All host cores for the CPU arm, whatever the launcher exported (torchrun sets
    OMP_NUM_THREADS=1). Must run before the BLAS library is loaded."""
    n = str(os.cpu_count() or 1)
    os.environ["OMP_NUM_THREADS"] = n
    os.environ["OPENBLAS_NUM_THREADS"] = n
    return int(n)


def cpu_reference(pkg, model, rows, first_embed, noise_seed, n_warm, n_frames, budget_s):
    """Times the same workload on the host with the reference's own CPU code: the 256-row prompt
    is prefilled by the reference (outside the timed frames; its time is the configuration-3
    figure), then n_warm untimed and up to n_frames timed frames (decoder step, acoustic frame,
    re-embedding). Also one decoder step at 64 cached positions and one acoustic frame
    (configurations 1 and 2). Returns a dict."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    cores = set_host_threads()
    import oracle_bind
    ref = oracle_bind.load_ref("blas")
    kind, what = "reference", "reference C sources, -DUSE_BLAS with scipy's OpenBLAS"
    if ref is None:
        ref = oracle_bind.load_ref("noblas")
        what = "reference C sources, portable build without BLAS"
    pos0 = rows.shape[0]
    per_config = {}
    t_frames, done = 0.0, 0
    if ref is not None:
        ref.open(model, kv_max=pos0 + n_warm + n_frames + 8)
        ref.seed(noise_seed)
        ref.set_kv_len(64)                       # 64 cached positions (their values do not change the work)
        ref.llm_forward(first_embed)             # pages the decoder weights in
        ref.set_kv_len(64)
        t0 = time.perf_counter()
        h = ref.llm_forward(first_embed)
        per_config["decoder_step_ms_at_64_cached_positions"] = (time.perf_counter() - t0) * 1000.0
        ref.acoustic_forward(h)
        t0 = time.perf_counter()
        ref.acoustic_forward(h)
        per_config["acoustic_frame_ms"] = (time.perf_counter() - t0) * 1000.0
        ref.set_kv_len(0)
        t0 = time.perf_counter()
        ref.llm_prefill(rows)
        per_config["prefill_s_256_rows"] = time.perf_counter() - t0
        ref.seed(noise_seed)
        e = first_embed
        t_start = time.perf_counter()
        for f in range(n_warm + n_frames):
            t0 = time.perf_counter()
            h = ref.llm_forward(e)
            codes = ref.acoustic_forward(h)
            e = ref.audio_embed(codes)
            dt = time.perf_counter() - t0
            if f >= n_warm:
                t_frames += dt
                done += 1
            elif time.perf_counter() - t_start > 0.4 * budget_s:
                n_warm = f + 1                   # the warm-up may not eat the budget
            if done and time.perf_counter() - t_start + t_frames / done > budget_s:
                break
        ref.close()
    else:
        kind, what = "port", "CPU restatement (oracle/vox_oracle.c, OpenMP over output rows)"
        orc = oracle_bind.Oracle()
        dec, ac = orc.decoder(model), orc.acoustic(model)
        k = np.zeros((26, pos0 + n_warm + n_frames + 8, 1024), dtype=np.float32)
        v = np.zeros_like(k)
        t0 = time.perf_counter()
        orc.llm_prefill(dec, k, v, 0, rows)
        per_config["prefill_s_256_rows"] = time.perf_counter() - t0
        st, e = orc.seed(noise_seed), first_embed
        t_start = time.perf_counter()
        for f in range(n_warm + n_frames):
            t0 = time.perf_counter()
            h = orc.llm_forward(dec, k, v, pos0 + f, e)
            codes, _, _, st = orc.acoustic_forward(ac, st, h)
            e = orc.audio_embed(model.audio_table(), codes)
            dt = time.perf_counter() - t0
            if f >= n_warm:
                t_frames += dt
                done += 1
            if done and time.perf_counter() - t_start + t_frames / done > budget_s:
                break
    fps = done / t_frames
    return {"value": fps, "unit": "frames/s", "cores": cores, "kind": kind, "per_config": per_config,
            "sample": f"{done} timed frame(s) of the same workload (decoder step at {pos0}+ cached positions of the "
                      f"prefilled prompt, acoustic frame, re-embedding) after {n_warm} warm-up frame(s); {what}; the "
                      f"M=1 decoder matvecs are single-threaded by construction, the M=3 acoustic GEMMs and the "
                      f"prefill use up to {cores} threads",
            "ms_per_frame": 1000.0 / fps}


def gpu_reference_worker(n_frames):
    """Runs in a process of its own (the reference's CUDA object exports the same symbol names as
    this repository's library): the reference's own CUDA backend, built unchanged for sm_100 into
    oracle/_ref/libvoxref_cuda.so, on the same synthetic weights: per frame tts_cuda_llm_forward
    and the 14 tts_cuda_predict_velocity calls of the Euler loop (voxtral_tts_acoustic.c:336-355),
    wall clock (every call ends with a blocking copy to the host). Prints one JSON line."""
    pkg = load_package()
    path = os.path.join(ROOT, "oracle", "_ref", "libvoxref_cuda.so")
    if not os.path.exists(path):
        print(json.dumps({"unavailable": "oracle/_ref/libvoxref_cuda.so not built (needs the reference checkout and cuBLAS at build time)"}))
        return
    try:
        R = C.CDLL(path)
    except OSError as e:
        print(json.dumps({"unavailable": f"cannot load the reference CUDA object: {e}"}))
        return
    model = pkg.SynthModel(seed=1234)
    tok = pkg.synth_bf16((pkg.VOCAB, pkg.DIM), 1234, "mm_audio_embeddings.tok_embeddings.weight")
    dec, ac = model.decoder_struct(), model.acoustic_struct()
    dec.tok_embeddings = tok.ctypes.data_as(pkg.u16p)
    R.tts_cuda_init.restype = C.c_int
    R.tts_cuda_upload_llm_weights.restype = C.c_int
    R.tts_cuda_upload_acoustic_weights.restype = C.c_int
    kv_max = PROMPT_ROWS + n_frames + 16
    if R.tts_cuda_init(kv_max) != 0 or R.tts_cuda_upload_llm_weights(C.byref(dec)) != 0 or \
            R.tts_cuda_upload_acoustic_weights(C.byref(ac)) != 0:
        print(json.dumps({"unavailable": "the reference's tts_cuda_init / weight upload failed on this GPU"}))
        return
    vp = C.c_void_p
    R.tts_cuda_llm_forward.argtypes = [vp, vp, C.c_int]
    R.tts_cuda_predict_velocity.argtypes = [vp, vp, vp, C.c_float]
    embed = (tok[24].astype(np.uint32) << 16).view(np.float32).copy()
    hidden = np.zeros(pkg.DIM, dtype=np.float32)
    zeros = np.zeros(pkg.DIM, dtype=np.float32)
    vc, vu = np.zeros(36, dtype=np.float32), np.zeros(36, dtype=np.float32)
    noise = noise_rows(5, n_frames + 1)
    ms = []
    for f in range(n_frames + 1):                # the first frame is the warm-up
        t0 = time.perf_counter()
        R.tts_cuda_llm_forward(hidden.ctypes.data, embed.ctypes.data, PROMPT_ROWS + f)
        x = noise[f].copy()
        for i in range(pkg.FLOW_STEPS - 1):
            t = np.float32(i) / np.float32(pkg.FLOW_STEPS - 1)
            R.tts_cuda_predict_velocity(vc.ctypes.data, x.ctypes.data, hidden.ctypes.data, C.c_float(float(t)))
            R.tts_cuda_predict_velocity(vu.ctypes.data, x.ctypes.data, zeros.ctypes.data, C.c_float(float(t)))
            x = x + (np.float32(1.2) * vc - np.float32(0.2) * vu) * np.float32(1.0 / (pkg.FLOW_STEPS - 1))
        if f:
            ms.append((time.perf_counter() - t0) * 1000.0)
    ok = bool(np.isfinite(hidden).all() and np.isfinite(x).all())
    R.tts_cuda_free()
    print(json.dumps({"ms_per_frame": float(np.mean(ms)), "frames_per_s": 1000.0 / float(np.mean(ms)), "frames": len(ms),
                      "finite_outputs": ok,
                      "what": "the reference's own CUDA backend (voxtral_tts_cuda.cu, cuBLAS SGEMM after a BF16->fp32 "
                              "expansion of every weight per call), built unchanged with -arch=sm_100: "
                              "tts_cuda_llm_forward at cache rows 256.. + 14 x tts_cuda_predict_velocity per frame, "
                              "wall clock; the semantic head, FSQ and re-embedding, which the reference leaves on the "
                              "CPU, are not included; cache rows below 256 are zero"}))


def gpu_reference(n_frames=4, timeout=600):
    """The GPU reference arm, from a child process. Returns a dict (with `unavailable` and the reason
    when it cannot run)."""
    try:
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "gpu_reference_worker", "--steps",
                            str(n_frames)], capture_output=True, text=True, timeout=timeout,
                           env={k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")})
    except subprocess.TimeoutExpired:
        return {"unavailable": f"the reference CUDA backend did not finish {n_frames} frames in {timeout} s"}
    for line in reversed(r.stdout.strip().splitlines()):
        try:
            return json.loads(line)
        except ValueError:
            continue
    return {"unavailable": f"the reference CUDA backend exited with {r.returncode}: {r.stderr.strip()[-300:]}"}


def micro_gemm(args):
    """The tensor-core GEMM kernel alone on one generated [n, k] matrix (no model upload): `reps`
    launches between two CUDA events. Not the headline metric: a small case for profiling and the
    per-shape table."""
    pkg = load_package()
    L = pkg.lib()
    ms, splits = C.c_float(0.0), C.c_int(0)
    rc = L.vb200_tc_gemm_probe(args.m, args.n, args.k, 1 if args.swiglu else 0,
                               (0 if args.untiled else 1) | (2 if args.l2_resident else 0), args.reps,
                               C.byref(ms), C.byref(splits))
    if rc != 0:
        raise SystemExit(f"vb200_tc_gemm_probe failed ({rc})")
    peak, src = measured_hbm_peak()
    us = ms.value * 1000.0 / args.reps
    gbs = 2.0 * args.n * args.k / (us * 1e-6) / 1e9
    print(json.dumps({"micro": "gemm", "m": args.m, "k": args.k, "n": args.n, "launches": args.reps,
                      "epilogue": "swiglu_terms" if args.swiglu else "split_k_partials", "splits": splits.value,
                      "tiled_weights": not args.untiled, "l2_resident": bool(args.l2_resident), "us_per_launch": us, "weight_bytes": 2 * args.n * args.k,
                      "achieved_gbs": gbs, "frac_of_peak": gbs / peak, "peak_source": src}))


def micro_stream(args):
    """The streaming decoder-step kernel alone on `--ops` GEMV ops over generated [n, k] matrices
    (no model upload; rotating copies so no op finds its weights in L2), with or without a grid
    barrier after every op. A small case for profiling and the per-shape table."""
    pkg = load_package()
    L = pkg.lib()
    ms, nb = C.c_float(0.0), C.c_double(0.0)
    rc = L.vb200_stream_probe(args.n, args.k, args.ops, 0 if args.no_sync else 1, args.reps, C.byref(ms), C.byref(nb))
    if rc != 0:
        raise SystemExit(f"vb200_stream_probe failed ({rc})")
    peak, src = measured_hbm_peak()
    us = ms.value * 1000.0 / args.reps
    gbs = nb.value / (us * 1e-6) / 1e9
    print(json.dumps({"micro": "stream", "k": args.k, "n": args.n, "ops_per_launch": args.ops, "launches": args.reps,
                      "grid_barrier_after_each_op": not args.no_sync, "us_per_launch": us, "us_per_op": us / args.ops,
                      "weight_bytes_per_launch": nb.value, "achieved_gbs": gbs, "frac_of_peak": gbs / peak,
                      "peak_source": src}))


def codec_leg(pkg, eng, codes, cpu_frames):
    """The codec decoder (vb200_codec_decode) on the utterance's codes: device time, wall time from
    host codes to host waveform, and the reference's own tts_codec_decode on the host cores on the
    first `cpu_frames` frames of the same codes (a bounded sample: its cost grows linearly with the
    frame count)."""
    codec = pkg.SynthCodec(seed=77)
    t0 = time.perf_counter()
    eng.codec_upload(codec)
    up_s = time.perf_counter() - t0
    eng.codec_decode(codes)
    wall, dev = [], []
    for _ in range(5):
        t0 = time.perf_counter()
        pcm, ms = eng.codec_decode(codes)
        wall.append((time.perf_counter() - t0) * 1e3)
        dev.append(ms)
    n = int(codes.shape[0])
    out = {"frames": n, "audio_s": n / 12.5, "samples": int(pcm.size), "device_ms": min(dev), "wall_ms": min(wall),
           "upload_s": up_s, "h2d_bytes": int(codes.nbytes), "d2h_bytes": int(pcm.nbytes),
           "weights": "seeded random-init codec decoder of the real shapes (8 transformer layers of width 1024, "
                      "4 convolutions)"}
    if cpu_frames > 0:
        try:
            sys.path.insert(0, os.path.join(ROOT, "tests"))
            import oracle_bind
            ref = oracle_bind.load_ref("blas") or oracle_bind.load_ref("noblas")
            if ref is not None and hasattr(ref.L, "refh_codec_decode"):
                k = min(cpu_frames, n)
                t0 = time.perf_counter()
                want = ref.codec_decode(codec.struct(), codes[:k])
                cpu_ms = (time.perf_counter() - t0) * 1e3
                got = pcm[:k * 1920].astype(np.float64)
                err = float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
                out["cpu_reference"] = {"frames": k, "ms": cpu_ms, "ms_per_frame": cpu_ms / k, "kind": ref.kind,
                                        "rel_l2_gpu_vs_reference": err}
        except Exception as e:                               # the extra leg never costs the main line
            out["cpu_reference"] = {"error": f"{type(e).__name__}: {e}"}
    return out


def micro_prefill(args):
    """tts_cuda_llm_prefill alone: `--m` prompt rows (host fp32 rows in, cache rows out), `--reps`
    calls, wall clock per call (the call is synchronous). Uploads the decoder only. The launch
    list of the prefill is taken from this command."""
    pkg = load_package()
    model = pkg.SynthModel(seed=1234)
    eng = pkg.Engine(kv_cache_max=max(64, args.m + 8))
    eng.upload(model, decoder=True, acoustic=False)
    rows = prompt_rows(pkg, model, utterance_seeds(0)["prompt"])[:args.m]
    eng.prefill(rows, 0)
    t = []
    for _ in range(args.reps):
        t0 = time.perf_counter()
        eng.prefill(rows, 0)
        t.append((time.perf_counter() - t0) * 1e3)
    print(json.dumps({"micro": "prefill", "rows": int(rows.shape[0]), "calls": args.reps, "ms_per_call_min": min(t),
                      "ms_per_call_median": sorted(t)[len(t) // 2]}))


def micro_codec(args):
    """vb200_codec_decode alone on `--m` frames of seeded codes (no decoder upload): `--reps` calls,
    device and wall time per call. The launch list of the codec decoder is taken from this command."""
    pkg = load_package()
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from cases import codec_codes
    eng = pkg.Engine(kv_cache_max=64)
    eng.codec_upload(pkg.SynthCodec(seed=77))
    codes = codec_codes(args.m)
    eng.codec_decode(codes)
    wall, dev = [], []
    for _ in range(args.reps):
        t0 = time.perf_counter()
        _, ms = eng.codec_decode(codes)
        wall.append((time.perf_counter() - t0) * 1e3)
        dev.append(ms)
    print(json.dumps({"micro": "codec", "frames": args.m, "calls": args.reps, "device_ms_min": min(dev),
                      "wall_ms_min": min(wall), "audio_s": args.m / 12.5}))


def micro(args):
    """One GEMV op of the frame kernel through tts_cuda_linear_bf16 on device buffers:
    y[m,n] = x[m,k] . W[n,k]^T. Not the headline metric: a small, self-contained case for profiling."""
    if args.micro == "gemm":
        return micro_gemm(args)
    if args.micro == "stream":
        return micro_stream(args)
    if args.micro == "prefill":
        return micro_prefill(args)
    if args.micro == "codec":
        return micro_codec(args)
    pkg = load_package()
    eng = pkg.Engine(kv_cache_max=64)
    L = eng.L
    M, K, N = args.m, args.k, args.n
    x = pkg.synth_f32((M, K), 1, "micro.x")
    W = pkg.synth_bf16((N, K), 2, "micro.W")
    dx, dW, dy = pkg.DeviceBuffer(x), pkg.DeviceBuffer(W), pkg.DeviceBuffer(nbytes=M * N * 4)
    for _ in range(3):
        L.tts_cuda_linear_bf16(dy.ptr, dx.ptr, None, M, K, N, dW.ptr)
    L.tts_cuda_sync()
    eng.engine_ms(reset=True)
    for _ in range(args.reps):
        L.tts_cuda_linear_bf16(dy.ptr, dx.ptr, None, M, K, N, dW.ptr)
    L.tts_cuda_sync()
    ms, n = eng.engine_ms()
    peak, src = measured_hbm_peak()
    gbs = 2.0 * N * K / (ms / 1000.0) / 1e9
    print(json.dumps({"micro": "gemv", "m": M, "k": K, "n": N, "launches": n, "us_per_launch": ms * 1000.0,
                      "weight_bytes": 2 * N * K, "achieved_gbs": gbs, "frac_of_peak": gbs / peak, "peak_source": src,
                      "status": L.vb200_last_status()}))
    eng.close()


# ----------------------------------------------------------------------------------------------
_RESULT_FD = None


def quiet_stdout():
    """Libraries (NCCL's version banner, the CUDA runtime) may write to stdout; the result line
    must be the only thing there. Everything else is sent to stderr from here on."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=212)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "gpu_reference_worker"])
    ap.add_argument("--no-gpu-reference", action="store_true", help="skip the reference's own CUDA backend (child process)")
    ap.add_argument("--no-tp-leg", action="store_true",
                    help="with N > 1 ranks: skip the extra one-utterance tensor-parallel measurement")
    ap.add_argument("--e2e-steps", type=int, default=0, help="frames of the host-ABI measurement (default: min(steps, 64))")
    ap.add_argument("--cpu-budget", type=float, default=25.0, help="seconds of CPU-baseline frames")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tp", action="store_true",
                    help="with N > 1 ranks: ONE utterance, the decoder tensor-parallel over the N GPUs (strong scaling) "
                         "instead of one utterance per GPU")
    ap.add_argument("--no-codec-leg", action="store_true", help="skip the codec-decoder leg")
    ap.add_argument("--no-streaming-leg", action="store_true",
                    help="skip the extra measurement with the decoder step on the persistent streaming kernel")
    ap.add_argument("--utterances", type=int, default=8,
                    help="utterances per GPU of the additional lock-step measurement (1 = skip it)")
    ap.add_argument("--swiglu", action="store_true", help="--micro gemm: SwiGLU epilogue instead of split-K partials")
    ap.add_argument("--untiled", action="store_true", help="--micro gemm: row-major weights instead of the tiled copy")
    ap.add_argument("--l2-resident", action="store_true",
                    help="--micro gemm: one weight copy (stays in L2 when it fits) instead of rotating copies")
    ap.add_argument("--ops", type=int, default=16, help="--micro stream: GEMV ops per launch")
    ap.add_argument("--no-sync", action="store_true", help="--micro stream: no grid barrier between the ops")
    ap.add_argument("--micro", default="", choices=["", "gemv", "gemm", "stream", "prefill", "codec"],
                    help="kernel micro-benchmark instead of the frame loop (reported separately; used for ncu captures)")
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--k", type=int, default=3072)
    ap.add_argument("--n", type=int, default=32768)
    ap.add_argument("--reps", type=int, default=8)
    args = ap.parse_args()
    if args.micro:
        return micro(args)
    if args.impl == "gpu_reference_worker":
        return gpu_reference_worker(max(args.steps, 1))
    quiet_stdout()
    K, W = max(args.steps, 1), max(args.warmup, 0)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    config = {"workload": "config 4: 256-row prompt prefilled, then one utterance per GPU generates frames "
                          "(decoder step at cache 256.. + acoustic frame 7 Euler x 2 CFG + re-embedding)",
              "prompt_rows": PROMPT_ROWS, "frames": K, "utterances_per_gpu": 1, "parallelism": f"dp{world}",
              "weights": "seeded random-init BF16 ~N(0,0.02), real shapes",
              "l2_policy": "inputs larger than L2 (11 GB of weights stream per frame)"}

    pkg = load_package()

    if args.impl == "reference":
        if rank != 0:
            return
        model = pkg.SynthModel(seed=1234)
        seeds = utterance_seeds(0)
        rows = prompt_rows(pkg, model, seeds["prompt"])
        first = model.token_rows([24])[0]
        budget = min(170.0, max(30.0, 6.0 * (K + W)))
        r = cpu_reference(pkg, model, rows, first, seeds["noise"], W, K, budget)
        cb = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample", "per_config")}
        line = {"impl": "reference", "metric": "frames_per_s", "value": r["value"], "unit": "frames/s",
                "n_gpus": args.gpus, "steps": K, "warmup": W, "ms_per_step": r["ms_per_frame"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f32 (BF16 weights, fp32 activations and accumulation)",
                "data": "synthetic", "config": config, "cpu_baseline": cb,
                "e2e": {"value": r["value"], "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        emit(line)
        return

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: the library has no CPU fallback "
                         "(use --impl reference for the CPU reference arm)")
    torch.cuda.set_device(local_rank)
    os.environ["VB200_DEVICE"] = str(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        try:
            torch.set_num_threads(max(1, (os.cpu_count() or 8) // world))
        except Exception:
            pass
        os.environ.setdefault("OMP_NUM_THREADS", str(max(1, (os.cpu_count() or 8) // world)))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(int(os.environ.get("VB200_DEVICE", local_rank)))
    sampler.start()
    model = pkg.SynthModel(seed=1234)
    kv_max = PROMPT_ROWS + W + K + 72
    eng = pkg.Engine(kv_cache_max=kv_max)
    eng.upload(model, decoder=True, acoustic=True, audio_table=True)
    up_s, up_b = eng.upload_stats()
    upload = {"seconds": up_s, "bytes": up_b, "gbs": up_b / up_s / 1e9 if up_s > 0 else None,
              "what": "tts_cuda_upload_llm_weights + tts_cuda_upload_acoustic_weights + vb200_upload_audio_embed from "
                      "pageable host memory: pinned staging ring filled by host threads, copies and repacking "
                      "kernels on one stream, one wait per call"}
    eng.L.vb200_set_option(b"ignore_end", 1)

    tp = bool(args.tp and world > 1)
    if tp:
        # every rank maps the others' exchange arenas (CUDA IPC handles gathered over the process group)
        handle = (C.c_ubyte * 64)()
        assert eng.L.vb200_tp_arena(rank, world, handle) == 0, "tensor-parallel arena"
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle))
        assert eng.L.vb200_tp_connect(b"".join(handles)) == 0, "tensor-parallel connect"
        barrier()
        config["parallelism"] = f"tp{world}"
        config["utterances_per_gpu"] = f"1 utterance over {world} GPUs"
    seeds = utterance_seeds(0 if tp else rank)               # tensor parallelism: all ranks decode the same utterance
    rows = prompt_rows(pkg, model, seeds["prompt"])
    eng.prefill(rows, 0)
    first = model.token_rows([24])[0]                      # embed(AUDIO), voxtral_tts.c:295
    noise = noise_rows(seeds["noise"], W + K)

    # ---- value: device-resident loop -------------------------------------------------------
    Lb = eng.L
    assert Lb.vb200_utterance_begin(first.ctypes.data, PROMPT_ROWS, noise.ctypes.data, W + K) == 0
    codes = np.zeros((W + K, pkg.CODES), dtype=np.int32)
    done, end, ms = C.c_int(0), C.c_int(0), C.c_float(0.0)
    if W:
        assert Lb.vb200_utterance_run(W) == 0
    torch.cuda.synchronize()
    barrier()
    sampler.begin()
    assert Lb.vb200_utterance_run(K) == 0
    torch.cuda.synchronize()
    barrier()
    sampler.end()
    clocks = sampler.stop()                                 # nvidia-smi polling must not run into the host-timed legs
    assert Lb.vb200_utterance_end(codes.ctypes.data, C.byref(done), C.byref(end), C.byref(ms)) == 0
    if done.value != W + K:
        raise SystemExit(f"device loop ran {done.value} of {W + K} frames (status {Lb.vb200_last_status()})")
    value, total_ms = aggregate(ms.value, K, dist, shared=tp)

    # ---- e2e: one host-facing call per frame, re-embedding on the host ------------------------
    Ke = args.e2e_steps or min(K, 64)
    table = model.audio_table()
    offs = np.concatenate([[0], 8194 + 23 * np.arange(36)]).astype(np.int64)
    # the prompt prefill through the reference-facing call (host rows in, synchronous): it also
    # rewinds the cache to the prompt
    prefill_ms = []
    for _ in range(3):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.prefill(rows, 0)
        torch.cuda.synchronize()
        prefill_ms.append((time.perf_counter() - t0) * 1000.0)
    e = first.copy()
    pos = PROMPT_ROWS
    for f in range(min(W, 3)):
        c, _ = eng.frame(e, noise[f], pos)
        pos += 1
        e = (table[offs + c].astype(np.uint32) << 16).view(np.float32).sum(axis=0, dtype=np.float32)
    barrier()
    t0 = time.perf_counter()
    for f in range(Ke):
        c, h = eng.frame(e, noise[min(W, 3) + f], pos)      # H2D embed+noise, kernel, D2H hidden+codes
        pos += 1
        e = (table[offs + c].astype(np.uint32) << 16).view(np.float32).sum(axis=0, dtype=np.float32)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e_value, _ = aggregate(e2e_s * 1000.0, Ke, dist, shared=tp)

    # ---- roofline of the dominant kernel --------------------------------------------------------
    peak, peak_src = measured_hbm_peak()
    on_tc = bool(Lb.vb200_frame_on_tensor_cores())
    head_bytes = 51_118_080 + 18_874_368                      # semantic head + llm_proj
    mean_frame_bytes = float(np.mean([frame_bytes(PROMPT_ROWS + W + f) for f in range(K)]))
    frame_ms = total_ms / K
    whole = {"algorithmic_bytes": mean_frame_bytes, "ms": frame_ms,
             "achieved": mean_frame_bytes / (frame_ms / 1000.0) / 1e9,
             "frac": mean_frame_bytes / (frame_ms / 1000.0) / 1e9 / peak}
    if on_tc:
        # A frame is one CUDA graph of 350 launches; 190 of them are vb_tc_gemm_kernel<16> and
        # carry every weight byte (104 decoder-layer GEMMs, 2 head GEMMs, 84 acoustic-layer
        # GEMMs). Launches inside a graph cannot be bracketed one by one, so the kernel's own
        # launch time is measured live on the decoder's 104 GEMMs launched back to back (every
        # decoder weight byte once per sweep: 6.05 GB, far beyond L2) between two CUDA events.
        sweeps = 10
        sms, sbytes, sn = C.c_float(0.0), C.c_double(0.0), C.c_int(0)
        assert Lb.vb200_gemm_sweep(0, 2, C.byref(sms), C.byref(sbytes), C.byref(sn)) == 0
        assert Lb.vb200_gemm_sweep(0, sweeps, C.byref(sms), C.byref(sbytes), C.byref(sn)) == 0
        launch_ms = sms.value / (sweeps * sn.value)
        bytes_per_launch = sbytes.value / sn.value
        achieved = bytes_per_launch / (launch_ms / 1000.0) / 1e9
        gemm_bytes_frame = LLM_WEIGHT_BYTES + ACOUSTIC_BYTES
        traffic = None
        try:
            with open(os.path.join(ROOT, "profiles", "tc_gemm_traffic.json")) as f:
                ratio = json.load(f).get("dram_bytes_over_algorithmic")
                traffic = bytes_per_launch * ratio if ratio else None
        except Exception:
            pass
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": traffic,
                    "kernel": "vb_tc_gemm_kernel<16> (tcgen05 skinny GEMM; 190 of a frame's 350 launches, all weight bytes)",
                    "algorithmic_bytes_per_launch": bytes_per_launch, "launch_ms": launch_ms,
                    "measured_on": f"{sweeps} sweeps of the decoder's {sn.value} layer GEMMs, back to back, CUDA events",
                    "share_of_frame_time": (gemm_bytes_frame / 1e9 / achieved * 1000.0) / frame_ms,
                    "peak_source": peak_src, "whole_frame": whole}
        launches_per_frame = int(Lb.vb200_batch_launches_per_frame())
    else:
        n_eng = C.c_int(0)
        eng_ms_total = float(Lb.vb200_utterance_engine_ms(C.byref(n_eng)))
        tc_ac = os.environ.get("VB200_NO_TC") is None
        dec_bytes = lambda pos: LLM_WEIGHT_BYTES + LLM_NORM_BYTES + 26 * (pos + 1) * 8192 + KV_WRITE_BYTES
        if tc_ac and n_eng.value == K:
            eng_bytes = float(np.mean([dec_bytes(PROMPT_ROWS + W + f) for f in range(K)])) + head_bytes + REEMBED_BYTES
            launch_ms = eng_ms_total / n_eng.value
            kernel_desc = "vb_engine_kernel (one launch per frame: re-embedding + decoder step + semantic head)"
        else:                                                     # whole frame inside the frame kernel
            eng_bytes = mean_frame_bytes
            launch_ms = (eng_ms_total / n_eng.value) if n_eng.value == K else frame_ms
            kernel_desc = "vb_engine_kernel (one launch = one whole frame)"
        achieved = eng_bytes / (launch_ms / 1000.0) / 1e9
        traffic = None
        try:
            with open(os.path.join(ROOT, "profiles", "frame_kernel_traffic.json")) as f:
                ratio = json.load(f).get("dram_read_over_algorithmic")
                traffic = eng_bytes * ratio if ratio else None
        except Exception:
            pass
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": traffic, "kernel": kernel_desc, "algorithmic_bytes_per_launch": eng_bytes,
                    "launch_ms": launch_ms, "share_of_frame_time": launch_ms / frame_ms, "peak_source": peak_src,
                    "whole_frame": whole}
        launches_per_frame = 1 + (84 + 42 + 21 + 14 + 1 if tc_ac else 0)

    # ---- several utterances per GPU in lock step (weights read once per frame for all) -----------
    batched = None
    if on_tc and args.utterances > 1 and not tp:
        Bu = args.utterances
        Kb, Wb = min(K, 64), min(W, 5)
        cap = Wb + Kb
        assert Lb.vb200_batch_open(Bu, PROMPT_ROWS + cap + 8, cap) == 0
        for u in range(Bu):
            pr = rows if u == 0 else prompt_rows(pkg, model, seeds["prompt"] + 17 * u)
            assert Lb.vb200_batch_prefill(u, pr.ctypes.data, PROMPT_ROWS) == 0
        nb = np.stack([noise_rows(seeds["noise"] + 31 * u, cap) for u in range(Bu)]).astype(np.float32)
        fe = np.ascontiguousarray(np.stack([first] * Bu), dtype=np.float32)
        sp = np.full(Bu, PROMPT_ROWS, dtype=np.int32)
        assert Lb.vb200_batch_begin(fe.ctypes.data, sp.ctypes.data, nb.ctypes.data) == 0
        assert Lb.vb200_batch_run(Wb) == 0
        torch.cuda.synchronize()
        barrier()
        assert Lb.vb200_batch_run(Kb) == 0
        bdone = np.zeros(Bu, dtype=np.int32)
        bms = C.c_float(0.0)
        assert Lb.vb200_batch_end(None, bdone.ctypes.data, None, C.byref(bms)) == 0
        if int(bdone.min()) != cap:
            raise SystemExit(f"batched loop ran {bdone.tolist()} of {cap} frames")
        Lb.vb200_batch_close()
        bval, bmax = aggregate(bms.value, Kb * Bu, dist)
        per_utt = float(np.mean([26 * (PROMPT_ROWS + Wb + f + 1) * 8192 for f in range(Kb)])) + KV_WRITE_BYTES + REEMBED_BYTES
        step_bytes = LLM_WEIGHT_BYTES + LLM_NORM_BYTES + ACOUSTIC_BYTES + Bu * per_utt
        batched = {"utterances_per_gpu": Bu, "value": bval, "unit": "frames/s", "steps": Kb, "ms_per_step": bmax / Kb,
                   "algorithmic_bytes_per_step": step_bytes,
                   "hbm_frac": step_bytes / (bmax / Kb / 1000.0) / 1e9 / peak,
                   "workload": "config 5 per GPU: 8 utterances, 256-row prompts, lock-step frames"}

    # ---- the other decoder-step kernel: one launch of the persistent streaming kernel per frame ----
    streaming = None
    if on_tc and not tp and not args.no_streaming_leg:
        Ks, Ws = min(K, 64), min(W, 5)
        assert Lb.vb200_set_option(b"decoder_kernel", 1) == 0
        try:
            eng.prefill(rows, 0)
            assert Lb.vb200_utterance_begin(first.ctypes.data, PROMPT_ROWS, noise.ctypes.data, Ws + Ks) == 0
            assert Lb.vb200_utterance_run(Ws) == 0
            torch.cuda.synchronize()
            barrier()
            assert Lb.vb200_utterance_run(Ks) == 0
            sdone, send, sms = C.c_int(0), C.c_int(0), C.c_float(0.0)
            assert Lb.vb200_utterance_end(None, C.byref(sdone), C.byref(send), C.byref(sms)) == 0
            sval, smax = aggregate(sms.value, Ks, dist)
            stms, stb = C.c_float(0.0), C.c_double(0.0)
            mid = PROMPT_ROWS + (W + K) // 2
            assert Lb.vb200_stream_step_ms(mid, 10, C.byref(stms), C.byref(stb)) == 0
            step_ms = stms.value / 10
            streaming = {"decoder_kernel": "vb_stream_kernel (26 layers + semantic head + llm token + argmax: one launch)",
                         "value": sval, "unit": "frames/s", "steps": Ks, "ms_per_step": smax / Ks,
                         "launches_per_frame": 1 + (pkg.FLOW_STEPS - 1) * (2 + pkg.AC_LAYERS * 7) + 1,
                         "step_launch_ms": step_ms, "step_cache_row": mid, "step_algorithmic_bytes": stb.value,
                         "step_achieved_gbs": stb.value / (step_ms / 1000.0) / 1e9,
                         "step_frac": stb.value / (step_ms / 1000.0) / 1e9 / peak}
        finally:
            Lb.vb200_set_option(b"decoder_kernel", 0)

    # ---- N > 1: ONE utterance with the decoder tensor-parallel over the N GPUs (strong scaling) ----
    tp_leg = None
    if world > 1 and not tp and not args.no_tp_leg:
        def all_ok(flag):
            t = torch.tensor([1 if flag else 0], dtype=torch.int32, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            return bool(t.item())

        Kt, Wt = min(K, 64), min(W, 5)
        stage, ok = "arena", True
        try:
            handle = (C.c_ubyte * 64)()
            ok = all_ok(Lb.vb200_tp_arena(rank, world, handle) == 0)
            if ok:
                stage = "connect"
                handles = [None] * world
                dist.all_gather_object(handles, bytes(handle))
                ok = all_ok(Lb.vb200_tp_connect(b"".join(handles)) == 0)
            tms, tcodes, run_ok = 0.0, None, False
            if ok:
                stage = "run"
                try:
                    s0 = utterance_seeds(0)                  # every rank decodes the same utterance
                    rows0 = rows if rank == 0 else prompt_rows(pkg, model, s0["prompt"])
                    noise0 = noise if rank == 0 else noise_rows(s0["noise"], W + K)
                    eng.prefill(rows0, 0)
                    run_ok = Lb.vb200_utterance_begin(first.ctypes.data, PROMPT_ROWS, noise0.ctypes.data, Wt + Kt) == 0
                    run_ok = run_ok and Lb.vb200_utterance_run(Wt) == 0
                except Exception:
                    run_ok = False
                ok = all_ok(run_ok)                          # also the barrier before the timed frames
                if ok:
                    torch.cuda.synchronize()
                    run_ok = Lb.vb200_utterance_run(Kt) == 0
                    tcodes = np.zeros((Wt + Kt, pkg.CODES), dtype=np.int32)
                    tdone, tend, tm = C.c_int(0), C.c_int(0), C.c_float(0.0)
                    run_ok = run_ok and Lb.vb200_utterance_end(tcodes.ctypes.data, C.byref(tdone), C.byref(tend),
                                                               C.byref(tm)) == 0 and tdone.value == Wt + Kt
                    tms = tm.value
                    ok = all_ok(run_ok)
            if ok:
                tval, tmax = aggregate(tms, Kt, dist, shared=True)
                tp_leg = {"parallelism": f"tp{world}", "ms_per_frame": tmax / Kt, "frames_per_s": tval, "steps": Kt,
                          "codes_equal_to_single_gpu": bool(np.array_equal(tcodes, codes[:Wt + Kt])) if rank == 0 else None,
                          "what": "one utterance, every decoder-layer GEMM sliced by output tiles over the ranks, "
                                  "results exchanged by peer stores over NVLink inside the GEMM epilogue"}
            else:
                tp_leg = {"error": f"tensor-parallel leg failed at stage '{stage}' on at least one rank"}
        except Exception as e:                              # never lose the main line to the extra leg
            tp_leg = {"error": f"{type(e).__name__}: {e}"}
        try:
            dist.barrier()                                   # nobody unmaps an arena a peer may still write to
            Lb.vb200_tp_close()
        except Exception:
            pass

    if tp:
        barrier()                                            # nobody unmaps an arena a peer may still write to
    if rank != 0:
        eng.close()
        if dist is not None:
            dist.destroy_process_group()
        return

    codec = None
    if not args.no_codec_leg:
        try:
            codec = codec_leg(pkg, eng, np.ascontiguousarray(codes[W:W + K]) if K <= 1024 else codes[W:W + 1024],
                              24 if world == 1 and not args.no_cpu_baseline else 0)
        except Exception as e:
            codec = {"error": f"{type(e).__name__}: {e}"}
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        r = cpu_reference(pkg, model, rows, first, seeds["noise"], 1, 6, args.cpu_budget)
        cpu = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample", "per_config")}
    eng.close()
    gpu_ref = None
    if world == 1 and not args.no_gpu_reference:
        gpu_ref = gpu_reference()                   # after eng.close(): the child has the GPU to itself

    line = {"metric": "frames_per_s", "value": value, "unit": "frames/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": total_ms / K, "higher_is_better": True, "scaling": "strong" if tp else "weak",
            "vs_baseline": None, "dtype": "f32 (BF16 weights, fp32 activations and accumulation)",
            "data": "synthetic", "config": config, "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "frames/s", "steps": Ke,
                    "h2d_bytes_per_step": 16 + 3072 * 4 + 36 * 4, "d2h_bytes_per_step": 176 + 3072 * 4},
            "gpu_launches": K * launches_per_frame, "roofline": roofline, "cpu_baseline": cpu,
            "gpu_reference": gpu_ref, "tp": tp_leg,
            "batched": batched, "streaming_decoder": streaming,
            "upload": upload, "codec": codec,
            "utterance": {"prefill_rows": PROMPT_ROWS, "prefill_ms": min(prefill_ms),
                          "first_frame_after_ms": min(prefill_ms) + 1000.0 * (1 if tp else world) / e2e_value,
                          "frames": 212,
                          "total_ms_at_measured_rates": min(prefill_ms) + 212 * 1000.0 * (1 if tp else world) / e2e_value,
                          "note": "tts_cuda_llm_prefill with host rows (wall clock, synchronous), then "
                                  "vb200_frame per frame; 212 frames = 16.96 s of audio at 12.5 frames/s"}}
    emit(line)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
