"""Host-side binding of libvoxtral_b200.so for tests and benchmarks.

The product is the C-ABI shared library (include/voxtral_b200.h and
include/voxtral_b200_ext.h). This module only loads it with ctypes and mirrors
the reference's call sequence (tts_cuda_init -> upload -> forward calls) in
Python. There is no fallback: a missing library or a missing sm_100 GPU raises.

The directory name is not a valid Python identifier; load it with
importlib (see tests/conftest.py: load_package()).
"""
import ctypes as C
import os
import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libvoxtral_b200.so")

DIM, DEC_LAYERS, AC_LAYERS = 3072, 26, 3
HEADS, KV_HEADS, HEAD_DIM, HIDDEN = 32, 8, 128, 9216
Q_DIM, KV_DIM = HEADS * HEAD_DIM, KV_HEADS * HEAD_DIM
VOCAB, ACOUSTIC_DIM, SEM_PADDED, SEM_VALID_END = 131072, 36, 8320, 8194
FLOW_STEPS, FSQ_LEVELS, CODES, CODE_END = 8, 21, 37, 1
AUDIO_ROWS = 8194 + 36 * 23
NORM_EPS, ROPE_THETA, CFG_ALPHA = 1e-5, 1e6, 1.2

u16p = C.POINTER(C.c_uint16)
f32p = C.POINTER(C.c_float)
i32p = C.POINTER(C.c_int)


class LayerWeights(C.Structure):
    _fields_ = [("wq", u16p), ("wk", u16p), ("wv", u16p), ("wo", u16p), ("attention_norm", f32p),
                ("w1", u16p), ("w2", u16p), ("w3", u16p), ("ffn_norm", f32p)]


class DecoderWeights(C.Structure):
    _fields_ = [("tok_embeddings", u16p), ("layers", LayerWeights * DEC_LAYERS), ("norm", f32p)]


class AcousticWeights(C.Structure):
    _fields_ = [("time_inv_freq", f32p), ("input_proj", u16p), ("time_proj", u16p), ("llm_proj", u16p),
                ("semantic_out", u16p), ("semantic_out_bias", f32p), ("acoustic_out", u16p), ("norm", f32p),
                ("layers", LayerWeights * AC_LAYERS)]


_lib = None


def lib():
    """The loaded shared library. Raises when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: run `python voxtral-tts.c_b200/build.py` "
                           "(there is no CPU fallback)")
    L = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    sig = {
        "tts_cuda_init": (C.c_int, [C.c_int]),
        "tts_cuda_upload_llm_weights": (C.c_int, [C.c_void_p]),
        "tts_cuda_upload_acoustic_weights": (C.c_int, [C.c_void_p]),
        "tts_cuda_free": (None, []),
        "tts_cuda_available": (C.c_int, []),
        "tts_cuda_linear_bf16": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
        "tts_cuda_rms_norm": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float]),
        "tts_cuda_apply_rope": (None, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]),
        "tts_cuda_compute_rope_freqs": (None, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float]),
        "tts_cuda_silu_mul": (None, [C.c_void_p, C.c_void_p, C.c_int]),
        "tts_cuda_add_inplace": (None, [C.c_void_p, C.c_void_p, C.c_int]),
        "tts_cuda_causal_attention_decode": (None, [C.c_void_p] * 4 + [C.c_int] * 4 + [C.c_float, C.c_int]),
        "tts_cuda_causal_attention_prefill": (None, [C.c_void_p] * 4 + [C.c_int] * 5 + [C.c_float]),
        "tts_cuda_bidirectional_attention": (None, [C.c_void_p] * 4 + [C.c_int] * 4 + [C.c_float]),
        "tts_cuda_embed_token": (None, [C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
        "tts_cuda_llm_forward": (None, [C.c_void_p, C.c_void_p, C.c_int]),
        "tts_cuda_llm_prefill": (None, [C.c_void_p, C.c_int, C.c_int]),
        "tts_cuda_predict_velocity": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float]),
        "tts_cuda_to_device": (None, [C.c_void_p, C.c_void_p, C.c_size_t]),
        "tts_cuda_to_host": (None, [C.c_void_p, C.c_void_p, C.c_size_t]),
        "tts_cuda_memset": (None, [C.c_void_p, C.c_int, C.c_size_t]),
        "tts_cuda_alloc": (C.c_void_p, [C.c_size_t]),
        "tts_cuda_free_ptr": (None, [C.c_void_p]),
        "tts_cuda_sync": (None, []),
        "vb200_frame": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
        "vb200_frame_chained": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
        "vb200_acoustic_frame": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
        "vb200_upload_audio_embed": (C.c_int, [C.c_void_p, C.c_int]),
        "vb200_prefill_prompt": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int]),
        "vb200_upload_stats": (None, [C.POINTER(C.c_double), C.POINTER(C.c_double)]),
        "vb200_codec_upload": (C.c_int, [C.c_void_p]),
        "vb200_codec_decode": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.POINTER(C.c_int)]),
        "vb200_codec_last_ms": (C.c_float, []),
        "vb200_utterance_begin": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int]),
        "vb200_utterance_run": (C.c_int, [C.c_int]),
        "vb200_batch_open": (C.c_int, [C.c_int, C.c_int, C.c_int]),
        "vb200_batch_prefill": (C.c_int, [C.c_int, C.c_void_p, C.c_int]),
        "vb200_batch_begin": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
        "vb200_batch_run": (C.c_int, [C.c_int]),
        "vb200_batch_end": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, f32p]),
        "vb200_batch_hidden": (C.c_int, [C.c_void_p]),
        "vb200_batch_launches_per_frame": (C.c_int, []),
        "vb200_batch_close": (None, []),
        "vb200_gemm_sweep": (C.c_int, [C.c_int, C.c_int, f32p, C.POINTER(C.c_double), i32p]),
        "vb200_frame_on_tensor_cores": (C.c_int, []),
        "vb200_tp_arena": (C.c_int, [C.c_int, C.c_int, C.c_void_p]),
        "vb200_tp_connect": (C.c_int, [C.c_void_p]),
        "vb200_tp_close": (None, []),
        "vb200_tp_plan": (C.c_int, [C.c_int, C.c_int, C.c_int, i32p]),
        "vb200_tc_gemm_probe": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, f32p, i32p]),
        "vb200_set_option": (C.c_int, [C.c_char_p, C.c_int]),
        "vb200_stream_step_ms": (C.c_int, [C.c_int, C.c_int, f32p, C.POINTER(C.c_double)]),
        "vb200_selftest_wait_expiry": (C.c_int, [C.c_int]),
        "vb200_stream_probe": (C.c_int, [C.c_int] * 5 + [f32p, C.POINTER(C.c_double)]),
        "vb200_frame_on_stream_kernel": (C.c_int, []),
        "vb200_utterance_engine_ms": (C.c_double, [i32p]),
        "vb200_utterance_end": (C.c_int, [C.c_void_p, i32p, i32p, f32p]),
        "vb200_kv_write": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
        "vb200_kv_read": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
        "vb200_tap_enable": (C.c_int, [C.c_int]),
        "vb200_tap_read": (C.c_int, [C.c_void_p]),
        "vb200_debug_gemv_plan": (C.c_int, [C.c_int] * 6 + [i32p]),
        "vb200_linear_bf16_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]),
        "vb200_linear_bf16_static_status": (C.c_int, []),
        "vb200_last_status": (C.c_int, []),
        "vb200_sm_count": (C.c_int, []),
        "vb200_engine_ms": (C.c_double, [C.c_int, i32p]),
        "vb200_synth_bf16": (None, [C.c_void_p, C.c_size_t, C.c_uint64, C.c_uint64, C.c_uint64, C.c_float]),
        "vb200_synth_f32": (None, [C.c_void_p, C.c_size_t, C.c_uint64, C.c_uint64, C.c_uint64, C.c_float, C.c_float]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


EXPORTED_SYMBOLS_REFERENCE = [
    "g_cuda", "tts_cuda_init", "tts_cuda_upload_llm_weights", "tts_cuda_upload_acoustic_weights",
    "tts_cuda_free", "tts_cuda_available", "tts_cuda_linear_bf16", "tts_cuda_rms_norm", "tts_cuda_apply_rope",
    "tts_cuda_compute_rope_freqs", "tts_cuda_silu_mul", "tts_cuda_add_inplace",
    "tts_cuda_causal_attention_decode", "tts_cuda_causal_attention_prefill",
    "tts_cuda_bidirectional_attention", "tts_cuda_embed_token", "tts_cuda_llm_forward", "tts_cuda_llm_prefill",
    "tts_cuda_predict_velocity", "tts_cuda_to_device", "tts_cuda_to_host", "tts_cuda_memset", "tts_cuda_alloc",
    "tts_cuda_free_ptr", "tts_cuda_sync",
]


class ConvWeights(C.Structure):
    """tts_conv_t (voxtral_tts.h:172-181)."""
    _fields_ = [("weight", C.c_void_p), ("bias", C.c_void_p), ("in_ch", C.c_int), ("out_ch", C.c_int),
                ("kernel", C.c_int), ("stride", C.c_int), ("is_transpose", C.c_int)]


class CodecLayerWeights(C.Structure):
    """tts_codec_layer_t (voxtral_tts.h:184-205)."""
    _fields_ = [(n, C.c_void_p) for n in ("wq", "wk", "wv", "wo", "q_norm", "k_norm", "attention_norm",
                                          "w1", "w2", "w3", "ffn_norm", "attn_scale", "ffn_scale")] + \
               [("window_size", C.c_int)]


class CodecWeights(C.Structure):
    """tts_codec_t (voxtral_tts.h:207-225)."""
    _fields_ = [("semantic_embedding", C.c_void_p), ("input_conv", ConvWeights),
                ("transformers", CodecLayerWeights * 8), ("stage_convs", ConvWeights * 4),
                ("output_proj", ConvWeights), ("alibi_slopes", C.c_float * 8)]


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


# --------------------------------------------------------------------------
# synthetic checkpoint (stands in for the real weights, which need the network)
# --------------------------------------------------------------------------
def stream_id(name):
    return zlib.crc32(name.encode())


_synth = None


def synth_lib():
    """The synthetic-tensor generator alone (lib/libvb_synth.so, plain C++, no CUDA): what the
    benchmark's CPU reference arm loads, so that it never maps the CUDA library."""
    global _synth
    if _synth is not None:
        return _synth
    path = os.path.join(HERE, "lib", "libvb_synth.so")
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing: run `python voxtral-tts.c_b200/build.py`")
    S = C.CDLL(path)
    S.vb200_synth_bf16.restype = None
    S.vb200_synth_bf16.argtypes = [C.c_void_p, C.c_size_t, C.c_uint64, C.c_uint64, C.c_uint64, C.c_float]
    S.vb200_synth_f32.restype = None
    S.vb200_synth_f32.argtypes = [C.c_void_p, C.c_size_t, C.c_uint64, C.c_uint64, C.c_uint64, C.c_float, C.c_float]
    S.vb200_randn_fill.restype = None
    S.vb200_randn_fill.argtypes = [C.POINTER(C.c_uint64), C.c_void_p, C.c_size_t]
    _synth = S
    return S


def randn(state, n):
    """n normals of the reference's generator from `state`; returns (values, new state)."""
    st = C.c_uint64(state)
    out = np.empty(n, dtype=np.float32)
    synth_lib().vb200_randn_fill(C.byref(st), _ptr(out), n)
    return out, st.value


def synth_bf16(shape, seed, name, sigma=0.02, first=0):
    out = np.empty(shape, dtype=np.uint16)
    synth_lib().vb200_synth_bf16(_ptr(out), out.size, seed, stream_id(name), first, sigma)
    return out


def synth_f32(shape, seed, name, mean=0.0, sigma=1.0, first=0):
    out = np.empty(shape, dtype=np.float32)
    synth_lib().vb200_synth_f32(_ptr(out), out.size, seed, stream_id(name), first, mean, sigma)
    return out


class SynthModel:
    """Seeded random-init weights with the tensor names and shapes of the real
    checkpoint (voxtral_tts_llm.c:50-95, voxtral_tts_acoustic.c:48-111,
    voxtral_tts_voice.c:257-283). Matrices: BF16 ~N(0, 0.02). Norm gains:
    1 + N(0, 0.02). The 131072-row token table is produced row by row on demand."""

    def __init__(self, seed=1234, decoder=True, acoustic=True, semantic_bias=False, audio_table=True,
                 dec_layers=DEC_LAYERS):
        self.seed = seed
        self.t = {}
        self.dec_layers = dec_layers
        if decoder:
            for i in range(DEC_LAYERS):
                # layers beyond dec_layers alias layer 0 (small-memory smoke runs only)
                src = i if i < dec_layers else 0
                self._layer(f"layers.{i}", f"layers.{src}")
            self.t["norm.weight"] = synth_f32(DIM, seed, "norm.weight", 1.0, 0.02)
        if acoustic:
            p = "acoustic_transformer"
            for i in range(AC_LAYERS):
                self._layer(f"{p}.layers.{i}", f"{p}.layers.{i}")
            self.t[f"{p}.input_projection.weight"] = synth_bf16((DIM, ACOUSTIC_DIM), seed, f"{p}.input_projection.weight")
            self.t[f"{p}.time_projection.weight"] = synth_bf16((DIM, DIM), seed, f"{p}.time_projection.weight")
            self.t[f"{p}.llm_projection.weight"] = synth_bf16((DIM, DIM), seed, f"{p}.llm_projection.weight")
            self.t[f"{p}.semantic_codebook_output.weight"] = synth_bf16(
                (SEM_PADDED, DIM), seed, f"{p}.semantic_codebook_output.weight")
            self.t[f"{p}.acoustic_codebook_output.weight"] = synth_bf16(
                (ACOUSTIC_DIM, DIM), seed, f"{p}.acoustic_codebook_output.weight")
            self.t[f"{p}.norm.weight"] = synth_f32(DIM, seed, f"{p}.norm.weight", 1.0, 0.02)
            if semantic_bias:
                self.t[f"{p}.semantic_codebook_output.bias"] = synth_f32(
                    SEM_PADDED, seed, f"{p}.semantic_codebook_output.bias", 0.0, 0.5)
            # exp(-ln(10000) * i / 1536) in fp32, voxtral_tts_acoustic.c:49-57
            i = np.arange(DIM // 2, dtype=np.float32)
            theta = np.float32(10000.0)
            self.t[f"{p}.time_embedding.inv_freq"] = np.exp(
                (-np.log(theta, dtype=np.float32) * i / np.float32(DIM // 2)).astype(np.float32)).astype(np.float32)
        if audio_table:
            n = "mm_audio_embeddings.audio_codebook_embeddings.embeddings.weight"
            self.t[n] = synth_bf16((AUDIO_ROWS, DIM), seed, n)

    def _layer(self, name, src):
        s = self.seed
        if src != name:
            for k in ("attention.wq", "attention.wk", "attention.wv", "attention.wo", "feed_forward.w1",
                      "feed_forward.w2", "feed_forward.w3", "attention_norm", "ffn_norm"):
                self.t[f"{name}.{k}.weight"] = self.t[f"{src}.{k}.weight"]
            return
        self.t[f"{name}.attention.wq.weight"] = synth_bf16((Q_DIM, DIM), s, f"{name}.attention.wq.weight")
        self.t[f"{name}.attention.wk.weight"] = synth_bf16((KV_DIM, DIM), s, f"{name}.attention.wk.weight")
        self.t[f"{name}.attention.wv.weight"] = synth_bf16((KV_DIM, DIM), s, f"{name}.attention.wv.weight")
        self.t[f"{name}.attention.wo.weight"] = synth_bf16((DIM, Q_DIM), s, f"{name}.attention.wo.weight")
        self.t[f"{name}.feed_forward.w1.weight"] = synth_bf16((HIDDEN, DIM), s, f"{name}.feed_forward.w1.weight")
        self.t[f"{name}.feed_forward.w2.weight"] = synth_bf16((DIM, HIDDEN), s, f"{name}.feed_forward.w2.weight")
        self.t[f"{name}.feed_forward.w3.weight"] = synth_bf16((HIDDEN, DIM), s, f"{name}.feed_forward.w3.weight")
        self.t[f"{name}.attention_norm.weight"] = synth_f32(DIM, s, f"{name}.attention_norm.weight", 1.0, 0.02)
        self.t[f"{name}.ffn_norm.weight"] = synth_f32(DIM, s, f"{name}.ffn_norm.weight", 1.0, 0.02)

    def token_rows(self, ids):
        """fp32 embedding rows of the token table (tts_embed_token_bf16,
        voxtral_tts_kernels.c:55-59) for the given ids."""
        out = np.empty((len(ids), DIM), dtype=np.float32)
        name = "mm_audio_embeddings.tok_embeddings.weight"
        for r, tid in enumerate(ids):
            row = synth_bf16(DIM, self.seed, name, first=int(tid) * DIM)
            out[r] = (row.astype(np.uint32) << 16).view(np.float32)
        return out

    def _fill_layer(self, L, name):
        g = self.t
        L.wq = g[f"{name}.attention.wq.weight"].ctypes.data_as(u16p)
        L.wk = g[f"{name}.attention.wk.weight"].ctypes.data_as(u16p)
        L.wv = g[f"{name}.attention.wv.weight"].ctypes.data_as(u16p)
        L.wo = g[f"{name}.attention.wo.weight"].ctypes.data_as(u16p)
        L.w1 = g[f"{name}.feed_forward.w1.weight"].ctypes.data_as(u16p)
        L.w2 = g[f"{name}.feed_forward.w2.weight"].ctypes.data_as(u16p)
        L.w3 = g[f"{name}.feed_forward.w3.weight"].ctypes.data_as(u16p)
        L.attention_norm = g[f"{name}.attention_norm.weight"].ctypes.data_as(f32p)
        L.ffn_norm = g[f"{name}.ffn_norm.weight"].ctypes.data_as(f32p)

    def token_table(self):
        """The whole 131072-row token table (0.8 GB), generated once on first use."""
        name = "mm_audio_embeddings.tok_embeddings.weight"
        if getattr(self, "_tok", None) is None:
            self._tok = synth_bf16((VOCAB, DIM), self.seed, name)
        return self._tok

    def decoder_struct(self, token_table=False):
        w = DecoderWeights()
        for i in range(DEC_LAYERS):
            self._fill_layer(w.layers[i], f"layers.{i}")
        w.norm = self.t["norm.weight"].ctypes.data_as(f32p)
        if token_table:
            w.tok_embeddings = self.token_table().ctypes.data_as(u16p)
        return w

    def acoustic_struct(self):
        p = "acoustic_transformer"
        w = AcousticWeights()
        g = self.t
        w.time_inv_freq = g[f"{p}.time_embedding.inv_freq"].ctypes.data_as(f32p)
        w.input_proj = g[f"{p}.input_projection.weight"].ctypes.data_as(u16p)
        w.time_proj = g[f"{p}.time_projection.weight"].ctypes.data_as(u16p)
        w.llm_proj = g[f"{p}.llm_projection.weight"].ctypes.data_as(u16p)
        w.semantic_out = g[f"{p}.semantic_codebook_output.weight"].ctypes.data_as(u16p)
        b = g.get(f"{p}.semantic_codebook_output.bias")
        if b is not None:
            w.semantic_out_bias = b.ctypes.data_as(f32p)
        w.acoustic_out = g[f"{p}.acoustic_codebook_output.weight"].ctypes.data_as(u16p)
        w.norm = g[f"{p}.norm.weight"].ctypes.data_as(f32p)
        for i in range(AC_LAYERS):
            self._fill_layer(w.layers[i], f"{p}.layers.{i}")
        return w

    def audio_table(self):
        return self.t["mm_audio_embeddings.audio_codebook_embeddings.embeddings.weight"]

    def write_safetensors(self, path, token_table=True):
        """Writes the tensors as a safetensors file the reference's reader accepts
        (voxtral_tts_safetensors.c:71-283: 8-byte little-endian header length, JSON with dtype /
        shape / data_offsets per tensor, then the raw data; matrices BF16, gains F32), so that
        tts_llm_load / tts_acoustic_load / tts_audio_embed_load can be run on the synthetic
        checkpoint. The 131072-row token table (0.8 GB) is generated on the way out."""
        import json
        import struct
        items = [(k, v) for k, v in self.t.items()]
        header, off = {}, 0
        tok_name = "mm_audio_embeddings.tok_embeddings.weight"
        sizes = []
        for name, a in items:
            dt = "BF16" if a.dtype == np.uint16 else "F32"
            n = a.size * a.dtype.itemsize
            header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + n]}
            sizes.append(n)
            off += n
        if token_table:
            n = VOCAB * DIM * 2
            header[tok_name] = {"dtype": "BF16", "shape": [VOCAB, DIM], "data_offsets": [off, off + n]}
            off += n
        blob = json.dumps(header, separators=(",", ":")).encode()
        blob += b" " * ((8 - len(blob) % 8) % 8)
        with open(path, "wb") as f:
            f.write(struct.pack("<Q", len(blob)))
            f.write(blob)
            for _, a in items:
                np.ascontiguousarray(a).tofile(f)
            if token_table:
                rows = 8192
                for r0 in range(0, VOCAB, rows):
                    synth_bf16((rows, DIM), self.seed, tok_name, first=r0 * DIM).tofile(f)
        return path


# --------------------------------------------------------------------------
# thin object over the C ABI (one context per process, like the reference)
# --------------------------------------------------------------------------
class SynthCodec:
    """Seeded random-init codec-decoder weights in the form tts_codec_load leaves them
    (voxtral_tts_codec.c:177-262): transformer matrices BF16-representable fp32 (the checkpoint
    stores BF16, the loader widens), effective (weight-normed) convolution weights plain fp32,
    semantic embedding ~N(0, 1), layer scales 0.5 + N(0, 0.1)."""

    CODEC_DIM, CODEC_HIDDEN, EMBED, PATCH = 1024, 4096, 292, 240

    def __init__(self, seed=77, qk_norm=True, layer_scale=True, conv_bias=True):
        D, Hd = self.CODEC_DIM, self.CODEC_HIDDEN
        self.seed = seed
        t = self.t = {}

        def mat(name, shape):
            # BF16 values widened to fp32: exactly what safetensors_get_f32 returns for a BF16 tensor
            b = synth_bf16(shape, seed, name, 0.02)
            return (b.astype(np.uint32) << 16).view(np.float32)

        t["semantic_embedding"] = synth_f32((8192, 256), seed, "codec.semantic_embedding", 0.0, 1.0)

        def conv(name, shape, fan_in, n_bias):
            t[f"{name}.weight"] = synth_f32(shape, seed, f"{name}.weight", 0.0, 1.0 / np.sqrt(fan_in))
            t[f"{name}.bias"] = synth_f32(n_bias, seed, f"{name}.bias", 0.0, 0.05) if conv_bias else None

        conv("input_conv", (D, self.EMBED, 3), self.EMBED * 3, D)
        for s_ in range(3):
            conv(f"up{s_}", (D, D, 4), D * 2, D)                 # [in_ch, out_ch, kernel]
        conv("output_proj", (self.PATCH, D, 7), D * 7, self.PATCH)
        for l in range(8):
            n = f"codec.layers.{l}"
            for k, shape in (("wq", (D, D)), ("wk", (D, D)), ("wv", (D, D)), ("wo", (D, D)),
                             ("w1", (Hd, D)), ("w2", (D, Hd)), ("w3", (Hd, D))):
                t[f"{n}.{k}"] = mat(f"{n}.{k}", shape)
            t[f"{n}.attention_norm"] = synth_f32(D, seed, f"{n}.attention_norm", 1.0, 0.02)
            t[f"{n}.ffn_norm"] = synth_f32(D, seed, f"{n}.ffn_norm", 1.0, 0.02)
            t[f"{n}.q_norm"] = synth_f32(D, seed, f"{n}.q_norm", 1.0, 0.05) if qk_norm else None
            t[f"{n}.k_norm"] = synth_f32(D, seed, f"{n}.k_norm", 1.0, 0.05) if qk_norm else None
            t[f"{n}.attn_scale"] = synth_f32(D, seed, f"{n}.attn_scale", 0.5, 0.1) if layer_scale else None
            t[f"{n}.ffn_scale"] = synth_f32(D, seed, f"{n}.ffn_scale", 0.5, 0.1) if layer_scale else None

    def write_safetensors(self, path):
        """The codec tensors in checkpoint form, under the names tts_codec_load reads
        (voxtral_tts_codec.c:177-262): embedding_sum / cluster_usage, the input and the three
        upsampling convolutions weight-normed (original0 = g, original1 = v), the output
        convolution plain, transformer matrices BF16, vectors F32. The effective weights a loader
        derives from this file are NOT the arrays of this object (g and v are fresh draws)."""
        import json
        import struct
        t, seed, D = self.t, self.seed, self.CODEC_DIM
        out = {}
        usage = np.abs(synth_f32(8192, seed, "codec.cluster_usage", 1.0, 0.5)).astype(np.float32)
        usage[:3] = (0.0, 1e-7, 2.0)                                   # the clamp at 1e-5
        out["audio_tokenizer.quantizer.semantic_codebook.cluster_usage"] = usage
        # sums chosen so that sum / max(usage, 1e-5) is again ~N(0, 1)
        out["audio_tokenizer.quantizer.semantic_codebook.embedding_sum"] = (
            t["semantic_embedding"] * np.maximum(usage, np.float32(1e-5))[:, None]).astype(np.float32)

        def wn(prefix, name, lead):
            v = t[f"{name}.weight"]
            out[f"{prefix}.conv.parametrizations.weight.original1"] = v
            out[f"{prefix}.conv.parametrizations.weight.original0"] = np.abs(
                synth_f32((lead, 1, 1), seed, f"{prefix}.g", 1.0, 0.2)).astype(np.float32)
            if t[f"{name}.bias"] is not None:
                out[f"{prefix}.conv.bias"] = t[f"{name}.bias"]

        B = "audio_tokenizer.decoder_blocks"
        wn(f"{B}.0", "input_conv", D)
        for s_ in range(3):
            wn(f"{B}.{2 + 2 * s_}", f"up{s_}", D)
        out["audio_tokenizer.output_proj.conv.weight"] = t["output_proj.weight"]
        if t["output_proj.bias"] is not None:
            out["audio_tokenizer.output_proj.conv.bias"] = t["output_proj.bias"]
        names = {"wq": "attention.wq.weight", "wk": "attention.wk.weight", "wv": "attention.wv.weight",
                 "wo": "attention.wo.weight", "w1": "feed_forward.w1.weight", "w2": "feed_forward.w2.weight",
                 "w3": "feed_forward.w3.weight", "q_norm": "attention.q_norm.weight", "k_norm": "attention.k_norm.weight",
                 "attention_norm": "attention_norm.weight", "ffn_norm": "ffn_norm.weight",
                 "attn_scale": "attention_scale", "ffn_scale": "ffn_scale"}
        for l in range(8):
            for k, full in names.items():
                a = t[f"codec.layers.{l}.{k}"]
                if a is None:
                    continue
                if a.ndim == 2:                                        # back to the BF16 the values came from
                    a = (a.view(np.uint32) >> 16).astype(np.uint16)
                out[f"{B}.{1 + 2 * (l // 2)}.layers.{l % 2}.{full}"] = a
        header, off = {}, 0
        for name, a in out.items():
            n = a.size * a.dtype.itemsize
            header[name] = {"dtype": "BF16" if a.dtype == np.uint16 else "F32", "shape": list(a.shape),
                            "data_offsets": [off, off + n]}
            off += n
        blob = json.dumps(header, separators=(",", ":")).encode()
        blob += b" " * ((8 - len(blob) % 8) % 8)
        with open(path, "wb") as f:
            f.write(struct.pack("<Q", len(blob)))
            f.write(blob)
            for a in out.values():
                np.ascontiguousarray(a).tofile(f)
        return path

    def struct(self):
        """A CodecWeights (== tts_codec_t) whose pointers reference this object's arrays."""
        t, w = self.t, CodecWeights()
        w._owner = self                                           # the arrays live as long as the struct
        D = self.CODEC_DIM

        def p(a):
            return None if a is None else _ptr(a)

        def conv(dst, name, in_ch, out_ch, kernel, stride, transpose):
            dst.weight, dst.bias = p(t[f"{name}.weight"]), p(t[f"{name}.bias"])
            dst.in_ch, dst.out_ch, dst.kernel, dst.stride, dst.is_transpose = in_ch, out_ch, kernel, stride, transpose

        w.semantic_embedding = p(t["semantic_embedding"])
        conv(w.input_conv, "input_conv", self.EMBED, D, 3, 1, 0)
        for s_ in range(3):
            conv(w.stage_convs[s_], f"up{s_}", D, D, 4, 2, 1)
        conv(w.output_proj, "output_proj", D, self.PATCH, 7, 1, 0)
        windows = (2, 4, 8, 16)                                   # voxtral_tts_codec.c:223
        for l in range(8):
            n, L = f"codec.layers.{l}", w.transformers[l]
            for k in ("wq", "wk", "wv", "wo", "q_norm", "k_norm", "attention_norm", "w1", "w2", "w3", "ffn_norm",
                      "attn_scale", "ffn_scale"):
                setattr(L, k, p(t[f"{n}.{k}"]))
            L.window_size = windows[l // 2]
        for h in range(8):
            w.alibi_slopes[h] = float(np.float32(2.0) ** np.float32(-8.0 / 8.0 * (h + 1)))   # voxtral_tts_codec.c:204-205
        return w


class Engine:
    def __init__(self, kv_cache_max=512):
        L = lib()
        if L.tts_cuda_init(kv_cache_max) != 0:
            raise RuntimeError("tts_cuda_init failed: an sm_100 GPU is required (no CPU fallback)")
        self.L = L
        self.kv_max = kv_cache_max
        self._keep = []

    def upload(self, model, decoder=True, acoustic=True, audio_table=False, token_table=False):
        if decoder:
            w = model.decoder_struct(token_table=token_table)
            self._keep.append(w)
            if self.L.tts_cuda_upload_llm_weights(C.byref(w)) != 0:
                raise RuntimeError("tts_cuda_upload_llm_weights failed")
        if acoustic:
            w = model.acoustic_struct()
            self._keep.append(w)
            if self.L.tts_cuda_upload_acoustic_weights(C.byref(w)) != 0:
                raise RuntimeError("tts_cuda_upload_acoustic_weights failed")
        if audio_table:
            t = model.audio_table()
            if self.L.vb200_upload_audio_embed(_ptr(t), t.shape[0]) != 0:
                raise RuntimeError("vb200_upload_audio_embed failed")

    def _ok(self, what, rc=0):
        if rc != 0 or self.L.vb200_last_status() != 0:
            raise RuntimeError(f"{what} failed (rc={rc}, device status={self.L.vb200_last_status()})")

    def llm_forward(self, embed, pos):
        embed = np.ascontiguousarray(embed, dtype=np.float32)
        out = np.empty(DIM, dtype=np.float32)
        self.L.tts_cuda_llm_forward(_ptr(out), _ptr(embed), int(pos))
        self._ok("tts_cuda_llm_forward")
        return out

    def prefill(self, embeds, start_pos=0):
        embeds = np.ascontiguousarray(embeds, dtype=np.float32)
        self.L.tts_cuda_llm_prefill(_ptr(embeds), embeds.shape[0], int(start_pos))
        self._ok("tts_cuda_llm_prefill")

    def codec_upload(self, codec):
        """vb200_codec_upload of a SynthCodec (or anything with .struct())."""
        w = codec.struct()
        self._keep.append((codec, w))
        if self.L.vb200_codec_upload(C.byref(w)) != 0:
            raise RuntimeError("vb200_codec_upload failed")

    def codec_decode(self, codes):
        """codes [n_frames, 37] -> (waveform float32 [n_frames * 1920], device ms)."""
        codes = np.ascontiguousarray(codes, dtype=np.int32).reshape(-1, CODES)
        out = np.empty(codes.shape[0] * 1920, dtype=np.float32)
        n = C.c_int(0)
        if self.L.vb200_codec_decode(_ptr(codes), codes.shape[0], _ptr(out), out.size, C.byref(n)) != 0:
            raise RuntimeError(f"vb200_codec_decode failed (device status={self.L.vb200_last_status()})")
        return out[:n.value], self.L.vb200_codec_last_ms()

    def upload_stats(self):
        """(seconds spent inside the weight-upload calls, bytes copied host -> device) so far."""
        s, b = C.c_double(0.0), C.c_double(0.0)
        self.L.vb200_upload_stats(C.byref(s), C.byref(b))
        return s.value, b.value

    def prefill_prompt(self, text_ids, voice_bf16, start_pos=0):
        """vb200_prefill_prompt: returns the number of prompt rows."""
        ids = np.ascontiguousarray(text_ids, dtype=np.int32)
        voice = np.ascontiguousarray(voice_bf16, dtype=np.uint16).reshape(-1, DIM)
        n = self.L.vb200_prefill_prompt(_ptr(ids) if ids.size else None, ids.size, _ptr(voice) if voice.size else None,
                                        voice.shape[0], int(start_pos))
        if n < 0:
            raise RuntimeError(f"vb200_prefill_prompt failed (device status={self.L.vb200_last_status()})")
        return n

    def predict_velocity(self, x_t, hidden, t):
        x_t = np.ascontiguousarray(x_t, dtype=np.float32)
        hidden = np.ascontiguousarray(hidden, dtype=np.float32)
        out = np.empty(ACOUSTIC_DIM, dtype=np.float32)
        self.L.tts_cuda_predict_velocity(_ptr(out), _ptr(x_t), _ptr(hidden), float(t))
        self._ok("tts_cuda_predict_velocity")
        return out

    def acoustic_frame(self, hidden, noise):
        hidden = np.ascontiguousarray(hidden, dtype=np.float32)
        noise = np.ascontiguousarray(noise, dtype=np.float32)
        codes = np.empty(CODES, dtype=np.int32)
        latent = np.empty(ACOUSTIC_DIM, dtype=np.float32)
        self._ok("vb200_acoustic_frame", self.L.vb200_acoustic_frame(_ptr(hidden), _ptr(noise), _ptr(codes), _ptr(latent)))
        return codes, latent

    def frame(self, embed, noise, pos, want_hidden=True):
        noise = np.ascontiguousarray(noise, dtype=np.float32)
        codes = np.empty(CODES, dtype=np.int32)
        hidden = np.empty(DIM, dtype=np.float32) if want_hidden else None
        hp = _ptr(hidden) if want_hidden else None
        if embed is None:
            rc = self.L.vb200_frame_chained(_ptr(noise), int(pos), hp, _ptr(codes))
        else:
            embed = np.ascontiguousarray(embed, dtype=np.float32)
            rc = self.L.vb200_frame(_ptr(embed), _ptr(noise), int(pos), hp, _ptr(codes))
        self._ok("vb200_frame", rc)
        return codes, hidden

    def utterance(self, first_embed, start_pos, noise, n_frames=None, batch=None):
        """Device-resident frame loop. Returns (codes [frames,37], hit_end, device_ms)."""
        noise = np.ascontiguousarray(noise, dtype=np.float32).reshape(-1, ACOUSTIC_DIM)
        n_frames = noise.shape[0] if n_frames is None else n_frames
        first_embed = np.ascontiguousarray(first_embed, dtype=np.float32)
        self._ok("vb200_utterance_begin",
                 self.L.vb200_utterance_begin(_ptr(first_embed), int(start_pos), _ptr(noise), n_frames))
        self._ok("vb200_utterance_run", self.L.vb200_utterance_run(n_frames if batch is None else batch))
        codes = np.zeros((n_frames, CODES), dtype=np.int32)
        done, end, ms = C.c_int(0), C.c_int(0), C.c_float(0.0)
        self._ok("vb200_utterance_end",
                 self.L.vb200_utterance_end(_ptr(codes), C.byref(done), C.byref(end), C.byref(ms)))
        return codes[:done.value], bool(end.value), ms.value

    def batch(self, prompts, first_embeds, noise, kv_max=None):
        """Decodes len(prompts) utterances in lock step. prompts: list of [rows, 3072] prompt
        embeddings; first_embeds [n, 3072]; noise [n, frames, 36]. Returns (codes list of
        [frames_done, 37], hit_end list, hidden [n, 3072], device_ms)."""
        n = len(prompts)
        noise = np.ascontiguousarray(noise, dtype=np.float32).reshape(n, -1, ACOUSTIC_DIM)
        frames = noise.shape[1]
        first_embeds = np.ascontiguousarray(first_embeds, dtype=np.float32).reshape(n, DIM)
        if kv_max is None:
            kv_max = max(p.shape[0] for p in prompts) + frames + 1
        self._ok("vb200_batch_open", self.L.vb200_batch_open(n, int(kv_max), frames))
        try:
            start = np.zeros(n, dtype=np.int32)
            for u, p in enumerate(prompts):
                p = np.ascontiguousarray(p, dtype=np.float32).reshape(-1, DIM)
                self._ok("vb200_batch_prefill", self.L.vb200_batch_prefill(u, _ptr(p), p.shape[0]))
                start[u] = p.shape[0]
            self._ok("vb200_batch_begin", self.L.vb200_batch_begin(_ptr(first_embeds), _ptr(start), _ptr(noise)))
            self._ok("vb200_batch_run", self.L.vb200_batch_run(frames))
            codes = np.zeros((n, frames, CODES), dtype=np.int32)
            done = np.zeros(n, dtype=np.int32)
            end = np.zeros(n, dtype=np.int32)
            ms = C.c_float(0.0)
            self._ok("vb200_batch_end", self.L.vb200_batch_end(_ptr(codes), _ptr(done), _ptr(end), C.byref(ms)))
            hidden = np.zeros((n, DIM), dtype=np.float32)
            self._ok("vb200_batch_hidden", self.L.vb200_batch_hidden(_ptr(hidden)))
        finally:
            self.L.vb200_batch_close()
        return [codes[u, :done[u]] for u in range(n)], [bool(e) for e in end], hidden, ms.value

    def kv_write(self, layer, pos0, k_rows, v_rows):
        k_rows = np.ascontiguousarray(k_rows, dtype=np.float32)
        v_rows = np.ascontiguousarray(v_rows, dtype=np.float32)
        self._ok("vb200_kv_write", self.L.vb200_kv_write(layer, pos0, k_rows.shape[0], _ptr(k_rows), _ptr(v_rows)))

    def kv_read(self, layer, pos0, n):
        k = np.empty((n, KV_DIM), dtype=np.float32)
        v = np.empty((n, KV_DIM), dtype=np.float32)
        self._ok("vb200_kv_read", self.L.vb200_kv_read(layer, pos0, n, _ptr(k), _ptr(v)))
        return k, v

    def tap(self, on=True):
        self._ok("vb200_tap_enable", self.L.vb200_tap_enable(1 if on else 0))

    def tap_read(self):
        out = np.empty((DEC_LAYERS, 2, DIM), dtype=np.float32)
        self._ok("vb200_tap_read", self.L.vb200_tap_read(_ptr(out)))
        return out

    def engine_ms(self, reset=False):
        n = C.c_int(0)
        ms = self.L.vb200_engine_ms(1 if reset else 0, C.byref(n))
        return ms, n.value

    def close(self):
        self.L.tts_cuda_free()


class DeviceBuffer:
    """A tts_cuda_alloc'd buffer (for the single-op entry points)."""

    def __init__(self, array=None, nbytes=None):
        L = lib()
        self.L = L
        if array is not None:
            array = np.ascontiguousarray(array)
            nbytes = array.nbytes
        self.nbytes = max(int(nbytes), 4)
        self.ptr = L.tts_cuda_alloc(self.nbytes)
        if not self.ptr:
            raise RuntimeError("tts_cuda_alloc failed")
        if array is not None and array.nbytes:
            L.tts_cuda_to_device(self.ptr, _ptr(array), array.nbytes)

    def get(self, shape, dtype=np.float32):
        out = np.empty(shape, dtype=dtype)
        self.L.tts_cuda_sync()
        if out.nbytes:
            self.L.tts_cuda_to_host(_ptr(out), self.ptr, out.nbytes)
        return out

    def free(self):
        if self.ptr:
            self.L.tts_cuda_free_ptr(self.ptr)
            self.ptr = None
