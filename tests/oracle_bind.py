"""ctypes bindings of the CPU checkers (test infrastructure only).

Oracle  -> oracle/liboracle.so, the independent restatement (oracle/vox_oracle.c)
Ref     -> oracle/_ref/libvoxref_{noblas,blas}.so, the reference's own CPU sources
           behind oracle/ref_harness.c
"""
import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")

u16p = C.POINTER(C.c_uint16)
f32p = C.POINTER(C.c_float)

DIM, DEC_LAYERS, AC_LAYERS = 3072, 26, 3
HEADS, KV_HEADS, HEAD_DIM, HIDDEN = 32, 8, 128, 9216
KV_DIM = KV_HEADS * HEAD_DIM


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class Dims(C.Structure):
    _fields_ = [("dim", C.c_int), ("n_layers", C.c_int), ("n_heads", C.c_int), ("n_kv_heads", C.c_int),
                ("head_dim", C.c_int), ("hidden", C.c_int), ("eps", C.c_float), ("rope_theta", C.c_float)]


class Layer(C.Structure):
    _fields_ = [("wq", u16p), ("wk", u16p), ("wv", u16p), ("wo", u16p), ("w1", u16p), ("w2", u16p), ("w3", u16p),
                ("attn_norm", f32p), ("ffn_norm", f32p)]


class Decoder(C.Structure):
    _fields_ = [("d", Dims), ("layers", C.POINTER(Layer)), ("final_norm", f32p)]


class Acoustic(C.Structure):
    _fields_ = [("d", Dims), ("layers", C.POINTER(Layer)), ("final_norm", f32p), ("time_inv_freq", f32p),
                ("input_proj", u16p), ("time_proj", u16p), ("llm_proj", u16p), ("semantic_out", u16p),
                ("semantic_bias", f32p), ("acoustic_out", u16p), ("n_acoustic", C.c_int), ("sem_padded", C.c_int),
                ("sem_valid_end", C.c_int), ("flow_steps", C.c_int), ("fsq_levels", C.c_int),
                ("cfg_alpha", C.c_float), ("noise_scale", C.c_float)]


def _layer_from(t, name):
    L = Layer()
    L.wq = t[f"{name}.attention.wq.weight"].ctypes.data_as(u16p)
    L.wk = t[f"{name}.attention.wk.weight"].ctypes.data_as(u16p)
    L.wv = t[f"{name}.attention.wv.weight"].ctypes.data_as(u16p)
    L.wo = t[f"{name}.attention.wo.weight"].ctypes.data_as(u16p)
    L.w1 = t[f"{name}.feed_forward.w1.weight"].ctypes.data_as(u16p)
    L.w2 = t[f"{name}.feed_forward.w2.weight"].ctypes.data_as(u16p)
    L.w3 = t[f"{name}.feed_forward.w3.weight"].ctypes.data_as(u16p)
    L.attn_norm = t[f"{name}.attention_norm.weight"].ctypes.data_as(f32p)
    L.ffn_norm = t[f"{name}.ffn_norm.weight"].ctypes.data_as(f32p)
    return L


class Oracle:
    def __init__(self):
        path = os.path.join(ORACLE_DIR, "liboracle.so")
        self.L = C.CDLL(path)
        L = self.L
        L.vox_randn.restype = C.c_float
        vp = C.c_void_p
        L.vox_linear_bf16.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int, C.c_int]
        L.vox_rms_norm.argtypes = [vp, vp, vp, C.c_int, C.c_int, C.c_float]
        L.vox_rope_table.argtypes = [vp, vp, C.c_int, C.c_int, C.c_float]
        L.vox_rope_apply.argtypes = [vp, vp, C.c_int, C.c_int, C.c_int]
        L.vox_silu_mul.argtypes = [vp, vp, C.c_int]
        L.vox_attention_causal.argtypes = [vp] * 4 + [C.c_int] * 5 + [C.c_float, C.c_int]
        L.vox_attention_full.argtypes = [vp] * 4 + [C.c_int] * 4 + [C.c_float]
        L.vox_llm_forward.argtypes = [vp, vp, vp, C.c_int, C.c_int, vp, vp, vp]
        L.vox_llm_prefill.argtypes = [vp, vp, vp, C.c_int, C.c_int, vp, C.c_int, vp]
        L.vox_predict_velocity.argtypes = [vp, vp, vp, C.c_float, vp]
        L.vox_acoustic_forward.argtypes = [vp, vp, vp, vp, vp, vp]
        L.vox_audio_embed.argtypes = [vp, C.c_int, vp, C.c_int, C.c_int, C.c_int, vp]
        L.vox_randn_fill.argtypes = [vp, vp, C.c_int]
        L.vox_rng_seed.argtypes = [vp, C.c_uint64]
        L.vox_time_embedding.argtypes = [vp, vp, C.c_float, C.c_int]
        self._keep = []

    # ---- model structs ----
    def decoder(self, model, n_layers=DEC_LAYERS, dims=None):
        arr = (Layer * n_layers)(*[_layer_from(model.t, f"layers.{i}") for i in range(n_layers)])
        d = Decoder()
        d.d = dims or Dims(DIM, n_layers, HEADS, KV_HEADS, HEAD_DIM, HIDDEN, 1e-5, 1e6)
        d.layers = C.cast(arr, C.POINTER(Layer))
        d.final_norm = model.t["norm.weight"].ctypes.data_as(f32p)
        self._keep.append((arr, model))
        return d

    def acoustic(self, model):
        p = "acoustic_transformer"
        arr = (Layer * AC_LAYERS)(*[_layer_from(model.t, f"{p}.layers.{i}") for i in range(AC_LAYERS)])
        a = Acoustic()
        a.d = Dims(DIM, AC_LAYERS, HEADS, KV_HEADS, HEAD_DIM, HIDDEN, 1e-5, 0.0)
        a.layers = C.cast(arr, C.POINTER(Layer))
        t = model.t
        a.final_norm = t[f"{p}.norm.weight"].ctypes.data_as(f32p)
        a.time_inv_freq = t[f"{p}.time_embedding.inv_freq"].ctypes.data_as(f32p)
        a.input_proj = t[f"{p}.input_projection.weight"].ctypes.data_as(u16p)
        a.time_proj = t[f"{p}.time_projection.weight"].ctypes.data_as(u16p)
        a.llm_proj = t[f"{p}.llm_projection.weight"].ctypes.data_as(u16p)
        a.semantic_out = t[f"{p}.semantic_codebook_output.weight"].ctypes.data_as(u16p)
        b = t.get(f"{p}.semantic_codebook_output.bias")
        if b is not None:
            a.semantic_bias = b.ctypes.data_as(f32p)
        a.acoustic_out = t[f"{p}.acoustic_codebook_output.weight"].ctypes.data_as(u16p)
        a.n_acoustic, a.sem_padded, a.sem_valid_end = 36, 8320, 8194
        a.flow_steps, a.fsq_levels, a.cfg_alpha, a.noise_scale = 8, 21, 1.2, 1.0
        self._keep.append((arr, model))
        return a

    # ---- primitives ----
    def linear(self, x, W, bias=None):
        x = np.ascontiguousarray(x, dtype=np.float32)
        x2 = x.reshape(-1, x.shape[-1])
        M, K = x2.shape
        N = W.shape[0]
        assert W.shape[1] == K and W.dtype == np.uint16
        y = np.empty((M, N), dtype=np.float32)
        self.L.vox_linear_bf16(_p(y), _p(x2), _p(W), _p(bias), M, K, N)
        return y if x.ndim > 1 else y[0]

    def rms_norm(self, x, w, eps=1e-5):
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, x.shape[-1])
        out = np.empty_like(x)
        self.L.vox_rms_norm(_p(out), _p(x), _p(w), x.shape[0], x.shape[1], eps)
        return out

    def rope_table(self, positions, head_dim=HEAD_DIM, theta=1e6):
        pos = np.ascontiguousarray(positions, dtype=np.int32)
        cs = np.empty((len(pos), head_dim // 2, 2), dtype=np.float32)
        self.L.vox_rope_table(_p(cs), _p(pos), len(pos), head_dim, theta)
        return cs

    def rope_apply(self, x, cs, heads, head_dim=HEAD_DIM):
        x = np.array(x, dtype=np.float32, copy=True).reshape(cs.shape[0], heads * head_dim)
        self.L.vox_rope_apply(_p(x), _p(cs), cs.shape[0], heads, head_dim)
        return x

    def silu_mul(self, gate, up):
        g = np.array(gate, dtype=np.float32, copy=True)
        self.L.vox_silu_mul(_p(g), _p(np.ascontiguousarray(up, dtype=np.float32)), g.size)
        return g

    def attention_causal(self, Q, K, V, n_heads, n_kv_heads, head_dim, scale, q_offset):
        Q = np.ascontiguousarray(Q, dtype=np.float32).reshape(-1, n_heads * head_dim)
        K = np.ascontiguousarray(K, dtype=np.float32)
        V = np.ascontiguousarray(V, dtype=np.float32)
        out = np.zeros_like(Q)
        self.L.vox_attention_causal(_p(out), _p(Q), _p(K), _p(V), Q.shape[0], K.shape[0], n_heads, n_kv_heads,
                                    head_dim, scale, q_offset)
        return out

    def attention_full(self, Q, K, V, n_heads, n_kv_heads, head_dim, scale):
        Q = np.ascontiguousarray(Q, dtype=np.float32).reshape(-1, n_heads * head_dim)
        K = np.ascontiguousarray(K, dtype=np.float32)
        V = np.ascontiguousarray(V, dtype=np.float32)
        out = np.zeros_like(Q)
        self.L.vox_attention_full(_p(out), _p(Q), _p(K), _p(V), Q.shape[0], n_heads, n_kv_heads, head_dim, scale)
        return out

    def time_embedding(self, inv_freq, t, dim=DIM):
        out = np.empty(dim, dtype=np.float32)
        self.L.vox_time_embedding(_p(out), _p(inv_freq), t, dim)
        return out

    # ---- rng ----
    def randn(self, state, n):
        st = C.c_uint64(state)
        buf = np.empty(n, dtype=np.float32)
        self.L.vox_randn_fill(C.byref(st), _p(buf), n)
        return buf, st.value

    def seed(self, seed):
        st = C.c_uint64(0)
        self.L.vox_rng_seed(C.byref(st), seed)
        return st.value

    # ---- model-level ----
    def llm_forward(self, dec, kv_k, kv_v, pos, embed, tap=False):
        kv_max = kv_k.shape[1]
        out = np.empty(dec.d.dim, dtype=np.float32)
        tapbuf = np.zeros((dec.d.n_layers, 2, dec.d.dim), dtype=np.float32) if tap else None
        embed = np.ascontiguousarray(embed, dtype=np.float32)
        self.L.vox_llm_forward(C.byref(dec), _p(kv_k), _p(kv_v), kv_max, pos, _p(embed), _p(out), _p(tapbuf))
        return (out, tapbuf) if tap else out

    def llm_prefill(self, dec, kv_k, kv_v, start, embeds, tap=False):
        kv_max = kv_k.shape[1]
        embeds = np.ascontiguousarray(embeds, dtype=np.float32)
        M = embeds.shape[0]
        tapbuf = np.zeros((dec.d.n_layers, 2, M, dec.d.dim), dtype=np.float32) if tap else None
        self.L.vox_llm_prefill(C.byref(dec), _p(kv_k), _p(kv_v), kv_max, start, _p(embeds), M, _p(tapbuf))
        return tapbuf

    def predict_velocity(self, ac, x_t, hidden, t):
        out = np.empty(ac.n_acoustic, dtype=np.float32)
        self.L.vox_predict_velocity(C.byref(ac), _p(np.ascontiguousarray(x_t, dtype=np.float32)),
                                    _p(np.ascontiguousarray(hidden, dtype=np.float32)), t, _p(out))
        return out

    def acoustic_forward(self, ac, rng_state, hidden):
        st = C.c_uint64(rng_state)
        codes = np.empty(37, dtype=np.int32)
        logits = np.empty(ac.sem_padded, dtype=np.float32)
        xf = np.empty(ac.n_acoustic, dtype=np.float32)
        self.L.vox_acoustic_forward(C.byref(ac), C.byref(st), _p(np.ascontiguousarray(hidden, dtype=np.float32)),
                                    _p(codes), _p(logits), _p(xf))
        return codes, logits, xf, st.value

    def audio_embed(self, table, codes):
        out = np.empty(table.shape[1], dtype=np.float32)
        codes = np.ascontiguousarray(codes, dtype=np.int32)
        self.L.vox_audio_embed(_p(table), table.shape[1], _p(codes), 37, 8194, 23, _p(out))
        return out


class Ref:
    """The reference's own CPU code on caller-supplied weights."""

    def __init__(self, L, kind):
        self.L, self.kind = L, kind
        vp = C.c_void_p
        L.refh_create.restype = vp
        L.refh_destroy.argtypes = [vp]
        L.refh_set_dec_layer.argtypes = [vp, C.c_int] + [vp] * 9
        L.refh_set_dec_misc.argtypes = [vp, vp, vp]
        L.refh_set_ac_layer.argtypes = [vp, C.c_int] + [vp] * 9
        L.refh_set_ac_misc.argtypes = [vp] * 9
        L.refh_set_audio_embed.argtypes = [vp, vp]
        L.refh_load_file.argtypes = [vp, C.c_char_p]
        L.refh_kv_alloc.argtypes = [vp, C.c_int]
        L.refh_kv_k.argtypes = [vp]
        L.refh_kv_k.restype = vp
        L.refh_kv_v.argtypes = [vp]
        L.refh_kv_v.restype = vp
        L.refh_kv_len.argtypes = [vp]
        L.refh_set_kv_len.argtypes = [vp, C.c_int]
        L.refh_seed.argtypes = [vp, C.c_uint64]
        L.refh_rng_state.argtypes = [vp]
        L.refh_rng_state.restype = C.c_uint64
        L.refh_set_rng_state.argtypes = [vp, C.c_uint64]
        L.refh_llm_forward.argtypes = [vp, vp, vp]
        L.refh_llm_prefill.argtypes = [vp, vp, C.c_int]
        L.refh_acoustic_forward.argtypes = [vp, vp, vp]
        L.refh_audio_embed.argtypes = [vp, vp, vp]
        L.refh_predict_velocity.argtypes = [vp, vp, vp, C.c_float, vp]
        L.refh_tap_set.argtypes = [vp, C.c_size_t]
        L.refh_tap_used.restype = C.c_size_t
        L.refh_constants.argtypes = [vp]
        L.refh_sizeof_ctx.restype = C.c_size_t
        L.refh_sizeof_decoder.restype = C.c_size_t
        L.refh_sizeof_acoustic.restype = C.c_size_t
        if hasattr(L, "refh_codec_decode"):
            L.refh_sizeof_codec.restype = C.c_size_t
            L.refh_codec_decode.argtypes = [vp, vp, vp, C.c_int, vp, C.c_int]
        L.refh_decoder_ptr.argtypes = [vp]
        L.refh_decoder_ptr.restype = vp
        L.refh_acoustic_ptr.argtypes = [vp]
        L.refh_acoustic_ptr.restype = vp
        for fn in ("tts_linear_nobias_bf16",):
            getattr(L, fn).argtypes = [vp, vp, vp, C.c_int, C.c_int, C.c_int]
        L.tts_linear_bf16.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int, C.c_int]
        L.tts_rms_norm.argtypes = [vp, vp, vp, C.c_int, C.c_int, C.c_float]
        L.tts_causal_attention.argtypes = [vp] * 4 + [C.c_int] * 5 + [C.c_float, C.c_int, C.c_int]
        L.tts_bidirectional_attention.argtypes = [vp] * 4 + [C.c_int] * 4 + [C.c_float]
        L.tts_compute_rope_freqs.argtypes = [vp, vp, C.c_int, C.c_int, C.c_float]
        L.tts_apply_rope.argtypes = [vp, vp, C.c_int, C.c_int, C.c_int]
        L.tts_silu.argtypes = [vp, C.c_int]
        L.tts_mul_inplace.argtypes = [vp, vp, C.c_int]
        L.tts_randn_fill.argtypes = [vp, vp, C.c_int]
        L.tts_rng_seed.argtypes = [vp, C.c_uint64]
        self.ctx = None
        self._keep = []

    def constants(self):
        out = np.zeros(16, dtype=np.int32)
        self.L.refh_constants(_p(out))
        return out

    def open(self, model, kv_max=512, decoder=True, acoustic=True):
        self.close()
        self.ctx = self.L.refh_create()
        t = model.t
        self._keep.append(model)

        def ptrs(name):
            return [_p(t[f"{name}.attention.{k}.weight"]) for k in ("wq", "wk", "wv", "wo")] + \
                   [_p(t[f"{name}.feed_forward.{k}.weight"]) for k in ("w1", "w2", "w3")] + \
                   [_p(t[f"{name}.attention_norm.weight"]), _p(t[f"{name}.ffn_norm.weight"])]

        if decoder:
            for i in range(DEC_LAYERS):
                self.L.refh_set_dec_layer(self.ctx, i, *ptrs(f"layers.{i}"))
            self.L.refh_set_dec_misc(self.ctx, None, _p(t["norm.weight"]))
            assert self.L.refh_kv_alloc(self.ctx, kv_max) == 0
            self.kv_max = kv_max
        if acoustic:
            p = "acoustic_transformer"
            for i in range(AC_LAYERS):
                self.L.refh_set_ac_layer(self.ctx, i, *ptrs(f"{p}.layers.{i}"))
            self.L.refh_set_ac_misc(self.ctx, _p(t[f"{p}.time_embedding.inv_freq"]),
                                    _p(t[f"{p}.input_projection.weight"]), _p(t[f"{p}.time_projection.weight"]),
                                    _p(t[f"{p}.llm_projection.weight"]),
                                    _p(t[f"{p}.semantic_codebook_output.weight"]),
                                    _p(t.get(f"{p}.semantic_codebook_output.bias")),
                                    _p(t[f"{p}.acoustic_codebook_output.weight"]), _p(t[f"{p}.norm.weight"]))
        n = "mm_audio_embeddings.audio_codebook_embeddings.embeddings.weight"
        if n in t:
            self.L.refh_set_audio_embed(self.ctx, _p(t[n]))
        return self

    def close(self):
        if self.ctx:
            self.L.refh_destroy(self.ctx)
            self.ctx = None

    def codec_decode(self, codec_struct, codes):
        """tts_codec_decode (voxtral_tts_codec.c:389-510) on a caller-filled tts_codec_t."""
        codes = np.ascontiguousarray(codes, dtype=np.int32).reshape(-1, 37)
        ctx = self.L.refh_create()
        out = np.empty(codes.shape[0] * 1920, dtype=np.float32)
        n = self.L.refh_codec_decode(ctx, C.byref(codec_struct), _p(codes), codes.shape[0], _p(out), out.size)
        self.L.refh_destroy(ctx)
        if n < 0:
            raise RuntimeError("reference tts_codec_decode failed")
        return out[:n]

    def kv(self):
        n = DEC_LAYERS * self.kv_max * KV_DIM
        k = np.ctypeslib.as_array(C.cast(self.L.refh_kv_k(self.ctx), f32p), shape=(n,)).reshape(
            DEC_LAYERS, self.kv_max, KV_DIM)
        v = np.ctypeslib.as_array(C.cast(self.L.refh_kv_v(self.ctx), f32p), shape=(n,)).reshape(
            DEC_LAYERS, self.kv_max, KV_DIM)
        return k, v

    def set_kv_len(self, n):
        self.L.refh_set_kv_len(self.ctx, n)

    def kv_len(self):
        return self.L.refh_kv_len(self.ctx)

    def llm_forward(self, embed, tap=False):
        out = np.empty(DIM, dtype=np.float32)
        tapbuf = np.zeros((DEC_LAYERS, 2, DIM), dtype=np.float32) if tap else None
        self.L.refh_tap_set(_p(tapbuf), tapbuf.size if tap else 0)
        self.L.refh_llm_forward(self.ctx, _p(np.ascontiguousarray(embed, dtype=np.float32)), _p(out))
        self.L.refh_tap_set(None, 0)
        return (out, tapbuf) if tap else out

    def llm_prefill(self, embeds, tap=False):
        embeds = np.ascontiguousarray(embeds, dtype=np.float32)
        M = embeds.shape[0]
        tapbuf = np.zeros((DEC_LAYERS, 2, M, DIM), dtype=np.float32) if tap else None
        self.L.refh_tap_set(_p(tapbuf), tapbuf.size if tap else 0)
        self.L.refh_llm_prefill(self.ctx, _p(embeds), M)
        self.L.refh_tap_set(None, 0)
        return tapbuf

    def seed(self, s):
        self.L.refh_seed(self.ctx, s)

    def rng_state(self):
        return self.L.refh_rng_state(self.ctx)

    def set_rng_state(self, s):
        self.L.refh_set_rng_state(self.ctx, s)

    def acoustic_forward(self, hidden):
        codes = np.empty(37, dtype=np.int32)
        self.L.refh_acoustic_forward(self.ctx, _p(np.ascontiguousarray(hidden, dtype=np.float32)), _p(codes))
        return codes

    def predict_velocity(self, x_t, hidden, t):
        out = np.empty(36, dtype=np.float32)
        rc = self.L.refh_predict_velocity(self.ctx, _p(np.ascontiguousarray(x_t, dtype=np.float32)),
                                          _p(np.ascontiguousarray(hidden, dtype=np.float32)), t, _p(out))
        assert rc == 0
        return out

    def audio_embed(self, codes):
        out = np.empty(DIM, dtype=np.float32)
        self.L.refh_audio_embed(self.ctx, _p(np.ascontiguousarray(codes, dtype=np.int32)), _p(out))
        return out

    # raw kernels of voxtral_tts_kernels.c
    def linear(self, x, W, bias=None):
        x = np.ascontiguousarray(x, dtype=np.float32)
        x2 = x.reshape(-1, x.shape[-1])
        y = np.empty((x2.shape[0], W.shape[0]), dtype=np.float32)
        self.L.tts_linear_bf16(_p(y), _p(x2), _p(W), _p(bias), x2.shape[0], x2.shape[1], W.shape[0])
        return y if x.ndim > 1 else y[0]

    def randn(self, state, n):
        st = C.c_uint64(state)
        buf = np.empty(n, dtype=np.float32)
        self.L.tts_randn_fill(C.byref(st), _p(buf), n)
        return buf, st.value


def load_ref(kind):
    path = os.path.join(ORACLE_DIR, "_ref", f"libvoxref_{kind}.so")
    if not os.path.exists(path):
        return None
    try:
        return Ref(C.CDLL(path), kind)
    except OSError:
        return None
