"""The shared library loads without a GPU and exports every symbol the headers declare."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b((?:tts_cuda|vb200)_[a-z0-9_]+)\s*\(", text))
    if "extern vb200_ref_cuda_ctx_t g_cuda" in text:
        names.add("g_cuda")
    return names


def test_reference_surface_is_complete(pkg):
    L = pkg.lib()
    names = _declared("voxtral_b200.h")
    assert names == set(pkg.EXPORTED_SYMBOLS_REFERENCE), names ^ set(pkg.EXPORTED_SYMBOLS_REFERENCE)
    assert len(names) == 25  # the 25 symbols the reference's CUDA object exports
    for n in names:
        assert hasattr(L, n), n


def test_extension_surface_is_exported(pkg):
    L = pkg.lib()
    for header in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if not header.endswith(".h") or header == "voxtral_b200.h":
            continue
        for n in _declared(header):
            assert hasattr(L, n), (header, n)


def test_g_cuda_layout_matches_reference(pkg, ref_noblas):
    """Struct sizes of the weight tables the upload calls receive match the reference's."""
    assert ref_noblas.L.refh_sizeof_decoder() == C.sizeof(pkg.DecoderWeights)
    assert ref_noblas.L.refh_sizeof_acoustic() == C.sizeof(pkg.AcousticWeights)
    ref_noblas.L.refh_sizeof_codec.restype = C.c_size_t
    assert ref_noblas.L.refh_sizeof_codec() == C.sizeof(pkg.CodecWeights)
    c = ref_noblas.constants()
    assert list(c[:14]) == [pkg.DIM, pkg.DEC_LAYERS, pkg.HEADS, pkg.KV_HEADS, pkg.HEAD_DIM, pkg.HIDDEN,
                            pkg.AC_LAYERS, pkg.ACOUSTIC_DIM, pkg.SEM_PADDED, pkg.FLOW_STEPS, pkg.FSQ_LEVELS,
                            pkg.CODES, 8192, pkg.VOCAB]


def test_init_without_gpu_fails_loudly(pkg):
    import torch
    if torch.cuda.is_available():
        return
    assert pkg.lib().tts_cuda_init(64) != 0
    assert pkg.lib().tts_cuda_available() == 0
    try:
        pkg.Engine(64)
    except RuntimeError:
        pass
    else:
        raise AssertionError("Engine() must raise without a GPU")
