"""Shared fixtures. GPU tests are marked `gpu`; everything else runs on CPU."""
import importlib.util
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "voxtral-tts.c_b200")
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


def load_package():
    """Import the package directory (its name is not a Python identifier)."""
    name = "voxtral_tts_c_b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(PKG_DIR, "__init__.py"),
                                                  submodule_search_locations=[PKG_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def _ensure_built():
    lib = os.path.join(PKG_DIR, "lib", "libvoxtral_b200.so")
    if not os.path.exists(lib):
        subprocess.check_call([sys.executable, os.path.join(PKG_DIR, "build.py")])
    port = os.path.join(ROOT, "oracle", "liboracle.so")
    if not os.path.exists(port):
        subprocess.check_call([sys.executable, os.path.join(ROOT, "oracle", "build_oracle.py")])


@pytest.fixture(scope="session")
def pkg():
    _ensure_built()
    return load_package()


@pytest.fixture(scope="session")
def oracle():
    _ensure_built()
    import oracle_bind
    return oracle_bind.Oracle()


@pytest.fixture(scope="session")
def ref_noblas():
    import oracle_bind
    r = oracle_bind.load_ref("noblas")
    if r is None:
        pytest.skip("oracle/_ref/libvoxref_noblas.so not built (needs the reference checkout)")
    return r


@pytest.fixture(scope="session")
def ref_blas():
    import oracle_bind
    r = oracle_bind.load_ref("blas")
    if r is None:
        pytest.skip("oracle/_ref/libvoxref_blas.so not available")
    return r


@pytest.fixture(scope="session")
def synth_model(pkg):
    from cases import MODEL_SEED
    return pkg.SynthModel(seed=MODEL_SEED)


@pytest.fixture(scope="session")
def engine(pkg, synth_model):
    """The process-wide GPU context (the library, like the reference, has one per process)
    with the full synthetic checkpoint uploaded."""
    e = pkg.Engine(kv_cache_max=512)
    e.upload(synth_model, decoder=True, acoustic=True, audio_table=True)
    yield e
    e.close()
