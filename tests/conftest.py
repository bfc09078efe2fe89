import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "icdm-2021_mascot_b200")
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def load_module(name, path):
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs on the B200 box)")


@pytest.fixture(scope="session")
def mascot():
    """ctypes binding of libmascot.so (the product)."""
    return load_module("mascot_binding", os.path.join(PKG, "mascot.py"))


@pytest.fixture(scope="session")
def synth():
    return load_module("mascot_synth", os.path.join(PKG, "synth.py"))


@pytest.fixture(scope="session")
def oracle():
    """CPU oracle (test infrastructure)."""
    import oracle as O
    O.lib()
    return O


@pytest.fixture(scope="session")
def golden():
    from bundle import read_bundle
    gdir = os.path.join(ROOT, "tests", "golden")
    return read_bundle(os.path.join(gdir, "harness_in.bin")), read_bundle(os.path.join(gdir, "harness_out.bin"))


@pytest.fixture(scope="session")
def setup_golden():
    """Inputs and outputs of the reference's m-quantization set-up functions (oracle/ref_harness.cu, kind 8)."""
    from bundle import read_bundle
    gdir = os.path.join(ROOT, "tests", "golden")
    return read_bundle(os.path.join(gdir, "setup_in.bin")), read_bundle(os.path.join(gdir, "setup_out.bin"))
