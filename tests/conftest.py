import importlib.util
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "apus-qwen3.6-35b-a3b_b200")
sys.path.insert(0, ROOT)


def load_package():
    """The package directory name is not an identifier: load it by path."""
    if "apus_b200" in sys.modules:
        return sys.modules["apus_b200"]
    spec = importlib.util.spec_from_file_location(
        "apus_b200", os.path.join(PKG_DIR, "__init__.py"),
        submodule_search_locations=[PKG_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["apus_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def be(pkg):
    """The CUDA library binding.  Built on demand where nvcc exists; loading
    it needs no GPU."""
    pkg.build.build()
    return pkg.Backend()


@pytest.fixture(scope="session")
def synth(pkg):
    import apus_b200.synth as s
    return s


@pytest.fixture(scope="session")
def orc():
    from oracle import oracle
    return oracle.Restatement()


@pytest.fixture(scope="session")
def ref():
    from oracle import oracle
    if not oracle.Reference.available():
        pytest.skip("oracle/_ref/libapus_ref.so not built")
    return oracle.Reference()


@pytest.fixture
def gpu(be):
    """Enable the backend on the device (fails loudly without one).  Each
    test gets a fresh residency table: the backend keys resident weights by
    host address (the engine's stable-pointer rule), and numpy reuses the
    addresses of arrays an earlier test freed."""
    be.enable()
    yield be
    be.disable()


def rel_l2(a, b):
    a = a.astype(np.float64).ravel()
    b = b.astype(np.float64).ravel()
    return float(np.linalg.norm(a - b) / (np.linalg.norm(b) + 1e-30))
