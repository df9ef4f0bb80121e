"""Test configuration: the ``gpu`` marker, and loaders for the CPU oracle (the checker, never the product)."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with `-m gpu` on the GPU box")


def pytest_collection_modifyitems(config, items):
    # Keep the file order alphabetical (test_zz_* last) whatever order paths were given in.
    items.sort(key=lambda it: (os.path.basename(str(it.fspath)), ))


@pytest.fixture(scope="session")
def oracle():
    from oracle_loader import load_oracle
    return load_oracle()


@pytest.fixture(scope="session")
def ref_kernels():
    from oracle_loader import load_ref_kernels
    lib = load_ref_kernels()
    if lib is None:
        pytest.skip("oracle/_ref/libsymplex_kernels.so not built (needs the reference checkout)")
    return lib


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_vectors.npz"))


@pytest.fixture(scope="session")
def lib():
    """The product library, built on demand (CPU-only boxes can still load it and query symbols)."""
    from symplex_b200 import _capi
    if not os.path.exists(_capi.LIB_PATH):
        from symplex_b200.build import build_library
        build_library()
    return _capi.load()


@pytest.fixture
def set_option(lib):
    """``set_option(name, value)``: a tuning override of the library for the duration of one test."""
    saved = {}

    def _set(name, value):
        key = name.encode()
        if key not in saved:
            saved[key] = lib.symplex_b200_get_option(key)
        assert lib.symplex_b200_set_option(key, int(value)) == 0

    yield _set
    for key, old in saved.items():
        lib.symplex_b200_set_option(key, old)
