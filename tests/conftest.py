"""Shared fixtures: library loaders and the gpu marker.

`-m "not gpu"` runs on a machine without a GPU (parsers, host logic, the
oracle against its fixtures, symbol checks); `-m gpu` holds the parity tests
that launch kernels.
"""
import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ENGINE_LIB = os.path.join(ROOT, "mini-caffe_b200", "lib", "libcaffe.so")
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libcaffe_ref.so")
# A checkout of the reference project (its example models and callers are test inputs where present):
# MINI_CAFFE_REFERENCE, else a directory `reference` beside this repository.
REFERENCE_CHECKOUT = os.environ.get("MINI_CAFFE_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pkg(name):
    """Import a module of the hyphenated package directory."""
    return importlib.import_module("mini-caffe_b200." + name)


@pytest.fixture(scope="session")
def capi():
    return pkg("capi")


@pytest.fixture(scope="session")
def engine(capi):
    if not os.path.isfile(ENGINE_LIB):
        pytest.fail("libcaffe.so is not built: run `python -c 'import __graft_entry__ as g; g.build()'`")
    return capi.CaffeLibrary(ENGINE_LIB)


@pytest.fixture(scope="session")
def kernels():
    """libcaffe.so as a plain ctypes handle, for the kernel-level C ABI
    (include/mcb200_kernels.h)."""
    import ctypes
    if not os.path.isfile(ENGINE_LIB):
        pytest.fail("libcaffe.so is not built: run `python -c 'import __graft_entry__ as g; g.build()'`")
    return ctypes.CDLL(ENGINE_LIB, mode=ctypes.RTLD_LOCAL)


_reference_library = {}


@pytest.fixture
def reflib(request, capi):
    """The reference project's CPU build (oracle/_ref), the checker of the parity tests.

    Without it a GPU parity test has nothing to compare with, so for a test marked `gpu` its absence
    is a failure (a run in which the checker did not travel with the repository must not look green).
    Host-only tests are skipped instead: the library can only be built where a checkout of the
    reference project is present."""
    if not os.path.isfile(REF_LIB):
        message = "oracle/_ref/libcaffe_ref.so is not built (build it with `make -C oracle REF=<mini-caffe checkout>`)"
        if request.node.get_closest_marker("gpu") is not None:
            pytest.fail(message)
        pytest.skip(message)
    if "lib" not in _reference_library:
        _reference_library["lib"] = capi.CaffeLibrary(REF_LIB)
    return _reference_library["lib"]
