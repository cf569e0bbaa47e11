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


@pytest.fixture(scope="session")
def reflib(capi):
    """The reference project's CPU build (oracle/_ref).  Tests that need it are
    skipped when it has not been built (it needs the reference checkout)."""
    if not os.path.isfile(REF_LIB):
        pytest.skip("oracle/_ref/libcaffe_ref.so not built")
    return capi.CaffeLibrary(REF_LIB)
