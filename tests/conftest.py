import ctypes as C
import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def capi():
    return importlib.import_module("s2pro-native_b200.capi")


@pytest.fixture(scope="session")
def synth():
    return importlib.import_module("s2pro-native_b200.synth")


@pytest.fixture(scope="session")
def mine(capi):
    """The product library; a missing build is an error, never a skip."""
    return capi.load_library()


@pytest.fixture(scope="session")
def testlib(capi):
    """Same objects with default visibility: reaches the internal launchers of cuda/ops.h."""
    p = os.path.join(os.path.dirname(capi.LIB_PATH), "libs2pro_b200_test.so")
    if not os.path.exists(p):
        pytest.fail(f"{p} missing: run `make -C s2pro-native_b200/csrc testlib` (or __graft_entry__.build())")
    lib = C.CDLL(p)
    capi.bind(lib, capi.PROTOTYPES)
    return lib


def _ref(name, capi):
    p = os.path.join(ROOT, "oracle", "_ref", name)
    if not os.path.exists(p):
        pytest.skip(f"{p} not built (the reference sources are not on this machine)")
    lib = C.CDLL(p)
    capi.bind(lib, capi.PROTOTYPES, strict=False)
    return lib


@pytest.fixture(scope="session")
def ref(capi):
    """The reference's own CUDA path rebuilt for sm_100a (oracle/Makefile `ref`)."""
    return _ref("libs2pref.so", capi)


@pytest.fixture(scope="session")
def ref_l2(capi):
    return _ref("libs2pref_l2.so", capi)


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle_api
    return oracle_api.load()
