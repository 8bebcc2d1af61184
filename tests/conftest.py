"""Shared fixtures.  GPU tests carry the `gpu` marker; everything else runs on a machine without a device."""
from __future__ import annotations

import ctypes as C
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; runs the CUDA path through the C ABI")


@pytest.fixture(scope="session")
def libs():
    """Builds (if stale) and loads the product libraries."""
    from det_b200 import build, capi
    build.build_all()
    return capi


@pytest.fixture(scope="session")
def oracle(libs):
    """The CPU oracle library (test infrastructure): restated spec + reference backend."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import importlib.util
    spec = importlib.util.spec_from_file_location("oracle_build", ROOT / "oracle" / "build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    libs.host()
    lib = C.CDLL(str(mod.build()))
    lib.orc_ref_backend_new.restype = C.c_void_p
    lib.orc_ref_backend_free.argtypes = [C.c_void_p]
    lib.orc_conformance.restype = C.c_int
    lib.orc_conformance.argtypes = [C.c_void_p, C.c_void_p, C.c_char_p, C.c_void_p, C.c_char_p, C.c_size_t]
    lib.orc_treesum.restype = C.c_float
    lib.orc_argmax.restype = C.c_int
    lib.orc_sample.restype = C.c_int
    lib.orc_sample.argtypes = [C.c_void_p, C.c_size_t, C.c_float, C.c_size_t, C.c_float, C.c_uint64]
    lib.orc_splitmix64.restype = C.c_uint64
    vp, sz = C.c_void_p, C.c_size_t
    lib.orc_gemm.argtypes = [vp, sz, sz, C.c_int, vp, vp, vp, sz, vp, C.c_int]
    lib.orc_quant.argtypes = [vp, sz, sz, vp, vp, vp]
    lib.orc_rmsnorm_quant.argtypes = [vp, vp, C.c_float, sz, sz, vp, vp, vp]
    lib.orc_silu_mul_quant.argtypes = [vp, vp, sz, sz, vp, vp, vp]
    lib.orc_unpack_row.argtypes = [vp, C.c_int, sz, vp]
    lib.orc_treesum.argtypes = [vp, sz]
    lib.orc_argmax.argtypes = [vp, sz]
    lib.orc_weights.argtypes = [vp, sz, C.c_float, vp]
    lib.orc_prim.argtypes = [C.c_int, vp, sz, sz, sz, vp, sz]
    lib.orc_splitmix64.argtypes = [C.POINTER(C.c_uint64)]
    return lib


@pytest.fixture(scope="session")
def ref_backend(oracle):
    b = oracle.orc_ref_backend_new()
    yield b
    oracle.orc_ref_backend_free(b)


@pytest.fixture(scope="session")
def cuda_backend(libs):
    h = libs.host()
    b = h.dh_cuda_backend_new(1, 1)
    assert b, h.dh_last_error()
    yield b
    h.dh_backend_free(b)
