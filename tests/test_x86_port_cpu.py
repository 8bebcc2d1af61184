"""The restated x86 backend (oracle/x86_backend.hpp: the timed CPU baseline and the CPU side of the large-model parity
checks) against the restated reference backend: the conformance suites on both dot-product paths, as the reference runs
its own x86 backend (crates/det/tests/backends.rs:59-70), and the tiny model end to end."""
import ctypes as C

import numpy as np
import pytest

SEED = 20261125


def _paths(oracle):
    level = oracle.orc_cpu_simd_level()
    if level == 0:
        pytest.skip("no AVX2 on this host")
    return [1, 0] if level == 2 else [0]


@pytest.fixture(scope="module")
def port(oracle):
    oracle.orc_cpu_backend_new.restype = C.c_void_p
    oracle.orc_cpu_backend_new.argtypes = [C.c_int]
    made = {}
    for vnni in _paths(oracle):
        made[vnni] = oracle.orc_cpu_backend_new(vnni)
        assert made[vnni]
    yield made
    for b in made.values():
        oracle.orc_ref_backend_free(b)


@pytest.mark.parametrize("suite", ["gemm", "norms", "attention", "gdn", "sampling"])
def test_conformance_suites_on_both_dot_product_paths(suite, oracle, ref_backend, port):
    for vnni, dut in port.items():
        if suite == "sampling" and vnni == 0 and len(port) == 2:
            continue     # sampling is the scalar spec on every CPU backend (x86/mod.rs:168-181): one run covers it
        buf = C.create_string_buffer(1 << 20)
        failed = oracle.orc_conformance(ref_backend, dut, suite.encode(), None, buf, len(buf))
        report = buf.value.decode()
        assert failed == 0, f"vnni={vnni}\n" + "\n".join(l for l in report.splitlines() if not l.startswith("ok"))
        assert report.count("ok ") > 0


def test_tiny_model_logits_and_tokens_equal_the_reference_backend(libs, ref_backend, port):
    h = libs.host()
    ids = np.zeros(24, np.int32)
    h.dh_synth_prompt(1, len(ids), 32768, ids.ctypes.data)
    results = []
    for backend in [ref_backend] + list(port.values()):
        m = h.dh_model_new_synth(backend, b"tiny", 0, SEED, 64, 16)
        assert m, h.dh_last_error()
        out, n = np.zeros(6, np.int32), C.c_size_t(0)
        assert h.dh_model_generate(m, ids.ctypes.data, len(ids), 6, 1, 1.0, 0, 1.0, 0, out.ctypes.data, C.byref(n)) == 0
        logits = np.zeros(32768, np.float32)
        h.dh_model_logits(m, logits.ctypes.data, logits.size)
        results.append((out.copy(), logits.view(np.uint32).copy()))
        h.dh_model_free(m)
    for toks, lg in results[1:]:
        assert np.array_equal(toks, results[0][0])
        assert np.array_equal(lg, results[0][1])
