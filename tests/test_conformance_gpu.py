"""The reference's acceptance test (`det conformance --backend cuda`, crates/det/src/conformance.rs:164-175) against
the B200 backend: every op through the C ABI vs the CPU oracle, bit for bit, edge cases included."""
import ctypes as C

import pytest

pytestmark = pytest.mark.gpu

SUITES = ["primitives", "gemm", "norms", "attention", "gdn", "sampling"]


@pytest.mark.parametrize("suite", SUITES)
def test_suite(suite, libs, oracle, ref_backend, cuda_backend):
    h = libs.host()
    report = C.create_string_buffer(1 << 20)
    hook = C.cast(h.dh_cuda_test_prim, C.c_void_p)
    failed = oracle.orc_conformance(ref_backend, cuda_backend, suite.encode(), hook, report, len(report))
    text = report.value.decode()
    bad = [l for l in text.splitlines() if not l.startswith("ok ")]
    assert failed == 0 and not bad, f"{suite}: {failed} failed checks\n" + "\n".join(bad[:40])
    assert text.count("ok ") > 0
