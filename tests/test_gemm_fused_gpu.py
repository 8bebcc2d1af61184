"""det_gemm_fused (activation quantization inside the GEMV prologue) against the unfused pipeline it replaces
(det_rmsnorm_quant / det_quant / det_silu_mul_quant, then det_gemm_ex), bit for bit, on the edge-case rows the
reference's norms suite uses (crates/det/src/conformance.rs:462-498): all-denormal rows, denormal/zero alternation,
mixed magnitudes, squares that underflow."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

PER32 = {8: 32, 6: 24, 4: 16}


def _rows(rng, m, n):
    x = np.zeros((m, n), np.float32)
    den = lambda size: (rng.integers(1, 1 << 23, size, dtype=np.uint32) | (rng.integers(0, 2, size, dtype=np.uint32) << 31)).view(np.float32)
    for r in range(m):
        kind = r % 6
        if kind == 0:
            x[r] = den(n)
        elif kind == 1:
            x[r, ::2] = den(n // 2)
        elif kind == 2:
            scales = np.array([1e-20, 1e-23, 0, 1.0, 0.0, 1e-30, -0.0, 1e3], np.float32)
            x[r] = (rng.random(n, dtype=np.float32) * 2 - 1) * scales[np.arange(n) % 8]
            x[r, 2::8] = den(len(x[r, 2::8]))
        elif kind == 3:
            x[r] = (rng.random(n, dtype=np.float32) * 2 - 1) * np.where(np.arange(n) % 5 == 0, 1e-19, 1e-38).astype(np.float32)
        else:
            x[r] = (rng.random(n, dtype=np.float32) * 2 - 1) * (10.0 ** -((np.arange(n) // 128) % 4)).astype(np.float32)
    return x


def _dev(d, arr):
    p = d.det_malloc(max(arr.nbytes, 16))
    d.det_memcpy(p, arr.ctypes.data, arr.nbytes, None)
    return p


def _host(d, p, like):
    out = np.zeros_like(like)
    d.det_memcpy(out.ctypes.data, p, out.nbytes, None)
    d.det_sync()
    return out


@pytest.mark.parametrize("n_out,k,bits,m", [(512, 2560, 6, 6), (384, 5120, 6, 1), (256, 17408, 6, 3), (640, 1024, 8, 8),
                                            (256, 2048, 4, 5)])
@pytest.mark.parametrize("kind", [1, 2, 3])
def test_fused_equals_unfused(n_out, k, bits, m, kind, libs):
    d = libs.cuda()
    rng = np.random.default_rng(k + bits + kind)
    g = k // 128
    nc = k // 32 * PER32[bits]
    wq = _dev(d, rng.integers(0, 256, n_out * nc, dtype=np.uint8))
    cc = _dev(d, (rng.random(n_out, dtype=np.float32) * 1e-6 + 1e-8).astype(np.float32))
    mm = _dev(d, rng.integers(1, 65536, n_out * g).astype(np.uint16))
    src = libs.QLinear(wq, cc, mm, n_out, k, bits)
    sp = d.det_malloc(d.det_linear_repack_bytes(n_out, k, bits))
    d.det_linear_repack(C.byref(src), sp, None)
    lin = libs.QLinear(sp, cc, mm, n_out, k, bits | libs.DET_LAYOUT_STREAM)
    a = _rows(rng, m, k)
    b = (1.0 + (rng.random(k, dtype=np.float32) * 2 - 1)).astype(np.float32) if kind == 1 else \
        np.where(np.arange(m * k).reshape(m, k) % 3 == 1, 1e-39, (rng.random((m, k), dtype=np.float32) * 6 - 3)).astype(np.float32)
    da, db = _dev(d, a), _dev(d, b)
    y0 = (rng.random((m, n_out), dtype=np.float32) * 2 - 1).astype(np.float32)
    outs = []
    for fused in (False, True):
        xq, sx, mx = d.det_malloc(m * k), d.det_malloc(m * 4), d.det_malloc(m * g * 2)
        y, yacc = d.det_malloc(m * n_out * 4), _dev(d, y0)
        if fused:
            s = libs.ActSource(kind, da, db, 1e-6, xq, sx, mx)
            d.det_gemm_fused(C.byref(lin), C.byref(s), m, y, 0, 0, None, None, None)
            s2 = libs.ActSource(kind, da, db, 1e-6, None, None, None)
            d.det_gemm_fused(C.byref(lin), C.byref(s2), m, yacc, 1, 0, None, None, None)
        else:
            if kind == 1:
                d.det_rmsnorm_quant(da, db, 1e-6, m, k, None, xq, sx, mx, None)
            elif kind == 2:
                d.det_quant(da, m, k, xq, sx, mx, None)
            else:
                d.det_silu_mul_quant(da, db, m, k, None, xq, sx, mx, None)
            d.det_gemm_ex(C.byref(lin), xq, sx, mx, m, y, 0, 0, None, None, None)
            d.det_gemm_ex(C.byref(lin), xq, sx, mx, m, yacc, 1, 0, None, None, None)
        outs.append((_host(d, y, y0).view(np.uint32), _host(d, yacc, y0).view(np.uint32),
                     _host(d, xq, np.zeros(m * k, np.int8)), _host(d, sx, np.zeros(m, np.float32)).view(np.uint32),
                     _host(d, mx, np.zeros(m * g, np.uint16))))
        for p in (xq, sx, mx, y, yacc):
            d.det_free(p)
    for name, u, f in zip(("y", "y accumulate", "codes", "scales", "multipliers"), outs[0], outs[1]):
        assert np.array_equal(u, f), f"{name}: {(u != f).sum()} of {u.size} differ"
    assert d.det_last_error() == 0
    for p in (wq, cc, mm, sp, da, db):
        d.det_free(p)
