"""det_argmax on decode-sized inputs (few rows, large vocabulary: the split kernel) against the oracle's spec argmax
(spec/sample.rs:6-14): lowest index of the maximum, +0 and -0 tie."""
import ctypes as C

import numpy as np
import pytest


def _rows():
    rng = np.random.default_rng(7)
    V = 248320
    a = rng.standard_normal(V).astype(np.float32)
    yield "random", a
    b = a.copy()
    top = b.max() + 1
    b[[7761, 100000, 248319]] = top          # the maximum three times, in three different chunks
    yield "tie across chunks", b
    c = np.full(V, -np.inf, np.float32)
    yield "all -inf", c
    e = np.full(V, -1.0, np.float32)
    e[200000] = -0.0
    e[5] = 0.0
    e[150000] = 0.0
    yield "signed zeros", e
    f = a.copy()
    f[-1] = 100.0
    yield "maximum last", f
    g = rng.standard_normal(32768).astype(np.float32)
    g[[3, 32767]] = 9.0
    yield "smaller vocabulary", g


@pytest.mark.gpu
def test_argmax_rows_match_spec(libs, oracle):
    d = libs.cuda()
    assert d.det_init() == 0
    for name, row in _rows():
        V = row.size
        for M in (1, 3, 8, 9):                 # 9 rows: the one-CTA-per-row kernel
            x = np.stack([np.roll(row, 1000 * t) for t in range(M)]).astype(np.float32)
            want = np.array([oracle.orc_argmax(x[t].ctypes.data, V) for t in range(M)], np.int32)
            dx, dout = d.det_malloc(x.nbytes), d.det_malloc(4 * M)
            d.det_memcpy(dx, x.ctypes.data, x.nbytes, None)
            d.det_argmax(dx, M, V, dout, None)
            got = np.zeros(M, np.int32)
            d.det_memcpy(got.ctypes.data, dout, 4 * M, None)
            d.det_sync()
            d.det_free(dx)
            d.det_free(dout)
            assert np.array_equal(got, want), (name, M, got, want)
