"""det_sample_topkp on a 248320-token vocabulary (the cluster-per-row kernel) and on a small one (one CTA per row)
against the oracle's spec sampler (spec/sample.rs:16-87): flat, peaked and heavily tied logits, top-k only, top-p only,
both, and degenerate parameters."""
import ctypes as C

import numpy as np
import pytest


def _cases(V):
    rng = np.random.default_rng(V)
    flat = (rng.standard_normal(V) * 0.3).astype(np.float32)
    peaked = (rng.standard_normal(V) * 4.0).astype(np.float32)
    peaked[V // 3] = 30.0
    tied = np.zeros(V, np.float32)
    tied[rng.integers(0, V, 5000)] = 1.0             # thousands of equal weights across all ranges
    tail = np.full(V, -40.0, np.float32)
    tail[-7:] = 3.0                                   # everything that matters sits in the last range
    return {"flat": flat, "peaked": peaked, "tied": tied, "tail": tail}


@pytest.mark.gpu
@pytest.mark.parametrize("V", [248320, 32768, 70001])
def test_topkp_matches_spec(V, libs, oracle):
    d = libs.cuda()
    assert d.det_init() == 0
    params = [(1.0 / 0.7, 40, 0.95), (1.0, 0, 0.5), (1.0, 7, 1.0), (2.0, 1, 0.9), (1.0, 100000, 0.999), (1.0, 40, 0.0)]
    M = 3
    scratch = d.det_malloc(d.det_sample_scratch_bytes(M, V))
    dl, dz, dout = d.det_malloc(M * V * 4), d.det_malloc(M * 8), d.det_malloc(M * 4)
    for name, row in _cases(V).items():
        x = np.stack([np.roll(row, 12345 * t) for t in range(M)]).astype(np.float32)
        d.det_memcpy(dl, x.ctypes.data, x.nbytes, None)
        for inv_temp, top_k, top_p in params:
            for draw in (0, 0x9E3779B97F4A7C15, 2**64 - 1):
                z = np.array([(draw + 977 * t) % 2**64 for t in range(M)], np.uint64)
                d.det_memcpy(dz, z.ctypes.data, z.nbytes, None)
                d.det_sample_topkp(dl, M, V, inv_temp, top_k, top_p, dz, dout, scratch, None)
                got = np.zeros(M, np.int32)
                d.det_memcpy(got.ctypes.data, dout, 4 * M, None)
                d.det_sync()
                want = np.array([oracle.orc_sample(x[t].ctypes.data, V, inv_temp, top_k, top_p, int(z[t])) for t in range(M)],
                                np.int32)
                assert np.array_equal(got, want), (name, inv_temp, top_k, top_p, draw, got, want)
    for p in (scratch, dl, dz, dout):
        d.det_free(p)
    assert d.det_last_error() == 0
