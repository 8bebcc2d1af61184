"""det_sample_topkp_static — the sampler for callers that are not allowed to allocate — must pick exactly the token
det_sample_topkp picks with a caller-provided scratch, and the token the CPU oracle's sampler picks.  Checked through the
C ABI on calls in a row (each one finds the previous one's weights still in the built-in array), on two rows at once
(the second row starts at a stride inside the shared array), on a vocabulary above 262144 (the one-CTA-per-row kernel),
plus the refusals.  This file sorts last on purpose: a run that stops at the first failure has then already been through
every other test."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _draws(zs):
    return np.array(zs, np.uint64)


def _run(d, oracle, rows, inv_temp, top_k, top_p, zs):
    """rows: [M][V] fp32 logits.  Returns (scratch version, static version, oracle) token ids."""
    m, v = rows.shape
    logits = d.det_malloc(rows.nbytes)
    z_dev, out_a, out_b = d.det_malloc(8 * m), d.det_malloc(4 * m), d.det_malloc(4 * m)
    scratch = d.det_malloc(d.det_sample_scratch_bytes(m, v))
    try:
        d.det_memcpy(logits, rows.ctypes.data, rows.nbytes, None)
        zz = _draws(zs)
        d.det_memcpy(z_dev, zz.ctypes.data, zz.nbytes, None)
        d.det_sample_topkp(logits, m, v, inv_temp, top_k, top_p, z_dev, out_a, scratch, None)
        assert d.det_sample_topkp_static(logits, m, v, inv_temp, top_k, top_p, z_dev, out_b, None) == 0
        a, b = np.zeros(m, np.int32), np.zeros(m, np.int32)
        d.det_memcpy(a.ctypes.data, out_a, a.nbytes, None)
        d.det_memcpy(b.ctypes.data, out_b, b.nbytes, None)
        d.det_sync()
        want = np.array([oracle.orc_sample(rows[i].ctypes.data, v, inv_temp, top_k, top_p, int(zz[i])) for i in range(m)],
                        np.int32)
        return a, b, want
    finally:
        for p in (logits, z_dev, out_a, out_b, scratch):
            d.det_free(p)


def test_static_scratch_sampler_matches_the_scratch_version_and_the_oracle(libs, oracle):
    d = libs.cuda()
    assert d.det_init() == 0
    v = 248320
    rng = np.random.default_rng(11)
    first = (rng.random(v, dtype=np.float32) * 24 - 12).astype(np.float32)
    second = np.where(np.arange(v) % 7 == 0, 3.0, (rng.random(v, dtype=np.float32) * 6 - 3)).astype(np.float32)
    calls = [(first[None], 1.0 / 0.7, 40, 0.95, [0x9E3779B97F4A7C15]), (second[None], 1.3, 0, 0.5, [12345678901234567]),
             (second[None], 0.8, 5, 1.0, [2 ** 64 - 1]), (first[None], 1.0, 0, 1.0, [77]),
             # two rows in one call: 496640 weights, the second row at offset V of the shared array
             (np.stack([first, second]), 1.0 / 0.7, 40, 0.95, [1234567, 7654321987654321]),
             (np.stack([second, first]), 1.1, 0, 0.3, [99, 2 ** 63 + 5])]
    for rows, inv_temp, top_k, top_p, zs in calls:          # consecutive calls share the built-in array
        rows = np.ascontiguousarray(rows)
        a, b, want = _run(d, oracle, rows, inv_temp, top_k, top_p, zs)
        assert np.array_equal(a, b), (inv_temp, top_k, top_p, a, b)
        assert np.array_equal(b, want), (inv_temp, top_k, top_p, b, want)
        assert ((0 <= b) & (b < v)).all()
    # a vocabulary above 262144 tokens takes the one-CTA-per-row kernel
    big = (rng.random(300000, dtype=np.float32) * 10 - 5).astype(np.float32)[None]
    a, b, want = _run(d, oracle, np.ascontiguousarray(big), 1.0 / 0.7, 40, 0.95, [424242424242])
    assert np.array_equal(a, b) and np.array_equal(b, want), (a, b, want)
    assert d.det_last_error() == 0


def test_static_scratch_sampler_refusals(libs):
    d = libs.cuda()
    assert d.det_init() == 0
    v = 248320
    logits, z_dev, out = d.det_malloc(3 * v * 4), d.det_malloc(24), d.det_malloc(12)
    try:
        # beyond the built-in scratch with a filter active: refused, nothing launched
        assert d.det_sample_topkp_static(logits, 3, v, 1.0, 40, 0.9, z_dev, out, None) == 1
        # not a vocabulary
        assert d.det_sample_topkp_static(logits, 1, 0, 1.0, 40, 0.9, z_dev, out, None) == 1
        # no filter active: no scratch needed, so the size limit does not apply
        assert d.det_sample_topkp_static(logits, 3, v, 1.0, 0, 1.0, z_dev, out, None) == 0
        got = np.full(3, -1, np.int32)
        d.det_memcpy(got.ctypes.data, out, 12, None)
        d.det_sync()
        assert ((0 <= got) & (got < v)).all()
        assert d.det_last_error() == 0
    finally:
        for p in (logits, z_dev, out):
            d.det_free(p)
