"""det_sample_topkp_static — the sampler for callers that are not allowed to allocate — must pick exactly the token
det_sample_topkp picks with a caller-provided scratch.  Checked through the C ABI on two calls in a row (the second one
finds the first one's weights still in the built-in array), plus the refusal of an oversized request.  This file sorts
last on purpose: a run that stops at the first failure has then already been through every other test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_static_scratch_sampler_matches_the_scratch_version(libs):
    d = libs.cuda()
    assert d.det_init() == 0
    v = 248320
    rng = np.random.default_rng(11)
    first = (rng.random(v, dtype=np.float32) * 24 - 12).astype(np.float32)
    second = np.where(np.arange(v) % 7 == 0, 3.0, (rng.random(v, dtype=np.float32) * 6 - 3)).astype(np.float32)
    logits = d.det_malloc(v * 4)
    z_dev, out_a, out_b = d.det_malloc(8), d.det_malloc(4), d.det_malloc(4)
    scratch = d.det_malloc(d.det_sample_scratch_bytes(1, v))
    calls = [(first, 1.0 / 0.7, 40, 0.95, 0x9E3779B97F4A7C15), (second, 1.3, 0, 0.5, 12345678901234567),
             (second, 0.8, 5, 1.0, 2 ** 64 - 1), (first, 1.0, 0, 1.0, 77)]
    try:
        for row, inv_temp, top_k, top_p, z in calls:          # consecutive calls share the built-in array
            d.det_memcpy(logits, row.ctypes.data, row.nbytes, None)
            zz = np.array([z], np.uint64)
            d.det_memcpy(z_dev, zz.ctypes.data, 8, None)
            d.det_sample_topkp(logits, 1, v, inv_temp, top_k, top_p, z_dev, out_a, scratch, None)
            assert d.det_sample_topkp_static(logits, 1, v, inv_temp, top_k, top_p, z_dev, out_b, None) == 0
            a, b = np.zeros(1, np.int32), np.zeros(1, np.int32)
            d.det_memcpy(a.ctypes.data, out_a, 4, None)
            d.det_memcpy(b.ctypes.data, out_b, 4, None)
            d.det_sync()
            assert a[0] == b[0], (inv_temp, top_k, top_p, int(a[0]), int(b[0]))
            assert 0 <= b[0] < v
        # beyond the built-in scratch: refused, nothing launched, the previous result stays
        assert d.det_sample_topkp_static(logits, 3, v, 1.0, 40, 0.9, z_dev, out_b, None) == 1
        d.det_sync()
        assert d.det_last_error() == 0
    finally:
        for p in (logits, z_dev, out_a, out_b, scratch):
            d.det_free(p)
