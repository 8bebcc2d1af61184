"""Batched serving decode on the CUDA backend (BASELINE configs[4] in miniature): sequences of different lengths advance
together, once through det_attention_rows / det_gdn_rows (one launch sequence over all rows) and once composed from the
single-sequence calls; every stream must equal the stream that sequence produces alone, which test_model_gpu ties to the
oracle."""
import numpy as np
import pytest

from test_serve_cpu import run_streams

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fused", [1, 0])
def test_batched_streams_equal_solo_streams(fused, libs, cuda_backend):
    h = libs.host()
    h.dh_cuda_set_fuse_rows(cuda_backend, fused)
    try:
        together, solo = run_streams(h, cuda_backend, n_new=40, layers=8, ctx=96)
    finally:
        h.dh_cuda_set_fuse_rows(cuda_backend, 1)
    for i, (a, b) in enumerate(zip(together, solo)):
        assert np.array_equal(a, b), (i, a, b)
    assert libs.cuda().det_last_error() == 0
