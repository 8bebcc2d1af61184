"""Batched serving decode on the CUDA backend (the 32-sequence serving configuration in miniature): sequences of different lengths advance
together, once through det_attention_rows / det_gdn_rows (one launch sequence over all rows) and once composed from the
single-sequence calls; every stream must equal the stream that sequence produces alone, which test_model_gpu ties to the
oracle."""
import numpy as np
import pytest

from test_serve_cpu import run_streams

pytestmark = pytest.mark.gpu


def test_nine_sequences_use_the_shared_prep_kernel(libs, cuda_backend):
    """From 8 sequences on the batched Gated DeltaNet step prepares its operands once per head (k_gdn_prep) instead of in
    every recurrence CTA; the streams must still equal the solo streams."""
    h = libs.host()
    together, solo = run_streams(h, cuda_backend, n_new=24, layers=8, ctx=96, prompts=[5, 17, 33, 9, 12, 3, 40, 21, 8])
    for i, (a, b) in enumerate(zip(together, solo)):
        assert np.array_equal(a, b), (i, a, b)
    assert libs.cuda().det_last_error() == 0


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


def test_fused_decode_launches_give_the_same_tokens_and_logits(libs, cuda_backend):
    """The decode step with its ops fused across launches (quantization as the GEMV prologue, a|b riding with qkv|z, the
    SwiGLU product from the gate|up epilogue, the Gated DeltaNet step in one cluster launch) against every op issued on its
    own: same tokens, same final logits."""
    import ctypes as C
    h = libs.host()
    ids = np.zeros(20, np.int32)
    h.dh_synth_prompt(3, ids.size, 32768, ids.ctypes.data)
    runs = []
    for fuse in (0, 1):
        h.dh_cuda_debug(cuda_backend, 0, fuse)
        try:
            m = h.dh_model_new_synth(cuda_backend, b"tiny", 8, 20261125, 96, 16)
            assert m, h.dh_last_error()
            out = np.zeros(48, np.int32)
            n = C.c_size_t(0)
            assert h.dh_model_generate(m, ids.ctypes.data, ids.size, 48, 1, 1.0, 0, 1.0, 0, out.ctypes.data, C.byref(n)) == 0
            logits = np.zeros(32768, np.float32)
            h.dh_model_logits(m, logits.ctypes.data, logits.size)
            runs.append((out[: n.value].copy(), logits.view(np.uint32).copy()))
            h.dh_model_free(m)
        finally:
            h.dh_cuda_debug(cuda_backend, 0, 1)
    assert np.array_equal(runs[0][0], runs[1][0])
    assert np.array_equal(runs[0][1], runs[1][1])
    assert libs.cuda().det_last_error() == 0
