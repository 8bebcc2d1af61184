"""End-to-end parity on the tiny seeded model (the benchmark's tiny configuration): every logit of a 64-token prompt and 64 greedy
tokens, CUDA backend vs the CPU oracle running the same driver; plus invariance to the prefill chunking."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SEED = 20261125


def _model(h, backend, max_batch, cfg=b"tiny", layers=0, max_ctx=192):
    m = h.dh_model_new_synth(backend, cfg, layers, SEED, max_ctx, max_batch)
    assert m, h.dh_last_error()
    return m


def _prompt(h, n, vocab):
    ids = np.zeros(n, np.int32)
    h.dh_synth_prompt(1, n, vocab, ids.ctypes.data)
    return ids


def _all_logits(h, m, ids):
    vocab = h.dh_model_vocab(m)
    assert h.dh_model_set_all_logits(m, 1) == 0
    assert h.dh_model_forward(m, ids.ctypes.data, len(ids)) == 0, h.dh_last_error()
    out = np.zeros(len(ids) * vocab, np.float32)
    h.dh_model_logits(m, out.ctypes.data, out.size)
    return out.view(np.uint32)


def _greedy(h, m, ids, n_new):
    out = np.zeros(n_new, np.int32)
    n = C.c_size_t(0)
    assert h.dh_model_generate(m, ids.ctypes.data, len(ids), n_new, 1, 1.0, 0, 1.0, 0, out.ctypes.data, C.byref(n)) == 0
    return out[: n.value]


def test_tiny_every_logit_and_greedy_tokens(libs, ref_backend, cuda_backend):
    h = libs.host()
    ids = _prompt(h, 64, 32768)
    ref, gpu = _model(h, ref_backend, 64), _model(h, cuda_backend, 64)
    try:
        a, b = _all_logits(h, ref, ids), _all_logits(h, gpu, ids)
        assert np.array_equal(a, b), f"{(a != b).sum()} of {a.size} logits differ"
        for m in (ref, gpu):
            h.dh_model_set_all_logits(m, 0)
            h.dh_model_reset(m)
        ta, tb = _greedy(h, ref, ids, 64), _greedy(h, gpu, ids, 64)
        assert np.array_equal(ta, tb), (ta, tb)
        la, lb = np.zeros(32768, np.float32), np.zeros(32768, np.float32)
        h.dh_model_logits(ref, la.ctypes.data, la.size)
        h.dh_model_logits(gpu, lb.ctypes.data, lb.size)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
    finally:
        h.dh_model_free(ref)
        h.dh_model_free(gpu)


@pytest.mark.parametrize("chunk", [1, 16])
def test_tiny_chunking_invariance(chunk, libs, cuda_backend):
    h = libs.host()
    ids = _prompt(h, 64, 32768)
    whole, parts = _model(h, cuda_backend, 64), _model(h, cuda_backend, chunk)
    try:
        assert h.dh_model_prefill(whole, ids.ctypes.data, 64) == 0
        assert h.dh_model_prefill(parts, ids.ctypes.data, 64) == 0
        la, lb = np.zeros(32768, np.float32), np.zeros(32768, np.float32)
        h.dh_model_logits(whole, la.ctypes.data, la.size)
        h.dh_model_logits(parts, lb.ctypes.data, lb.size)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
    finally:
        h.dh_model_free(whole)
        h.dh_model_free(parts)


def test_long_context_decode_equals_chunked_prefill(libs, cuda_backend):
    """Context of 5200 keys on a 4-layer tiny model (one attention layer): the last 400 tokens are fed one at a time (the fused decode attention
    kernel, two key tiles per CTA, key ranges merged through the global cells) on one model and in 64-token
    batches (the separate max / acc / fin kernels) on the other; the final logits must be the same bits."""
    h = libs.host()
    n = 5200
    ids = _prompt(h, n, 32768)
    a = _model(h, cuda_backend, 64, layers=4, max_ctx=n + 8)
    b = _model(h, cuda_backend, 64, layers=4, max_ctx=n + 8)
    try:
        assert h.dh_model_prefill(a, ids.ctypes.data, n) == 0, h.dh_last_error()
        assert h.dh_model_prefill(b, ids.ctypes.data, n - 400) == 0, h.dh_last_error()
        for i in range(n - 400, n):
            assert h.dh_model_forward(b, ids[i:].ctypes.data, 1) == 0, h.dh_last_error()
        la, lb = np.zeros(32768, np.float32), np.zeros(32768, np.float32)
        h.dh_model_logits(a, la.ctypes.data, la.size)
        h.dh_model_logits(b, lb.ctypes.data, lb.size)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32)), f"{(la.view(np.uint32) != lb.view(np.uint32)).sum()} logits differ"
        assert libs.cuda().det_last_error() == 0
    finally:
        h.dh_model_free(a)
        h.dh_model_free(b)


def test_4b_chunking_1_64_512(libs, cuda_backend):
    """The 4B configuration (32 layers, hidden 2560, vocabulary 248320): a 512-token prompt prefilled in
    chunks of 512 (tensor-core GEMM), 64 and 1 (streaming GEMV), then 32 greedy tokens; last-position logits and all
    tokens must be the same bits for the three chunkings."""
    h = libs.host()
    vocab = 248320
    ids = _prompt(h, 512, vocab)
    results = []
    for chunk in (512, 64, 1):
        m = _model(h, cuda_backend, chunk, cfg=b"4b", max_ctx=512 + 40)
        try:
            assert h.dh_model_prefill(m, ids.ctypes.data, 512) == 0, h.dh_last_error()
            logits = np.zeros(vocab, np.float32)
            h.dh_model_logits(m, logits.ctypes.data, logits.size)
            h.dh_model_reset(m)
            toks = _greedy(h, m, ids, 32)
            results.append((logits.view(np.uint32).copy(), toks.copy()))
        finally:
            h.dh_model_free(m)
    for lg, tk in results[1:]:
        assert np.array_equal(lg, results[0][0]), f"{(lg != results[0][0]).sum()} logits differ"
        assert np.array_equal(tk, results[0][1]), (tk, results[0][1])
    assert libs.cuda().det_last_error() == 0
