"""Parity of the CUDA path with a CPU path at the large benchmark shapes, where the scalar reference backend would take
hours: the CPU side is the restated x86 backend (oracle/x86_backend.hpp), which tests/test_x86_port_cpu.py pins to the
reference backend suite by suite.  Covered: the 4B configuration (512-token prompt, logits and greedy tokens), the 27B
shape at reduced depth (the first 8 layers — two attention and six Gated DeltaNet layers, every 27B kernel shape — plus
the W8 head: 2048-token prompt in 512- and 64-token chunks, logits after the prompt and after 16 decode steps), and the
graph-replayed decode step against the eager loop on one GPU."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SEED = 20261125
VOCAB = 248320


@pytest.fixture(scope="module")
def cpu_port(oracle, libs):
    if oracle.orc_cpu_simd_level() == 0:
        pytest.skip("no AVX2 on this host")
    oracle.orc_cpu_backend_new.restype = C.c_void_p
    oracle.orc_cpu_backend_new.argtypes = [C.c_int]
    h = libs.host()
    h.dh_use_cuda_synth_rows(1)        # identical det rows from the device generator: seconds instead of minutes
    b = oracle.orc_cpu_backend_new(-1)
    assert b
    yield b
    h.dh_use_cuda_synth_rows(0)
    oracle.orc_ref_backend_free(b)


def _prompt(h, n, vocab=VOCAB):
    ids = np.zeros(n, np.int32)
    h.dh_synth_prompt(1, n, vocab, ids.ctypes.data)
    return ids


def _logits(h, m, vocab=VOCAB):
    out = np.zeros(vocab, np.float32)
    h.dh_model_logits(m, out.ctypes.data, out.size)
    return out.view(np.uint32).copy()


def _run(h, backend, cfg, layers, chunk, ids, n_new, vocab=VOCAB):
    """Prefill in `chunk`-token batches, then n_new greedy steps.  Returns (logits after the prompt, tokens, final logits)."""
    m = h.dh_model_new_synth(backend, cfg, layers, SEED, len(ids) + n_new + 8, chunk)
    assert m, h.dh_last_error()
    try:
        assert h.dh_model_prefill(m, ids.ctypes.data, len(ids)) == 0, h.dh_last_error()
        after_prompt = _logits(h, m, vocab)
        toks = []
        tok, rng = C.c_int32(0), C.c_uint64(0)
        for _ in range(n_new):
            assert h.dh_model_pick(m, 1, 1.0, 0, 1.0, C.byref(rng), C.byref(tok)) == 0
            toks.append(tok.value)
            one = np.array([tok.value], np.int32)
            assert h.dh_model_forward(m, one.ctypes.data, 1) == 0, h.dh_last_error()
        return after_prompt, np.array(toks, np.int32), _logits(h, m, vocab)
    finally:
        h.dh_model_free(m)


def _same(name, a, b):
    for what, x, y in zip(("logits after the prompt", "tokens", "final logits"), a, b):
        assert np.array_equal(x, y), f"{name}: {what}: {int((x != y).sum())} of {x.size} differ"


def test_4b_logits_and_tokens_match_the_cpu_port(libs, cuda_backend, cpu_port):
    h = libs.host()
    ids = _prompt(h, 512)
    cpu = _run(h, cpu_port, b"4b", 0, 256, ids, 8)
    _same("4B, 512-token chunk", _run(h, cuda_backend, b"4b", 0, 512, ids, 8), cpu)
    _same("4B, 64-token chunk", _run(h, cuda_backend, b"4b", 0, 64, ids, 8), cpu)
    assert libs.cuda().det_last_error() == 0


def test_27b_shape_reduced_depth_matches_the_cpu_port(libs, cuda_backend, cpu_port):
    h = libs.host()
    ids = _prompt(h, 2048)
    cpu = _run(h, cpu_port, b"27b", 8, 256, ids, 16)
    _same("27B shape, 512-token chunks", _run(h, cuda_backend, b"27b", 8, 512, ids, 16), cpu)
    _same("27B shape, 64-token chunks", _run(h, cuda_backend, b"27b", 8, 64, ids, 16), cpu)
    assert libs.cuda().det_last_error() == 0


@pytest.mark.parametrize("cfg,layers,vocab", [(b"tiny", 0, 32768), (b"27b", 4, VOCAB)])
def test_graph_replayed_decode_equals_the_eager_loop(cfg, layers, vocab, libs, cuda_backend):
    h = libs.host()
    ids = _prompt(h, 40, vocab)
    n_new = 12
    _, eager, eager_logits = _run(h, cuda_backend, cfg, layers, 64, ids, n_new, vocab)
    m = h.dh_model_new_synth(cuda_backend, cfg, layers, SEED, len(ids) + n_new + 8, 64)
    assert m, h.dh_last_error()
    try:
        assert h.dh_model_prefill(m, ids.ctypes.data, len(ids)) == 0
        tok, rng = C.c_int32(0), C.c_uint64(0)
        assert h.dh_model_pick(m, 1, 1.0, 0, 1.0, C.byref(rng), C.byref(tok)) == 0
        assert tok.value == eager[0]
        dec = h.dh_graph_decoder_new(m)
        assert dec, h.dh_last_error()
        # two enqueue calls: the second replays the graph captured by the first
        got = []
        last = tok.value
        for part in (5, n_new - 1 - 5):
            assert h.dh_graph_decoder_enqueue(dec, last, part, 1) == 0, h.dh_last_error()
            out = np.zeros(part, np.int32)
            assert h.dh_graph_decoder_finish(dec, out.ctypes.data, part) == part
            got += [int(x) for x in out]
            last = got[-1]
        h.dh_graph_decoder_free(dec)
        assert got == [int(x) for x in eager[1:]], (got, eager)
        assert libs.cuda().det_last_error() == 0
    finally:
        h.dh_model_free(m)
