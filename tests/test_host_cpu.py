"""Host logic without a GPU: the model driver over the CPU oracle backend (chunking invariance, error paths), the
synthetic generator and the quantizer (port of the reference's unit test, crates/det/src/quantize.rs:102-141)."""
import ctypes as C

import numpy as np
import pytest

SEED = 20261125


def _model(h, backend, max_batch, layers=4, max_ctx=64):
    m = h.dh_model_new_synth(backend, b"tiny", layers, SEED, max_ctx, max_batch)
    assert m, h.dh_last_error()
    return m


def _logits(h, m):
    out = np.zeros(h.dh_model_vocab(m), np.float32)
    h.dh_model_logits(m, out.ctypes.data, out.size)
    return out.view(np.uint32)


def test_chunking_invariance_on_the_oracle(libs, ref_backend):
    h = libs.host()
    ids = np.zeros(12, np.int32)
    h.dh_synth_prompt(1, 12, 32768, ids.ctypes.data)
    outs = []
    for chunk in (12, 5, 1):
        m = _model(h, ref_backend, chunk)
        assert h.dh_model_prefill(m, ids.ctypes.data, 12) == 0, h.dh_last_error()
        assert h.dh_model_pos(m) == 12
        outs.append(_logits(h, m))
        h.dh_model_free(m)
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])


def test_input_errors_are_reported_not_fatal(libs, ref_backend):
    h = libs.host()
    m = _model(h, ref_backend, 4, max_ctx=8)
    bad = np.array([32768], np.int32)
    assert h.dh_model_forward(m, bad.ctypes.data, 1) != 0 and b"outside the embedding table" in h.dh_last_error()
    neg = np.array([-1], np.int32)
    assert h.dh_model_forward(m, neg.ctypes.data, 1) != 0
    five = np.zeros(5, np.int32)
    assert h.dh_model_forward(m, five.ctypes.data, 5) != 0 and b"batch of 5" in h.dh_last_error()
    assert h.dh_model_forward(m, five.ctypes.data, 0) != 0
    four = np.zeros(4, np.int32)
    assert h.dh_model_forward(m, four.ctypes.data, 4) == 0
    assert h.dh_model_forward(m, four.ctypes.data, 4) == 0
    assert h.dh_model_forward(m, four.ctypes.data, 1) != 0 and b"exceed the context" in h.dh_last_error()
    assert h.dh_model_pos(m) == 8                      # failed calls left the state untouched
    tok, rng = C.c_int32(0), C.c_uint64(0)
    assert h.dh_model_pick(m, 0, float("nan"), 0, 1.0, C.byref(rng), C.byref(tok)) != 0
    assert h.dh_model_pick(m, 0, 1.0, 0, float("nan"), C.byref(rng), C.byref(tok)) != 0
    assert rng.value == 0
    assert h.dh_model_pick(m, 0, 1.0, 40, 0.95, C.byref(rng), C.byref(tok)) == 0
    assert rng.value == 0x9E3779B97F4A7C15 and 0 <= tok.value < 32768
    h.dh_model_free(m)


def test_sampled_generation_is_reproducible(libs, ref_backend):
    h = libs.host()
    ids = np.zeros(4, np.int32)
    h.dh_synth_prompt(2, 4, 32768, ids.ctypes.data)
    runs = []
    for _ in range(2):
        m = _model(h, ref_backend, 4)
        out, n = np.zeros(6, np.int32), C.c_size_t(0)
        assert h.dh_model_generate(m, ids.ctypes.data, 4, 6, 0, 1.0 / 0.7, 40, 0.95, 1234, out.ctypes.data, C.byref(n)) == 0
        runs.append(out[: n.value].copy())
        h.dh_model_free(m)
    assert len(runs[0]) == 6 and np.array_equal(runs[0], runs[1])


@pytest.mark.parametrize("bits", [4, 6, 8])
def test_quantizer_round_trip_and_error_bound(bits, libs, oracle):
    """det rows of the synthetic generator: codes within range, unpack(pack) is the identity, and every weight is
    reproduced within half a step of its group scale (quantize.rs:102-141)."""
    h = libs.host()
    n, k = 8, 512
    rb = h.dh_det_row_bytes(bits, k)
    rows = np.zeros(n * rb, np.uint8)
    h.dh_synth_det_rows(SEED, 77, n, k, bits, rows.ctypes.data)
    again = np.zeros_like(rows)
    h.dh_synth_det_rows(SEED, 77, n, k, bits, again.ctypes.data)
    assert np.array_equal(rows, again)
    qmax = (1 << (bits - 1)) - 1
    nc = rb - 4 - k // 128 * 2
    for r in range(n):
        row = np.ascontiguousarray(rows[r * rb:(r + 1) * rb])
        codes = np.zeros(k, np.int8)
        oracle.orc_unpack_row(row.ctypes.data, bits, k, codes.ctypes.data)
        assert codes.min() >= -qmax and codes.max() <= qmax
        c = row[nc:nc + 4].view(np.float32)[0]
        m = row[nc + 4:].view(np.uint16)
        assert c > 0 and m.min() >= 1 and m.max() == 65535     # the largest group scale maps to the top multiplier
        w = (np.float64(c) * m.astype(np.float64))[:, None] * codes.reshape(-1, 128).astype(np.float64)
        assert np.isfinite(w).all() and np.abs(w).max() < 0.2    # ~N(0, 0.02) weights
