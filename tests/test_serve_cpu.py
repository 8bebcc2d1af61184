"""Batched serving decode on the CPU reference backend: four sequences of different prompt lengths advance together
(rows stacked for the linears, attention / Gated DeltaNet per row against each sequence's own cache and state, one
sampler state per sequence).  Every stream must equal the stream that sequence produces alone."""
import ctypes as C

import numpy as np
import pytest

SEED = 20261125
VOCAB = 32768
PROMPTS = [5, 17, 33, 9]
SAMPLING = dict(greedy=0, inv_temp=1.0 / 0.7, top_k=40, top_p=0.95)


def _prompt(h, seed, n):
    ids = np.zeros(n, np.int32)
    h.dh_synth_prompt(seed, n, VOCAB, ids.ctypes.data)
    return ids


def run_streams(h, backend, n_new, layers=4, ctx=64, prompts=None):
    """(batched streams, solo streams) for the prompts above (or the given prompt lengths)."""
    PROMPTS = prompts or globals()["PROMPTS"]
    model = h.dh_model_new_synth(backend, b"tiny", layers, SEED, ctx, 16)
    assert model, h.dh_last_error()
    solo = []
    for i, n in enumerate(PROMPTS):
        ids = _prompt(h, 100 + i, n)
        out = np.zeros(n_new, np.int32)
        cnt = C.c_size_t(0)
        assert h.dh_model_reset(model) == 0
        assert h.dh_model_generate(model, ids.ctypes.data, n, n_new, SAMPLING["greedy"], SAMPLING["inv_temp"],
                                   SAMPLING["top_k"], SAMPLING["top_p"], 7000 + i, out.ctypes.data, C.byref(cnt)) == 0, h.dh_last_error()
        solo.append(out[: cnt.value].copy())
    batch = h.dh_batch_new(model, len(PROMPTS), ctx)
    assert batch, h.dh_last_error()
    for i, n in enumerate(PROMPTS):
        ids = _prompt(h, 100 + i, n)
        assert h.dh_batch_prefill(batch, i, ids.ctypes.data, n, SAMPLING["greedy"], SAMPLING["inv_temp"],
                                  SAMPLING["top_k"], SAMPLING["top_p"], 7000 + i) == 0, h.dh_last_error()
    assert h.dh_batch_step(batch, n_new - 1) == 0, h.dh_last_error()
    together = []
    for i in range(len(PROMPTS)):
        out = np.zeros(n_new, np.int32)
        assert h.dh_batch_tokens(batch, i, out.ctypes.data, n_new) == n_new
        together.append(out)
    h.dh_batch_free(batch)
    h.dh_model_free(model)
    return together, solo


def test_batched_streams_equal_solo_streams_on_the_reference_backend(libs, ref_backend):
    together, solo = run_streams(libs.host(), ref_backend, n_new=6)
    for i, (a, b) in enumerate(zip(together, solo)):
        assert np.array_equal(a, b), (i, a, b)


def test_mixed_sampling_parameters_per_sequence(libs, ref_backend):
    """Sequences with different sampling settings (greedy, plain temperature, top-k / top-p) in one batch: the step then
    samples row by row; each stream must still equal its solo stream."""
    h = libs.host()
    settings = [(1, 1.0, 0, 1.0), (0, 1.0 / 0.9, 0, 1.0), (0, 1.0 / 0.7, 40, 0.95), (0, 2.0, 5, 1.0)]
    n_new, ctx = 5, 64
    model = h.dh_model_new_synth(ref_backend, b"tiny", 4, SEED, ctx, 16)
    assert model, h.dh_last_error()
    solo = []
    for i, (n, (greedy, inv_temp, top_k, top_p)) in enumerate(zip(PROMPTS, settings)):
        ids = _prompt(h, 200 + i, n)
        out = np.zeros(n_new, np.int32)
        cnt = C.c_size_t(0)
        assert h.dh_model_reset(model) == 0
        assert h.dh_model_generate(model, ids.ctypes.data, n, n_new, greedy, inv_temp, top_k, top_p, 9000 + i,
                                   out.ctypes.data, C.byref(cnt)) == 0, h.dh_last_error()
        solo.append(out[: cnt.value].copy())
    batch = h.dh_batch_new(model, len(PROMPTS), ctx)
    assert batch, h.dh_last_error()
    for i, (n, (greedy, inv_temp, top_k, top_p)) in enumerate(zip(PROMPTS, settings)):
        ids = _prompt(h, 200 + i, n)
        assert h.dh_batch_prefill(batch, i, ids.ctypes.data, n, greedy, inv_temp, top_k, top_p, 9000 + i) == 0, h.dh_last_error()
    assert h.dh_batch_step(batch, n_new - 1) == 0, h.dh_last_error()
    for i in range(len(PROMPTS)):
        out = np.zeros(n_new, np.int32)
        assert h.dh_batch_tokens(batch, i, out.ctypes.data, n_new) == n_new
        assert np.array_equal(out, solo[i]), (i, out, solo[i])
    h.dh_batch_free(batch)
    h.dh_model_free(model)


def test_prefilling_a_slot_again_starts_a_fresh_conversation(libs, ref_backend):
    """A slot that is prefilled a second time must forget its first conversation (position, recurrent state): the second
    stream equals the stream of a decoder that only ever saw the second prompt."""
    h = libs.host()
    n_new, ctx = 5, 64
    model = h.dh_model_new_synth(ref_backend, b"tiny", 4, SEED, ctx, 16)
    assert model, h.dh_last_error()
    first, second = _prompt(h, 300, 21), _prompt(h, 301, 12)

    def stream(prompts):
        batch = h.dh_batch_new(model, 2, ctx)
        assert batch, h.dh_last_error()
        other = _prompt(h, 302, 7)
        assert h.dh_batch_prefill(batch, 1, other.ctypes.data, len(other), 0, 1.0 / 0.7, 40, 0.95, 5) == 0
        for ids in prompts:
            assert h.dh_batch_prefill(batch, 0, ids.ctypes.data, len(ids), 0, 1.0 / 0.7, 40, 0.95, 4242) == 0, h.dh_last_error()
            if ids is not prompts[-1]:
                assert h.dh_batch_step(batch, 3) == 0, h.dh_last_error()
                assert h.dh_batch_prefill(batch, 1, other.ctypes.data, len(other), 0, 1.0 / 0.7, 40, 0.95, 5) == 0
        assert h.dh_batch_step(batch, n_new - 1) == 0, h.dh_last_error()
        out = np.zeros(n_new, np.int32)
        assert h.dh_batch_tokens(batch, 0, out.ctypes.data, n_new) == n_new
        h.dh_batch_free(batch)
        return out

    again, fresh = stream([first, second]), stream([second])
    h.dh_model_free(model)
    assert np.array_equal(again, fresh), (again, fresh)
