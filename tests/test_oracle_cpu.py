"""Pins the CPU oracle (oracle/spec.hpp) against the committed known-answer vectors of tests/golden (an independent
numpy restatement of the spec's primitives) and against the spec's literal constants."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

G = np.load(Path(__file__).resolve().parent / "golden" / "spec_vectors.npz")


def _prim(oracle, op, x, m=1, n=None):
    x = np.ascontiguousarray(x, np.float32)
    n = len(x) if n is None else n
    out = np.zeros(max(len(x), m), np.float32)
    oracle.orc_prim(op, x.ctypes.data, len(x), m, n, out.ctypes.data, len(out))
    return out


def _same(a, b):
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    return np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_elementwise_primitives(oracle):
    x = G["x"]
    for op, key in ((0, "exp"), (3, "sigmoid"), (4, "silu"), (2, "softplus")):
        got = _prim(oracle, op, x)[: len(x)]
        bad = np.flatnonzero(got.view(np.uint32) != G[key].view(np.uint32))
        bad = [i for i in bad if not (np.isnan(got[i]) and np.isnan(G[key][i]))]
        assert not bad, f"{key}: {len(bad)} differ, first x={x[bad[0]]!r} oracle={got[bad[0]]!r} numpy={G[key][bad[0]]!r}"
    assert _same(_prim(oracle, 1, G["pos"])[: len(G["pos"])], G["log"])


def test_treesum(oracle):
    rows = G["tree_rows"]
    for i, n in enumerate(G["tree_len"]):
        row = np.ascontiguousarray(rows[i, :n])
        assert _same([oracle.orc_treesum(row.ctypes.data, int(n))], [G["tree_out"][i]]), f"row {i} of length {n}"


def test_quant_act_i8g(oracle):
    qx = np.ascontiguousarray(G["qx"])
    m, n = qx.shape
    q, sx, mx = np.zeros((m, n), np.int8), np.zeros(m, np.float32), np.zeros((m, n // 128), np.uint16)
    oracle.orc_quant(qx.ctypes.data, m, n, q.ctypes.data, sx.ctypes.data, mx.ctypes.data)
    assert np.array_equal(q, G["q_codes"])
    assert np.array_equal(mx, G["q_mx"])
    assert _same(sx, G["q_sx"])


def test_unpack_and_gemm_row(oracle):
    k = 512
    rows = {}
    for bits in (4, 6, 8):
        packed = np.ascontiguousarray(G[f"packed{bits}"])
        codes = np.zeros(k, np.int8)
        oracle.orc_unpack_row(packed.ctypes.data, bits, k, codes.ctypes.data)
        assert np.array_equal(codes, G[f"codes{bits}"]), f"W{bits}"
        c = np.array([3.1e-7], np.float32)
        rows[bits] = np.concatenate([packed, c.view(np.uint8), G["gemm_m"].view(np.uint8)])
    xq, mx = np.ascontiguousarray(G["gemm_xq"]), np.ascontiguousarray(G["gemm_mx"])
    sx = np.array([1.7e-3], np.float32)
    for i, bits in enumerate((4, 6, 8)):
        y = np.zeros(1, np.float32)
        row = np.ascontiguousarray(rows[bits])
        oracle.orc_gemm(row.ctypes.data, 1, k, bits, xq.ctypes.data, sx.ctypes.data, mx.ctypes.data, 1, y.ctypes.data, 0)
        assert _same(y, G["gemm_out"][i:i + 1]), f"W{bits}"


def test_splitmix64_and_sampling_weights(oracle):
    state = C.c_uint64(0)
    for want_state, want_out in zip(G["sm_states"], G["sm_outs"]):
        assert oracle.orc_splitmix64(C.byref(state)) == int(want_out)
        assert state.value == int(want_state)
    logits = np.ascontiguousarray(G["logits"])
    for key, inv_temp in (("weights_1", np.float32(1.0)), ("weights_07", np.float32(1.0) / np.float32(0.7))):
        w = np.zeros(len(logits), np.uint64)
        oracle.orc_weights(logits.ctypes.data, len(logits), float(inv_temp), w.ctypes.data)
        assert np.array_equal(w, G[key]), key


def test_literal_constants(oracle):
    """The constants the reference pins literally (spec/layers.rs:16,147; model.rs:47; spec/prim.rs:204-211)."""
    assert _prim(oracle, 0, [0.0])[0] == 1.0
    one = np.array([1.0], np.float32)
    w = np.zeros(1, np.uint64)
    oracle.orc_weights(one.ctypes.data, 1, 1.0, w.ctypes.data)
    assert int(w[0]) == 1 << 32                      # the largest weight is exactly 2^32 (33 bits)
    assert np.float32(1.0 / 1024.0) == np.float32(2.0 ** -10)
    assert np.array([0x3DB504F3], np.uint32).view(np.float32)[0] == np.float32(1.0 / np.sqrt(np.float32(128.0)))


def test_sampler_properties(oracle):
    """top_p <= 0 keeps the first candidate only; top_k = 1 is argmax; a huge top_k is the plain sampler."""
    rng = np.random.default_rng(5)
    logits = np.ascontiguousarray((rng.random(5000) * 10).astype(np.float32))
    best = oracle.orc_argmax(logits.ctypes.data, len(logits))
    for z in (0, 1, 2 ** 63, 2 ** 64 - 1):
        assert oracle.orc_sample(logits.ctypes.data, len(logits), 1.0, 0, 0.0, z) == best
        assert oracle.orc_sample(logits.ctypes.data, len(logits), 1.0, 1, 1.0, z) == best
        a = oracle.orc_sample(logits.ctypes.data, len(logits), 0.5, 0, 1.0, z)
        b = oracle.orc_sample(logits.ctypes.data, len(logits), 0.5, len(logits) + 5, 1.0, z)
        assert a == b


def test_restated_x86_gemm_equals_gemm_row(oracle):
    """The strip-repacked, K-blocked integer GEMM of the timed CPU baseline (oracle/x86_backend.hpp, the restated
    crates/det/src/x86/gemm.rs) against the scalar spec gemm_row, on both dot-product paths, every weight width, extreme
    codes, ragged row counts (a partial strip pair) and token counts on both sides of the 4-token tile and the 64-token
    chunk."""
    import ctypes as C
    if oracle.orc_cpu_simd_level() == 0:
        pytest.skip("no AVX2 on this host")
    oracle.orc_gemm_x86.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_size_t, C.c_void_p, C.c_int]
    rng = np.random.default_rng(5)
    paths = [0, 1] if oracle.orc_cpu_simd_level() == 2 else [0]
    for bits, n, k, m in [(6, 96, 1024, 3), (8, 40, 512, 1), (4, 64, 2560, 5), (6, 33, 128, 2), (6, 50, 2560, 70), (8, 17, 1152, 9)]:
        per32 = {8: 32, 6: 24, 4: 16}[bits]
        g = k // 128
        nc = k // 32 * per32
        rows = np.zeros((n, nc + 4 + 2 * g), np.uint8)
        rows[:, :nc] = rng.integers(0, 256, (n, nc), dtype=np.uint8)
        rows[0, :nc] = 0xFF          # extreme codes
        rows[1, :nc] = 0x00
        c = (1e-8 + rng.random(n) * 1e-6).astype(np.float32)
        mm = rng.integers(1, 65536, (n, g)).astype(np.uint16)
        mm[2] = 65535
        rows[:, nc:nc + 4] = c.view(np.uint8).reshape(n, 4)
        rows[:, nc + 4:] = mm.view(np.uint8).reshape(n, 2 * g)
        xq = rng.integers(-127, 128, (m, k)).astype(np.int8)
        xq[0] = 127
        if m > 1:
            xq[1] = -127
        sx = (1e-3 * (0.5 + rng.random(m))).astype(np.float32)
        mx = rng.integers(1, 65536, (m, g)).astype(np.uint16)
        mx[0] = 65535
        want = np.zeros((m, n), np.float32)
        got = np.zeros((m, n), np.float32)
        oracle.orc_gemm(rows.ctypes.data, n, k, bits, xq.ctypes.data, sx.ctypes.data, mx.ctypes.data, m, want.ctypes.data, 0)
        for vnni in paths:
            got[:] = 0
            oracle.orc_gemm_x86(rows.ctypes.data, n, k, bits, xq.ctypes.data, sx.ctypes.data, mx.ctypes.data, m,
                                got.ctypes.data, vnni)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (bits, n, k, m, vnni)
