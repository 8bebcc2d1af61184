"""Generates tests/golden/spec_vectors.npz: known-answer vectors for the oracle.

The reference ships no golden files (its tests are differential), and its Rust cannot be built here.  This script is a
second, independent restatement of the spec's primitives (crates/det/src/spec/prim.rs, quant.rs, sample.rs) in numpy —
every step is one np.float32 operation, the equivalence the spec's own comments state (prim.rs:4, prim.rs:72) — and
its outputs pin the C++ oracle (oracle/spec.hpp) in tests/test_oracle_cpu.py.  Run: python tests/golden/make_golden.py
"""
from __future__ import annotations

from pathlib import Path

import numpy as np

f32 = np.float32
OUT = Path(__file__).resolve().parent / "spec_vectors.npz"

LOG2E = f32(1.44269504088896341)
EXP_C1, EXP_C2 = f32(0.693359375), f32(-2.12194440e-4)
EXP_P = [f32(v) for v in (1.9875691500E-4, 1.3981999507E-3, 8.3334519073E-3, 4.1665795894E-2, 1.6666665459E-1,
                          5.0000001201E-1)]
LOG_SQRTHF = f32(0.707106781186547524)
LOG_P = [f32(v) for v in (7.0376836292E-2, -1.1514610310E-1, 1.1676998740E-1, -1.2420140846E-1, 1.4249322787E-1,
                          -1.6668057665E-1, 2.0000714765E-1, -2.4999993993E-1, 3.3333331174E-1)]


def exp_f(x: np.ndarray) -> np.ndarray:
    x = np.minimum(x.astype(f32), f32(88.0))
    small = x < f32(-87.0)
    xs = np.where(small, f32(0.0), x)
    n = np.floor(xs * LOG2E + f32(0.5)).astype(f32)
    r = xs - n * EXP_C1
    r = r - n * EXP_C2
    z = r * r
    y = np.full_like(r, EXP_P[0])
    for c in EXP_P[1:]:
        y = y * r + c
    y = y * z + r
    y = y + f32(1.0)
    scale = ((n.astype(np.int32) + 127) << 23).astype(np.uint32).view(f32)
    return np.where(small, f32(0.0), y * scale).astype(f32)


def log_f(x: np.ndarray) -> np.ndarray:
    b = x.astype(f32).view(np.uint32)
    e = ((b >> 23) & 0xFF).astype(np.int32) - 126
    m = ((b & 0x007FFFFF) | 0x3F000000).astype(np.uint32).view(f32)
    lt = m < LOG_SQRTHF
    e = np.where(lt, e - 1, e)
    m = np.where(lt, (m + m) - f32(1.0), m - f32(1.0)).astype(f32)
    z = m * m
    y = np.full_like(m, LOG_P[0])
    for c in LOG_P[1:]:
        y = y * m + c
    y = y * m
    y = y * z
    ef = e.astype(f32)
    y = y + EXP_C2 * ef
    y = y + f32(-0.5) * z
    r = m + y
    r = r + EXP_C1 * ef
    return r.astype(f32)


def softplus_f(x):
    x = x.astype(f32)
    mid = log_f(f32(1.0) + exp_f(np.minimum(x, f32(20.0))))
    return np.where(x > f32(20.0), x, np.where(x < f32(-15.0), exp_f(x), mid)).astype(f32)


def sigmoid_f(x):
    x = x.astype(f32)
    xs = np.maximum(x, f32(-80.0))
    with np.errstate(over="ignore"):
        main = f32(1.0) / (f32(1.0) + exp_f(-xs))
    return np.where(x < f32(-80.0), exp_f(x), main).astype(f32)


def silu_f(x):
    return (x.astype(f32) * sigmoid_f(x)).astype(f32)


def treesum(x: np.ndarray) -> np.float32:
    p = 1
    while p < len(x):
        p *= 2
    s = np.zeros(p, f32)
    s[: len(x)] = x
    while len(s) > 1:
        s = (s[0::2] + s[1::2]).astype(f32)
    return s[0]


def quant_act_i8g(x: np.ndarray):
    g = len(x) // 128
    xs = x.reshape(g, 128).astype(f32)
    s_g = (np.abs(xs).max(axis=1) / f32(127.0)).astype(f32)
    smax = s_g.max()
    sx = f32(1.0) if smax == 0 else f32(smax / f32(65535.0))
    m = np.rint(s_g / sx).astype(f32)
    m = np.clip(m, f32(1.0), f32(65535.0))
    mx = m.astype(np.uint16)
    inv = (f32(1.0) / (sx * mx.astype(f32))).astype(f32)
    q = np.clip(np.rint(xs * inv[:, None]), -127, 127).astype(np.int8)
    return q.reshape(-1), sx, mx


def unpack_row(packed: np.ndarray, bits: int, k: int) -> np.ndarray:
    out = np.zeros(k, np.int8)
    if bits == 8:
        return packed.view(np.int8).copy()
    per = 16 if bits == 4 else 24
    for blk in range(k // 32):
        b = packed[blk * per:(blk + 1) * per].astype(np.int32)
        lo = np.concatenate([b[:16] & 0xF, b[:16] >> 4])
        if bits == 4:
            out[blk * 32:(blk + 1) * 32] = lo - 8
        else:
            hi = np.array([(b[16 + i % 8] >> (2 * (i // 8))) & 3 for i in range(32)])
            out[blk * 32:(blk + 1) * 32] = (lo | (hi << 4)) - 32
    return out


def gemm_row(wq, c, m, xq, sx, mx):
    k = len(wq)
    acc = 0
    for g in range(k // 128):
        part = int(np.dot(wq[g * 128:(g + 1) * 128].astype(np.int64), xq[g * 128:(g + 1) * 128].astype(np.int64)))
        acc += int(m[g]) * int(mx[g]) * part
    return f32(f32(f32(acc) * f32(c)) * f32(sx))


def splitmix64(state: int):
    mask = (1 << 64) - 1
    state = (state + 0x9E3779B97F4A7C15) & mask
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    return state, z ^ (z >> 31)


def sample_weights(logits: np.ndarray, inv_temp: np.float32) -> np.ndarray:
    l = (logits.astype(f32) * f32(inv_temp)).astype(f32)
    return np.rint(exp_f(l - l.max()).astype(f32) * f32(4294967296.0)).astype(np.uint64)


def main():
    rng = np.random.default_rng(20261125)
    x = np.concatenate([
        (rng.random(4000) * 200 - 100).astype(f32),
        (rng.integers(0, 1 << 23, 500, dtype=np.uint32)).view(f32),                      # positive denormals
        (rng.integers(0, 1 << 23, 500, dtype=np.uint32) | np.uint32(0x80000000)).view(f32),  # negative denormals
        np.array([0.0, -0.0, 88.0, 89.0, -87.0, -87.00001, -86.99999, 20.0, 20.000002, -15.0, -15.000001, -80.0,
                  -80.00001, np.inf, -np.inf, 1e-38, -1e-38, 1.0, -1.0, 0.5], f32),
    ])
    pos = (np.abs(x) + f32(1e-30)).astype(f32)
    pos = pos[np.isfinite(pos)]
    rows = (rng.random((6, 5120)) * 2 - 1).astype(f32)
    rows[:, ::97] = (rng.integers(1, 1 << 23, rows[:, ::97].shape, dtype=np.uint32)).view(f32)
    tree_in = [rows[i, :n] for i, n in enumerate((5120, 4096, 1000, 128, 3, 1))]
    qx = (rng.random((5, 1024)) * 2 - 1).astype(f32) * np.array([1.0, 1e-3, 1e-20, 0.0, 1e3], f32)[:, None]
    qx[2, ::2] = (rng.integers(1, 1 << 23, 512, dtype=np.uint32)).view(f32)
    q_out, sx_out, mx_out = zip(*(quant_act_i8g(r) for r in qx))
    k = 512
    packed = {b: rng.integers(0, 256, k // 32 * per, dtype=np.uint8) for b, per in ((4, 16), (6, 24), (8, 32))}
    unpacked = {b: unpack_row(p, b, k) for b, p in packed.items()}
    xq = rng.integers(-127, 128, k).astype(np.int8)
    m, mx = rng.integers(1, 65536, k // 128).astype(np.uint16), rng.integers(1, 65536, k // 128).astype(np.uint16)
    gemm_out = np.array([gemm_row(unpacked[b], 3.1e-7, m, xq, 1.7e-3, mx) for b in (4, 6, 8)], f32)
    states, outs, s = [], [], 0
    for _ in range(8):
        s, z = splitmix64(s)
        states.append(s)
        outs.append(z)
    logits = (rng.random(4096) * 24 - 12).astype(f32)
    np.savez_compressed(
        OUT, x=x, exp=exp_f(x), sigmoid=sigmoid_f(x), silu=silu_f(x), softplus=softplus_f(x), pos=pos, log=log_f(pos),
        tree_rows=rows, tree_len=np.array([len(t) for t in tree_in]), tree_out=np.array([treesum(t) for t in tree_in], f32),
        qx=qx, q_codes=np.stack(q_out), q_sx=np.array(sx_out, f32), q_mx=np.stack(mx_out),
        packed4=packed[4], packed6=packed[6], packed8=packed[8], codes4=unpacked[4], codes6=unpacked[6], codes8=unpacked[8],
        gemm_xq=xq, gemm_m=m, gemm_mx=mx, gemm_out=gemm_out,
        sm_states=np.array(states, np.uint64), sm_outs=np.array(outs, np.uint64),
        logits=logits, weights_1=sample_weights(logits, f32(1.0)), weights_07=sample_weights(logits, f32(1.0) / f32(0.7)))
    print("wrote", OUT, OUT.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
