"""Prefill attention on the tensor cores against the CUDA-core kernels of the same library, through det_attention.

The CUDA-core path is pinned to the CPU oracle by the conformance suite (tests/test_conformance_gpu.py, which also runs
its batches of 16, 40, 100 and 200 tokens through the tensor path); here the two paths meet on shapes the oracle would
take minutes for: the 27B head geometry (24 q heads on 4 kv heads, head_dim 256), chunked prefill behind a filled
cache, a context past 16384 keys (the key-split launch), a workspace so small that the rows go in several rounds, and a
batch with probabilities that hit 2^24 in many columns (equal scores).  Everything must agree bit for bit, cache rows
included."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HD, ROT = 256, 64


class Dev:
    def __init__(self, cu):
        self.cu, self.bufs = cu, []

    def up(self, a):
        a = np.ascontiguousarray(a)
        p = self.cu.det_malloc(a.nbytes)
        assert p
        self.cu.det_memcpy(p, a.ctypes.data, a.nbytes, None)
        self.bufs.append(p)
        return p

    def zeros(self, nbytes):
        p = self.cu.det_malloc(nbytes)
        assert p
        self.bufs.append(p)
        return p

    def down(self, p, shape, dtype):
        out = np.zeros(shape, dtype)
        self.cu.det_memcpy(out.ctypes.data, p, out.nbytes, None)
        self.cu.det_sync()
        return out

    def free(self):
        self.cu.det_sync()
        for p in self.bufs:
            self.cu.det_free(p)
        self.bufs = []


def run_case(libs, rng, n_h, n_kv, chunks, pos_start, tc, ctx=None, equal_scores=False):
    """Runs the chunks (list of batch sizes) one after the other from position pos_start behind a cache whose first
    pos_start rows hold random codes; returns every output and the final cache."""
    cu = libs.cuda()
    cu.det_debug_set_attn_tc(1 if tc else 0, 0)
    d = Dev(cu)
    total = pos_start + sum(chunks)
    ctx = ctx or total
    kq = np.zeros((ctx, n_kv, HD), np.int8)
    sk = np.zeros((ctx, n_kv), np.float32)
    vq = np.zeros((ctx, n_kv, HD), np.int16)
    kq[:pos_start] = rng.integers(-127, 128, (pos_start, n_kv, HD), dtype=np.int8)
    sk[:pos_start] = rng.uniform(0.001, 0.02, (pos_start, n_kv)).astype(np.float32)
    vq[:pos_start] = rng.integers(-32767, 32768, (pos_start, n_kv, HD), dtype=np.int16)
    if equal_scores:
        kq[:pos_start] = kq[0]
        sk[:pos_start] = sk[0]
    d_kq, d_sk, d_vq = d.up(kq), d.up(sk), d.up(vq)
    layer = libs.AttnLayer(d.up(rng.uniform(0.5, 1.5, HD).astype(np.float32)), d.up(rng.uniform(0.5, 1.5, HD).astype(np.float32)),
                           d.up(np.full(n_kv, 1 / 1024, np.float32)), d.up(np.full(n_kv, 1024.0, np.float32)))
    cache = libs.KvCache(d_kq, d_sk, d_vq, ctx, None, None)
    ang = np.arange(ctx)[:, None] * (1e7 ** (-np.arange(ROT // 2) * 2.0 / ROT))[None, :]
    d_cos, d_sin = d.up(np.cos(ang).astype(np.float32)), d.up(np.sin(ang).astype(np.float32))
    outs, pos = [], pos_start
    for m in chunks:
        qg = rng.standard_normal((m, n_h, 2 * HD)).astype(np.float32)
        k = rng.standard_normal((m, n_kv, HD)).astype(np.float32)
        v = (rng.standard_normal((m, n_kv, HD)) * 3).astype(np.float32)
        if equal_scores:
            qg[:, :, :HD] = 0          # every score is 0: every unmasked probability is exactly 2^24
        d_o = d.zeros(m * n_h * HD * 4)
        scratch = d.zeros(cu.det_attn_scratch_bytes(m, n_h, HD))
        cu.det_attention(C.byref(layer), C.byref(cache), d.up(qg), d.up(k), d.up(v), d_cos, d_sin, ROT, 1e-6, m, pos, n_h,
                         n_kv, HD, d_o, scratch, None)
        outs.append(d.down(d_o, (m, n_h, HD), np.float32))
        pos += m
    res = (outs, d.down(d_kq, kq.shape, np.int8), d.down(d_sk, sk.shape, np.float32), d.down(d_vq, vq.shape, np.int16))
    assert cu.det_last_error() == 0
    d.free()
    cu.det_debug_set_attn_tc(1, 0)
    return res


def same(a, b):
    outs_a, kq_a, sk_a, vq_a = a
    outs_b, kq_b, sk_b, vq_b = b
    assert np.array_equal(kq_a, kq_b) and np.array_equal(vq_a, vq_b) and np.array_equal(sk_a.view(np.uint32), sk_b.view(np.uint32))
    for i, (x, y) in enumerate(zip(outs_a, outs_b)):
        assert np.isfinite(x).all()
        bad = np.argwhere(x.view(np.uint32) != y.view(np.uint32))
        assert bad.size == 0, (i, len(bad), bad[:4], x[tuple(bad[0])], y[tuple(bad[0])])


@pytest.mark.parametrize("n_h,n_kv,chunks,pos_start", [
    (24, 4, [512, 512], 0),          # 27B geometry, two prefill chunks from an empty cache
    (24, 4, [16, 100, 21, 200], 37), # ragged batches behind a filled cache; 21 tokens x 6 heads = 126 rows: a short tile
    (16, 4, [256], 1500),            # 4B geometry deep in a context
    (8, 2, [64, 64], 130),           # tiny geometry (rep 4)
    (8, 8, [48], 200),               # one q head per kv head
])
def test_tensor_path_equals_cuda_core_path(libs, n_h, n_kv, chunks, pos_start):
    assert libs.cuda().det_init() == 0
    a = run_case(libs, np.random.default_rng(42), n_h, n_kv, chunks, pos_start, tc=True)
    b = run_case(libs, np.random.default_rng(42), n_h, n_kv, chunks, pos_start, tc=False)
    same(a, b)


def test_context_past_16384_keys_uses_the_key_split(libs):
    assert libs.cuda().det_init() == 0
    a = run_case(libs, np.random.default_rng(7), 24, 4, [64], 16500, tc=True)
    b = run_case(libs, np.random.default_rng(7), 24, 4, [64], 16500, tc=False)
    same(a, b)


def test_probabilities_of_exactly_two_to_the_24(libs):
    """All scores equal: every unmasked p is 2^24 = (2^24 - 1) + 1, so all three byte slices are 255 everywhere and the
    separate plane of ones carries the rest."""
    assert libs.cuda().det_init() == 0
    a = run_case(libs, np.random.default_rng(3), 24, 4, [128], 300, tc=True, equal_scores=True)
    b = run_case(libs, np.random.default_rng(3), 24, 4, [128], 300, tc=False, equal_scores=True)
    same(a, b)


def test_small_workspace_runs_in_rounds_and_none_falls_back(libs):
    cu = libs.cuda()
    assert cu.det_init() == 0
    want = run_case(libs, np.random.default_rng(11), 24, 4, [384], 640, tc=False)
    # 1024 keys: V planes 2 MB + 2 MB per row tile; 7 MB holds two of the 18 row tiles per round
    ws = cu.det_malloc(7 << 20)
    cu.det_attn_set_workspace(ws, 7 << 20)
    try:
        same(run_case(libs, np.random.default_rng(11), 24, 4, [384], 640, tc=True), want)
        cu.det_attn_set_workspace(None, 0)      # no workspace: the CUDA-core kernels take the call
        same(run_case(libs, np.random.default_rng(11), 24, 4, [384], 640, tc=True), want)
    finally:
        big = cu.det_malloc(256 << 20)
        cu.det_attn_set_workspace(big, 256 << 20)
        cu.det_free(ws)
