"""Single-linear integer GEMM at the benchmark shapes (the GEMM-sweep configuration: K=5120 x N=17408 and the transposed FFN
shape), through det_gemm_ex on both weight layouts, bit for bit against the oracle's gemm_row."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

PER32 = {8: 32, 6: 24, 4: 16}


def _det_rows(rng, n, k, bits):
    """Random det rows: random code bytes (every code value occurs), c in [1e-8, 1e-6], m in [1, 65535]."""
    nc = k // 32 * PER32[bits]
    g = k // 128
    rows = np.zeros((n, nc + 4 + 2 * g), np.uint8)
    rows[:, :nc] = rng.integers(0, 256, (n, nc), dtype=np.uint8)
    c = (rng.random(n, dtype=np.float32) * 1e-6 + 1e-8).astype(np.float32)
    m = rng.integers(1, 65536, (n, g)).astype(np.uint16)
    rows[:, nc:nc + 4] = c.view(np.uint8).reshape(n, 4)
    rows[:, nc + 4:] = m.view(np.uint8).reshape(n, 2 * g)
    return rows, c, m, nc


@pytest.mark.parametrize("n,k,bits,ms", [
    (17408, 5120, 6, [1, 4, 8, 16, 70]),
    (17408, 5120, 8, [1, 3]),
    (17408, 5120, 4, [1, 5]),
    (5120, 17408, 6, [1, 2, 40]),
    (5120, 6144, 6, [1]),
])
def test_gemm_matches_oracle(n, k, bits, ms, libs, oracle):
    d = libs.cuda()
    rng = np.random.default_rng(n + k + bits)
    rows, c, m, nc = _det_rows(rng, n, k, bits)
    g = k // 128
    wq, cc, mm = d.det_malloc(n * nc), d.det_malloc(n * 4), d.det_malloc(n * g * 2)
    codes = np.ascontiguousarray(rows[:, :nc])
    d.det_memcpy(wq, codes.ctypes.data, codes.nbytes, None)
    d.det_memcpy(cc, c.ctypes.data, c.nbytes, None)
    d.det_memcpy(mm, m.ctypes.data, m.nbytes, None)
    src = libs.QLinear(wq, cc, mm, n, k, bits)
    sp = d.det_malloc(d.det_linear_repack_bytes(n, k, bits))
    d.det_linear_repack(C.byref(src), sp, None)
    stream = libs.QLinear(sp, cc, mm, n, k, bits | libs.DET_LAYOUT_STREAM)
    w8 = d.det_malloc(d.det_linear_expand_bytes(n, k))
    d.det_linear_expand(C.byref(src), w8, None)
    tensor = libs.QLinear(w8, cc, mm, n, k, bits | libs.DET_LAYOUT_INT8)
    try:
        for mtok in ms:
            xq = rng.integers(-127, 128, (mtok, k)).astype(np.int8)
            sx = (1e-3 * (0.5 + rng.random(mtok))).astype(np.float32)
            mx = rng.integers(1, 65536, (mtok, g)).astype(np.uint16)
            want = np.zeros((mtok, n), np.float32)
            oracle.orc_gemm(rows.ctypes.data, n, k, bits, xq.ctypes.data, sx.ctypes.data, mx.ctypes.data, mtok,
                            want.ctypes.data, 0)
            dx, ds, dm, dy = d.det_malloc(xq.nbytes), d.det_malloc(sx.nbytes), d.det_malloc(mx.nbytes), d.det_malloc(want.nbytes)
            d.det_memcpy(dx, xq.ctypes.data, xq.nbytes, None)
            d.det_memcpy(ds, sx.ctypes.data, sx.nbytes, None)
            d.det_memcpy(dm, mx.ctypes.data, mx.nbytes, None)
            cases = [("stream", stream, 0), ("rowmajor", src, 0)]
            # every tile instantiation of the tensor-core kernel (0 = the one the shape selects)
            cases += [(f"int8 tensor-core, tile variant {v}", tensor, v) for v in (0, 1, 2, 3)]
            # K split over several CTAs per tile (takes effect on the shapes with few row tiles)
            cases += [(f"int8 tensor-core, split K, tile variant {v}", tensor, v | 0x100) for v in (0, 1, 2)]
            for name, lin, variant in cases:
                got = np.zeros_like(want)
                d.det_memset(dy, 0xFF, want.nbytes, None)
                d.det_debug_set_tc_variant(variant | (0 if variant & 0x100 else 0x200))   # K split only where asked for
                d.det_gemm(C.byref(lin), dx, ds, dm, mtok, dy, None)
                d.det_debug_set_tc_variant(0x100)                                         # back to the defaults
                d.det_memcpy(got.ctypes.data, dy, got.nbytes, None)
                d.det_sync()
                bad = int((got.view(np.uint32) != want.view(np.uint32)).sum())
                assert bad == 0, f"{name} layout, M={mtok}: {bad} of {want.size} outputs differ"
            for p in (dx, ds, dm, dy):
                d.det_free(p)
        assert d.det_last_error() == 0
    finally:
        for p in (wq, cc, mm, sp, w8):
            d.det_free(p)


def _upload(d, arr):
    p = d.det_malloc(arr.nbytes)
    d.det_memcpy(p, arr.ctypes.data, arr.nbytes, None)
    return p


@pytest.mark.parametrize("n,k,bits,ms", [
    (17408, 5120, 6, [64, 512, 2048]),
    (17408, 5120, 8, [512]),
    (17408, 5120, 4, [512]),
    (5120, 17408, 6, [64, 512]),
])
def test_large_batch_gemm_matches_oracle(n, k, bits, ms, libs, oracle):
    """The prefill sizes of the GEMM sweep (M = 64, 512, 2048 at K=5120 x N=17408, W6 / W8 / W4, and the transposed FFN
    shape): every tile instantiation of the tensor-core kernel against spec gemm_row.  gemm_row over all M * N outputs
    would take minutes of scalar CPU time, so the oracle computes complete 128-row tiles — the first, the last and three
    seeded ones, every token — and the remaining rows are compared with this backend's row-major CUDA-core kernel, a
    different kernel that the small-M test above pins to gemm_row on its own."""
    d = libs.cuda()
    rng = np.random.default_rng(7 * n + k + bits)
    rows, c, m, nc = _det_rows(rng, n, k, bits)
    g = k // 128
    codes = np.ascontiguousarray(rows[:, :nc])
    wq, cc, mm = _upload(d, codes), _upload(d, c), _upload(d, m)
    src = libs.QLinear(wq, cc, mm, n, k, bits)
    w8 = d.det_malloc(d.det_linear_expand_bytes(n, k))
    d.det_linear_expand(C.byref(src), w8, None)
    tensor = libs.QLinear(w8, cc, mm, n, k, bits | libs.DET_LAYOUT_INT8)
    tiles = sorted({0, n // 128 - 1, *(int(x) for x in rng.integers(1, n // 128 - 1, 3))})
    pick = np.concatenate([np.arange(t * 128, t * 128 + 128) for t in tiles])
    sub = np.ascontiguousarray(rows[pick])
    try:
        for mtok in ms:
            xq = rng.integers(-127, 128, (mtok, k)).astype(np.int8)
            sx = (1e-3 * (0.5 + rng.random(mtok))).astype(np.float32)
            mx = rng.integers(1, 65536, (mtok, g)).astype(np.uint16)
            want = np.zeros((mtok, len(pick)), np.float32)
            oracle.orc_gemm(sub.ctypes.data, len(pick), k, bits, xq.ctypes.data, sx.ctypes.data, mx.ctypes.data, mtok,
                            want.ctypes.data, 0)
            dx, ds, dm = _upload(d, xq), _upload(d, sx), _upload(d, mx)
            dy = d.det_malloc(mtok * n * 4)
            base = np.zeros((mtok, n), np.float32)
            d.det_gemm(C.byref(src), dx, ds, dm, mtok, dy, None)
            d.det_memcpy(base.ctypes.data, dy, base.nbytes, None)
            d.det_sync()
            bad = int((base[:, pick].view(np.uint32) != want.view(np.uint32)).sum())
            assert bad == 0, f"row-major kernel, M={mtok}: {bad} of {want.size} outputs differ from gemm_row"
            for variant in libs.TC_VARIANTS_LARGE:
                got = np.zeros_like(base)
                d.det_memset(dy, 0xFF, base.nbytes, None)
                d.det_debug_set_tc_variant(variant)
                d.det_gemm(C.byref(tensor), dx, ds, dm, mtok, dy, None)
                d.det_debug_set_tc_variant(0x200)
                d.det_memcpy(got.ctypes.data, dy, got.nbytes, None)
                d.det_sync()
                bad = int((got[:, pick].view(np.uint32) != want.view(np.uint32)).sum())
                assert bad == 0, f"tensor-core variant {variant:#x}, M={mtok}: {bad} of {want.size} outputs differ from gemm_row"
                bad = int((got.view(np.uint32) != base.view(np.uint32)).sum())
                assert bad == 0, f"tensor-core variant {variant:#x}, M={mtok}: {bad} of {base.size} outputs differ from the row-major kernel"
            # accumulate form on the tile the shape selects: y += result is one fp32 add per element
            prev = (rng.random((mtok, n), dtype=np.float32) - 0.5).astype(np.float32)
            d.det_memcpy(dy, prev.ctypes.data, prev.nbytes, None)
            d.det_gemm_ex(C.byref(tensor), dx, ds, dm, mtok, dy, 1, 0, None, None, None)
            got = np.zeros_like(base)
            d.det_memcpy(got.ctypes.data, dy, got.nbytes, None)
            d.det_sync()
            assert np.array_equal(got.view(np.uint32), (prev + base).view(np.uint32)), f"accumulate, M={mtok}"
            for p in (dx, ds, dm, dy):
                d.det_free(p)
        assert d.det_last_error() == 0
    finally:
        for p in (wq, cc, mm, w8):
            d.det_free(p)


def _expanded(d, libs, rng, n, k, bits):
    rows, c, m, nc = _det_rows(rng, n, k, bits)
    g = k // 128
    wq, cc, mm = d.det_malloc(n * nc), d.det_malloc(n * 4), d.det_malloc(n * g * 2)
    codes = np.ascontiguousarray(rows[:, :nc])
    d.det_memcpy(wq, codes.ctypes.data, codes.nbytes, None)
    d.det_memcpy(cc, c.ctypes.data, c.nbytes, None)
    d.det_memcpy(mm, m.ctypes.data, m.nbytes, None)
    src = libs.QLinear(wq, cc, mm, n, k, bits)
    w8 = d.det_malloc(d.det_linear_expand_bytes(n, k))
    d.det_linear_expand(C.byref(src), w8, None)
    d.det_sync()
    return libs.QLinear(w8, cc, mm, n, k, bits | libs.DET_LAYOUT_INT8), [wq, cc, mm, w8]


@pytest.mark.parametrize("n1,n2,k,mtok", [(1000, 96, 1024, 32), (16384, 96, 5120, 32), (640, 300, 2560, 100), (5120, 96, 6144, 20),
                                          (2048, 96, 5120, 512)])
def test_pair_launch_equals_two_launches(n1, n2, k, mtok, libs):
    """det_gemm_pair — a W6 linear and a small W8 linear over the same rows in one tensor-core launch, each with two
    routed parts — against two det_gemm_ex calls, bit for bit (ragged last row tiles, the K split, every token tile)."""
    d = libs.cuda()
    rng = np.random.default_rng(n1 + n2 + k + mtok)
    g = k // 128
    l1, b1 = _expanded(d, libs, rng, n1, k, 6)
    l2, b2 = _expanded(d, libs, rng, n2, k, 8)
    xq = rng.integers(-127, 128, (mtok, k)).astype(np.int8)
    sx = (1e-3 * (0.5 + rng.random(mtok))).astype(np.float32)
    mx = rng.integers(1, 65536, (mtok, g)).astype(np.uint16)
    dx, ds, dm = d.det_malloc(xq.nbytes), d.det_malloc(sx.nbytes), d.det_malloc(mx.nbytes)
    d.det_memcpy(dx, xq.ctypes.data, xq.nbytes, None)
    d.det_memcpy(ds, sx.ctypes.data, sx.nbytes, None)
    d.det_memcpy(dm, mx.ctypes.data, mx.nbytes, None)
    d.det_debug_set_tc_variant(0x100)
    cut1, cut2 = n1 // 2 // 4 * 4, n2 // 3
    widths = [(cut1, n1 - cut1), (cut2, n2 - cut2)]
    outs = []
    for pair in (False, True):
        bufs = [[d.det_malloc(mtok * w * 4) for w in ws] for ws in widths]
        for ws, bs in zip(widths, bufs):
            for w, b in zip(ws, bs):
                d.det_memset(b, 0xFF, mtok * w * 4, None)
        offs = [(C.c_int * 2)(0, ws[0]) for ws in widths]
        dsts = [(C.c_void_p * 2)(*bs) for bs in bufs]
        if pair:
            d.det_gemm_pair(C.byref(l1), C.byref(l2), dx, ds, dm, mtok, 2, offs[0], dsts[0], 2, offs[1], dsts[1], None)
        else:
            d.det_gemm_ex(C.byref(l1), dx, ds, dm, mtok, None, 0, 2, offs[0], dsts[0], None)
            d.det_gemm_ex(C.byref(l2), dx, ds, dm, mtok, None, 0, 2, offs[1], dsts[1], None)
        got = []
        for ws, bs in zip(widths, bufs):
            for w, b in zip(ws, bs):
                a = np.zeros((mtok, w), np.float32)
                d.det_memcpy(a.ctypes.data, b, a.nbytes, None)
                d.det_sync()
                got.append(a.view(np.uint32))
                d.det_free(b)
        outs.append(got)
    for i, (u, f) in enumerate(zip(*outs)):
        assert np.isfinite(u.view(np.float32)).all() and np.array_equal(u, f), f"part {i}: {(u != f).sum()} of {u.size} differ"
    assert d.det_last_error() == 0
    for p in b1 + b2 + [dx, ds, dm]:
        d.det_free(p)
