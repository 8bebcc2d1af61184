"""det_gemv — one decode GEMV launch with its neighbours fused in — against the separate calls it replaces
(det_rmsnorm_quant / det_quant, det_gemm_ex per linear, det_silu_mul_quant), bit for bit: the activation quantization as
the prologue (on the edge-case rows the reference's norms suite uses, crates/det/src/conformance.rs:462-498: all-denormal
rows, denormal/zero alternation, mixed magnitudes, squares that underflow), a second W8 linear riding in the same launch,
the pairs layout with plain outputs, and the SwiGLU product from the epilogue."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

PER32 = {8: 32, 6: 24, 4: 16}


def _rows(rng, m, n):
    x = np.zeros((m, n), np.float32)
    den = lambda size: (rng.integers(1, 1 << 23, size, dtype=np.uint32) | (rng.integers(0, 2, size, dtype=np.uint32) << 31)).view(np.float32)
    for r in range(m):
        kind = r % 6
        if kind == 0:
            x[r] = den(n)
        elif kind == 1:
            x[r, ::2] = den(n // 2)
        elif kind == 2:
            scales = np.array([1e-20, 1e-23, 0, 1.0, 0.0, 1e-30, -0.0, 1e3], np.float32)
            x[r] = (rng.random(n, dtype=np.float32) * 2 - 1) * scales[np.arange(n) % 8]
            x[r, 2::8] = den(len(x[r, 2::8]))
        elif kind == 3:
            x[r] = (rng.random(n, dtype=np.float32) * 2 - 1) * np.where(np.arange(n) % 5 == 0, 1e-19, 1e-38).astype(np.float32)
        else:
            x[r] = (rng.random(n, dtype=np.float32) * 2 - 1) * (10.0 ** -((np.arange(n) // 128) % 4)).astype(np.float32)
    return x


def _dev(d, arr):
    p = d.det_malloc(max(arr.nbytes, 16))
    d.det_memcpy(p, arr.ctypes.data, arr.nbytes, None)
    return p


def _host(d, p, like):
    out = np.zeros_like(like)
    d.det_memcpy(out.ctypes.data, p, out.nbytes, None)
    d.det_sync()
    return out


def _linear(d, libs, rng, n, k, bits, pairs=False):
    """(reference-layout linear, streaming-layout linear, buffers to free)"""
    g, nc = k // 128, k // 32 * PER32[bits]
    wq = _dev(d, rng.integers(0, 256, n * nc, dtype=np.uint8))
    cc = _dev(d, (rng.random(n, dtype=np.float32) * 1e-6 + 1e-8).astype(np.float32))
    mm = _dev(d, rng.integers(1, 65536, n * g).astype(np.uint16))
    src = libs.QLinear(wq, cc, mm, n, k, bits)
    sp = d.det_malloc(d.det_linear_repack_bytes(n, k, bits))
    if pairs:
        d.det_linear_repack_pairs(C.byref(src), sp, None)
    else:
        d.det_linear_repack(C.byref(src), sp, None)
    tag = bits | libs.DET_LAYOUT_STREAM | (libs.DET_LAYOUT_PAIRS if pairs else 0)
    return src, libs.QLinear(sp, cc, mm, n, k, tag), [wq, cc, mm, sp]


@pytest.mark.parametrize("n_out,k,bits,m", [(512, 2560, 6, 6), (384, 5120, 6, 1), (640, 1024, 8, 8),
                                            (256, 2048, 4, 5), (130, 384, 6, 2), (96, 6144, 8, 1)])
@pytest.mark.parametrize("kind", [1, 2])
def test_prologue_equals_separate_quantization(n_out, k, bits, m, kind, libs):
    d = libs.cuda()
    rng = np.random.default_rng(k + bits + kind)
    g = k // 128
    src, lin, bufs = _linear(d, libs, rng, n_out, k, bits)
    a = _rows(rng, m, k)
    b = (1.0 + (rng.random(k, dtype=np.float32) * 2 - 1)).astype(np.float32)
    da, db = _dev(d, a), _dev(d, b)
    y0 = (rng.random((m, n_out), dtype=np.float32) * 2 - 1).astype(np.float32)
    outs = []
    for fused in (False, True):
        xq, sx, mx = d.det_malloc(m * k), d.det_malloc(m * 4), d.det_malloc(m * g * 2)
        y, yacc = d.det_malloc(m * n_out * 4), _dev(d, y0)
        if fused:
            s = libs.ActSource(kind, da, db, 1e-6, xq, sx, mx)
            op = libs.GemvOp(lin=C.pointer(lin), src=C.pointer(s), M=m, y=y)
            d.det_gemv(C.byref(op), None)
            s2 = libs.ActSource(kind, da, db, 1e-6, None, None, None)
            op2 = libs.GemvOp(lin=C.pointer(lin), src=C.pointer(s2), M=m, y=yacc, accumulate=1)
            d.det_gemv(C.byref(op2), None)
        else:
            if kind == 1:
                d.det_rmsnorm_quant(da, db, 1e-6, m, k, None, xq, sx, mx, None)
            else:
                d.det_quant(da, m, k, xq, sx, mx, None)
            d.det_gemm_ex(C.byref(src), xq, sx, mx, m, y, 0, 0, None, None, None)      # the row-major kernel
            d.det_gemm_ex(C.byref(lin), xq, sx, mx, m, yacc, 1, 0, None, None, None)   # the streaming kernel, no prologue
        outs.append((_host(d, y, y0).view(np.uint32), _host(d, yacc, y0).view(np.uint32),
                     _host(d, xq, np.zeros(m * k, np.int8)), _host(d, sx, np.zeros(m, np.float32)).view(np.uint32),
                     _host(d, mx, np.zeros(m * g, np.uint16))))
        for p in (xq, sx, mx, y, yacc):
            d.det_free(p)
    for name, u, f in zip(("y", "y accumulate", "codes", "scales", "multipliers"), outs[0], outs[1]):
        assert np.array_equal(u, f), f"{name}: {(u != f).sum()} of {u.size} differ"
    assert d.det_last_error() == 0
    for p in bufs + [da, db]:
        d.det_free(p)


@pytest.mark.parametrize("n1,n2,k,m", [(1024, 96, 5120, 1), (600, 32, 1024, 3), (16384, 96, 5120, 2)])
def test_second_linear_rides_in_the_same_launch(n1, n2, k, m, libs):
    """qkv|z (W6, two parts) + a|b (W8, two parts) over the same RMSNorm-quantized row: one det_gemv launch against
    det_rmsnorm_quant + two det_gemm_ex."""
    d = libs.cuda()
    rng = np.random.default_rng(n1 + n2 + k)
    g = k // 128
    src1, lin1, b1 = _linear(d, libs, rng, n1, k, 6)
    src2, lin2, b2 = _linear(d, libs, rng, n2, k, 8)
    x = (rng.standard_normal((m, k)) * 0.7).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    dx, dw = _dev(d, x), _dev(d, w)
    cut1, cut2 = (n1 // 8) * 5, n2 // 2
    want = None
    for fused in (False, True):
        xq, sx, mx = d.det_malloc(m * k), d.det_malloc(m * 4), d.det_malloc(m * g * 2)
        pa, pb = d.det_malloc(m * cut1 * 4), d.det_malloc(m * (n1 - cut1) * 4)
        pc, pd = d.det_malloc(m * cut2 * 4), d.det_malloc(m * (n2 - cut2) * 4)
        offs1, offs2 = (C.c_int * 2)(0, cut1), (C.c_int * 2)(0, cut2)
        dsts1, dsts2 = (C.c_void_p * 2)(pa, pb), (C.c_void_p * 2)(pc, pd)
        if fused:
            s = libs.ActSource(libs.DET_ACT_RMSNORM, dx, dw, 1e-6, None, None, None)
            op = libs.GemvOp(lin=C.pointer(lin1), lin2=C.pointer(lin2), src=C.pointer(s), M=m, nparts=2, offs=offs1,
                             dsts=dsts1, nparts2=2, offs2=offs2, dsts2=dsts2)
            d.det_gemv(C.byref(op), None)
        else:
            d.det_rmsnorm_quant(dx, dw, 1e-6, m, k, None, xq, sx, mx, None)
            d.det_gemm_ex(C.byref(src1), xq, sx, mx, m, None, 0, 2, offs1, dsts1, None)
            d.det_gemm_ex(C.byref(src2), xq, sx, mx, m, None, 0, 2, offs2, dsts2, None)
        got = [_host(d, p, np.zeros(m * wd, np.float32)).view(np.uint32) for p, wd in
               ((pa, cut1), (pb, n1 - cut1), (pc, cut2), (pd, n2 - cut2))]
        if want is None:
            want = got
        else:
            for i, (u, f) in enumerate(zip(want, got)):
                assert np.array_equal(u, f), f"part {i}: {(u != f).sum()} of {u.size} differ"
        for p in (xq, sx, mx, pa, pb, pc, pd):
            d.det_free(p)
    assert d.det_last_error() == 0
    for p in b1 + b2 + [dx, dw]:
        d.det_free(p)


@pytest.mark.parametrize("half,k,m", [(1536, 1024, 1), (17408, 5120, 1), (640, 2560, 4), (17408, 5120, 3), (9216, 2560, 8)])
def test_pairs_layout_plain_outputs_and_swiglu_epilogue(half, k, m, libs):
    """gate|up stored with interleaved rows: plain two-part outputs come back in the linear's own order, and the SwiGLU
    product from the epilogue followed by the plain-quantization prologue of a second GEMV equals det_silu_mul_quant +
    det_gemm_ex."""
    d = libs.cuda()
    rng = np.random.default_rng(half + k)
    n, g = 2 * half, k // 128
    src, lin, b1 = _linear(d, libs, rng, n, k, 6, pairs=True)
    n_down = 256
    src_d, lin_d, b2 = _linear(d, libs, rng, n_down, half, 6)
    xq = _dev(d, rng.integers(-127, 128, (m, k)).astype(np.int8))
    sx = _dev(d, (1e-3 * (0.5 + rng.random(m))).astype(np.float32))
    mx = _dev(d, rng.integers(1, 65536, (m, g)).astype(np.uint16))
    pg, pu = d.det_malloc(m * half * 4), d.det_malloc(m * half * 4)
    offs, dsts = (C.c_int * 2)(0, half), (C.c_void_p * 2)(pg, pu)
    # reference: row-major kernel -> gate, up; det_silu_mul_quant; down projection
    d.det_gemm_ex(C.byref(src), xq, sx, mx, m, None, 0, 2, offs, dsts, None)
    want_g, want_u = _host(d, pg, np.zeros(m * half, np.float32)), _host(d, pu, np.zeros(m * half, np.float32))
    hq, sh, mh = d.det_malloc(m * half), d.det_malloc(m * 4), d.det_malloc(m * (half // 128) * 2)
    yd = d.det_malloc(m * n_down * 4)
    d.det_silu_mul_quant(pg, pu, m, half, None, hq, sh, mh, None)
    d.det_gemm_ex(C.byref(src_d), hq, sh, mh, m, yd, 0, 0, None, None, None)
    want_y = _host(d, yd, np.zeros(m * n_down, np.float32)).view(np.uint32)
    want_hq = _host(d, hq, np.zeros(m * half, np.int8))
    # pairs layout, plain outputs
    d.det_memset(pg, 0xFF, m * half * 4, None)
    d.det_memset(pu, 0xFF, m * half * 4, None)
    d.det_gemm_ex(C.byref(lin), xq, sx, mx, m, None, 0, 2, offs, dsts, None)
    assert np.array_equal(_host(d, pg, want_g).view(np.uint32), want_g.view(np.uint32))
    assert np.array_equal(_host(d, pu, want_u).view(np.uint32), want_u.view(np.uint32))
    # SwiGLU epilogue, then the quantization of the product as the next GEMV's prologue
    h = d.det_malloc(m * half * 4)
    op = libs.GemvOp(lin=C.pointer(lin), xq=xq, sx=sx, mx=mx, M=m, h=h)
    d.det_gemv(C.byref(op), None)
    d.det_memset(hq, 0, m * half, None)
    d.det_memset(yd, 0xFF, m * n_down * 4, None)
    if half <= 8192:
        s = libs.ActSource(libs.DET_ACT_PLAIN, h, None, 0.0, hq, sh, mh)
        op2 = libs.GemvOp(lin=C.pointer(lin_d), src=C.pointer(s), M=m, y=yd)
    else:      # rows longer than the prologue takes: quantized by the row kernel
        d.det_quant(h, m, half, hq, sh, mh, None)
        op2 = libs.GemvOp(lin=C.pointer(lin_d), xq=hq, sx=sh, mx=mh, M=m, y=yd)
    d.det_gemv(C.byref(op2), None)
    assert np.array_equal(_host(d, yd, np.zeros(m * n_down, np.float32)).view(np.uint32), want_y)
    assert np.array_equal(_host(d, hq, want_hq), want_hq)
    # the same pair with the group maxima handed from the epilogue to the prologue (any row length), twice in a row: the
    # consumer has to leave the maxima zero for the next producer
    groups = half // 128
    amax = d.det_malloc((4 + 8 * m * groups) * 4)
    for _ in range(2):
        d.det_memset(hq, 0, m * half, None)
        d.det_memset(yd, 0xFF, m * n_down * 4, None)
        op = libs.GemvOp(lin=C.pointer(lin), xq=xq, sx=sx, mx=mx, M=m, h=h, h_amax=amax)
        d.det_gemv(C.byref(op), None)
        got_amax = _host(d, amax, np.zeros(4 + 8 * m * groups, np.uint32))
        hv = _host(d, h, np.zeros((m, groups, 128), np.float32))
        folded = got_amax[4:].reshape(m, groups, 8).max(axis=2)     # eight cells per group
        assert got_amax[0] == 0 and np.array_equal(folded.reshape(-1), np.abs(hv).max(axis=2).reshape(-1).view(np.uint32))
        s = libs.ActSource(libs.DET_ACT_PLAIN, h, None, 0.0, hq, sh, mh, amax)
        op2 = libs.GemvOp(lin=C.pointer(lin_d), src=C.pointer(s), M=m, y=yd)
        d.det_gemv(C.byref(op2), None)
        assert np.array_equal(_host(d, yd, np.zeros(m * n_down, np.float32)).view(np.uint32), want_y)
        assert np.array_equal(_host(d, hq, want_hq), want_hq)
        assert not _host(d, amax, np.zeros(4 + 8 * m * groups, np.uint32)).any()
    assert d.det_last_error() == 0
    for p in b1 + b2 + [xq, sx, mx, pg, pu, hq, sh, mh, yd, h, amax]:
        d.det_free(p)


@pytest.mark.parametrize("kind,m", [("rms", 1), ("plain", 1), ("rms", 2)])
def test_exchange_prologue_on_a_loopback_handle(kind, m, libs):
    """The tensor-parallel prologue (push the local slice, poll the gathered row, residual add, RMSNorm / quantization
    inside the GEMV) on a loopback exchange of size 2, where the gathered row is the local slice twice: it must equal
    the ordinary prologue on that doubled row (plus the residual), twice in a row (two staging slots)."""
    d = libs.cuda()
    rng = np.random.default_rng(5)
    k, n_out, slice_ = 2048, 1024, 1024
    _, lin, bufs = _linear(d, libs, rng, n_out, k, 6)
    x = d.det_xchg_create(16 * 8 * k + 4096, 0, 2)
    d.det_xchg_open_loopback(x)
    w = _dev(d, (1 + 0.1 * rng.standard_normal(k)).astype(np.float32))
    y1, y2 = d.det_malloc(m * n_out * 4), d.det_malloc(m * n_out * 4)
    hq, sh, mh = d.det_malloc(m * k), d.det_malloc(m * 4), d.det_malloc(m * (k // 128) * 2)
    for it in range(2):
        local = (rng.standard_normal((m, slice_)) * (0.3 + it)).astype(np.float32)
        resid = (rng.standard_normal((m, k)) * 0.5).astype(np.float32)
        full = np.concatenate([local, local], axis=1)
        p_local, p_res, p_out = _dev(d, local), _dev(d, resid), d.det_malloc(m * k * 4)
        if kind == "rms":
            want_rows = _dev(d, (resid + full).astype(np.float32))      # one fp32 add per element, as the kernel does
            s_ref = libs.ActSource(libs.DET_ACT_RMSNORM, want_rows, w, 1e-6, None, None, None, None, None, None, 0, None)
            s_x = libs.ActSource(libs.DET_ACT_RMSNORM, p_res, w, 1e-6, hq, sh, mh, None, x, p_local, slice_, p_out)
        else:
            want_rows = _dev(d, full)
            s_ref = libs.ActSource(libs.DET_ACT_PLAIN, want_rows, None, 0.0, None, None, None, None, None, None, 0, None)
            s_x = libs.ActSource(libs.DET_ACT_PLAIN, None, None, 0.0, hq, sh, mh, None, x, p_local, slice_, None)
        d.det_gemv(C.byref(libs.GemvOp(lin=C.pointer(lin), src=C.pointer(s_ref), M=m, y=y1)), None)
        d.det_gemv(C.byref(libs.GemvOp(lin=C.pointer(lin), src=C.pointer(s_x), M=m, y=y2)), None)
        a, b = _host(d, y1, np.zeros(m * n_out, np.float32)), _host(d, y2, np.zeros(m * n_out, np.float32))
        assert a.any() and np.array_equal(a.view(np.uint32), b.view(np.uint32))
        if kind == "rms":
            got = _host(d, p_out, np.zeros((m, k), np.float32))
            assert np.array_equal(got.view(np.uint32), (resid + full).astype(np.float32).view(np.uint32))
        for p in (p_local, p_res, p_out, want_rows):
            d.det_free(p)
    assert d.det_last_error() == 0
    d.det_xchg_destroy(x)
    for p in bufs + [w, y1, y2, hq, sh, mh]:
        d.det_free(p)
