"""One linear of a chosen shape through the C ABI, timed with CUDA events: the small stand-alone case of the two GEMM
kernels that a profiler capture needs (a few hundred MB on the device, a handful of launches).

    python bench_kernel.py gemv    [N K bits M]    # k_gemv_stream, default 17408 5120 6 1
    python bench_kernel.py gemm_tc [N K bits M [variant]]   # k_gemm_tc, default 17408 5120 6 512, tile by shape
    python bench_kernel.py umma_peak                        # int8 tcgen05.mma issue rate with resident operands
    python bench_kernel.py stream_peak                      # HBM read rate with nothing to compute: plain loads, GEMV rings
    python bench_kernel.py attn [n_h n_kv M pos0 [tc]]      # prefill attention, default 24 4 512 1536, tensor path on

attn: one det_attention call of M tokens behind pos0 cached positions (head_dim 256, random cache contents); tc = 0
keeps it on the CUDA-core kernels; 2 warm-up calls, then 5 timed ones.

gemv: six copies of the weights (seeded, generated on the device, repacked into the streaming layout) are cycled through
so that no launch finds its weights in the 126 MB L2; 6 warm-up launches, then 12 timed ones.
gemm_tc: one int8-expanded copy; 3 warm-up launches, then 10 timed ones.
"""
from __future__ import annotations

import ctypes as C
import sys

import numpy as np

import os
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from det_b200 import capi

PER32 = {8: 32, 6: 24, 4: 16}


class _Events:
    def __init__(self, stream):
        self.rt = C.CDLL("libcudart.so.12")
        self.stream = C.c_void_p(stream)

    def record(self):
        e = C.c_void_p()
        assert self.rt.cudaEventCreate(C.byref(e)) == 0
        assert self.rt.cudaEventRecord(e, self.stream) == 0
        return e

    def ms(self, a, b):
        assert self.rt.cudaEventSynchronize(b) == 0
        out = C.c_float()
        assert self.rt.cudaEventElapsedTime(C.byref(out), a, b) == 0
        return out.value


def _linear(d, n, k, bits, tensor_id):
    g = k // 128
    wq = d.det_malloc(n * (k // 32) * PER32[bits])
    c = d.det_malloc(n * 4)
    m = d.det_malloc(n * g * 2)
    scratch = d.det_malloc(n * g * 8)
    d.det_synth_linear(20261125, tensor_id, 0, n, k, bits, 0, wq, c, m, scratch, None)
    d.det_sync()
    d.det_free(scratch)
    return capi.QLinear(wq, c, m, n, k, bits)


def _activations(d, m, k, n):
    rng = np.random.default_rng(1)
    g = k // 128
    xq, sx, mx, y = d.det_malloc(m * k), d.det_malloc(m * 4), d.det_malloc(m * g * 2), d.det_malloc(m * n * 4)
    hx = rng.integers(-127, 128, m * k).astype(np.int8)
    hs = (rng.random(m, dtype=np.float32) * 1e-3 + 1e-4).astype(np.float32)
    hm = rng.integers(1, 65536, m * g).astype(np.uint16)
    d.det_memcpy(xq, hx.ctypes.data, hx.nbytes, None)
    d.det_memcpy(sx, hs.ctypes.data, hs.nbytes, None)
    d.det_memcpy(mx, hm.ctypes.data, hm.nbytes, None)
    d.det_sync()
    return xq, sx, mx, y


def attn(argv):
    n_h, n_kv, m, pos0 = (24, 4, 512, 1536) if len(argv) < 5 else map(int, argv[1:5])
    tc = int(argv[5]) if len(argv) >= 6 else 1
    hd, rot, ctx = 256, 64, pos0 + m
    d = capi.cuda()
    assert d.det_init() == 0
    d.det_debug_set_attn_tc(tc, 0)
    rng = np.random.default_rng(1)

    def up(a):
        a = np.ascontiguousarray(a)
        p = d.det_malloc(a.nbytes)
        d.det_memcpy(p, a.ctypes.data, a.nbytes, None)
        return p

    layer = capi.AttnLayer(up(np.ones(hd, np.float32)), up(np.ones(hd, np.float32)), up(np.full(n_kv, 1 / 1024, np.float32)),
                           up(np.full(n_kv, 1024.0, np.float32)))
    cache = capi.KvCache(up(rng.integers(-127, 128, (ctx, n_kv, hd), dtype=np.int8)),
                         up(rng.uniform(0.001, 0.02, (ctx, n_kv)).astype(np.float32)),
                         up(rng.integers(-32767, 32768, (ctx, n_kv, hd), dtype=np.int16)), ctx, None, None)
    ang = np.arange(ctx)[:, None] * (1e7 ** (-np.arange(rot // 2) * 2.0 / rot))[None, :]
    cos, sin = up(np.cos(ang).astype(np.float32)), up(np.sin(ang).astype(np.float32))
    qg = up(rng.standard_normal((m, n_h, 2 * hd)).astype(np.float32))
    k = up(rng.standard_normal((m, n_kv, hd)).astype(np.float32))
    v = up(rng.standard_normal((m, n_kv, hd)).astype(np.float32))
    o, scratch = d.det_malloc(m * n_h * hd * 4), d.det_malloc(d.det_attn_scratch_bytes(m, n_h, hd))
    ev = _Events(d.det_cuda_stream())

    def call():
        d.det_attention(C.byref(layer), C.byref(cache), qg, k, v, cos, sin, rot, 1e-6, m, pos0, n_h, n_kv, hd, o, scratch, None)

    for _ in range(2):
        call()
    a = ev.record()
    for _ in range(5):
        call()
    b = ev.record()
    us = ev.ms(a, b) / 5 * 1e3
    # causal pairs: token t sees pos0 + t + 1 keys; two contractions of hd MACs per (q head, token, key) pair
    pairs = n_h * sum(pos0 + t + 1 for t in range(m))
    print(f"det_attention n_h={n_h} n_kv={n_kv} M={m} pos0={pos0} {'tensor' if tc else 'cuda-core'} path: {us:.1f} us/call, "
          f"{4 * pairs * hd / us / 1e6:.1f} TOPS of 2 x hd MACs per pair; device error word {d.det_last_error()}")
    d.det_sync()


def main(argv):
    kind = argv[0] if argv else "gemv"
    if kind == "umma_peak":
        d = capi.cuda()
        assert d.det_init() == 0
        for iters in (2048, 8192):
            print(f"tcgen05.mma kind::i8 128x256x32, {iters} x 4 per SM: {d.det_debug_umma_peak(iters):.0f} TOPS; "
                  f"device error word {d.det_last_error()}")
        return
    if kind == "stream_peak":
        d = capi.cuda()
        assert d.det_init() == 0
        size = 2 << 30
        buf = d.det_malloc(size)
        d.det_memset(buf, 1, size, None)
        d.det_sync()
        # (record bytes, warps, slots per warp, records per quad); 3136 x 16 x 4 x 5 is the 27B W6 GEMV at K = 5120
        rings = ((3136, 16, 4, 5), (3136, 16, 2, 5), (3136, 16, 3, 5), (4096, 16, 3, 4), (8192, 16, 1, 2), (8192, 8, 3, 2),
                 (16384, 4, 3, 1), (2048, 16, 6, 8),
                 # half an SM or less: the successor's CTA is resident while this one runs
                 (3136, 8, 4, 5), (3136, 8, 3, 5), (6272, 8, 2, 5), (4096, 8, 3, 4), (8192, 4, 3, 2), (8192, 6, 2, 2), (3136, 16, 1, 5))
        # per launch: the whole buffer, then the size of one 17408 x 5120 W6 linear, then of a 5120 x 6144 one
        for piece, regions, reps in ((size, 1, 5), (68 * 1024 * 1024 // 256 * 256, 30, 60), (24 * 1024 * 1024, 85, 170)):
            label = f"{piece / 1e6:.0f} MB per launch"
            r = d.det_debug_stream_peak(buf, piece, regions, 0, 0, 0, 0, 0, reps)
            print(f"{label}: plain 16-byte loads {r:.0f} GB/s = {piece / r / 1e3:.2f} us")
            for rec, warps, slots, nch in rings:
                out = []
                for mode in (1, 2):
                    r = d.det_debug_stream_peak(buf, piece, regions, mode, rec, warps, slots, nch, reps)
                    out.append(f"{r:.0f} GB/s = {piece / r / 1e3:.2f} us")
                print(f"{label}: ring of {rec} B records, {warps} warps x {slots} slots ({rec * warps * slots >> 10} KB per SM), "
                      f"{nch} per quad: dealt {out[0]}, contiguous {out[1]}; device error word {d.det_last_error()}")
        d.det_free(buf)
        return
    if kind == "attn":
        return attn(argv)
    if kind not in ("gemv", "gemm_tc"):
        raise SystemExit(__doc__)
    n, k, bits, m = (17408, 5120, 6, 1 if kind == "gemv" else 512)
    if len(argv) >= 5:
        n, k, bits, m = map(int, argv[1:5])
    d = capi.cuda()
    assert d.det_init() == 0
    if len(argv) >= 6:
        if kind == "gemv":
            d.det_debug_set_gemv(int(argv[5]))
        else:
            d.det_debug_set_tc_variant(int(argv[5]))
    ev = _Events(d.det_cuda_stream())
    xq, sx, mx, y = _activations(d, m, k, n)
    g = k // 128
    if kind == "gemv":
        lins = []
        for copy in range(6):
            src = _linear(d, n, k, bits, 100 + copy)
            sp = d.det_malloc(d.det_linear_repack_bytes(n, k, bits))
            d.det_linear_repack(C.byref(src), sp, None)
            d.det_sync()
            d.det_free(src.wq)
            lins.append(capi.QLinear(sp, src.c, src.m, n, k, bits | capi.DET_LAYOUT_STREAM))
        for it in range(6):
            d.det_gemm(C.byref(lins[it % 6]), xq, sx, mx, m, y, None)
        a = ev.record()
        for it in range(12):
            d.det_gemm(C.byref(lins[it % 6]), xq, sx, mx, m, y, None)
        b = ev.record()
        us = ev.ms(a, b) / 12 * 1e3
        nbytes = n * (k // 32 * PER32[bits] + 4 + g * 2) + m * (k + 4 + g * 2) + m * n * 4
        print(f"k_gemv_stream N={n} K={k} W{bits} M={m}: {us:.2f} us/launch, {nbytes / 1e6:.2f} MB algorithmic, "
              f"{nbytes / us / 1e3:.0f} GB/s; device error word {d.det_last_error()}")
    else:
        src = _linear(d, n, k, bits, 100)
        w8 = d.det_malloc(d.det_linear_expand_bytes(n, k))
        d.det_linear_expand(C.byref(src), w8, None)
        d.det_sync()
        tc = capi.QLinear(w8, src.c, src.m, n, k, bits | capi.DET_LAYOUT_INT8)
        for _ in range(3):
            d.det_gemm(C.byref(tc), xq, sx, mx, m, y, None)
        a = ev.record()
        for _ in range(10):
            d.det_gemm(C.byref(tc), xq, sx, mx, m, y, None)
        b = ev.record()
        us = ev.ms(a, b) / 10 * 1e3
        print(f"k_gemm_tc N={n} K={k} W{bits} M={m}: {us:.1f} us/launch, {2 * m * n * k / us / 1e6:.0f} TOPS; "
              f"device error word {d.det_last_error()}")
    d.det_sync()


if __name__ == "__main__":
    main(sys.argv[1:])
