"""det files on the B200: a det GGUF loaded onto the CUDA backend gives the CPU reference backend's logits; the device
quantizer behind `det convert` writes the host quantizer's bytes; the calibration fold on the device gives the host
fold's scales; every observer tap of a run on the CUDA backend equals the same tap on the CPU reference backend; the
device-resident greedy loop reads its tokens' embedding rows from the file's own table."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SEED = 20261125
LAYERS = 4
N_POS = 96
VOCAB = 32768
HIDDEN = 1024


def _prompt(h, n, seed=11):
    ids = np.zeros(n, np.int32)
    h.dh_synth_prompt(seed, n, VOCAB, ids.ctypes.data)
    return ids


def _logits(h, model, ids):
    assert h.dh_model_reset(model) == 0
    assert h.dh_model_forward(model, ids.ctypes.data, len(ids)) == 0, h.dh_last_error()
    out = np.zeros(VOCAB, np.float32)
    assert h.dh_model_logits(model, out.ctypes.data, VOCAB) == VOCAB
    return out


@pytest.fixture(scope="module")
def det_file(libs, tmp_path_factory):
    h = libs.host()
    path = tmp_path_factory.mktemp("gguf") / "tiny-det-w6.gguf"
    assert h.dh_write_synthetic_gguf(b"tiny", LAYERS, SEED, str(path).encode(), N_POS) == 0, h.dh_last_error()
    return path


def test_loaded_model_on_the_device_equals_the_cpu_reference(libs, ref_backend, cuda_backend, det_file):
    h = libs.host()
    for n in (1, 9, 16):
        ids = _prompt(h, n, seed=20 + n)
        cpu = h.dh_model_load(ref_backend, str(det_file).encode(), 64, 16)
        gpu = h.dh_model_load(cuda_backend, str(det_file).encode(), 64, 16)
        assert cpu and gpu, h.dh_last_error()
        want, got = _logits(h, cpu, ids), _logits(h, gpu, ids)
        h.dh_model_free(cpu)
        h.dh_model_free(gpu)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), n


def test_graph_decoder_reads_the_files_embedding_table(libs, cuda_backend, det_file):
    h = libs.host()
    ids = _prompt(h, 7)
    model = h.dh_model_load(cuda_backend, str(det_file).encode(), 64, 16)
    assert model, h.dh_last_error()
    toks = np.zeros(6, np.int32)
    cnt = C.c_size_t()
    assert h.dh_model_generate(model, ids.ctypes.data, 7, 6, 1, 1.0, 0, 1.0, 0, toks.ctypes.data, C.byref(cnt)) == 0
    assert h.dh_model_reset(model) == 0 and h.dh_model_prefill(model, ids.ctypes.data, 7) == 0
    first, rng = C.c_int32(), C.c_uint64(0)
    assert h.dh_model_pick(model, 1, 1.0, 0, 1.0, C.byref(rng), C.byref(first)) == 0 and first.value == toks[0]
    dec = h.dh_graph_decoder_new(model)
    assert dec, h.dh_last_error()
    assert h.dh_graph_decoder_enqueue(dec, first.value, 5, 1) == 0, h.dh_last_error()
    out = np.zeros(5, np.int32)
    assert h.dh_graph_decoder_finish(dec, out.ctypes.data, 5) == 5
    h.dh_graph_decoder_free(dec)
    h.dh_model_free(model)
    assert list(out) == list(toks[1:6])


def test_typed_embedding_lookup(libs):
    cu = libs.cuda()
    assert cu.det_init() == 0
    rng = np.random.default_rng(5)
    table = rng.standard_normal((50, 256)).astype(np.float32)
    ids = np.array([3, 49, 0, 17], np.int32)
    d_ids = cu.det_malloc(ids.nbytes)
    d_x = cu.det_malloc(4 * 256 * 4)
    cu.det_memcpy(d_ids, ids.ctypes.data, ids.nbytes, None)
    for type_id, host in ((0, table), (1, table.astype(np.float16)), (30, (table.view(np.uint32) >> 16).astype(np.uint16))):
        d_t = cu.det_malloc(host.nbytes)
        cu.det_memcpy(d_t, host.ctypes.data, host.nbytes, None)
        cu.det_embed_table(d_t, type_id, d_ids, 4, 256, d_x, None)
        out = np.zeros((4, 256), np.float32)
        cu.det_memcpy(out.ctypes.data, d_x, out.nbytes, None)
        cu.det_sync()
        want = host[ids].astype(np.float32) if type_id != 30 else (host[ids].astype(np.uint32) << 16).view(np.float32)
        assert np.array_equal(out.view(np.uint32), want.view(np.uint32)), type_id
        cu.det_free(d_t)
    cu.det_free(d_ids)
    cu.det_free(d_x)


@pytest.mark.parametrize("f32_linears", [0, 1])
def test_device_convert_reproduces_the_det_file(libs, cuda_backend, det_file, tmp_path, f32_linears):
    h = libs.host()
    src, out = tmp_path / "tiny-BF16.gguf", tmp_path / "out.gguf"
    assert h.dh_write_synthetic_source_gguf(b"tiny", LAYERS, SEED, str(src).encode(), N_POS, f32_linears) == 0, h.dh_last_error()
    assert h.dh_convert(str(src).encode(), str(out).encode(), None, 0, 1) == 0, h.dh_last_error()
    assert out.read_bytes() == det_file.read_bytes()


def test_device_quantizer_on_f16_rows_and_w4_w8(libs):
    """det_quantize_rows against the host quantizer on an fp16 source with both permutations, at every width."""
    cu, h = libs.cuda(), libs.host()
    assert cu.det_init() == 0
    rng = np.random.default_rng(9)
    n, k = 24, 384
    src = (rng.standard_normal((n, k)) * 0.05).astype(np.float16)
    src[3, 128:256] = 0   # an all-zero group takes scale 1 (quantize.rs:36-38)
    rp = rng.permutation(n).astype(np.int32)
    cp = rng.permutation(k).astype(np.int32)
    d_src, d_rp, d_cp = cu.det_malloc(src.nbytes), cu.det_malloc(rp.nbytes), cu.det_malloc(cp.nbytes)
    cu.det_memcpy(d_src, src.ctypes.data, src.nbytes, None)
    cu.det_memcpy(d_rp, rp.ctypes.data, rp.nbytes, None)
    cu.det_memcpy(d_cp, cp.ctypes.data, cp.nbytes, None)
    d_tmp = cu.det_malloc(n * (k // 128) * 8)
    for bits in (4, 6, 8):
        rb = h.dh_det_row_bytes(bits, k)
        d_out = cu.det_malloc(n * rb)
        cu.det_quantize_rows(d_src, 1, d_rp, d_cp, n, k, bits, d_out, d_tmp, None)
        got = np.zeros((n, rb), np.uint8)
        cu.det_memcpy(got.ctypes.data, d_out, got.nbytes, None)
        cu.det_sync()
        cu.det_free(d_out)
        want = np.zeros((n, rb), np.uint8)
        for r in range(n):
            row = np.ascontiguousarray(src[rp[r]].astype(np.float32)[cp])
            h.dh_quantize_row(row.ctypes.data, k, bits, want[r].ctypes.data)
        assert np.array_equal(got, want), bits
    for p in (d_src, d_rp, d_cp, d_tmp):
        cu.det_free(p)


def test_calibration_fold_on_the_device_equals_the_host_fold(libs, ref_backend, cuda_backend, det_file):
    h = libs.host()
    ids = np.zeros(45, np.int32)
    h.dh_calibration_ids(None, 0, VOCAB, 45, ids.ctypes.data)
    res = []
    for backend in (ref_backend, cuda_backend):
        model = h.dh_model_load(backend, str(det_file).encode(), 64, 16)
        assert model, h.dh_last_error()
        scales = np.zeros(2, np.float32)
        n = C.c_size_t()
        assert h.dh_v_scales(model, ids.ctypes.data, len(ids), scales.ctypes.data, 2, C.byref(n)) == 0, h.dh_last_error()
        h.dh_model_free(model)
        res.append(scales)
    assert np.all(res[0] > 0) and np.array_equal(res[0].view(np.uint32), res[1].view(np.uint32))


def test_observer_taps_equal_the_cpu_reference(libs, ref_backend, cuda_backend, det_file):
    """Prefill of 12 tokens, then two single-token steps (the fused decode path): every fp32 tap, in order."""
    h = libs.host()
    sizes = {"Residual": HIDDEN, "PostMixer": HIDDEN, "MixerOut": 2048, "AttnV": 2 * 256, "AttnOut": 8 * 256,
             "GdnIn": 8 * (256 + 2 * 128 + 4), "GdnOut": 16 * 128}
    runs = []
    for backend in (ref_backend, cuda_backend):
        model = h.dh_model_load(backend, str(det_file).encode(), 64, 16)
        assert model, h.dh_last_error()
        events = []

        def tap(user, kind, layer, pos0, t, data, length, tid, rng, backend=backend, events=events):
            name = libs.TAP_KINDS[kind]
            n = VOCAB if name == "Logits" else sizes.get(name, 0) * t
            v = np.zeros(n, np.float32)
            if n:
                h.dh_backend_read(backend, data, v.ctypes.data, n)
            events.append((name, layer, pos0, t, v))

        cb = libs.TAP_FN(tap)
        ids = _prompt(h, 14)
        assert h.dh_model_forward_observed(model, ids.ctypes.data, 12, cb, None, 1) == 0, h.dh_last_error()
        for i in (12, 13):
            assert h.dh_model_forward_observed(model, ids[i:].ctypes.data, 1, cb, None, 1) == 0, h.dh_last_error()
        h.dh_model_free(model)
        runs.append(events)
    assert len(runs[0]) == len(runs[1]) == 3 * (LAYERS * 6 + 2)
    for a, b in zip(*runs):
        assert a[:4] == b[:4]
        assert np.array_equal(a[4].view(np.uint32), b[4].view(np.uint32)), a[:4]
