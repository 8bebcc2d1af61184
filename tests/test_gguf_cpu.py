"""det files on the CPU: the GGUF container (header, metadata, tensor table), Config from its metadata, Model::load,
`det convert` (host quantizer), `det calibrate` and the observer taps.  Mirrors crates/det/src/gguf.rs, config.rs,
model.rs:164-365, convert.rs, calibrate.rs and hooks.rs; the model under test is the seeded synthetic one at the tiny
shape, so every loaded-model result is compared with the same model built directly from the generator."""
import ctypes as C
import struct

import numpy as np
import pytest

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


def _tensors(h, g):
    out = {}
    for i in range(h.dh_gguf_n_tensors(g)):
        name = C.create_string_buffer(128)
        dims = (C.c_size_t * 4)()
        nd, off, nbytes, ty = C.c_size_t(), C.c_size_t(), C.c_size_t(), C.c_uint32()
        assert h.dh_gguf_tensor(g, i, name, 128, dims, C.byref(nd), C.byref(ty), C.byref(off), C.byref(nbytes)) == 0
        out[name.value.decode()] = (list(dims[: nd.value]), ty.value, off.value, nbytes.value)
    return out


def test_container_metadata_and_tensor_table(libs, det_file):
    h = libs.host()
    g = h.dh_gguf_open(str(det_file).encode())
    assert g, h.dh_last_error()
    cfg = C.create_string_buffer(1024)
    assert h.dh_gguf_config(g, cfg, 1024) == 0, h.dh_last_error()
    kv = dict(line.split("=") for line in cfg.value.decode().split())
    assert (int(kv["hidden"]), int(kv["n_layers"]), int(kv["vocab"])) == (HIDDEN, LAYERS, VOCAB)
    assert (int(kv["n_heads"]), int(kv["n_kv"]), int(kv["head_dim"]), int(kv["rot_dim"])) == (8, 2, 256, 64)
    assert (int(kv["gdn_k_heads"]), int(kv["gdn_v_heads"]), int(kv["gdn_dk"]), int(kv["gdn_dv"]), int(kv["conv_k"])) == (8, 16, 128, 128, 4)
    assert float(kv["rope_theta"]) == 1e7 and np.float32(kv["eps"]) == np.float32(1e-6)
    t = _tensors(h, g)
    # 5 globals + per layer: 2 norms + 3 ffn, then 6 (attention) or 9 (GDN) tensors
    assert len(t) == 5 + LAYERS * 5 + (LAYERS // 4) * 6 + (LAYERS - LAYERS // 4) * 9
    assert t["token_embd.weight"][:2] == ([HIDDEN, VOCAB], 30)
    assert t["output.weight"][:2] == ([HIDDEN, VOCAB], 0xDE08)
    assert t["blk.0.ssm_alpha.weight"][1] == 0xDE08 and t["blk.0.ffn_down.weight"][1] == 0xDE06
    assert t["rope_cos"][:2] == ([32, N_POS], 0)
    assert t["blk.0.ffn_down.weight"][3] == HIDDEN * h.dh_det_row_bytes(6, 3072)
    assert all(off % 32 == 0 for _, _, off, _ in t.values()) and h.dh_gguf_data_start(g) % 32 == 0
    buf = C.create_string_buffer(256)
    assert h.dh_gguf_get(g, b"general.architecture", buf, 256) == 0 and buf.value == b"qwen35"
    assert h.dh_gguf_get(g, b"det.v_scale", buf, 256) == 0 and buf.value.decode() == "[0.0009765625, 0.0009765625]"
    assert h.dh_gguf_get(g, b"no.such.key", buf, 256) == 1
    assert h.dh_gguf_check_finite(g) == 0, h.dh_last_error()
    h.dh_gguf_close(g)


def test_loaded_model_equals_the_generated_model(libs, ref_backend, det_file):
    h = libs.host()
    ids = _prompt(h, 9)
    direct = h.dh_model_new_synth(ref_backend, b"tiny", LAYERS, SEED, 64, 16)
    want = _logits(h, direct, ids)
    h.dh_model_free(direct)
    loaded = h.dh_model_load(ref_backend, str(det_file).encode(), 64, 16)
    assert loaded, h.dh_last_error()
    assert h.dh_model_vocab(loaded) == VOCAB and h.dh_model_calibrated(loaded) == 0
    got = _logits(h, loaded, ids)
    h.dh_model_free(loaded)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_load_refuses_a_context_beyond_the_rope_tables(libs, ref_backend, det_file):
    h = libs.host()
    assert not h.dh_model_load(ref_backend, str(det_file).encode(), N_POS + 1, 16)
    assert b"rope tables cover 96 positions" in h.dh_last_error()


def _patched(path, out, offset, data):
    blob = bytearray(path.read_bytes())
    blob[offset : offset + len(data)] = data
    out.write_bytes(blob)
    return out


def test_open_and_load_error_cases(libs, ref_backend, det_file, tmp_path):
    h = libs.host()
    blob = det_file.read_bytes()
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + blob[4:4096])
    assert not h.dh_gguf_open(str(bad).encode()) and b"not a GGUF file" in h.dh_last_error()
    bad.write_bytes(blob[:4] + struct.pack("<I", 1) + blob[8:4096])
    assert not h.dh_gguf_open(str(bad).encode()) and b"unsupported GGUF version 1" in h.dh_last_error()
    bad.write_bytes(blob[:200])
    assert not h.dh_gguf_open(str(bad).encode()) and b"truncated GGUF header" in h.dh_last_error()
    bad.write_bytes(blob[: len(blob) // 2])
    assert not h.dh_gguf_open(str(bad).encode()) and b"does not fit the file" in h.dh_last_error()
    assert not h.dh_gguf_open(str(tmp_path / "absent.gguf").encode())
    # a non-finite value: fp32 vector element, bf16 table element, det row scale
    g = h.dh_gguf_open(str(det_file).encode())
    t, start = _tensors(h, g), h.dh_gguf_data_start(g)
    h.dh_gguf_close(g)
    cases = [("output_norm.weight", 8, struct.pack("<f", float("inf"))),
             ("token_embd.weight", 2 * 77, struct.pack("<H", 0x7FC0)),
             ("blk.1.ffn_up.weight", 1024 // 32 * 24, struct.pack("<f", float("nan")))]
    for name, rel, data in cases:
        p = _patched(det_file, bad, start + t[name][2] + rel, data)
        assert not h.dh_model_load(ref_backend, str(p).encode(), 64, 16)
        assert h.dh_last_error() == f"{name}: non-finite value".encode()
    # an unsupported tensor type (Q4_0 = 2) in the table
    hdr = blob[:start]
    at = hdr.index(b"output_norm.weight") + len(b"output_norm.weight") + 4 + 8
    bad.write_bytes(hdr[:at] + struct.pack("<I", 2) + hdr[at + 4 :] + blob[start:])
    assert not h.dh_gguf_open(str(bad).encode()) and b"unsupported type Q4_0" in h.dh_last_error()


@pytest.mark.parametrize("f32_linears", [0, 1])
def test_convert_reproduces_the_det_file_byte_for_byte(libs, det_file, tmp_path, f32_linears):
    """A float source with the unconverted Gated DeltaNet head order -> `det convert` -> the synthetic det file: covers the
    row / column head permutations, the quantizer on bf16 and fp32 sources, the tied head, the rope tables, the vector
    permutations, the metadata copy and the reserved det.v_scale array."""
    h = libs.host()
    src, out = tmp_path / "tiny-BF16.gguf", tmp_path / "out.gguf"
    assert h.dh_write_synthetic_source_gguf(b"tiny", LAYERS, SEED, str(src).encode(), N_POS, f32_linears) == 0, h.dh_last_error()
    assert h.dh_convert(str(src).encode(), str(out).encode(), None, 0, 0) == 0, h.dh_last_error()
    assert out.read_bytes() == det_file.read_bytes()


def test_convert_bit_width_options_and_output_name(libs, det_file, tmp_path):
    h = libs.host()
    src, out = tmp_path / "m-BF16-00001-of-00002.gguf", tmp_path / "w4.gguf"
    name = C.create_string_buffer(512)
    assert h.dh_convert_default_output(str(src).encode(), b"4,output=8", name, 512) == 0
    assert name.value.decode() == str(tmp_path / "m-det-w4.gguf")
    assert h.dh_convert_default_output(b"x-f16.gguf", None, name, 512) == 0 and name.value == b"x-det-w6.gguf"
    assert h.dh_convert_default_output(b"x.gguf", b"5", name, 512) != 0 and b"bit width 5 is not 4, 6 or 8" in h.dh_last_error()
    assert h.dh_convert_default_output(b"x.gguf", b"six", name, 512) != 0 and b"bad bit width" in h.dh_last_error()
    assert h.dh_write_synthetic_source_gguf(b"tiny", LAYERS, SEED, str(src).encode(), N_POS, 0) == 0
    # split.count = 1 is not in the file, so the single part is the whole model
    assert h.dh_convert(str(src).encode(), str(out).encode(), b"4,output=8,ffn_down=8", 48, 0) == 0, h.dh_last_error()
    g = h.dh_gguf_open(str(out).encode())
    t = _tensors(h, g)
    h.dh_gguf_close(g)
    assert t["blk.0.ffn_gate.weight"][1] == 0xDE04 and t["blk.0.ffn_down.weight"][1] == 0xDE08
    assert t["blk.0.ssm_alpha.weight"][1] == 0xDE04 and t["output.weight"][1] == 0xDE08
    assert t["rope_cos"][0] == [32, 48]


def test_calibrate_sets_the_value_scales(libs, ref_backend, det_file, tmp_path):
    h = libs.host()
    path = tmp_path / "cal.gguf"
    path.write_bytes(det_file.read_bytes())
    model = h.dh_model_load(ref_backend, str(path).encode(), 64, 16)
    assert model, h.dh_last_error()
    prefix = np.array([5, 6, 7], np.int32)
    ids = np.zeros(3 + 40, np.int32)
    h.dh_calibration_ids(prefix.ctypes.data, 3, VOCAB, 40, ids.ctypes.data)
    assert list(ids[:3]) == [5, 6, 7] and ids[3:].min() >= 0 and ids[3:].max() < VOCAB
    # the generator part is splitmix64 from the golden-ratio state (calibrate.rs:55-62)
    z = (0x9E3779B97F4A7C15 * 2) & (2**64 - 1)
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & (2**64 - 1)
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & (2**64 - 1)
    assert ids[3] == (z ^ (z >> 31)) % VOCAB
    scales = np.zeros(8, np.float32)
    n = C.c_size_t()
    assert h.dh_v_scales(model, ids.ctypes.data, len(ids), scales.ctypes.data, 8, C.byref(n)) == 0, h.dh_last_error()
    assert n.value == 2 and np.all(scales[:2] > 0) and np.all(np.isfinite(scales[:2]))

    # the same numbers from the AttnV tap of an observed run, folded here
    seen = []

    def tap(user, kind, layer, pos0, t, data, length, tid, rng):
        if libs.TAP_KINDS[kind] == "AttnV":
            v = np.zeros(t * 2 * 256, np.float32)
            h.dh_backend_read(ref_backend, data, v.ctypes.data, v.size)
            seen.append(np.abs(v.reshape(t, 2, 256)).max(axis=(0, 2)))

    cb = libs.TAP_FN(tap)
    assert h.dh_model_reset(model) == 0
    for i in range(0, len(ids), 16):
        chunk = ids[i : i + 16]
        assert h.dh_model_forward_observed(model, chunk.ctypes.data, len(chunk), cb, None, 0) == 0, h.dh_last_error()
    absmax = np.max(np.stack(seen), axis=0).astype(np.float32)
    want = absmax * np.float32(8.0) / np.float32(32767.0)
    assert np.array_equal(want.view(np.uint32), scales[:2].view(np.uint32))

    assert h.dh_write_scales_in_place(model, scales.ctypes.data, 2, str(path).encode()) == 0, h.dh_last_error()
    h.dh_model_free(model)
    model = h.dh_model_load(ref_backend, str(path).encode(), 64, 16)
    assert model and h.dh_model_calibrated(model) == 1
    g = h.dh_gguf_open(str(path).encode())
    buf = C.create_string_buffer(256)
    assert h.dh_gguf_get(g, b"det.v_scale", buf, 256) == 0
    assert [np.float32(x) for x in buf.value.decode().strip("[]").split(", ")] == list(scales[:2])
    h.dh_gguf_close(g)
    # the tensor data is untouched by the in-place header rewrite
    a, b = det_file.read_bytes(), path.read_bytes()
    assert len(a) == len(b) and a[-(1 << 20):] == b[-(1 << 20):]
    # a copy with more scales than the header has room for is a new file; a wrong count is refused at load
    copy = tmp_path / "copy.gguf"
    many = np.full(64, 0.5, np.float32)
    assert h.dh_write_scales_in_place(model, many.ctypes.data, 64, str(path).encode()) == 2
    assert h.dh_write_scales_copy(model, many.ctypes.data, 64, str(copy).encode()) == 0, h.dh_last_error()
    h.dh_model_free(model)
    assert not h.dh_model_load(ref_backend, str(copy).encode(), 64, 16)
    assert b"det.v_scale: expected 2 positive floats" in h.dh_last_error()


def test_observer_sees_the_taps_in_network_order(libs, ref_backend):
    h = libs.host()
    model = h.dh_model_new_synth(ref_backend, b"tiny", LAYERS, SEED, 64, 16)
    ids = _prompt(h, 5)
    events = []

    def tap(user, kind, layer, pos0, t, data, length, tid, rng):
        rec = [libs.TAP_KINDS[kind], layer, pos0, t, None, tid, rng]
        if data and libs.TAP_KINDS[kind] in ("Residual", "Logits", "GdnIn", "GdnOut", "MixerOut"):
            n = {"Residual": t * HIDDEN, "Logits": VOCAB, "GdnIn": t * 8 * (256 + 2 * 128 + 4), "GdnOut": t * 16 * 128,
                 "MixerOut": t * 2048}[libs.TAP_KINDS[kind]]
            v = np.zeros(n, np.float32)
            h.dh_backend_read(ref_backend, data, v.ctypes.data, n)
            rec[4] = v
        events.append(rec)

    cb = libs.TAP_FN(tap)
    assert h.dh_model_forward_observed(model, ids.ctypes.data, 5, cb, None, 1) == 0, h.dh_last_error()
    kinds = [(e[0], e[1]) for e in events]
    gdn = lambda l: [("Residual", l), ("GdnIn", l), ("GdnOut", l), ("GdnState", l), ("MixerOut", l), ("PostMixer", l)]
    attn = lambda l: [("Residual", l), ("AttnV", l), ("Kv", l), ("AttnOut", l), ("MixerOut", l), ("PostMixer", l)]
    assert kinds == gdn(0) + gdn(1) + gdn(2) + attn(3) + [("Residual", 4), ("Logits", 0)]
    assert all(e[2] == 0 and e[3] == 5 for e in events)
    # the first residual is the embedding rows; the logits tap equals the model's logits; the export is non-trivial
    first = events[0][4].reshape(5, HIDDEN)
    assert first.any() and np.all(np.abs(first) < 1.0)
    out = np.zeros(VOCAB, np.float32)
    h.dh_model_logits(model, out.ctypes.data, VOCAB)
    assert np.array_equal(events[-1][4].view(np.uint32), out.view(np.uint32))
    assert events[1][4].any() and events[2][4].any()
    # without the export request the GdnIn / GdnOut taps are absent and the results are the same
    events.clear()
    assert h.dh_model_reset(model) == 0
    assert h.dh_model_forward_observed(model, ids.ctypes.data, 5, cb, None, 0) == 0
    assert ("GdnIn", 0) not in [(e[0], e[1]) for e in events]
    assert np.array_equal(events[-1][4].view(np.uint32), out.view(np.uint32))
    # generate: a Token tap after every pick, carrying the generator state after the draw
    events.clear()
    toks = np.zeros(4, np.int32)
    cnt = C.c_size_t()
    assert h.dh_model_reset(model) == 0
    assert h.dh_model_generate_observed(model, ids.ctypes.data, 5, 4, 0, 1.25, 40, 0.95, 99, toks.ctypes.data, C.byref(cnt),
                                        cb, None, 0) == 0, h.dh_last_error()
    tok_events = [e for e in events if e[0] == "Token"]
    assert [e[5] for e in tok_events] == list(toks[: cnt.value]) and cnt.value == 4
    assert [e[2] for e in tok_events] == [4, 5, 6, 7]
    golden = 0x9E3779B97F4A7C15
    assert [e[6] for e in tok_events] == [(99 + golden * (i + 1)) & (2**64 - 1) for i in range(4)]
    h.dh_model_free(model)


def test_row_helpers_round_trip(libs):
    """dequant_row on the three float types (spec/tensor.rs:8-30, 73-93) and on det rows written by the quantizer."""
    h = libs.host()
    rng = np.random.default_rng(3)
    x = rng.standard_normal(256).astype(np.float32)
    out = np.zeros(256, np.float32)
    assert h.dh_dequant_row(0, x.ctypes.data, 256, out.ctypes.data) == 0 and np.array_equal(out, x)
    half = np.concatenate([x[:250].astype(np.float16), np.array([0, -0.0, 6e-8, -6.1e-5, 65504, 1e-7], np.float16)])
    assert h.dh_dequant_row(1, half.ctypes.data, 256, out.ctypes.data) == 0
    assert np.array_equal(out.view(np.uint32), half.astype(np.float32).view(np.uint32))
    b16 = (x.view(np.uint32) >> 16).astype(np.uint16)
    assert h.dh_dequant_row(30, b16.ctypes.data, 256, out.ctypes.data) == 0
    assert np.array_equal(out.view(np.uint32), b16.astype(np.uint32) << 16)
    assert h.dh_dequant_row(2, x.ctypes.data, 256, out.ctypes.data) != 0
    for bits, tid in ((4, 0xDE04), (6, 0xDE06), (8, 0xDE08)):
        row = np.zeros(h.dh_det_row_bytes(bits, 256), np.uint8)
        h.dh_quantize_row(x.ctypes.data, 256, bits, row.ctypes.data)
        assert h.dh_dequant_row(tid, row.ctypes.data, 256, out.ctypes.data) == 0
        qmax = (1 << (bits - 1)) - 1
        for g in range(2):
            step = np.abs(x[g * 128 : (g + 1) * 128]).max() / qmax
            assert np.abs(out[g * 128 : (g + 1) * 128] - x[g * 128 : (g + 1) * 128]).max() <= max(0.55, 0.2 * qmax + 0.05) * step  # the scale search may go down to 0.8 x amax / qmax, clipping the largest values by 0.2 x amax


def _py_gguf(path):
    """An independent reading of the GGUF v3 container (little-endian header: magic, version, tensor count, kv count;
    kv = string key, u32 type, value; tensor = string name, u32 rank, u64 dims, u32 type, u64 offset; data section at the
    next multiple of general.alignment, default 32)."""
    blob = path.read_bytes()
    pos = 0

    def take(fmt):
        nonlocal pos
        v = struct.unpack_from("<" + fmt, blob, pos)
        pos += struct.calcsize("<" + fmt)
        return v[0] if len(v) == 1 else v

    def string():
        nonlocal pos
        n = take("Q")
        s = blob[pos : pos + n].decode()
        pos += n
        return s

    scalar = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 7: "?", 10: "Q", 11: "q", 12: "d"}

    def value(ty):
        if ty == 8:
            return string()
        if ty == 9:
            et, n = take("I"), take("Q")
            return [value(et) for _ in range(n)]
        return take(scalar[ty])

    assert blob[:4] == b"GGUF"
    pos = 4
    version, n_tensors, n_kv = take("I"), take("Q"), take("Q")
    kv = []
    for _ in range(n_kv):
        key = string()
        kv.append((key, value(take("I"))))
    tensors = []
    for _ in range(n_tensors):
        name = string()
        dims = [take("Q") for _ in range(take("I"))]
        tensors.append((name, dims, take("I"), take("Q")))
    align = dict(kv).get("general.alignment", 32)
    return version, kv, tensors, (pos + align - 1) // align * align, blob


def test_written_file_reads_back_through_an_independent_parser(libs, det_file):
    """The container this library writes, read by a parser written from the format description alone, and the tensor
    payloads it points at checked against what they must hold (rope tables in binary64 rounded once, convert.rs:370-385;
    unit norm weights; negative decay rates; the W8 head's row layout [codes][c][m], spec/tensor.rs:43-55)."""
    h = libs.host()
    version, kv, tensors, data_start, blob = _py_gguf(det_file)
    assert version == 3
    meta = dict(kv)
    assert [k for k, _ in kv][:3] == ["general.architecture", "general.name", "qwen35.block_count"]
    assert meta["general.architecture"] == "qwen35" and meta["qwen35.block_count"] == LAYERS
    assert meta["qwen35.embedding_length"] == HIDDEN and meta["qwen35.full_attention_interval"] == 4
    assert meta["qwen35.ssm.inner_size"] == 16 * 128 and meta["qwen35.ssm.time_step_rank"] == 16
    assert meta["qwen35.rope.freq_base"] == 1e7 and abs(meta["qwen35.attention.layer_norm_rms_epsilon"] - 1e-6) < 1e-12
    assert meta["det.v_scale"] == [1.0 / 1024] * 2
    g = h.dh_gguf_open(str(det_file).encode())
    assert h.dh_gguf_data_start(g) == data_start
    mine = _tensors(h, g)
    h.dh_gguf_close(g)
    assert [t[0] for t in tensors] == list(mine)            # same order
    table = {name: (dims, ty, off) for name, dims, ty, off in tensors}
    for name, (dims, ty, off, _) in mine.items():
        assert table[name] == (dims, ty, off)
    # payloads
    def f32s(name):
        dims, ty, off = table[name]
        assert ty == 0
        return np.frombuffer(blob, np.float32, int(np.prod(dims)), data_start + off)

    half, theta = 32, 1e7
    ang = np.arange(N_POS, dtype=np.float64)[:, None] * (theta ** (-(2.0 * np.arange(half)) / 64.0))[None, :]
    assert np.array_equal(f32s("rope_cos"), np.cos(ang).astype(np.float32).reshape(-1))
    assert np.array_equal(f32s("rope_sin"), np.sin(ang).astype(np.float32).reshape(-1))
    assert np.all(f32s("output_norm.weight") == 1.0) and np.all(f32s("blk.3.attn_q_norm.weight") == 1.0)
    a = f32s("blk.0.ssm_a")
    assert a.shape == (16,) and np.all(a <= -1.0) and np.all(a > -16.0)
    dims, ty, off = table["output.weight"]
    assert ty == 0xDE08 and dims == [HIDDEN, VOCAB]
    rb = HIDDEN + 4 + HIDDEN // 128 * 2
    row = np.frombuffer(blob, np.uint8, rb, data_start + off + 5 * rb)
    c = row[HIDDEN : HIDDEN + 4].view(np.float32)[0]
    m = row[HIDDEN + 4 :].view(np.uint16)
    assert np.isfinite(c) and c > 0 and m.max() == 65535 and m.min() >= 1     # the widest group takes the full multiplier
    out = np.zeros(HIDDEN, np.float32)
    assert h.dh_dequant_row(0xDE08, row.ctypes.data, HIDDEN, out.ctypes.data) == 0
    want = (np.float32(c) * m.astype(np.float32)).repeat(128) * row[:HIDDEN].view(np.int8).astype(np.float32)
    assert np.array_equal(out, want)
    # the W8 head quantizes the bf16 embedding table: row 5 of both must agree to half a step of the row's scale
    dims_e, ty_e, off_e = table["token_embd.weight"]
    emb = (np.frombuffer(blob, np.uint16, HIDDEN, data_start + off_e + 5 * HIDDEN * 2).astype(np.uint32) << 16).view(np.float32)
    assert np.abs(out - emb).max() <= 0.62 * np.abs(emb).reshape(-1, 128).max(axis=1).repeat(128).max() / 127
