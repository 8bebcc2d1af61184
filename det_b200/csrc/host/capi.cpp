// C entry points of the host driver library for the Python package (ctypes): backend objects, the synthetic model,
// the token loop.  Every function that can fail returns 0 on success and leaves a message for dh_last_error().
#include "convert.hpp"
#include "cuda_backend.hpp"
#include "graph_decode.hpp"
#include "model.hpp"
#include "serve.hpp"
#include <cstring>
#include <functional>
#include <string>

namespace {
thread_local std::string g_err;
int fail(const std::string& e) {
    g_err = e;
    return 1;
}
template <class F>
int guarded(F&& f) {
    try {
        std::string e = f();
        return e.empty() ? 0 : fail(e);
    } catch (const std::exception& ex) {
        return fail(ex.what());
    }
}
}  // namespace

extern "C" {

const char* dh_last_error() { return g_err.c_str(); }

// ---- backends.  A backend handle is a det::Backend*; the CUDA backend is created here, test code may pass handles of
// other implementations of the same interface.
void* dh_cuda_backend_new(int stream_layout, int keep_rowmajor) {
    try {
        auto* b = new det::CudaBackend();
        b->stream_layout = stream_layout != 0;
        b->keep_rowmajor = keep_rowmajor != 0;
        return static_cast<det::Backend*>(b);
    } catch (const std::exception& ex) {
        g_err = ex.what();
        return nullptr;
    }
}
void dh_backend_free(void* b) { delete static_cast<det::Backend*>(b); }
int dh_backend_name(void* b, char* out, size_t cap) {
    return guarded([&] {
        snprintf(out, cap, "%s", static_cast<det::Backend*>(b)->name().c_str());
        return std::string();
    });
}
// Profiling / measurement switches of a CUDA backend handle (see CudaBackend::skip_mask, fuse_decode).
void dh_cuda_debug(void* b, unsigned skip_mask, int fuse_decode) {
    auto* cb = dynamic_cast<det::CudaBackend*>(static_cast<det::Backend*>(b));
    if (!cb) return;
    cb->flush();
    cb->skip_mask = skip_mask;
    cb->fuse_decode = (fuse_decode & 1) != 0;
    cb->swiglu_amax = (fuse_decode & 2) == 0;   // bit 1 set: the SwiGLU product is quantized by its own launch again
}
// The primitive test hook of the CUDA backend (cuda.rs:474-490).
void dh_cuda_test_prim(int op, const float* x, size_t len, size_t m, size_t n, float* out, size_t out_len) {
    static det::CudaBackend* hook = new det::CudaBackend();
    std::vector<float> r = hook->test_prim(op, std::vector<float>(x, x + len), m, n);
    std::memcpy(out, r.data(), (out_len < r.size() ? out_len : r.size()) * sizeof(float));
}

// ---- model
void* dh_model_new_synth(void* backend, const char* config, size_t layers, uint64_t seed, size_t max_ctx,
                         size_t max_batch) {
    try {
        det::Config cfg = det::config_by_name(config, layers);
        return det::Model::load_synthetic(cfg, seed, static_cast<det::Backend*>(backend), max_ctx, max_batch).release();
    } catch (const std::exception& ex) {
        g_err = ex.what();
        return nullptr;
    }
}
// ---- det files: Model::load, the synthetic writers, convert, calibrate
void* dh_model_load(void* backend, const char* path, size_t max_ctx, size_t max_batch) {
    try {
        std::string err;
        std::unique_ptr<det::Model> m = det::Model::load(path, static_cast<det::Backend*>(backend), max_ctx, max_batch, err);
        if (!m) g_err = err;
        return m.release();
    } catch (const std::exception& ex) {
        g_err = ex.what();
        return nullptr;
    }
}
int dh_model_calibrated(void* m) { return static_cast<det::Model*>(m)->calibrated ? 1 : 0; }
int dh_write_synthetic_gguf(const char* config, size_t layers, uint64_t seed, const char* path, size_t n_pos) {
    return guarded([&] { return det::write_synthetic_gguf(det::config_by_name(config, layers), seed, path, n_pos); });
}
int dh_write_synthetic_source_gguf(const char* config, size_t layers, uint64_t seed, const char* path, size_t n_pos,
                                   int f32_linears) {
    return guarded([&] {
        return det::write_synthetic_source_gguf(det::config_by_name(config, layers), seed, path, n_pos, f32_linears != 0);
    });
}
// `bits` as `det convert --bits` takes it (NULL: the default widths); rope_positions 0 takes the source's context length;
// on_device != 0 quantizes with the CUDA backend's kernel instead of the host threads (same bytes).
int dh_convert(const char* src_path, const char* out_path, const char* bits, size_t rope_positions, int on_device) {
    return guarded([&] {
        det::Source src;
        std::string err;
        if (!det::Source::open(src_path, src, err)) return err;
        det::ConvertOptions opt;
        err = det::Bits::parse(bits ? bits : det::DEFAULT_BITS, opt.bits);
        if (!err.empty()) return err;
        opt.rope_positions = rope_positions;
        if (on_device)
            opt.quantizer = [](const uint8_t* s, det::GgmlType ty, size_t src_rows, const std::vector<int>* rp,
                               const std::vector<int>* cp, size_t n, size_t k, int b, uint8_t* out) {
                det::cuda_quantize_rows(s, (int)ty, src_rows, rp, cp, n, k, b, out);
            };
        return det::convert(src, out_path, opt);
    });
}
// Writes the default output name of `det convert` for src_path and `bits` into out (convert.rs:404-420).
int dh_convert_default_output(const char* src_path, const char* bits, char* out, size_t cap) {
    return guarded([&] {
        det::Bits b;
        std::string err = det::Bits::parse(bits ? bits : det::DEFAULT_BITS, b);
        if (!err.empty()) return err;
        snprintf(out, cap, "%s", det::default_output(src_path, b).c_str());
        return std::string();
    });
}
// calibrate.rs:66-89: the value scales [attention layers][kv heads] from a run over `ids`; returns their count in *n_out.
int dh_v_scales(void* m, const int32_t* ids, size_t n, float* out, size_t cap, size_t* n_out) {
    return guarded([&] {
        std::vector<float> s;
        std::string e = det::v_scales(*static_cast<det::Model*>(m), ids, n, s);
        if (!e.empty()) return e;
        *n_out = s.size();
        std::memcpy(out, s.data(), std::min(cap, s.size()) * sizeof(float));
        return std::string();
    });
}
void dh_calibration_ids(const int32_t* prefix, size_t n_prefix, size_t vocab, size_t n_random, int32_t* out) {
    std::vector<int32_t> ids = det::calibration_ids(std::vector<int32_t>(prefix, prefix + n_prefix), vocab, n_random);
    std::memcpy(out, ids.data(), ids.size() * sizeof(int32_t));
}
// calibrate.rs:91-109.  in_place: 0 on success, 2 when the header has no room (nothing written); copy: 0 on success.
int dh_write_scales_in_place(void* m, const float* scales, size_t n, const char* path) {
    std::string err;
    if (det::write_scales_in_place(*static_cast<det::Model*>(m), std::vector<float>(scales, scales + n), path, err)) return 0;
    if (err.empty()) return 2;
    return fail(err);
}
int dh_write_scales_copy(void* m, const float* scales, size_t n, const char* out) {
    std::string err;
    return det::write_scales_copy(*static_cast<det::Model*>(m), std::vector<float>(scales, scales + n), out, err) ? 0 : fail(err);
}
// ---- container access for tools and tests: a handle is a std::shared_ptr<det::Gguf>*
void* dh_gguf_open(const char* path) {
    std::string err;
    std::shared_ptr<det::Gguf> g = det::Gguf::open(path, err);
    if (!g) {
        g_err = err;
        return nullptr;
    }
    return new std::shared_ptr<det::Gguf>(g);
}
void dh_gguf_close(void* g) { delete static_cast<std::shared_ptr<det::Gguf>*>(g); }
size_t dh_gguf_n_tensors(void* g) { return (*static_cast<std::shared_ptr<det::Gguf>*>(g))->tensors.size(); }
size_t dh_gguf_data_start(void* g) { return (*static_cast<std::shared_ptr<det::Gguf>*>(g))->data_start; }
// Tensor i: name into `name`, up to 4 dims into dims (count returned through *nd), type id, offset and byte size.
int dh_gguf_tensor(void* g, size_t i, char* name, size_t cap, size_t* dims, size_t* nd, uint32_t* type_id, size_t* offset,
                   size_t* bytes) {
    return guarded([&] {
        const det::GgufTensor& t = (*static_cast<std::shared_ptr<det::Gguf>*>(g))->tensors.at(i);
        snprintf(name, cap, "%s", t.name.c_str());
        *nd = t.dims.size();
        for (size_t d = 0; d < t.dims.size() && d < 4; d++) dims[d] = t.dims[d];
        *type_id = t.type_id;
        *offset = t.offset;
        *bytes = t.bytes();
        return std::string();
    });
}
// Metadata as text: integers and floats printed, strings as they are, arrays as "[a, b, ...]"; 1 when the key is absent.
int dh_gguf_get(void* g, const char* key, char* out, size_t cap) {
    const det::GgufValue* v = (*static_cast<std::shared_ptr<det::Gguf>*>(g))->get(key);
    if (!v) return 1;
    std::function<std::string(const det::GgufValue&)> text = [&](const det::GgufValue& x) -> std::string {
        char buf[64];
        switch (x.type) {
            case 8: return x.s;
            case 6: case 12: snprintf(buf, sizeof buf, "%.9g", x.f); return buf;
            case 9: {
                std::string s = "[";
                for (size_t i = 0; i < x.arr.size(); i++) s += (i ? ", " : "") + text(x.arr[i]);
                return s + "]";
            }
            case 1: case 3: case 5: case 11: return std::to_string((int64_t)x.u);
            default: return std::to_string(x.u);
        }
    };
    snprintf(out, cap, "%s", text(*v).c_str());
    return 0;
}
// config.rs:34-92 as "key=value" lines (hidden, n_layers, full_attention_interval, vocab, eps, n_heads, n_kv, head_dim,
// rot_dim, rope_theta, intermediate, gdn_k_heads, gdn_v_heads, gdn_dk, gdn_dv, conv_k).
int dh_gguf_config(void* g, char* out, size_t cap) {
    return guarded([&] {
        det::Config c;
        std::string e = det::config_from_gguf(**static_cast<std::shared_ptr<det::Gguf>*>(g), c);
        if (!e.empty()) return e;
        snprintf(out, cap,
                 "hidden=%zu\nn_layers=%zu\nfull_attention_interval=%zu\nvocab=%zu\neps=%.9g\nn_heads=%zu\nn_kv=%zu\nhead_dim=%zu\n"
                 "rot_dim=%zu\nrope_theta=%.17g\nintermediate=%zu\ngdn_k_heads=%zu\ngdn_v_heads=%zu\ngdn_dk=%zu\ngdn_dv=%zu\nconv_k=%zu\n",
                 c.hidden, c.n_layers, c.full_attention_interval, c.vocab, (double)c.eps, c.n_heads, c.n_kv, c.head_dim, c.rot_dim,
                 c.rope_theta, c.intermediate, c.gdn_k_heads, c.gdn_v_heads, c.gdn_dk, c.gdn_dv, c.conv_k);
        return std::string();
    });
}
int dh_gguf_check_finite(void* g) {
    return guarded([&] { return det::check_finite(**static_cast<std::shared_ptr<det::Gguf>*>(g)); });
}
// Host-side row helpers of the spec for tests: dequantize one row of ggml type `type_id`, quantize one row.
int dh_dequant_row(uint32_t type_id, const uint8_t* row, size_t k, float* out) {
    return guarded([&] {
        det::GgmlType t;
        if (!det::ggml_type_from_id(type_id, t)) return std::string("unsupported type");
        det::dequant_row(t, row, k, out);
        return std::string();
    });
}
void dh_quantize_row(const float* w, size_t k, int bits, uint8_t* out) { det::quantize_row(w, k, bits, out); }

// ---- observers: a C callback sees every tap of a forward pass (hooks.rs:7-70).  kind follows det::Tap::Kind; `data` is
// the tap's fp32 buffer in backend memory (NULL for Kv / GdnState / Token taps), readable with dh_backend_read.
typedef void (*dh_tap_fn)(void* user, int kind, size_t layer, size_t pos0, size_t t, const float* data, size_t len,
                          int32_t id, uint64_t rng);
namespace {
struct CallbackObserver : det::Observer {
    dh_tap_fn fn;
    void* user;
    bool gdn_io;
    bool wants_gdn_io() const override { return gdn_io; }
    void observe(const det::Ctx& ctx, const det::Tap& tap) override {
        fn(user, (int)tap.kind, tap.layer, ctx.pos0, ctx.t, tap.x ? tap.x->ptr() : nullptr, tap.x ? tap.x->len() : 0, tap.id, tap.rng);
    }
};
}  // namespace
int dh_model_forward_observed(void* m, const int32_t* ids, size_t t, dh_tap_fn fn, void* user, int gdn_io) {
    return guarded([&] {
        CallbackObserver o;
        o.fn = fn;
        o.user = user;
        o.gdn_io = gdn_io != 0;
        return static_cast<det::Model*>(m)->forward(ids, t, &o);
    });
}
int dh_model_generate_observed(void* m, const int32_t* prompt, size_t n_prompt, size_t n_new, int greedy, float inv_temp,
                               size_t top_k, float top_p, uint64_t rng, int32_t* out, size_t* n_out, dh_tap_fn fn, void* user,
                               int gdn_io) {
    return guarded([&] {
        det::Sampling s;
        s.greedy = greedy != 0;
        s.inv_temp = inv_temp;
        s.top_k = top_k;
        s.top_p = top_p;
        s.rng = rng;
        CallbackObserver o;
        o.fn = fn;
        o.user = user;
        o.gdn_io = gdn_io != 0;
        std::vector<int32_t> ids;
        std::string e = static_cast<det::Model*>(m)->generate(prompt, n_prompt, n_new, s, {}, ids, nullptr, &o);
        std::memcpy(out, ids.data(), ids.size() * sizeof(int32_t));
        *n_out = ids.size();
        return e;
    });
}
// Copies `n` floats of backend memory to the host after the backend's pending work (Ctx::read, hooks.rs:52-62).
void dh_backend_read(void* backend, const float* src, float* out, size_t n) {
    static_cast<det::Backend*>(backend)->read_bytes(src, out, n * sizeof(float));
}

// ---- tensor parallel: a communicator handle is a det::Comm*
void dh_nccl_unique_id(uint8_t* out128) { det::NcclComm::unique_id(out128); }
void* dh_nccl_comm_new(const uint8_t* id128, int rank, int size) {
    try {
        return static_cast<det::Comm*>(new det::NcclComm(id128, rank, size));
    } catch (const std::exception& ex) {
        g_err = ex.what();
        return nullptr;
    }
}
// One-kernel exchanges over NVLink peer memory for up to 8 rows, NCCL (id128, may be null: none) above that.
// Collective set-up: new on every rank, exchange the 64-byte handles, open with all of them in rank order.
void* dh_peer_comm_new(const uint8_t* id128, int rank, int size, size_t region_bytes) {
    try {
        std::unique_ptr<det::Comm> bulk;
        if (id128) bulk = std::make_unique<det::NcclComm>(id128, rank, size);
        return static_cast<det::Comm*>(new det::PeerComm(rank, size, region_bytes, std::move(bulk)));
    } catch (const std::exception& ex) {
        g_err = ex.what();
        return nullptr;
    }
}
void dh_peer_comm_handle(void* c, uint8_t* out64) { static_cast<det::PeerComm*>(static_cast<det::Comm*>(c))->handle(out64); }
void dh_peer_comm_open(void* c, const uint8_t* handles) { static_cast<det::PeerComm*>(static_cast<det::Comm*>(c))->open(handles); }
void dh_peer_comm_open_loopback(void* c) { static_cast<det::PeerComm*>(static_cast<det::Comm*>(c))->open_loopback(); }
// Measurement switch: 0 runs every exchange as its own launch followed by the consumer kernels (same values).
// bit 0: exchange + consumer row kernel as one launch; bit 1: exchanges as prologues of the decode GEMVs they feed
void dh_peer_comm_set_fuse(void* c, int on) {
    auto* p = static_cast<det::PeerComm*>(static_cast<det::Comm*>(c));
    p->fuse = (on & 1) != 0;
    p->fuse_gemv = (on & 2) != 0;
}
// gather(local, gathered, bytes): fills gathered[size][bytes] with every rank's block (host memory).
void* dh_callback_comm_new(int rank, int size, void (*gather)(const void*, void*, size_t)) {
    return static_cast<det::Comm*>(new det::CallbackComm(rank, size, gather));
}
void dh_comm_free(void* c) { delete static_cast<det::Comm*>(c); }
void* dh_model_new_synth_tp(void* backend, const char* config, size_t layers, uint64_t seed, size_t max_ctx,
                            size_t max_batch, void* comm) {
    try {
        det::Config cfg = det::config_by_name(config, layers);
        return det::Model::load_synthetic(cfg, seed, static_cast<det::Backend*>(backend), max_ctx, max_batch,
                                          static_cast<det::Comm*>(comm)).release();
    } catch (const std::exception& ex) {
        g_err = ex.what();
        return nullptr;
    }
}
void dh_model_free(void* m) { delete static_cast<det::Model*>(m); }
size_t dh_model_vocab(void* m) { return static_cast<det::Model*>(m)->cfg.vocab; }
size_t dh_model_pos(void* m) { return static_cast<det::Model*>(m)->pos; }
int dh_model_set_all_logits(void* m, int all) {
    return guarded([&] {
        static_cast<det::Model*>(m)->set_all_logits(all != 0);
        return std::string();
    });
}
int dh_model_reset(void* m) {
    return guarded([&] {
        static_cast<det::Model*>(m)->reset();
        return std::string();
    });
}
int dh_model_forward(void* m, const int32_t* ids, size_t t) {
    return guarded([&] { return static_cast<det::Model*>(m)->forward(ids, t); });
}
int dh_model_prefill(void* m, const int32_t* ids, size_t n) {
    return guarded([&] { return static_cast<det::Model*>(m)->prefill(ids, n); });
}
// Copies the logits of the last forward ([vocab], or [t][vocab] in all-logits mode); returns the element count.
size_t dh_model_logits(void* m, float* out, size_t cap) {
    std::vector<float> l = static_cast<det::Model*>(m)->logits();
    const size_t n = l.size() < cap ? l.size() : cap;
    std::memcpy(out, l.data(), n * sizeof(float));
    return l.size();
}
// greedy != 0 ignores the sampling parameters.  `rng` is the splitmix64 state, advanced by every draw.
int dh_model_pick(void* m, int greedy, float inv_temp, size_t top_k, float top_p, uint64_t* rng, int32_t* id) {
    return guarded([&] {
        det::Sampling s;
        s.greedy = greedy != 0;
        s.inv_temp = inv_temp;
        s.top_k = top_k;
        s.top_p = top_p;
        s.rng = *rng;
        std::string e = static_cast<det::Model*>(m)->pick(s, *id);
        *rng = s.rng;
        return e;
    });
}
// Prefill + up to n_new tokens; writes the ids to `out` and their count to *n_out.
int dh_model_generate(void* m, const int32_t* prompt, size_t n_prompt, size_t n_new, int greedy, float inv_temp,
                      size_t top_k, float top_p, uint64_t rng, int32_t* out, size_t* n_out) {
    return guarded([&] {
        det::Sampling s;
        s.greedy = greedy != 0;
        s.inv_temp = inv_temp;
        s.top_k = top_k;
        s.top_p = top_p;
        s.rng = rng;
        std::vector<int32_t> ids;
        std::string e = static_cast<det::Model*>(m)->generate(prompt, n_prompt, n_new, s, {}, ids);
        std::memcpy(out, ids.data(), ids.size() * sizeof(int32_t));
        *n_out = ids.size();
        return e;
    });
}
// ---- device-resident greedy decode (CUDA backend only)
void* dh_graph_decoder_new(void* m) {
    try {
        return new det::GraphDecoder(*static_cast<det::Model*>(m));
    } catch (const std::exception& ex) {
        g_err = ex.what();
        return nullptr;
    }
}
void dh_graph_decoder_free(void* d) { delete static_cast<det::GraphDecoder*>(d); }
// Queues n steps starting from token first_id (returns without waiting); use_graph replays the captured step.
int dh_graph_decoder_enqueue(void* d, int32_t first_id, size_t n, int use_graph) {
    return guarded([&] { return static_cast<det::GraphDecoder*>(d)->enqueue(first_id, n, use_graph != 0); });
}
// Waits for the queued steps and copies their tokens; returns the count.
size_t dh_graph_decoder_finish(void* d, int32_t* out, size_t cap) {
    std::vector<int32_t> ids = static_cast<det::GraphDecoder*>(d)->finish();
    std::memcpy(out, ids.data(), (ids.size() < cap ? ids.size() : cap) * sizeof(int32_t));
    return ids.size();
}

// Measurement switch of the CUDA backend: 0 composes a batched step from per-sequence attention / GDN calls.
void dh_cuda_set_fuse_rows(void* backend, int on) {
    if (auto* c = dynamic_cast<det::CudaBackend*>(static_cast<det::Backend*>(backend))) c->fuse_rows = on != 0;
}
// ---- batched serving decode (serve.hpp)
void* dh_batch_new(void* model, size_t n_seq, size_t ctx) {
    try {
        return new det::BatchDecoder(*static_cast<det::Model*>(model), n_seq, ctx);
    } catch (const std::exception& ex) {
        g_err = ex.what();
        return nullptr;
    }
}
void dh_batch_free(void* b) { delete static_cast<det::BatchDecoder*>(b); }
int dh_batch_prefill(void* b, size_t i, const int32_t* ids, size_t n, int greedy, float inv_temp, size_t top_k, float top_p,
                     uint64_t seed) {
    return guarded([&] {
        det::Sampling s;
        s.greedy = greedy != 0;
        s.inv_temp = inv_temp;
        s.top_k = top_k;
        s.top_p = top_p;
        s.rng = seed;
        return static_cast<det::BatchDecoder*>(b)->prefill(i, ids, n, s);
    });
}
int dh_batch_step(void* b, size_t steps) {
    return guarded([&] {
        for (size_t i = 0; i < steps; i++) {
            std::string e = static_cast<det::BatchDecoder*>(b)->step();
            if (!e.empty()) return e;
        }
        return std::string();
    });
}
// Tokens produced so far by sequence i (the first one comes from the prefill); returns their number.
size_t dh_batch_tokens(void* b, size_t i, int32_t* out, size_t cap) {
    const std::vector<int32_t>& t = static_cast<det::BatchDecoder*>(b)->seqs[i].out;
    const size_t n = std::min(cap, t.size());
    std::memcpy(out, t.data(), n * sizeof(int32_t));
    return t.size();
}

// One decoded token's GEMVs, `reps` times, without syncing in between (the caller times it with events on the queue).
int dh_gemv_sweep(void* m, int reps, size_t* bytes, size_t* launches) {
    return guarded([&] {
        det::GemvSweep r = det::gemv_sweep(*static_cast<det::Model*>(m), reps);
        *bytes = r.bytes;
        *launches = r.launches;
        return std::string();
    });
}
// Routes the default (host-side) synthetic weight path through the device generator: identical rows, built in seconds.
void dh_use_cuda_synth_rows(int on) { det::set_synth_rows_provider(on ? det::cuda_synth_det_rows : nullptr); }

void dh_synth_prompt(uint64_t seed, size_t n, size_t vocab, int32_t* out) {
    std::vector<int32_t> ids = det::synth_prompt(seed, n, vocab);
    std::memcpy(out, ids.data(), n * sizeof(int32_t));
}
// Host twin of the synthetic generator: `n` det rows of tensor `tid` (for checking the device twin).
void dh_synth_det_rows(uint64_t seed, uint64_t tid, size_t n, size_t k, int bits, uint8_t* out) {
    std::vector<uint8_t> rows = det::synth_det_rows(seed, tid, n, k, bits, 0);
    std::memcpy(out, rows.data(), rows.size());
}
size_t dh_det_row_bytes(int bits, size_t k) { return det::det_row_bytes(bits, k); }

}  // extern "C"
