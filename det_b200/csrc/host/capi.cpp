// C entry points of the host driver library for the Python package (ctypes): backend objects, the synthetic model,
// the token loop.  Every function that can fail returns 0 on success and leaves a message for dh_last_error().
#include "cuda_backend.hpp"
#include "graph_decode.hpp"
#include "model.hpp"
#include "serve.hpp"
#include <cstring>
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
    cb->fuse_decode = fuse_decode != 0;
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
void dh_peer_comm_set_fuse(void* c, int on) { static_cast<det::PeerComm*>(static_cast<det::Comm*>(c))->fuse = on != 0; }
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
