// The model, its activation buffers and the token loop — the C++ mirror of crates/det/src/model.rs (Proj, Attn, Gdn,
// Layer, Work, Sampling, Model::{load, set_all_logits, reset, embed_rows, project, forward, logits, pick, prefill,
// generate}) and of the network's op sequence crates/det/src/qwen35.rs:8-172.  It talks to a backend only through
// the op set of backend.hpp, so the same driver runs the CUDA backend and, in tests, the CPU reference backend.
#pragma once
#include "backend.hpp"
#include "comm.hpp"
#include "gguf.hpp"
#include "hooks.hpp"
#include "synth.hpp"
#include <functional>
#include <memory>
#include <string>
#include <vector>

namespace det {

constexpr float DEFAULT_V_SCALE = 1.0f / 1024.0f;   // model.rs:47

struct Proj {   // model.rs:51-53
    std::vector<std::unique_ptr<Linear>> lins;
};
struct Attn {   // model.rs:55-63
    Proj qkv, o;
    Buf<float> q_norm, k_norm, v_scale, v_inv_scale;
    KvCache kv;
};
struct Gdn {   // model.rs:65-74
    Proj qkvz, ab, out;
    Buf<float> conv, a, dt_bias, norm;
    GdnState state;
};
struct Layer {   // model.rs:81-87
    Buf<float> attn_norm, ffn_norm;
    Proj gu, down;
    bool is_attn = false;
    Attn attn;
    Gdn gdn;
};
struct Work {   // model.rs:89-118
    Buf<float> x;
    Buf<int8_t> xq;
    Buf<float> sx;
    Buf<uint16_t> mx;
    Buf<float> qg, k, v, o;
    Buf<int8_t> oq;
    Buf<float> so;
    Buf<uint16_t> mo;
    Buf<float> qkv, z, a, b, on;
    Buf<int8_t> onq;
    Buf<float> son;
    Buf<uint16_t> mon;
    Buf<float> g, u;
    Buf<int8_t> hq;
    Buf<float> sh;
    Buf<uint16_t> mh;
    Buf<float> logits;
    Buf<float> gin, gout;   // GDN mixer export (model.rs:343-344); sized on the first observed step that asks for them
};
struct Sampling {   // model.rs:120-141
    bool greedy = true;
    float inv_temp = 1.0f;
    size_t top_k = 0;
    float top_p = 1.0f;
    uint64_t rng = 0;
};

// The per-sequence caches / states behind the rows of a batched decode step (serve.hpp): with it the network takes row b
// of the step's activations as the current token of sequence b, at the position pos[b] of that sequence.
struct RowsCtx {
    const std::vector<std::unique_ptr<RowSet>>* sets;   // one per layer
    const Buf<int32_t>* pos;                            // [rows], backend memory
    size_t max_pos;                                     // host bound on the positions
};

class Model {
  public:
    // A seeded random-init model of shape `cfg` (the stand-in for Model::load on a converted checkpoint).
    // `comm` (optional) makes this the shard of rank comm->rank in a tensor-parallel group of comm->size: linears are
    // cut by output rows, attention by q heads, Gated DeltaNet by k heads, the FFN by 128-column groups, the head by
    // vocabulary rows; the residual stream and the norms stay replicated (see network_tp in model.cpp).
    static std::unique_ptr<Model> load_synthetic(const Config& cfg, uint64_t seed, Backend* backend, size_t max_ctx,
                                                 size_t max_batch, Comm* comm = nullptr);

    // Model::load (model.rs:164-365): a det GGUF written by `det convert` (or write_synthetic_gguf).  Null and a message in
    // `err` when the file is unreadable, not a qwen35 det file, holds a non-finite value, or lacks a tensor.
    static std::unique_ptr<Model> load(const std::string& path, Backend* backend, size_t max_ctx, size_t max_batch,
                                       std::string& err);

    void set_all_logits(bool all);                                   // model.rs:367-375
    void reset();                                                    // model.rs:377-387
    std::string embed_rows(const int32_t* ids, size_t t);            // model.rs:389-413; "" on success
    void project(const Proj& p, const Buf<int8_t>& xq, const Buf<float>& sx, const Buf<uint16_t>& mx, size_t t,
                 const std::vector<const Buf<float>*>& dsts);        // model.rs:415-437
    std::string forward(const int32_t* ids, size_t t, Observer* obs = nullptr);            // model.rs:439-465
    std::vector<float> logits();                                     // model.rs:467-470
    std::string pick(Sampling& s, int32_t& id);                      // model.rs:472-496
    std::string pick_row(const Buf<float>& logits_row, Sampling& s, int32_t& id);   // the same draw on a given logits row
    static uint64_t next_draw(Sampling& s);   // advances the generator once, returns z (model.rs:484-485)
    std::string prefill(const int32_t* ids, size_t n, Observer* obs = nullptr);            // model.rs:498-508
    std::string generate(const int32_t* prompt, size_t n_prompt, size_t n_new, Sampling s,
                         const std::vector<int32_t>& stop, std::vector<int32_t>& out,
                         const std::function<void(int32_t)>& on_token = nullptr, Observer* obs = nullptr);   // model.rs:510-547

    Config cfg;
    Backend* backend = nullptr;
    uint64_t seed = 0;
    std::shared_ptr<Gguf> gguf;   // the mapped file of a loaded model (null for a synthetic one); owns the embedding rows
    GgufTensor embed;             // token_embd.weight of `gguf`
    bool calibrated = false;      // the file carries value scales other than the default (model.rs:236-244)
    Buf<float> final_norm, rope_cos, rope_sin;
    Proj lm_head;
    std::vector<Layer> layers;
    Work w;
    size_t max_ctx = 0, max_batch = 0, pos = 0;
    bool all_logits = false;

    void network(size_t pos0, size_t t, Observer* obs = nullptr, const RowsCtx* rows = nullptr);   // qwen35.rs:8-172

    // ---- tensor parallel state (comm == nullptr: none of it is used)
    Comm* comm = nullptr;
    struct Tp {
        size_t heads = 0, kv = 0;        // local q heads / kv heads of an attention layer
        size_t k_heads = 0, v_heads = 0; // local GDN heads
        size_t ffn = 0, hid = 0, voc = 0;   // local FFN columns, hidden rows, vocabulary rows
        Buf<float> mix_full;   // [mb][n_h*hd] gathered mixer output
        Buf<float> h_l, h_full;      // SwiGLU product, local and gathered
        Buf<float> y_l, y_full;      // projection back to hidden, local rows and gathered
        Buf<float> logits_l;
        Buf<float> tmp;              // all-gather scratch
        Buf<float> x_alt;            // second copy of the residual stream (an exchange fused into a GEMV stores the sums here)
    } tp;

  private:
    void network_tp(size_t pos0, size_t t, const RowsCtx* rows);
};

}  // namespace det
