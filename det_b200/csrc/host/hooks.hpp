// Observation points of a forward pass (crates/det/src/hooks.rs:7-70).  An observer sees the values a run produces, in the
// backend's buffers, as they are produced: the residual stream before every layer, the attention inputs and outputs, the
// Gated DeltaNet mixer's inputs, outputs and state, the logits and the sampled token.  The tap sites are those of
// crates/det/src/qwen35.rs:25-171 and crates/det/src/model.rs:524-538.
#pragma once
#include "backend.hpp"

namespace det {

struct Tap {   // hooks.rs:7-34
    enum Kind {
        Residual,    // x: residual stream before layer `layer` (layer == n_layers: before the final norm), [t][hidden]
        MixerOut,    // x: the mixer's output as fed to its out projection, [t][n_h*hd] or [t][n_v*dv]
        PostMixer,   // x: residual stream after the mixer of `layer`, before its MLP, [t][hidden]
        AttnV,       // x: value projections before quantization, [t][n_kv][hd]
        Kv,          // kv: the cache after the rows of this batch were written
        AttnOut,     // x: gated attention output, [t][n_h][hd]
        GdnIn,       // x: mixer inputs per k head, [t][n_k][2*dk + rep*dv + 2*rep] (q, k, then v, beta, decay of its v heads)
        GdnOut,      // x: mixer output before the gated norm, [t][n_v][dv]
        GdnStateTap, // state: S[n_v][dk][dv] and the conv window after the batch
        Logits,      // x: logits of the last position of the batch, [vocab]
        Token        // id, rng: the token sampled from the last logits and the generator state after the draw
    } kind;
    size_t layer = 0;
    const Buf<float>* x = nullptr;
    const KvCache* kv = nullptr;
    const GdnState* state = nullptr;
    int32_t id = 0;
    uint64_t rng = 0;
};

// hooks.rs:36-62 — the batch covers positions pos0 .. pos0 + t.  read() copies (part of) a tap's buffer to the host after
// the backend's pending work; sync() only waits, for observers that enqueue work of their own on the backend's queue.
struct Ctx {
    size_t pos0 = 0, t = 0;
    Backend* backend = nullptr;
    void sync() const { backend->sync(); }
    template <class T>
    std::vector<T> read(const Buf<T>& b, size_t offset, size_t n) const {
        std::vector<T> v(n);
        backend->read(b, offset, v.data(), n);
        return v;
    }
};

struct Observer {   // hooks.rs:64-70
    virtual ~Observer() = default;
    // Whether the GDN mixer should export its inputs and outputs (GdnIn, GdnOut), which costs extra writes in the kernel.
    virtual bool wants_gdn_io() const { return false; }
    virtual void observe(const Ctx& ctx, const Tap& tap) = 0;
};

}  // namespace det
