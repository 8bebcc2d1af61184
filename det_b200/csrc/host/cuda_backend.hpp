// The CUDA backend over the C ABI (the mirror of `Cuda` / `CudaLinear`, crates/det/src/cuda.rs:15-33,96-472).
#pragma once
#include "backend.hpp"
#include "det_b200.h"

namespace det {

// cuda.rs:24-33, plus the streaming copy of the same weights for the decode GEMV.
struct CudaLinear : Linear {
    Buf<uint8_t> wq;       // reference layout [N][K/32 * bytes_per_32] (empty when only the streaming copy is kept)
    Buf<float> c;          // [N]
    Buf<uint16_t> m;       // [N][K/128]
    Buf<uint8_t> stream;   // det_linear_repack layout
    Buf<uint8_t> wq8;      // det_linear_expand layout (signed int8 codes) for the tensor-core GEMM
};

class CudaBackend : public Backend {
  public:
    CudaBackend();
    ~CudaBackend() override;
    std::string name() const override;
    void* alloc_bytes(size_t bytes) override;
    void free_bytes(void* p) override;
    void write_bytes(void* dst, const void* host_src, size_t bytes) override;
    void read_bytes(const void* src, void* host_dst, size_t bytes) override;
    void zero_bytes(void* p, size_t bytes) override;
    void sync() override;
    void flush() override { flush_pending(); }
    std::unique_ptr<Linear> linear(const std::vector<LinearPart>& parts, size_t k, int bits) override;
    std::unique_ptr<Linear> linear_synth(uint64_t seed, const std::vector<SynthPart>& parts, size_t k,
                                         int bits) override;
    void rmsnorm_quant(const Buf<float>& x, const Buf<float>& w, float eps, size_t m, size_t n, const Buf<int8_t>& xq,
                       const Buf<float>& sx, const Buf<uint16_t>& mx) override;
    void quant(const Buf<float>& x, size_t m, size_t n, const Buf<int8_t>& xq, const Buf<float>& sx,
               const Buf<uint16_t>& mx) override;
    void gemm(const Linear& lin, const Buf<int8_t>& xq, const Buf<float>& sx, const Buf<uint16_t>& mx, size_t m,
              const GemmOut& out) override;
    void silu_mul_quant(const Buf<float>& g, const Buf<float>& u, size_t m, size_t n, const Buf<int8_t>& hq,
                        const Buf<float>& sh, const Buf<uint16_t>& mh) override;
    void attention(const AttnLayer& l, const KvCache& kv, const Shape& s, const Buf<float>& qg, const Buf<float>& k,
                   const Buf<float>& v, const Buf<float>& o) override;
    void gdn(const GdnLayer& l, const GdnState& st, const GdnShape& s, const Buf<float>& qkv, const Buf<float>& z,
             const Buf<float>& a, const Buf<float>& b, const Buf<float>& on, const GdnExport& ex) override;
    // batched decode: one launch sequence over all rows (det_attention_rows / det_gdn_rows); `fuse_rows = false` falls back
    // to the composed per-row calls of the base class (measurement switch; same values)
    std::unique_ptr<RowSet> make_rowset(std::vector<const KvCache*> kv, std::vector<const GdnState*> st) override;
    void attention_rows(const AttnLayer& l, const RowSet& rows, const Buf<int32_t>& pos, size_t max_pos, const Shape& s,
                        const Buf<float>& qg, const Buf<float>& k, const Buf<float>& v, const Buf<float>& o) override;
    void gdn_rows(const GdnLayer& l, const RowSet& rows, const GdnShape& s, const Buf<float>& qkv, const Buf<float>& z,
                  const Buf<float>& a, const Buf<float>& b, const Buf<float>& on) override;
    std::vector<int32_t> argmax_rows(const Buf<float>& logits, size_t rows, size_t v) override;
    std::vector<int32_t> sample_rows(const Buf<float>& logits, size_t rows, size_t v, float inv_temp, size_t top_k,
                                     float top_p, const std::vector<uint64_t>& z) override;
    bool gdn_decode_ab(const GdnLayer& l, const GdnState* st, const RowSet* rows, const GdnShape& s, const Linear& ab,
                       const Buf<int8_t>& xq, const Buf<float>& sx, const Buf<uint16_t>& mx, const Buf<float>& qkv,
                       const Buf<float>& z, const Buf<float>& on) override;
    // gdn_decode_ab is off by default: measured on the 27B shape it lengthens every recurrence CTA's critical path by more
    // than the a|b GEMV launch it removes costs (6.79 vs 6.55 ms per token)
    bool fold_ab = false;
    // held-back single-token gdn() + quant as det_gdn_quant: off by default — measured slower on the 27B shape (6.57 vs
    // 6.21 ms per token: the one CTA that quantizes the row is slower than the cluster kernel it replaces)
    bool fuse_gdn_quant = false;
    bool fuse_rows = true;
    void add(const Buf<float>& x, const Buf<float>& y, size_t n) override;
    void silu_mul(const Buf<float>& g, const Buf<float>& u, size_t m, size_t n, const Buf<float>& h) override;
    int32_t argmax(const Buf<float>& logits, size_t v) override;
    int32_t sample(const Buf<float>& logits, size_t v, float inv_temp, size_t top_k, float top_p, uint64_t z) override;

    // The primitive test hook (cuda.rs:474-490).
    std::vector<float> test_prim(int op, const std::vector<float>& x, size_t m, size_t n);

    // Weight-layout policy, fixed before the first linear() (a choice by configuration, never by timing):
    bool stream_layout = true;    // build the streaming copy for the decode GEMV
    bool keep_rowmajor = true;    // keep the reference layout too (needed by the large-M GEMM)
    int stream_max_m = 8;         // batches up to this many tokens go through the streaming GEMV
    bool int8_layout = true;      // build the int8-expanded copy; larger batches then run on the tensor cores

    // Fuse the activation quantization (rmsnorm_quant / quant / silu_mul_quant) into the prologue of the GEMM that
    // consumes it when that GEMM is a decode-sized streaming GEMV (det_gemm_fused).  The quantization call is held
    // back until the next op: a matching gemm() absorbs it, anything else runs it on its own first.  Results are
    // bit-identical either way.  Off by default: measured on the 27B decode step the redundant per-CTA prologue costs
    // more than the separate cluster kernels it removes (+0.3 to +0.9 ms per token depending on the kind).
    bool fuse_activations = false;
    unsigned fuse_kinds = 0xE;   // bit DET_ACT_* set: that kind may be fused

    // Profiling aid: op families in this mask are not launched at all (results are then meaningless); the time a
    // decode step loses without a family is that family's cost.  1 rmsnorm_quant, 2 quant, 4 silu_mul_quant, 8 gemm,
    // 16 attention, 32 gdn.
    unsigned skip_mask = 0;

    // Device-position mode (graph replay): when set, attention() reads pos0 from this device word
    // (det_attention_dev) and sizes its launch for positions up to max_pos.
    const int* pos_dev = nullptr;
    int max_pos = 0;

  private:
    struct PendingAct {
        int kind = 0;   // 0 none, else DET_ACT_*
        const float* a = nullptr;
        const float* b = nullptr;
        float eps = 0.0f;
        size_t m = 0, n = 0;
        int8_t* xq = nullptr;
        float* sx = nullptr;
        uint16_t* mx = nullptr;
    } pending_;
    // A single-token gdn() is held back for one call: when the quantization of its output follows, both run as
    // det_gdn_quant (one launch less); anything else issues it as it is.
    struct PendingGdn {
        bool on = false;
        det_gdn_layer layer{};
        det_gdn_state state{};
        const float *qkv = nullptr, *z = nullptr, *a = nullptr, *b = nullptr;
        float* out = nullptr;
        float eps = 0.0f;
        int n_k = 0, n_v = 0, dk = 0, dv = 0;
    } pending_gdn_;
    bool hold(int kind, const float* a, const float* b, float eps, size_t m, size_t n, int8_t* xq, float* sx,
              uint16_t* mx);
    void flush_pending();
    void flush_gdn();
    void* scratch(Buf<uint8_t>& slot, size_t bytes);
    void finish_linear(CudaLinear& l);
    Buf<uint8_t> attn_scratch_, gdn_scratch_, sample_scratch_, synth_scratch_;
    Buf<int32_t> pick_, picks_;
    Buf<uint64_t> z_, zs_;
};

std::vector<uint8_t> cuda_synth_det_rows(uint64_t seed, uint64_t tid, size_t src0, size_t n, size_t k, int bits);

class Model;
struct GemvSweep {
    size_t bytes;      // algorithmic bytes moved: weights + scales + activations in + outputs
    size_t launches;
};
// Issues the GEMV of every linear of the model at M = 1 (one decoded token's worth), `reps` times, into the model's
// logits buffer; no allocation and no sync inside.  The caller brackets it with events to get the GEMV-only rate.
GemvSweep gemv_sweep(Model& m, int reps);

}  // namespace det
