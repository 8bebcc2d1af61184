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
    bool pairs = false;    // the streaming copy interleaves the rows of two equal halves (det_linear_repack_pairs)
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
    bool fuse_rows = true;
    void absmax_heads(const Buf<float>& v, size_t t, size_t heads, size_t hd, const Buf<float>& slots) override;
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

    // Decode-sized calls (at most stream_max_m rows on the streaming layout) are fused across ops.  A quantization call
    // (rmsnorm_quant / quant) is held back until the next op: a matching gemm() absorbs it as its prologue, anything else
    // runs it on its own first.  A gemm() with several output parts is held back the same way: when a small W8 linear
    // over the same input follows (the GDN a|b projection after qkv|z) both go out as ONE launch; when
    // silu_mul_quant() over its two parts follows and the linear is stored in the pairs layout, the GEMV emits the SwiGLU
    // product from its epilogue and the quantization of that product becomes the next GEMV's prologue.  Results are
    // bit-identical either way (tests/test_gemv_fused_gpu.py); `fuse_decode = false` issues every op on its own.
    bool fuse_decode = true;
    // Tensor parallel: an exchange whose gathered rows feed a decode GEMV is held back like a quantization and becomes that
    // GEMV's prologue (det_act_source.xchg).  Returns false when the shape does not qualify (the caller then runs the
    // exchange kernel itself).  kind DET_ACT_RMSNORM: rows = x_in + gathered, stored to x_out (!= x_in), then RMSNorm with w;
    // DET_ACT_PLAIN: rows = gathered.  Either way the codes / scale / multipliers also land in xq / sx / mx.
    bool hold_exchange(int kind, void* xchg, const float* local, size_t slice, size_t size, const float* x_in, float* x_out,
                       const float* w, float eps, size_t m, int8_t* xq, float* sx, uint16_t* mx);
    // The SwiGLU epilogue also folds the group maxima of its product, and the down projection's GEMV quantizes the product
    // in its prologue from them (no separate quantization launch for the 17408-value row).  Same values either way.
    bool swiglu_amax = true;
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
        unsigned* amax = nullptr;   // group maxima of `a` left by the SwiGLU epilogue that produced it (det_gemv_op.h_amax)
        // tensor parallel: the rows are gathered from every rank's `local` slice through the exchange handle `xchg`; with
        // acc_out the residual `a` plus the gathered rows is what gets normalized, and lands in acc_out
        void* xchg = nullptr;
        const float* local = nullptr;
        size_t slice = 0;
        float* acc_out = nullptr;
    } pending_;
    struct PendingGemm {
        bool on = false;
        const CudaLinear* lin = nullptr;
        PendingAct act;                 // the quantization it absorbed (kind 0: none)
        const int8_t* xq = nullptr;
        const float* sx = nullptr;
        const uint16_t* mx = nullptr;
        size_t m = 0;
        std::vector<float*> dsts;       // one per part
        bool accumulate = false;
        bool tc = false;                // a batch for the tensor-core GEMM (int8 layout), held for a second linear only
    } pending_gemm_;
    bool hold(int kind, const float* a, const float* b, float eps, size_t m, size_t n, int8_t* xq, float* sx,
              uint16_t* mx, unsigned* amax = nullptr);
    void flush_pending();
    void issue_gemv(const PendingGemm& g, const CudaLinear* second, const std::vector<float*>* dsts2, float* h,
                    unsigned* h_amax = nullptr);
    void issue_gemm_tc(const PendingGemm& g, const CudaLinear* second, const std::vector<float*>* dsts2);
    void* scratch(Buf<uint8_t>& slot, size_t bytes);
    void finish_linear(CudaLinear& l);
    Buf<uint8_t> attn_scratch_, gdn_scratch_, sample_scratch_, synth_scratch_;
    Buf<float> swiglu_h_;            // SwiGLU product of a fused gate|up GEMV (the next GEMV quantizes it in its prologue)
    Buf<uint32_t> swiglu_amax_;      // its group maxima, folded by that GEMV's epilogue and consumed by the next one's prologue
    Buf<int32_t> pick_, picks_;
    Buf<uint64_t> z_, zs_;
};

std::vector<uint8_t> cuda_synth_det_rows(uint64_t seed, uint64_t tid, size_t src0, size_t n, size_t k, int bits);
// The device row quantizer for convert() (a RowQuantizer, convert.hpp): uploads the source tensor, runs
// det_quantize_rows in chunks of rows and copies the det file rows back.  Same bytes as host_quantize_rows.
void cuda_quantize_rows(const uint8_t* src, int ggml_type, size_t src_rows, const std::vector<int>* row_perm,
                        const std::vector<int>* col_perm, size_t n, size_t k, int bits, uint8_t* out);

class Model;
struct GemvSweep {
    size_t bytes;      // algorithmic bytes moved: weights + scales + activations in + outputs
    size_t launches;
};
// Issues the GEMV of every linear of the model at M = 1 (one decoded token's worth), `reps` times, into the model's
// logits buffer; no allocation and no sync inside.  The caller brackets it with events to get the GEMV-only rate.
GemvSweep gemv_sweep(Model& m, int reps);

}  // namespace det
