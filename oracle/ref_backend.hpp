// TEST INFRASTRUCTURE — not part of the product.  The reference backend (`--backend ref`, crates/det/src/cpu.rs:73-411)
// behind the driver's Backend interface, so that tests can run the same model driver and conformance suites against it
// that the CUDA backend runs under.  Buffers are plain host memory.
#pragma once
#include "../det_b200/csrc/host/backend.hpp"
#include "ref_ops.hpp"
#include <omp.h>

namespace oracle {

struct RefLinear : det::Linear {
    std::vector<std::vector<uint8_t>> rows;   // owned copies of the det rows, one per fused part
    refops::Linear view;
};

class RefBackend : public det::Backend {
  public:
    std::string name() const override { return "ref (restated crates/det/src/cpu.rs)"; }
    void* alloc_bytes(size_t bytes) override { return std::calloc(bytes ? bytes : 1, 1); }
    void free_bytes(void* p) override { std::free(p); }
    void write_bytes(void* dst, const void* src, size_t bytes) override { std::memcpy(dst, src, bytes); }
    void read_bytes(const void* src, void* dst, size_t bytes) override { std::memcpy(dst, src, bytes); }
    void zero_bytes(void* p, size_t bytes) override { std::memset(p, 0, bytes); }
    void sync() override {}

    std::unique_ptr<det::Linear> linear(const std::vector<det::LinearPart>& parts, size_t k, int bits) override {
        auto l = std::make_unique<RefLinear>();
        l->k = k;
        l->bits = bits;
        l->view.k = k;
        l->view.bits = bits;
        const size_t rb = spec::det_row_bytes(bits, k);
        for (const det::LinearPart& p : parts) {
            l->rows.emplace_back(p.rows, p.rows + p.n * rb);
            l->widths.push_back(p.n);
            l->view.widths.push_back(p.n);
        }
        for (auto& r : l->rows) l->view.parts.push_back(r.data());
        return l;
    }

    void rmsnorm_quant(const det::Buf<float>& x, const det::Buf<float>& w, float eps, size_t m, size_t n,
                       const det::Buf<int8_t>& xq, const det::Buf<float>& sx, const det::Buf<uint16_t>& mx) override {
        refops::rmsnorm_quant(x.ptr(), w.ptr(), eps, m, n, xq.ptr(), sx.ptr(), mx.ptr());
    }
    void quant(const det::Buf<float>& x, size_t m, size_t n, const det::Buf<int8_t>& xq, const det::Buf<float>& sx,
               const det::Buf<uint16_t>& mx) override {
        refops::quant(x.ptr(), m, n, xq.ptr(), sx.ptr(), mx.ptr());
    }
    void gemm(const det::Linear& lin, const det::Buf<int8_t>& xq, const det::Buf<float>& sx,
              const det::Buf<uint16_t>& mx, size_t m, const det::GemmOut& out) override {
        const RefLinear& l = static_cast<const RefLinear&>(lin);
        std::vector<float*> dsts;
        for (const det::Buf<float>* d : out.dst) dsts.push_back(d->ptr());
        const refops::Out mode = out.kind == det::GemmOut::Write ? refops::Out::Write
                                 : out.kind == det::GemmOut::Accumulate ? refops::Out::Accumulate
                                                                        : refops::Out::Parts;
        refops::gemm(l.view, xq.ptr(), sx.ptr(), mx.ptr(), m, mode, dsts.data(), &l.widths);
    }
    void silu_mul_quant(const det::Buf<float>& g, const det::Buf<float>& u, size_t m, size_t n,
                        const det::Buf<int8_t>& hq, const det::Buf<float>& sh, const det::Buf<uint16_t>& mh) override {
        refops::silu_mul_quant(g.ptr(), u.ptr(), m, n, hq.ptr(), sh.ptr(), mh.ptr());
    }
    void attention(const det::AttnLayer& l, const det::KvCache& kv, const det::Shape& s, const det::Buf<float>& qg,
                   const det::Buf<float>& k, const det::Buf<float>& v, const det::Buf<float>& o) override {
        refops::AttnLayer rl{l.q_norm->ptr(), l.k_norm->ptr(), l.v_scale->ptr(), l.v_inv_scale->ptr(),
                             l.rope_cos->ptr(), l.rope_sin->ptr()};
        refops::KvCache rk{kv.kq.ptr(), kv.sk.ptr(), kv.vq.ptr(), kv.capacity};
        refops::Shape rs{s.m, s.pos0, s.n_h, s.n_kv, s.hd, s.rot, s.eps};
        refops::attention(rl, rk, rs, qg.ptr(), k.ptr(), v.ptr(), o.ptr());
    }
    void gdn(const det::GdnLayer& l, const det::GdnState& st, const det::GdnShape& s, const det::Buf<float>& qkv,
             const det::Buf<float>& z, const det::Buf<float>& a, const det::Buf<float>& b, const det::Buf<float>& on,
             const det::GdnExport& ex) override {
        refops::GdnLayer rl{l.conv->ptr(), l.a->ptr(), l.dt_bias->ptr(), l.norm->ptr()};
        refops::GdnState rst{st.conv_state.ptr(), st.s.ptr()};
        refops::GdnShape rs{s.m, s.n_k, s.n_v, s.dk, s.dv, s.eps};
        refops::gdn(rl, rst, rs, qkv.ptr(), z.ptr(), a.ptr(), b.ptr(), on.ptr(), ex.gin ? ex.gin->ptr() : nullptr,
                    ex.gout ? ex.gout->ptr() : nullptr);
    }
    void add(const det::Buf<float>& x, const det::Buf<float>& y, size_t n) override {
        for (size_t i = 0; i < n; i++) x.ptr()[i] = x.ptr()[i] + y.ptr()[i];   // the add of GemmOut::Accumulate (cpu.rs:172-175)
    }
    void silu_mul(const det::Buf<float>& g, const det::Buf<float>& u, size_t m, size_t n, const det::Buf<float>& h) override {
        for (size_t i = 0; i < m * n; i++) h.ptr()[i] = spec::silu_f(g.ptr()[i]) * u.ptr()[i];   // cpu.rs:207
    }
    int32_t argmax(const det::Buf<float>& logits, size_t v) override { return (int32_t)spec::argmax(logits.ptr(), v); }
    int32_t sample(const det::Buf<float>& logits, size_t v, float inv_temp, size_t top_k, float top_p,
                   uint64_t z) override {
        return (int32_t)spec::sample_with_draw(logits.ptr(), v, inv_temp, top_k, top_p, z);
    }
};

// The spec primitives under the op numbers of the det_test_prim hook (kernels/cuda/det_cuda.h:114-118), as the
// `primitives` conformance suite expects them (conformance.rs:231-344).
std::vector<float> prim_ref(int op, const std::vector<float>& x, size_t m, size_t n);

}  // namespace oracle
