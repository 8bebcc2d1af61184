// The CUDA backend: device buffers and kernels reached through the C ABI of include/det_b200.h — the C++ mirror of
// crates/det/src/cuda.rs:15-490 (Cuda, CudaLinear, impl Backend for Cuda, test_prim).  Like the reference glue it keeps
// lazily grown scratch buffers for attention, GDN and sampling, builds the device weight layout in linear(), and reads
// picks back through a one-element device buffer.  The B200-specific part is linear(): besides the reference layout
// (kept for large-M GEMMs) it builds the streaming layout the decode GEMV reads (det_linear_repack).
#include "cuda_backend.hpp"
#include "model.hpp"
#include <cstdio>
#include <cstdlib>
#include <stdexcept>

namespace det {

namespace {
constexpr cudaStream_t ST = nullptr;   // the library's own in-order queue (cuda.rs:13)

size_t bytes_per_32(int bits) { return bits == 8 ? 32 : (bits == 6 ? 24 : 16); }
}  // namespace

CudaBackend::CudaBackend() {
    if (det_init() != 0) throw std::runtime_error("CUDA runtime failed to initialize");
    pick_ = alloc<int32_t>(1);
    z_ = alloc<uint64_t>(1);
}
CudaBackend::~CudaBackend() = default;

std::string CudaBackend::name() const { return det_device_name(); }
void* CudaBackend::alloc_bytes(size_t bytes) {
    void* p = det_malloc(bytes < 16 ? 16 : bytes);   // cuda.rs:39-44
    if (!p) {
        fprintf(stderr, "det_malloc(%zu) failed\n", bytes);
        abort();
    }
    return p;
}
void CudaBackend::free_bytes(void* p) {
    flush_pending();
    det_free(p);
}
void CudaBackend::write_bytes(void* dst, const void* src, size_t bytes) {
    flush_pending();
    det_memcpy(dst, src, bytes, ST);
}
void CudaBackend::read_bytes(const void* src, void* dst, size_t bytes) {
    flush_pending();
    det_memcpy(dst, src, bytes, ST);
    det_sync();
}
void CudaBackend::zero_bytes(void* p, size_t bytes) {
    flush_pending();
    det_memset(p, 0, bytes, ST);
}
void CudaBackend::sync() {
    flush_pending();
    det_sync();
}

// Holds an activation quantization back so that the next gemm() can absorb it.  Returns false when it does not qualify.
bool CudaBackend::hold(int kind, const float* a, const float* b, float eps, size_t m, size_t n, int8_t* xq, float* sx,
                       uint16_t* mx, unsigned* amax) {
    flush_pending();
    // rows of more than 8192 values only qualify when their group maxima come with them
    if (!fuse_decode || !stream_layout || m > (size_t)stream_max_m || n % 128 != 0 || (n > 8192 && !amax) || !mx) return false;
    pending_ = PendingAct();
    pending_.kind = kind;
    pending_.amax = amax;
    pending_.a = a; pending_.b = b; pending_.eps = eps;
    pending_.m = m; pending_.n = n;
    pending_.xq = xq; pending_.sx = sx; pending_.mx = mx;
    return true;
}
bool CudaBackend::hold_exchange(int kind, void* xchg, const float* local, size_t slice, size_t size, const float* x_in,
                                float* x_out, const float* w, float eps, size_t m, int8_t* xq, float* sx, uint16_t* mx) {
    flush_pending();
    const size_t n = slice * size;
    if (!fuse_decode || !stream_layout || m > 2 || n % 128 != 0 || n > 8192 || slice % 2 != 0 || !mx) return false;
    pending_ = PendingAct();
    pending_.kind = kind;
    pending_.a = x_in; pending_.b = w; pending_.eps = eps;
    pending_.m = m; pending_.n = n;
    pending_.xq = xq; pending_.sx = sx; pending_.mx = mx;
    pending_.xchg = xchg; pending_.local = local; pending_.slice = slice;
    pending_.acc_out = x_out;
    return true;
}
void CudaBackend::flush_pending() {
    if (pending_gemm_.on) {
        const PendingGemm g = pending_gemm_;
        pending_gemm_.on = false;
        if (g.tc) issue_gemm_tc(g, nullptr, nullptr);
        else issue_gemv(g, nullptr, nullptr, nullptr);
    }
    if (!pending_.kind) return;
    const PendingAct p = pending_;
    pending_ = PendingAct();
    if (p.xchg) {
        // no GEMV took the exchange as its prologue: the exchange kernels run it (in place on x, then the sums are copied
        // to where the fused form would have put them)
        if (p.kind == DET_ACT_RMSNORM) {
            det_xchg_add_rmsnorm_quant(p.xchg, p.local, (int)p.slice, const_cast<float*>(p.a), p.b, p.eps, (int)p.m, p.xq, p.sx, p.mx, ST);
            det_memcpy(p.acc_out, p.a, p.m * p.n * sizeof(float), ST);
        } else {
            det_xchg_quant(p.xchg, p.local, nullptr, (int)p.slice, (int)p.m, p.xq, p.sx, p.mx, ST);
        }
        return;
    }
    if (p.kind == DET_ACT_RMSNORM)
        det_rmsnorm_quant(p.a, p.b, p.eps, (int)p.m, (int)p.n, nullptr, p.xq, p.sx, p.mx, ST);
    else
        det_quant(p.a, (int)p.m, (int)p.n, p.xq, p.sx, p.mx, ST);
    // group maxima that no GEMV consumed: clear them for the next producer
    if (p.amax) det_memset(p.amax, 0, (4 + 8 * p.m * (p.n / 128)) * sizeof(unsigned), ST);
}

// One decode GEMV launch: linear g.lin (with the quantization it absorbed as its prologue), optionally a second W8
// linear over the same rows, optionally the SwiGLU product instead of the outputs of g.lin.
void CudaBackend::issue_gemv(const PendingGemm& g, const CudaLinear* second, const std::vector<float*>* dsts2, float* h,
                             unsigned* h_amax) {
    auto describe = [](const CudaLinear& l) {
        det_qlinear q;
        q.wq = l.stream.ptr();
        q.c = l.c.ptr();
        q.m = l.m.ptr();
        q.N = (int)l.n();
        q.K = (int)l.k;
        q.bits = l.bits | DET_LAYOUT_STREAM | (l.pairs ? DET_LAYOUT_PAIRS : 0);
        return q;
    };
    auto offsets = [](const CudaLinear& l) {
        std::vector<int> offs;
        int acc = 0;
        for (size_t w : l.widths) {
            offs.push_back(acc);
            acc += (int)w;
        }
        return offs;
    };
    const det_qlinear q1 = describe(*g.lin);
    det_qlinear q2{};
    const std::vector<int> offs1 = offsets(*g.lin);
    std::vector<int> offs2;
    det_act_source src{};
    det_gemv_op op{};
    op.lin = &q1;
    if (g.act.kind) {
        src.kind = g.act.kind;
        src.a = g.act.a; src.b = g.act.b; src.eps = g.act.eps;
        src.xq = g.act.xq; src.sx = g.act.sx; src.mx = g.act.mx;
        src.amax = g.act.amax;
        src.xchg = g.act.xchg; src.local = g.act.local; src.slice = (int)g.act.slice; src.acc_out = g.act.acc_out;
        op.src = &src;
    } else {
        op.xq = g.xq; op.sx = g.sx; op.mx = g.mx;
    }
    op.M = (int)g.m;
    if (g.accumulate) {
        op.y = g.dsts[0];
        op.accumulate = 1;
    } else {
        op.nparts = (int)g.dsts.size();
        op.offs = offs1.data();
        op.dsts = g.dsts.data();
    }
    if (second) {
        q2 = describe(*second);
        offs2 = offsets(*second);
        op.lin2 = &q2;
        op.nparts2 = (int)dsts2->size();
        op.offs2 = offs2.data();
        op.dsts2 = dsts2->data();
    }
    op.h = h;
    op.h_amax = h_amax;
    det_gemv(&op, ST);
}

// One tensor-core GEMM launch over a batch: linear g.lin with one output buffer per part, optionally a second linear over
// the same rows in the same launch (det_gemm_pair).
void CudaBackend::issue_gemm_tc(const PendingGemm& g, const CudaLinear* second, const std::vector<float*>* dsts2) {
    auto describe = [](const CudaLinear& l) {
        return det_qlinear{l.wq8.ptr(), l.c.ptr(), l.m.ptr(), (int)l.n(), (int)l.k, l.bits | DET_LAYOUT_INT8};
    };
    auto offsets = [](const CudaLinear& l) {
        std::vector<int> offs;
        int acc = 0;
        for (size_t w : l.widths) {
            offs.push_back(acc);
            acc += (int)w;
        }
        return offs;
    };
    const det_qlinear q1 = describe(*g.lin);
    const std::vector<int> offs1 = offsets(*g.lin);
    if (!second) {
        det_gemm_ex(&q1, g.xq, g.sx, g.mx, (int)g.m, nullptr, 0, (int)offs1.size(), offs1.data(), g.dsts.data(), ST);
        return;
    }
    const det_qlinear q2 = describe(*second);
    const std::vector<int> offs2 = offsets(*second);
    det_gemm_pair(&q1, &q2, g.xq, g.sx, g.mx, (int)g.m, (int)offs1.size(), offs1.data(), g.dsts.data(), (int)offs2.size(),
                  offs2.data(), dsts2->data(), ST);
}

void* CudaBackend::scratch(Buf<uint8_t>& slot, size_t bytes) {   // cuda.rs:81-87
    if (slot.len() < bytes) slot = alloc<uint8_t>(bytes < 256 ? 256 : bytes);
    return slot.ptr();
}

void CudaBackend::finish_linear(CudaLinear& l) {
    det_qlinear src{l.wq.ptr(), l.c.ptr(), l.m.ptr(), (int)l.n(), (int)l.k, l.bits};
    if (int8_layout) {
        l.wq8 = alloc<uint8_t>(det_linear_expand_bytes((int)l.n(), (int)l.k));
        det_linear_expand(&src, l.wq8.ptr(), ST);
    }
    if (!stream_layout) return;
    // two equal halves of a narrow-code linear (gate | up): rows interleaved, so that a decode GEMV can emit the SwiGLU
    // product of a (gate, up) pair from its epilogue (det_linear_repack_pairs); plain outputs are routed back per part
    l.pairs = l.widths.size() == 2 && l.widths[0] == l.widths[1] && l.bits != 8;
    l.stream = alloc<uint8_t>(det_linear_repack_bytes((int)l.n(), (int)l.k, l.bits));
    if (l.pairs) det_linear_repack_pairs(&src, l.stream.ptr(), ST);
    else det_linear_repack(&src, l.stream.ptr(), ST);
    if (!keep_rowmajor) {
        det_sync();
        l.wq = Buf<uint8_t>();
    }
}

// cuda.rs:139-163 — codes row-major, c and m split out; then the streaming copy
std::unique_ptr<Linear> CudaBackend::linear(const std::vector<LinearPart>& parts, size_t k, int bits) {
    auto lin = std::make_unique<CudaLinear>();
    lin->k = k;
    lin->bits = bits;
    size_t n = 0;
    for (const LinearPart& p : parts) {
        lin->widths.push_back(p.n);
        n += p.n;
    }
    const size_t nc = k / 32 * bytes_per_32(bits), g = k / 128, rb = nc + 4 + 2 * g;
    std::vector<uint8_t> wq(n * nc);
    std::vector<float> c(n);
    std::vector<uint16_t> m(n * g);
    size_t r = 0;
    for (const LinearPart& p : parts)
        for (size_t i = 0; i < p.n; i++, r++) {
            const uint8_t* row = p.rows + i * rb;
            std::memcpy(wq.data() + r * nc, row, nc);
            std::memcpy(&c[r], row + nc, 4);
            std::memcpy(m.data() + r * g, row + nc + 4, 2 * g);
        }
    lin->wq = upload(wq);
    lin->c = upload(c);
    lin->m = upload(m);
    det_sync();   // the staging vectors die here
    finish_linear(*lin);
    return lin;
}

std::unique_ptr<Linear> CudaBackend::linear_synth(uint64_t seed, const std::vector<SynthPart>& parts, size_t k,
                                                  int bits) {
    auto lin = std::make_unique<CudaLinear>();
    lin->k = k;
    lin->bits = bits;
    size_t n = 0, nmax = 0;
    for (const SynthPart& p : parts) {
        lin->widths.push_back(p.n);
        n += p.n;
        nmax = p.n > nmax ? p.n : nmax;
    }
    const size_t nc = k / 32 * bytes_per_32(bits), g = k / 128;
    lin->wq = alloc<uint8_t>(n * nc);
    lin->c = alloc<float>(n);
    lin->m = alloc<uint16_t>(n * g);
    double* tmp = static_cast<double*>(scratch(synth_scratch_, nmax * g * sizeof(double)));
    size_t row0 = 0;
    for (const SynthPart& p : parts) {
        det_synth_linear(seed, p.tensor_id, (long long)p.row0, (int)p.n, (int)k, bits, (int)row0, lin->wq.ptr(), lin->c.ptr(),
                         lin->m.ptr(), tmp, ST);
        row0 += p.n;
    }
    finish_linear(*lin);
    return lin;
}

void CudaBackend::rmsnorm_quant(const Buf<float>& x, const Buf<float>& w, float eps, size_t m, size_t n,
                                const Buf<int8_t>& xq, const Buf<float>& sx, const Buf<uint16_t>& mx) {
    if (skip_mask & 1) return;
    if (hold(DET_ACT_RMSNORM, x.ptr(), w.ptr(), eps, m, n, xq.ptr(), sx.ptr(), mx.ptr())) return;
    det_rmsnorm_quant(x.ptr(), w.ptr(), eps, (int)m, (int)n, nullptr, xq.ptr(), sx.ptr(), mx.ptr(), ST);
}
void CudaBackend::quant(const Buf<float>& x, size_t m, size_t n, const Buf<int8_t>& xq, const Buf<float>& sx,
                        const Buf<uint16_t>& mx) {
    if (skip_mask & 2) return;
    if (hold(DET_ACT_PLAIN, x.ptr(), nullptr, 0.0f, m, n, xq.ptr(), sx.ptr(), mx.ptr())) return;
    det_quant(x.ptr(), (int)m, (int)n, xq.ptr(), sx.ptr(), mx.ptr(), ST);
}

// cuda.rs:209-289
void CudaBackend::gemm(const Linear& lin_, const Buf<int8_t>& xq, const Buf<float>& sx, const Buf<uint16_t>& mx,
                       size_t m, const GemmOut& out) {
    const CudaLinear& lin = static_cast<const CudaLinear&>(lin_);
    if (skip_mask & 8) {
        pending_.kind = 0;
        pending_gemm_.on = false;
        return;
    }
    const bool use_stream = lin.stream.ptr() && (m <= (size_t)stream_max_m || !lin.wq.ptr());
    if (out.kind == GemmOut::Parts && out.dst.size() != lin.widths.size()) throw std::logic_error("gemm: part count mismatch");
    std::vector<float*> ptrs;
    for (const Buf<float>* d : out.dst) ptrs.push_back(d->ptr());
    // a held multi-part GEMV takes a small W8 linear over the same rows into its launch (qkv|z + a|b)
    if (pending_gemm_.on) {
        const PendingGemm& g = pending_gemm_;
        const bool same_rows = g.act.kind ? (g.act.xq == xq.ptr() && g.act.sx == sx.ptr() && g.act.mx == mx.ptr())
                                          : (g.xq == xq.ptr() && g.sx == sx.ptr() && g.mx == mx.ptr());
        // a held batch GEMM takes a small W8 linear over the same rows into its launch too (qkv|z + a|b)
        if (g.tc && !use_stream && same_rows && g.m == m && lin.bits == 8 && lin.wq8.ptr() && lin.k == g.lin->k &&
            lin.n() <= 4096 && out.kind == GemmOut::Parts) {
            const PendingGemm first = g;
            pending_gemm_.on = false;
            issue_gemm_tc(first, &lin, &ptrs);
            return;
        }
        if (!g.tc && use_stream && same_rows && g.m == m && lin.bits == 8 && !lin.pairs && lin.k == g.lin->k && lin.n() <= 4096 &&
            out.kind != GemmOut::Accumulate) {
            const PendingGemm first = g;
            pending_gemm_.on = false;
            issue_gemv(first, &lin, &ptrs, nullptr);
            return;
        }
        flush_pending();
    }
    // absorb a held activation quantization when this GEMM is its consumer and nothing it writes feeds the producer
    PendingAct act;
    if (pending_.kind) {
        bool ok = use_stream && pending_.xq == xq.ptr() && pending_.sx == sx.ptr() && pending_.mx == mx.ptr() &&
                  pending_.m == m && pending_.n == lin.k;
        for (float* d : ptrs)
            if (d == pending_.a || d == pending_.b || d == pending_.local || d == pending_.acc_out) ok = false;
        if (ok) {
            act = pending_;
            pending_ = PendingAct();
        } else {
            flush_pending();
        }
    }
    if (use_stream && m <= (size_t)stream_max_m) {
        PendingGemm g;
        g.on = true;
        g.lin = &lin;
        g.act = act;
        g.xq = xq.ptr(); g.sx = sx.ptr(); g.mx = mx.ptr();
        g.m = m;
        g.dsts = ptrs;
        g.accumulate = out.kind == GemmOut::Accumulate;
        if (fuse_decode && out.kind == GemmOut::Parts) {      // may still grow into a dual or a SwiGLU launch
            pending_gemm_ = g;
            return;
        }
        issue_gemv(g, nullptr, nullptr, nullptr);
        return;
    }
    if (!use_stream && lin.wq8.ptr() && fuse_decode && out.kind == GemmOut::Parts && lin.widths.size() <= 4) {
        PendingGemm g;      // may still grow into a pair launch
        g.on = true;
        g.tc = true;
        g.lin = &lin;
        g.xq = xq.ptr(); g.sx = sx.ptr(); g.mx = mx.ptr();
        g.m = m;
        g.dsts = ptrs;
        pending_gemm_ = g;
        return;
    }
    det_qlinear q;
    q.wq = use_stream ? lin.stream.ptr() : lin.wq.ptr();
    q.c = lin.c.ptr();
    q.m = lin.m.ptr();
    q.N = (int)lin.n();
    q.K = (int)lin.k;
    q.bits = use_stream ? (lin.bits | DET_LAYOUT_STREAM | (lin.pairs ? DET_LAYOUT_PAIRS : 0)) : lin.bits;
    if (!use_stream && lin.wq8.ptr()) {
        q.wq = lin.wq8.ptr();
        q.bits = lin.bits | DET_LAYOUT_INT8;
    }
    switch (out.kind) {
        case GemmOut::Write:
            det_gemm_ex(&q, xq.ptr(), sx.ptr(), mx.ptr(), (int)m, ptrs[0], 0, 0, nullptr, nullptr, ST);
            break;
        case GemmOut::Accumulate:
            det_gemm_ex(&q, xq.ptr(), sx.ptr(), mx.ptr(), (int)m, ptrs[0], 1, 0, nullptr, nullptr, ST);
            break;
        case GemmOut::Parts: {
            std::vector<int> offs;
            int acc = 0;
            for (size_t w : lin.widths) {
                offs.push_back(acc);
                acc += (int)w;
            }
            det_gemm_ex(&q, xq.ptr(), sx.ptr(), mx.ptr(), (int)m, nullptr, 0, (int)offs.size(), offs.data(), ptrs.data(), ST);
            break;
        }
    }
}

void CudaBackend::silu_mul_quant(const Buf<float>& g, const Buf<float>& u, size_t m, size_t n, const Buf<int8_t>& hq,
                                 const Buf<float>& sh, const Buf<uint16_t>& mh) {
    if (skip_mask & 4) return;
    // the held gate|up GEMV emits the product itself; its quantization becomes the next GEMV's prologue
    if (pending_gemm_.on && !pending_gemm_.tc && pending_gemm_.lin->pairs && pending_gemm_.dsts.size() == 2 && pending_gemm_.dsts[0] == g.ptr() &&
        pending_gemm_.dsts[1] == u.ptr() && pending_gemm_.m == m && pending_gemm_.lin->n() == 2 * n && n % 128 == 0) {
        const PendingGemm first = pending_gemm_;
        pending_gemm_.on = false;
        if (swiglu_h_.len() < (size_t)stream_max_m * n) {
            swiglu_h_ = alloc<float>((size_t)stream_max_m * n);
            swiglu_amax_ = alloc<uint32_t>(4 + 8 * (size_t)stream_max_m * (n / 128));   // zero-filled
        }
        unsigned* amax = swiglu_amax ? swiglu_amax_.ptr() : nullptr;
        issue_gemv(first, nullptr, nullptr, swiglu_h_.ptr(), amax);
        if (hold(DET_ACT_PLAIN, swiglu_h_.ptr(), nullptr, 0.0f, m, n, hq.ptr(), sh.ptr(), mh.ptr(), amax)) return;
        det_quant(swiglu_h_.ptr(), (int)m, (int)n, hq.ptr(), sh.ptr(), mh.ptr(), ST);
        if (amax) det_memset(amax, 0, swiglu_amax_.bytes(), ST);
        return;
    }
    flush_pending();
    det_silu_mul_quant(g.ptr(), u.ptr(), (int)m, (int)n, nullptr, hq.ptr(), sh.ptr(), mh.ptr(), ST);
}

// cuda.rs:316-364
void CudaBackend::attention(const AttnLayer& l, const KvCache& kv, const Shape& s, const Buf<float>& qg,
                            const Buf<float>& k, const Buf<float>& v, const Buf<float>& o) {
    if (skip_mask & 16) return;
    flush_pending();
    det_attn_layer layer{l.q_norm->ptr(), l.k_norm->ptr(), l.v_scale->ptr(), l.v_inv_scale->ptr()};
    det_kv_cache cache{kv.kq.ptr(), kv.sk.ptr(), kv.vq.ptr(), (int)kv.capacity, nullptr, nullptr};
    void* sc = scratch(attn_scratch_, det_attn_scratch_bytes((int)s.m, (int)s.n_h, (int)s.hd));
    if (pos_dev)
        det_attention_dev(&layer, &cache, qg.ptr(), k.ptr(), v.ptr(), l.rope_cos->ptr(), l.rope_sin->ptr(), (int)s.rot,
                          s.eps, (int)s.m, pos_dev, max_pos, (int)s.n_h, (int)s.n_kv, (int)s.hd, o.ptr(), sc, ST);
    else
        det_attention(&layer, &cache, qg.ptr(), k.ptr(), v.ptr(), l.rope_cos->ptr(), l.rope_sin->ptr(), (int)s.rot,
                      s.eps, (int)s.m, (int)s.pos0, (int)s.n_h, (int)s.n_kv, (int)s.hd, o.ptr(), sc, ST);
}

// cuda.rs:366-423
void CudaBackend::gdn(const GdnLayer& l, const GdnState& st, const GdnShape& s, const Buf<float>& qkv,
                      const Buf<float>& z, const Buf<float>& a, const Buf<float>& b, const Buf<float>& on,
                      const GdnExport& ex) {
    if (skip_mask & 32) return;
    flush_pending();
    det_gdn_layer layer{l.conv->ptr(), l.a->ptr(), l.dt_bias->ptr(), l.norm->ptr()};
    det_gdn_state state{st.conv_state.ptr(), st.s.ptr()};
    void* sc = scratch(gdn_scratch_, det_gdn_scratch_bytes((int)s.m, (int)s.n_k, (int)s.n_v, (int)s.dk, (int)s.dv));
    det_gdn_ex(&layer, &state, qkv.ptr(), z.ptr(), a.ptr(), b.ptr(), s.eps, (int)s.m, (int)s.n_k, (int)s.n_v,
               (int)s.dk, (int)s.dv, on.ptr(), sc, ex.gin ? ex.gin->ptr() : nullptr, ex.gout ? ex.gout->ptr() : nullptr,
               ST);
}

// ---- batched decode: device tables of the per-sequence caches / states of one layer
namespace {
struct CudaRowSet : RowSet {
    Buf<uint8_t> table;   // det_kv_cache[rows] or det_gdn_state[rows] in device memory
};
}  // namespace

std::vector<int32_t> CudaBackend::argmax_rows(const Buf<float>& logits, size_t rows, size_t v) {
    if (!fuse_rows) return Backend::argmax_rows(logits, rows, v);
    flush_pending();
    if (picks_.len() < rows) picks_ = alloc<int32_t>(rows);
    det_argmax(logits.ptr(), (int)rows, (int)v, picks_.ptr(), ST);
    std::vector<int32_t> out(rows);
    read(picks_, 0, out.data(), rows);
    return out;
}
std::vector<int32_t> CudaBackend::sample_rows(const Buf<float>& logits, size_t rows, size_t v, float inv_temp, size_t top_k,
                                              float top_p, const std::vector<uint64_t>& z) {
    if (!fuse_rows) return Backend::sample_rows(logits, rows, v, inv_temp, top_k, top_p, z);
    flush_pending();
    if (picks_.len() < rows) picks_ = alloc<int32_t>(rows);
    if (zs_.len() < rows) zs_ = alloc<uint64_t>(rows);
    write(zs_, 0, z.data(), rows);
    const unsigned long long* zp = reinterpret_cast<const unsigned long long*>(zs_.ptr());
    if (top_k == 0 && top_p >= 1.0f) {
        det_sample(logits.ptr(), (int)rows, (int)v, inv_temp, zp, picks_.ptr(), ST);
    } else {
        void* sc = scratch(sample_scratch_, det_sample_scratch_bytes((int)rows, (int)v));
        det_sample_topkp(logits.ptr(), (int)rows, (int)v, inv_temp, (int)top_k, top_p, zp, picks_.ptr(), sc, ST);
    }
    std::vector<int32_t> out(rows);
    read(picks_, 0, out.data(), rows);
    return out;
}


std::unique_ptr<RowSet> CudaBackend::make_rowset(std::vector<const KvCache*> kv, std::vector<const GdnState*> st) {
    auto r = std::make_unique<CudaRowSet>();
    if (!kv.empty()) {
        std::vector<det_kv_cache> t;
        for (const KvCache* c : kv) t.push_back(det_kv_cache{c->kq.ptr(), c->sk.ptr(), c->vq.ptr(), (int)c->capacity, nullptr, nullptr});
        r->table = upload(reinterpret_cast<const uint8_t*>(t.data()), t.size() * sizeof(det_kv_cache));
    } else {
        std::vector<det_gdn_state> t;
        for (const GdnState* g : st) t.push_back(det_gdn_state{g->conv_state.ptr(), g->s.ptr()});
        r->table = upload(reinterpret_cast<const uint8_t*>(t.data()), t.size() * sizeof(det_gdn_state));
    }
    r->kv = std::move(kv);
    r->st = std::move(st);
    return r;
}

void CudaBackend::attention_rows(const AttnLayer& l, const RowSet& rows, const Buf<int32_t>& pos, size_t max_pos,
                                 const Shape& s, const Buf<float>& qg, const Buf<float>& k, const Buf<float>& v,
                                 const Buf<float>& o) {
    const CudaRowSet* rs = dynamic_cast<const CudaRowSet*>(&rows);
    if (!fuse_rows || !rs) return Backend::attention_rows(l, rows, pos, max_pos, s, qg, k, v, o);
    if (skip_mask & 16) return;
    flush_pending();
    for (const KvCache* c : rows.kv)
        if (max_pos + 1 > c->capacity) throw std::runtime_error("a sequence's position exceeds its cache");
    det_attn_layer layer{l.q_norm->ptr(), l.k_norm->ptr(), l.v_scale->ptr(), l.v_inv_scale->ptr()};
    void* sc = scratch(attn_scratch_, det_attn_scratch_bytes((int)s.m, (int)s.n_h, (int)s.hd));
    det_attention_rows(&layer, reinterpret_cast<const det_kv_cache*>(rs->table.ptr()), pos.ptr(), (int)max_pos, qg.ptr(),
                       k.ptr(), v.ptr(), l.rope_cos->ptr(), l.rope_sin->ptr(), (int)s.rot, s.eps, (int)s.m, (int)s.n_h,
                       (int)s.n_kv, (int)s.hd, o.ptr(), sc, ST);
}

void CudaBackend::gdn_rows(const GdnLayer& l, const RowSet& rows, const GdnShape& s, const Buf<float>& qkv,
                           const Buf<float>& z, const Buf<float>& a, const Buf<float>& b, const Buf<float>& on) {
    const CudaRowSet* rs = dynamic_cast<const CudaRowSet*>(&rows);
    if (!fuse_rows || !rs) return Backend::gdn_rows(l, rows, s, qkv, z, a, b, on);
    if (skip_mask & 32) return;
    flush_pending();
    det_gdn_layer layer{l.conv->ptr(), l.a->ptr(), l.dt_bias->ptr(), l.norm->ptr()};
    void* sc = scratch(gdn_scratch_, det_gdn_scratch_bytes((int)s.m, (int)s.n_k, (int)s.n_v, (int)s.dk, (int)s.dv));
    det_gdn_rows(&layer, reinterpret_cast<const det_gdn_state*>(rs->table.ptr()), qkv.ptr(), z.ptr(), a.ptr(), b.ptr(), s.eps,
                 (int)s.m, (int)s.n_k, (int)s.n_v, (int)s.dk, (int)s.dv, on.ptr(), sc, ST);
}

void CudaBackend::add(const Buf<float>& x, const Buf<float>& y, size_t n) {
    flush_pending();
    det_add(x.ptr(), y.ptr(), (long long)n, ST);
}
void CudaBackend::silu_mul(const Buf<float>& g, const Buf<float>& u, size_t m, size_t n, const Buf<float>& h) {
    flush_pending();
    det_silu_mul_quant(g.ptr(), u.ptr(), (int)m, (int)n, h.ptr(), nullptr, nullptr, nullptr, ST);
}

// cuda.rs:425-471
int32_t CudaBackend::argmax(const Buf<float>& logits, size_t v) {
    flush_pending();
    det_argmax(logits.ptr(), 1, (int)v, pick_.ptr(), ST);
    return download(pick_)[0];
}
int32_t CudaBackend::sample(const Buf<float>& logits, size_t v, float inv_temp, size_t top_k, float top_p,
                            uint64_t z) {
    flush_pending();
    write(z_, 0, &z, 1);
    const unsigned long long* zp = reinterpret_cast<const unsigned long long*>(z_.ptr());
    if (top_k == 0 && top_p >= 1.0f) {
        det_sample(logits.ptr(), 1, (int)v, inv_temp, zp, pick_.ptr(), ST);
    } else {
        void* sc = scratch(sample_scratch_, det_sample_scratch_bytes(1, (int)v));
        det_sample_topkp(logits.ptr(), 1, (int)v, inv_temp, (int)top_k, top_p, zp, pick_.ptr(), sc, ST);
    }
    return download(pick_)[0];
}

// det rows [codes | c | m] of a synthetic tensor, generated on the device and copied to the host
std::vector<uint8_t> cuda_synth_det_rows(uint64_t seed, uint64_t tid, size_t src0, size_t n, size_t k, int bits) {
    const size_t nc = k / 32 * bytes_per_32(bits), g = k / 128, rb = nc + 4 + 2 * g;
    void* wq = det_malloc(n * nc);
    void* c = det_malloc(n * 4);
    void* m = det_malloc(n * g * 2);
    void* tmp = det_malloc(n * g * sizeof(double));
    if (!wq || !c || !m || !tmp) throw std::runtime_error("cuda_synth_det_rows: out of device memory");
    det_synth_linear(seed, tid, (long long)src0, (int)n, (int)k, bits, 0, (uint8_t*)wq, (float*)c, (uint16_t*)m, (double*)tmp, ST);
    std::vector<uint8_t> hw(n * nc), hm(n * g * 2), out(n * rb);
    std::vector<float> hc(n);
    det_memcpy(hw.data(), wq, hw.size(), ST);
    det_memcpy(hc.data(), c, n * 4, ST);
    det_memcpy(hm.data(), m, hm.size(), ST);
    det_sync();
    for (void* p : {wq, c, m, tmp}) det_free(p);
    for (size_t r = 0; r < n; r++) {
        std::memcpy(out.data() + r * rb, hw.data() + r * nc, nc);
        std::memcpy(out.data() + r * rb + nc, &hc[r], 4);
        std::memcpy(out.data() + r * rb + nc + 4, hm.data() + r * g * 2, g * 2);
    }
    return out;
}

void cuda_quantize_rows(const uint8_t* src, int ggml_type, size_t src_rows, const std::vector<int>* row_perm,
                        const std::vector<int>* col_perm, size_t n, size_t k, int bits, uint8_t* out) {
    const size_t esz = ggml_type == 0 ? 4 : 2, g = k / 128, rb = k / 32 * bytes_per_32(bits) + 4 + 2 * g;
    const size_t chunk = std::min<size_t>(n, std::max<size_t>(1, ((size_t)256 << 20) / rb));   // <= 256 MB of rows per pass
    void* dsrc = det_malloc(src_rows * k * esz);
    void* drows = det_malloc(chunk * rb);
    void* tmp = det_malloc(chunk * g * sizeof(double));
    void* drp = row_perm ? det_malloc(n * sizeof(int)) : nullptr;
    void* dcp = col_perm ? det_malloc(k * sizeof(int)) : nullptr;
    if (!dsrc || !drows || !tmp || (row_perm && !drp) || (col_perm && !dcp))
        throw std::runtime_error("cuda_quantize_rows: out of device memory");
    det_memcpy(dsrc, src, src_rows * k * esz, ST);
    if (drp) det_memcpy(drp, row_perm->data(), n * sizeof(int), ST);
    if (dcp) det_memcpy(dcp, col_perm->data(), k * sizeof(int), ST);
    for (size_t r0 = 0; r0 < n; r0 += chunk) {
        const size_t rows = std::min(chunk, n - r0);
        // without a row permutation the chunk starts at source row r0; with one, the permutation is offset instead
        const void* base = drp ? dsrc : static_cast<const uint8_t*>(dsrc) + r0 * k * esz;
        det_quantize_rows(base, ggml_type, drp ? static_cast<const int*>(drp) + r0 : nullptr, static_cast<const int*>(dcp),
                          (int)rows, (int)k, bits, static_cast<uint8_t*>(drows), static_cast<double*>(tmp), ST);
        det_memcpy(out + r0 * rb, drows, rows * rb, ST);
        det_sync();
    }
    for (void* p : {dsrc, drows, tmp, drp, dcp})
        if (p) det_free(p);
}

void CudaBackend::absmax_heads(const Buf<float>& v, size_t t, size_t heads, size_t hd, const Buf<float>& slots) {
    flush_pending();
    det_absmax_heads(v.ptr(), (int)t, (int)heads, (int)hd, slots.ptr(), ST);
}

// Every linear of the model once at M = 1 (the launches of one decoded token's GEMVs), `reps` times.
GemvSweep gemv_sweep(Model& m, int reps) {
    GemvSweep r{0, 0};
    CudaBackend* bk = dynamic_cast<CudaBackend*>(m.backend);
    if (!bk) throw std::runtime_error("gemv_sweep needs the CUDA backend");
    const Buf<float>& y = m.w.logits;   // widest output of any linear; nothing is allocated or freed in here
    auto run = [&](const Proj& p, const Buf<int8_t>& xq, const Buf<float>& sx, const Buf<uint16_t>& mx) {
        for (const auto& lin : p.lins) {
            bk->gemm(*lin, xq, sx, mx, 1, GemmOut::write(y));
            const size_t n = lin->n(), k = lin->k;
            r.bytes += n * (k / 32 * bytes_per_32(lin->bits) + 4 + k / 128 * 2) + (k + 4 + k / 128 * 2) + n * 4;
            r.launches++;
        }
    };
    for (int i = 0; i < reps; i++) {
        for (Layer& l : m.layers) {
            if (l.is_attn) {
                run(l.attn.qkv, m.w.xq, m.w.sx, m.w.mx);
                run(l.attn.o, m.w.oq, m.w.so, m.w.mo);
            } else {
                run(l.gdn.qkvz, m.w.xq, m.w.sx, m.w.mx);
                run(l.gdn.ab, m.w.xq, m.w.sx, m.w.mx);
                run(l.gdn.out, m.w.onq, m.w.son, m.w.mon);
            }
            run(l.gu, m.w.xq, m.w.sx, m.w.mx);
            run(l.down, m.w.hq, m.w.sh, m.w.mh);
        }
        run(m.lm_head, m.w.xq, m.w.sx, m.w.mx);
    }
    bk->flush();
    return r;
}

// cuda.rs:474-490
std::vector<float> CudaBackend::test_prim(int op, const std::vector<float>& x, size_t m, size_t n) {
    Buf<float> xb = upload(x);
    Buf<float> out = alloc<float>(x.size() > m ? x.size() : m);
    det_test_prim(op, xb.ptr(), (int)m, (int)n, out.ptr(), ST);
    return download(out);
}

}  // namespace det
