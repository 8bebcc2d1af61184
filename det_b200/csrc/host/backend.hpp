// The op set a backend implements and its buffer type — the C++ mirror of det's plugin boundary
// (crates/det/src/backend.rs:13-302: Buf<T>, GemmOut, AttnLayer, KvCache, GdnLayer, GdnState, GdnExport, Shape,
// GdnShape, trait Backend).  Names, argument order and meaning follow the trait so that the driver
// (model.hpp, the mirror of qwen35.rs / model.rs) and the conformance suites read like the reference's.
#pragma once
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace det {

class Backend;

// backend.rs:13-134 — a typed span owned by a backend (released through it) or a borrowed view.
template <class T>
class Buf {
  public:
    Buf() = default;
    Buf(Backend* owner, T* p, size_t len) : owner_(owner), p_(p), len_(len) {}
    static Buf view(T* p, size_t len) { return Buf(nullptr, p, len); }
    Buf(const Buf&) = delete;
    Buf& operator=(const Buf&) = delete;
    Buf(Buf&& o) noexcept { steal(o); }
    Buf& operator=(Buf&& o) noexcept {
        if (this != &o) {
            release();
            steal(o);
        }
        return *this;
    }
    ~Buf() { release(); }
    T* ptr() const { return p_; }
    T* ptr_at(size_t off) const { return p_ + off; }
    size_t len() const { return len_; }
    size_t bytes() const { return len_ * sizeof(T); }
    Backend* owner() const { return owner_; }

  private:
    void steal(Buf& o) {
        owner_ = o.owner_; p_ = o.p_; len_ = o.len_;
        o.owner_ = nullptr; o.p_ = nullptr; o.len_ = 0;
    }
    void release();
    Backend* owner_ = nullptr;
    T* p_ = nullptr;
    size_t len_ = 0;
};

// A quantized linear, possibly several tensors fused along N (backend.rs:229-231).
struct Linear {
    virtual ~Linear() = default;
    std::vector<size_t> widths;
    size_t k = 0;
    int bits = 0;
    size_t n() const {
        size_t s = 0;
        for (size_t w : widths) s += w;
        return s;
    }
};
// One tensor of det rows in host memory: `n` rows of det_row_bytes(bits, k) bytes (spec/tensor.rs:43-55).
struct LinearPart {
    const uint8_t* rows;
    size_t n;
};
// One tensor of a seeded synthetic model: rows are produced by the generator in synth.hpp from (seed, tensor_id).
struct SynthPart {
    uint64_t tensor_id;
    size_t n;
    size_t row0 = 0;   // first row of the tensor this part takes (a tensor-parallel rank takes a slice of the rows)
};

// Optional source of synthetic det rows for Backend::linear_synth's default path (n rows of tensor tid).  When unset the
// rows come from the host generator; a benchmark may plug in the device generator to build a CPU-side model quickly.
using SynthRowsProvider = std::vector<uint8_t> (*)(uint64_t seed, uint64_t tid, size_t row0, size_t n, size_t k, int bits);
void set_synth_rows_provider(SynthRowsProvider p);

// backend.rs:136-142
struct GemmOut {
    enum Kind { Write, Accumulate, Parts } kind;
    std::vector<const Buf<float>*> dst;
    static GemmOut write(const Buf<float>& y) { return GemmOut{Write, {&y}}; }
    static GemmOut accumulate(const Buf<float>& y) { return GemmOut{Accumulate, {&y}}; }
    static GemmOut parts(std::vector<const Buf<float>*> d) { return GemmOut{Parts, std::move(d)}; }
};

// backend.rs:144-151
struct AttnLayer {
    const Buf<float>*q_norm, *k_norm, *v_scale, *v_inv_scale, *rope_cos, *rope_sin;
};
// backend.rs:153-162 (the Metal-only V planes are not carried)
struct KvCache {
    Buf<int8_t> kq;
    Buf<float> sk;
    Buf<int16_t> vq;
    size_t capacity = 0;
};
// backend.rs:164-169
struct GdnLayer {
    const Buf<float>*conv, *a, *dt_bias, *norm;
};
// backend.rs:171-175
struct GdnState {
    Buf<float> conv_state;
    Buf<float> s;
};
// backend.rs:177-182
struct GdnExport {
    const Buf<float>* gin = nullptr;
    const Buf<float>* gout = nullptr;
};
// backend.rs:184-192
struct Shape {
    size_t m, pos0, n_h, n_kv, hd, rot;
    float eps;
};
// backend.rs:194-201
struct GdnShape {
    size_t m, n_k, n_v, dk, dv;
    float eps;
};

// The per-sequence caches (attention layer) or states (GDN layer) behind the rows of a batched decode step: row b of
// the step's activations is the current token of sequence b.  A backend may attach its own lookup tables.
struct RowSet {
    virtual ~RowSet() = default;
    std::vector<const KvCache*> kv;
    std::vector<const GdnState*> st;
};

// backend.rs:203-302
class Backend {
  public:
    virtual ~Backend() = default;
    virtual std::string name() const = 0;

    // raw storage (typed helpers below)
    virtual void* alloc_bytes(size_t bytes) = 0;   // zero-filled
    virtual void free_bytes(void* p) = 0;
    virtual void write_bytes(void* dst, const void* host_src, size_t bytes) = 0;
    virtual void read_bytes(const void* src, void* host_dst, size_t bytes) = 0;   // waits for the producers
    virtual void zero_bytes(void* p, size_t bytes) = 0;
    virtual void sync() = 0;
    virtual void flush() {}   // issues anything a backend holds back (nothing by default); does not wait

    virtual std::unique_ptr<Linear> linear(const std::vector<LinearPart>& parts, size_t k, int bits) = 0;
    // A linear of the seeded synthetic model.  The default builds the det rows on the host and calls linear();
    // a device backend may generate the identical rows in place.
    virtual std::unique_ptr<Linear> linear_synth(uint64_t seed, const std::vector<SynthPart>& parts, size_t k, int bits);

    virtual void rmsnorm_quant(const Buf<float>& x, const Buf<float>& w, float eps, size_t m, size_t n,
                               const Buf<int8_t>& xq, const Buf<float>& sx, const Buf<uint16_t>& mx) = 0;
    virtual void quant(const Buf<float>& x, size_t m, size_t n, const Buf<int8_t>& xq, const Buf<float>& sx,
                       const Buf<uint16_t>& mx) = 0;
    virtual void gemm(const Linear& lin, const Buf<int8_t>& xq, const Buf<float>& sx, const Buf<uint16_t>& mx,
                      size_t m, const GemmOut& out) = 0;
    virtual void silu_mul_quant(const Buf<float>& g, const Buf<float>& u, size_t m, size_t n, const Buf<int8_t>& hq,
                                const Buf<float>& sh, const Buf<uint16_t>& mh) = 0;
    virtual void attention(const AttnLayer& l, const KvCache& kv, const Shape& s, const Buf<float>& qg,
                           const Buf<float>& k, const Buf<float>& v, const Buf<float>& o) = 0;
    virtual void gdn(const GdnLayer& l, const GdnState& st, const GdnShape& s, const Buf<float>& qkv,
                     const Buf<float>& z, const Buf<float>& a, const Buf<float>& b, const Buf<float>& on,
                     const GdnExport& ex) = 0;
    // Not in the reference trait (its token loop is single-device): the two elementwise steps a tensor-parallel step
    // needs on their own — the residual add that GemmOut::Accumulate otherwise fuses (x[i] = x[i] + y[i]), and the
    // SwiGLU product without quantization (h[i] = silu_f(g[i]) * u[i]) — each exactly one spec operation per element.
    virtual void add(const Buf<float>& x, const Buf<float>& y, size_t n) = 0;
    virtual void silu_mul(const Buf<float>& g, const Buf<float>& u, size_t m, size_t n, const Buf<float>& h) = 0;
    // The calibration fold (crates/det/src/calibrate.rs:21-36; an observer's own work in the reference):
    // slots[h] = max(slots[h], largest |v[row][h][0..hd)|) over the t rows.  The default reads v back and folds on the
    // host; a device backend may fold in place on its queue.
    virtual void absmax_heads(const Buf<float>& v, size_t t, size_t heads, size_t hd, const Buf<float>& slots) {
        std::vector<float> x(t * heads * hd), s(heads);
        read(v, 0, x.data(), x.size());
        read(slots, 0, s.data(), heads);
        for (size_t r = 0; r < t; r++)
            for (size_t h = 0; h < heads; h++) {
                float m = 0.0f;
                for (size_t i = 0; i < hd; i++) {
                    const float a = std::fabs(x[(r * heads + h) * hd + i]);
                    m = a > m ? a : m;   // a NaN never wins, as with f32::max
                }
                s[h] = m > s[h] ? m : s[h];
            }
        write(slots, 0, s.data(), heads);
    }
    // Batched serving decode (not in the reference trait, whose Model holds one sequence): `rows` sequences advance one
    // token each.  Row b of qg/k/v/o (or qkv/z/a/b/on) belongs to sequence b, with its own cache or state and its own
    // position pos[b] (a backend buffer of rows int32).  The defaults compose the step from the unchanged single-
    // sequence ops on row views — each row is exactly attention(m=1, pos0=pos[b]) / gdn(m=1) of its sequence; a backend
    // may override them with one launch over all rows (same values).
    virtual std::unique_ptr<RowSet> make_rowset(std::vector<const KvCache*> kv, std::vector<const GdnState*> st) {
        auto r = std::make_unique<RowSet>();
        r->kv = std::move(kv);
        r->st = std::move(st);
        return r;
    }
    virtual void attention_rows(const AttnLayer& l, const RowSet& rows, const Buf<int32_t>& pos, size_t max_pos,
                                const Shape& s /* m = rows; pos0 unused */, const Buf<float>& qg, const Buf<float>& k,
                                const Buf<float>& v, const Buf<float>& o);
    virtual void gdn_rows(const GdnLayer& l, const RowSet& rows, const GdnShape& s /* m = rows */, const Buf<float>& qkv,
                          const Buf<float>& z, const Buf<float>& a, const Buf<float>& b, const Buf<float>& on);
    // argmax / sample of `rows` logits rows at once (row r uses draw z[r]); the defaults loop over the single-row ops.
    virtual std::vector<int32_t> argmax_rows(const Buf<float>& logits, size_t rows, size_t v) {
        std::vector<int32_t> out(rows);
        for (size_t r = 0; r < rows; r++) out[r] = argmax(Buf<float>::view(logits.ptr_at(r * v), v), v);
        return out;
    }
    virtual std::vector<int32_t> sample_rows(const Buf<float>& logits, size_t rows, size_t v, float inv_temp, size_t top_k,
                                             float top_p, const std::vector<uint64_t>& z) {
        std::vector<int32_t> out(rows);
        for (size_t r = 0; r < rows; r++) out[r] = sample(Buf<float>::view(logits.ptr_at(r * v), v), v, inv_temp, top_k, top_p, z[r]);
        return out;
    }
    virtual int32_t argmax(const Buf<float>& logits, size_t v) = 0;
    virtual int32_t sample(const Buf<float>& logits, size_t v, float inv_temp, size_t top_k, float top_p,
                           uint64_t z) = 0;

    // ---- typed helpers (backend.rs:209-227)
    template <class T>
    Buf<T> alloc(size_t len) {
        return Buf<T>(this, static_cast<T*>(alloc_bytes((len ? len : 1) * sizeof(T))), len);
    }
    template <class T>
    Buf<T> upload(const T* data, size_t len) {
        Buf<T> b = alloc<T>(len);
        write_bytes(b.ptr(), data, len * sizeof(T));
        return b;
    }
    template <class T>
    Buf<T> upload(const std::vector<T>& v) { return upload(v.data(), v.size()); }
    template <class T>
    void write(const Buf<T>& b, size_t offset, const T* data, size_t len) {
        write_bytes(b.ptr_at(offset), data, len * sizeof(T));
    }
    template <class T>
    void read(const Buf<T>& b, size_t offset, T* out, size_t len) {
        read_bytes(b.ptr_at(offset), out, len * sizeof(T));
    }
    template <class T>
    std::vector<T> download(const Buf<T>& b) {
        std::vector<T> v(b.len());
        read_bytes(b.ptr(), v.data(), b.bytes());
        return v;
    }
    template <class T>
    void zero(const Buf<T>& b) { zero_bytes(b.ptr(), b.bytes()); }
};

inline void Backend::attention_rows(const AttnLayer& l, const RowSet& rows, const Buf<int32_t>& pos, size_t,
                                    const Shape& s, const Buf<float>& qg, const Buf<float>& k, const Buf<float>& v,
                                    const Buf<float>& o) {
    std::vector<int32_t> p(s.m);
    read(pos, 0, p.data(), s.m);
    for (size_t b = 0; b < s.m; b++) {
        Shape one{1, (size_t)p[b], s.n_h, s.n_kv, s.hd, s.rot, s.eps};
        attention(l, *rows.kv[b], one, Buf<float>::view(qg.ptr_at(b * s.n_h * 2 * s.hd), s.n_h * 2 * s.hd),
                  Buf<float>::view(k.ptr_at(b * s.n_kv * s.hd), s.n_kv * s.hd),
                  Buf<float>::view(v.ptr_at(b * s.n_kv * s.hd), s.n_kv * s.hd),
                  Buf<float>::view(o.ptr_at(b * s.n_h * s.hd), s.n_h * s.hd));
    }
}
inline void Backend::gdn_rows(const GdnLayer& l, const RowSet& rows, const GdnShape& s, const Buf<float>& qkv,
                              const Buf<float>& z, const Buf<float>& a, const Buf<float>& b, const Buf<float>& on) {
    const size_t conv_dim = 2 * s.n_k * s.dk + s.n_v * s.dv, vd = s.n_v * s.dv;
    for (size_t r = 0; r < s.m; r++) {
        GdnShape one{1, s.n_k, s.n_v, s.dk, s.dv, s.eps};
        gdn(l, *rows.st[r], one, Buf<float>::view(qkv.ptr_at(r * conv_dim), conv_dim), Buf<float>::view(z.ptr_at(r * vd), vd),
            Buf<float>::view(a.ptr_at(r * s.n_v), s.n_v), Buf<float>::view(b.ptr_at(r * s.n_v), s.n_v),
            Buf<float>::view(on.ptr_at(r * vd), vd), GdnExport{});
    }
}

template <class T>
void Buf<T>::release() {
    if (owner_ && p_) owner_->free_bytes(p_);
    owner_ = nullptr;
    p_ = nullptr;
    len_ = 0;
}

}  // namespace det
