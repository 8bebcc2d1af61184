// TEST AND CPU-BASELINE INFRASTRUCTURE — not part of the product.  The reference's x86 backend (`--backend cpu`,
// crates/det/src/x86/{mod,gemm,glue,attn,gdn,simd}.rs) restated in C++ intrinsics behind the driver's Backend
// interface.  It is the timed CPU baseline of the benchmark and the CPU side of the large-model parity checks (a 27B
// forward through the scalar reference backend would take hours).  Like the reference it
//   * repacks every linear at load into strips of 8 rows whose codes stay packed (6 bits per W6 weight in memory),
//     blocks of 16 k holding the unsigned codes u = wq + OFF as [row][4 k] bytes (gemm.rs:59-134);
//   * runs a work item = a pair of strips x up to 64 tokens, K in chunks of 1024 unpacked once into an L1 scratch,
//     four tokens at a time, group sums corrected by OFF * sum(xq), multiplied by m * mx into int64 (gemm.rs:136-372);
//   * builds the spec's treesum from in-register pair sums, quantizes on 8 lanes (glue.rs), runs attention with
//     sign-moved byte dots and 12-bit-split probabilities (attn.rs) and the Gated DeltaNet recurrence over 32-column
//     state blocks with a running balanced tree (gdn.rs);
//   * exists in two builds, AVX-VNNI (vpdpbusd / vpdpwssd) and plain AVX2, and the conformance suites run on both
//     (crates/det/tests/backends.rs:59-70).  Sampling and argmax are the scalar spec (x86/mod.rs:168-181).
// Threads: OpenMP over independent work items, rows, heads and tokens, where the reference uses rayon.
#pragma once
#include "ref_backend.hpp"
#if defined(__x86_64__)
#include <immintrin.h>

namespace x86port {

constexpr size_t ROWS = 8, PAIR = 16, BLOCK = 16, KC = 1024, TC = 64;
inline size_t block_bytes(int bits) { return 4 * spec::bytes_per_32(bits); }

// A linear repacked into strips (gemm.rs:22-57): [codes: k/16 blocks][m: k/128 x 8 rows u16][c: 8 fp32], 64-byte padded.
struct StripLinear {
    uint8_t* data = nullptr;
    size_t n = 0, k = 0, strip_bytes = 0, m_off = 0, c_off = 0, strips = 0;
    int bits = 0;
    const uint8_t* strip(size_t s) const { return data + s * strip_bytes; }
    const uint16_t* m(size_t s, size_t g) const { return reinterpret_cast<const uint16_t*>(strip(s) + m_off + g * ROWS * 2); }
    float c(size_t row) const {
        float v;
        std::memcpy(&v, strip(row / ROWS) + c_off + (row % ROWS) * 4, 4);
        return v;
    }
    size_t bytes() const { return strips * strip_bytes; }
    StripLinear() = default;
    StripLinear(const StripLinear&) = delete;
    StripLinear& operator=(const StripLinear&) = delete;
    ~StripLinear() { std::free(data); }
};

// gemm.rs:59-134
inline void repack(const refops::Linear& src, StripLinear& out) {
    const size_t k = src.k, n = src.n();
    const int bits = src.bits;
    if (k % spec::GROUP != 0) throw std::runtime_error("x86 port: K must be a multiple of 128");
    const size_t strips = (n + PAIR - 1) / PAIR * 2, bb = block_bytes(bits), g = k / spec::GROUP;
    out.n = n; out.k = k; out.bits = bits; out.strips = strips;
    out.m_off = k / BLOCK * bb;
    out.c_off = out.m_off + g * ROWS * 2;
    out.strip_bytes = (out.c_off + ROWS * 4 + 63) / 64 * 64;
    out.data = static_cast<uint8_t*>(std::aligned_alloc(64, std::max<size_t>(64, strips * out.strip_bytes)));
    if (!out.data) throw std::runtime_error("x86 port: out of memory");
    const int o = 1 << (bits - 1);
#pragma omp parallel for schedule(static)
    for (long s = 0; s < (long)strips; s++) {
        uint8_t* d = out.data + (size_t)s * out.strip_bytes;
        std::memset(d, 0, out.strip_bytes);
        std::vector<uint8_t> u(ROWS * k);
        std::vector<int8_t> wq(k);
        for (size_t r = 0; r < ROWS; r++) {
            const size_t row = (size_t)s * ROWS + r;
            float c = 0.0f;
            if (row < n) {
                const spec::DetRow dr = spec::det_row(bits, k, src.row(row));
                spec::unpack_row(dr.codes, bits, k, wq.data());
                for (size_t i = 0; i < k; i++) u[r * k + i] = (uint8_t)((int)wq[i] + o);
                c = dr.c;
                for (size_t gi = 0; gi < g; gi++) {
                    const uint16_t mg = dr.m(gi);
                    std::memcpy(d + out.m_off + (gi * ROWS + r) * 2, &mg, 2);
                }
            } else {
                std::fill(u.begin() + r * k, u.begin() + (r + 1) * k, (uint8_t)o);   // value 0, m = 1, c = 0
                const uint16_t one = 1;
                for (size_t gi = 0; gi < g; gi++) std::memcpy(d + out.m_off + (gi * ROWS + r) * 2, &one, 2);
            }
            std::memcpy(d + out.c_off + 4 * r, &c, 4);
        }
        for (size_t b = 0; b < k / BLOCK; b++) {
            uint8_t* blk = d + b * bb;
            for (size_t r = 0; r < ROWS; r++)
                for (size_t kk = 0; kk < 4; kk++) {
                    auto q = [&](size_t i) { return u[r * k + b * BLOCK + i * 4 + kk]; };
                    const size_t i = r * 4 + kk;
                    if (bits == 8) {
                        for (size_t qi = 0; qi < 4; qi++) blk[qi * 32 + i] = q(qi);
                    } else if (bits == 4) {
                        blk[i] = (uint8_t)(q(0) | q(1) << 4);
                        blk[32 + i] = (uint8_t)(q(2) | q(3) << 4);
                    } else {
                        blk[i] = (uint8_t)((q(0) & 15) | (q(1) & 15) << 4);
                        blk[32 + i] = (uint8_t)((q(2) & 15) | (q(3) & 15) << 4);
                        blk[64 + i] = (uint8_t)((q(0) >> 4) | (q(1) >> 4) << 2 | (q(2) >> 4) << 4 | (q(3) >> 4) << 6);
                    }
                }
        }
    }
}

inline bool have_avx2() { return __builtin_cpu_supports("avx2"); }
inline bool have_vnni() { return __builtin_cpu_supports("avxvnni"); }

}  // namespace x86port

#pragma GCC push_options
#pragma GCC target("avx2,avxvnni")
namespace x86vnni {
#define X86_VNNI 1
#include "x86_kernels.inc"
#undef X86_VNNI
}  // namespace x86vnni
#pragma GCC pop_options
#pragma GCC push_options
#pragma GCC target("avx2")
namespace x86avx2 {
#define X86_VNNI 0
#include "x86_kernels.inc"
#undef X86_VNNI
}  // namespace x86avx2
#pragma GCC pop_options

namespace oracle {

struct X86LinearObj : det::Linear {
    x86port::StripLinear strips;
};

// x86/mod.rs:27-182
class X86Backend : public RefBackend {
  public:
    bool vnni;
    explicit X86Backend(bool use_vnni) : vnni(use_vnni) {
        if (!x86port::have_avx2() || (use_vnni && !x86port::have_vnni()))
            throw std::runtime_error("x86 port: this CPU lacks the requested instruction set");
    }
    std::string name() const override {
        return std::string("x86 port (") + (vnni ? "avx-vnni" : "avx2") + ", " + std::to_string(omp_get_max_threads()) +
               " threads; restated crates/det/src/x86)";
    }
    std::unique_ptr<det::Linear> linear(const std::vector<det::LinearPart>& parts, size_t k, int bits) override {
        auto l = std::make_unique<X86LinearObj>();
        l->k = k;
        l->bits = bits;
        refops::Linear view;
        view.k = k;
        view.bits = bits;
        for (const det::LinearPart& p : parts) {
            l->widths.push_back(p.n);
            view.widths.push_back(p.n);
            view.parts.push_back(p.rows);
        }
        x86port::repack(view, l->strips);   // the det rows are not kept: the strips hold everything
        return l;
    }
    void rmsnorm_quant(const det::Buf<float>& x, const det::Buf<float>& w, float eps, size_t m, size_t n,
                       const det::Buf<int8_t>& xq, const det::Buf<float>& sx, const det::Buf<uint16_t>& mx) override {
        if (vnni) x86vnni::rmsnorm_quant(x.ptr(), w.ptr(), eps, m, n, xq.ptr(), sx.ptr(), mx.ptr());
        else x86avx2::rmsnorm_quant(x.ptr(), w.ptr(), eps, m, n, xq.ptr(), sx.ptr(), mx.ptr());
    }
    void quant(const det::Buf<float>& x, size_t m, size_t n, const det::Buf<int8_t>& xq, const det::Buf<float>& sx,
               const det::Buf<uint16_t>& mx) override {
        if (vnni) x86vnni::quant(x.ptr(), m, n, xq.ptr(), sx.ptr(), mx.ptr());
        else x86avx2::quant(x.ptr(), m, n, xq.ptr(), sx.ptr(), mx.ptr());
    }
    void gemm(const det::Linear& lin, const det::Buf<int8_t>& xq, const det::Buf<float>& sx,
              const det::Buf<uint16_t>& mx, size_t m, const det::GemmOut& out) override {
        const X86LinearObj& l = static_cast<const X86LinearObj&>(lin);
        std::vector<float*> dsts;
        for (const det::Buf<float>* d : out.dst) dsts.push_back(d->ptr());
        const refops::Out mode = out.kind == det::GemmOut::Write ? refops::Out::Write
                                 : out.kind == det::GemmOut::Accumulate ? refops::Out::Accumulate
                                                                        : refops::Out::Parts;
        if (vnni) x86vnni::gemm(l.strips, xq.ptr(), sx.ptr(), mx.ptr(), m, mode, dsts.data(), l.widths);
        else x86avx2::gemm(l.strips, xq.ptr(), sx.ptr(), mx.ptr(), m, mode, dsts.data(), l.widths);
    }
    void silu_mul_quant(const det::Buf<float>& g, const det::Buf<float>& u, size_t m, size_t n,
                        const det::Buf<int8_t>& hq, const det::Buf<float>& sh, const det::Buf<uint16_t>& mh) override {
        if (vnni) x86vnni::silu_mul_quant(g.ptr(), u.ptr(), m, n, hq.ptr(), sh.ptr(), mh.ptr());
        else x86avx2::silu_mul_quant(g.ptr(), u.ptr(), m, n, hq.ptr(), sh.ptr(), mh.ptr());
    }
    void attention(const det::AttnLayer& l, const det::KvCache& kv, const det::Shape& s, const det::Buf<float>& qg,
                   const det::Buf<float>& k, const det::Buf<float>& v, const det::Buf<float>& o) override {
        refops::AttnLayer rl{l.q_norm->ptr(), l.k_norm->ptr(), l.v_scale->ptr(), l.v_inv_scale->ptr(),
                             l.rope_cos->ptr(), l.rope_sin->ptr()};
        refops::KvCache rk{kv.kq.ptr(), kv.sk.ptr(), kv.vq.ptr(), kv.capacity};
        refops::Shape rs{s.m, s.pos0, s.n_h, s.n_kv, s.hd, s.rot, s.eps};
        if (vnni) x86vnni::attention(rl, rk, rs, qg.ptr(), k.ptr(), v.ptr(), o.ptr());
        else x86avx2::attention(rl, rk, rs, qg.ptr(), k.ptr(), v.ptr(), o.ptr());
    }
    void gdn(const det::GdnLayer& l, const det::GdnState& st, const det::GdnShape& s, const det::Buf<float>& qkv,
             const det::Buf<float>& z, const det::Buf<float>& a, const det::Buf<float>& b, const det::Buf<float>& on,
             const det::GdnExport& ex) override {
        refops::GdnLayer rl{l.conv->ptr(), l.a->ptr(), l.dt_bias->ptr(), l.norm->ptr()};
        refops::GdnState rst{st.conv_state.ptr(), st.s.ptr()};
        refops::GdnShape rs{s.m, s.n_k, s.n_v, s.dk, s.dv, s.eps};
        float* gin = ex.gin ? ex.gin->ptr() : nullptr;
        float* gout = ex.gout ? ex.gout->ptr() : nullptr;
        if (vnni) x86vnni::gdn(rl, rst, rs, qkv.ptr(), z.ptr(), a.ptr(), b.ptr(), on.ptr(), gin, gout);
        else x86avx2::gdn(rl, rst, rs, qkv.ptr(), z.ptr(), a.ptr(), b.ptr(), on.ptr(), gin, gout);
    }
};

}  // namespace oracle
#endif   // __x86_64__
