// TEST INFRASTRUCTURE — not part of the product.  The reference backend (`--backend ref`, crates/det/src/cpu.rs)
// restated over plain host pointers: every op is the spec function applied row by row; threads only split independent
// rows, heads or output columns, which cannot change a result (cpu.rs:1-3).
#pragma once
#include "spec.hpp"

namespace refops {

// A fused linear over det rows in memory (cpu.rs:19-71): part i holds widths[i] rows of det_row_bytes(bits, k) bytes.
struct Linear {
    std::vector<const uint8_t*> parts;
    std::vector<size_t> widths;
    size_t k = 0;
    int bits = 0;
    size_t n() const {
        size_t s = 0;
        for (size_t w : widths) s += w;
        return s;
    }
    const uint8_t* row(size_t n) const {
        size_t rb = spec::det_row_bytes(bits, k);
        for (size_t i = 0; i < widths.size(); i++) {
            if (n < widths[i]) return parts[i] + n * rb;
            n -= widths[i];
        }
        throw std::runtime_error("row out of range");
    }
};

// cpu.rs:104-127
inline void rmsnorm_quant(const float* x, const float* w, float eps, size_t m, size_t n, int8_t* xq, float* sx,
                          uint16_t* mx) {
    const size_t g = n / spec::GROUP;
#pragma omp parallel for schedule(static)
    for (long t = 0; t < (long)m; t++) {
        std::vector<float> y(n);
        spec::rmsnorm(x + t * n, w, eps, y.data(), n);
        sx[t] = spec::quant_act_i8g(y.data(), xq + t * n, mx + t * g, n);
    }
}
// cpu.rs:129-140
inline void quant(const float* x, size_t m, size_t n, int8_t* xq, float* sx, uint16_t* mx) {
    const size_t g = n / spec::GROUP;
#pragma omp parallel for schedule(static)
    for (long t = 0; t < (long)m; t++) sx[t] = spec::quant_act_i8g(x + t * n, xq + t * n, mx + t * g, n);
}

enum class Out { Write, Accumulate, Parts };
// cpu.rs:142-186.  The per-token unpack of cpu.rs:159-167 is hoisted out of the token loop (integers; legal).
// `out_widths` (Parts only) are the widths of the destination buffers; they default to the widths of the source parts.
inline void gemm(const Linear& lin, const int8_t* xq, const float* sx, const uint16_t* mx, size_t m, Out mode,
                 float* const* dsts /* Write/Accumulate: dsts[0] */, const std::vector<size_t>* out_widths = nullptr) {
    const size_t k = lin.k, n = lin.n(), g = k / spec::GROUP;
    std::vector<float> y(m * n);
#pragma omp parallel for schedule(static)
    for (long j = 0; j < (long)n; j++) {
        spec::DetRow r = spec::det_row(lin.bits, k, lin.row(j));
        std::vector<int8_t> wq(k);
        std::vector<uint16_t> mrow(g);
        spec::unpack_row(r.codes, lin.bits, k, wq.data());
        for (size_t gi = 0; gi < g; gi++) mrow[gi] = r.m(gi);
        for (size_t t = 0; t < m; t++)
            y[t * n + j] = spec::gemm_row(wq.data(), r.c, mrow.data(), xq + t * k, sx[t], mx ? mx + t * g : nullptr, k);
    }
    for (size_t t = 0; t < m; t++) {
        const float* yt = y.data() + t * n;
        switch (mode) {
            case Out::Write:
                std::memcpy(dsts[0] + t * n, yt, n * sizeof(float));
                break;
            case Out::Accumulate: {
                float* d = dsts[0] + t * n;
                for (size_t j = 0; j < n; j++) d[j] = d[j] + yt[j];
                break;
            }
            case Out::Parts: {
                size_t off = 0;
                const std::vector<size_t>& ws = out_widths ? *out_widths : lin.widths;
                for (size_t i = 0; i < ws.size(); i++) {
                    size_t w = ws[i];
                    std::memcpy(dsts[i] + t * w, yt + off, w * sizeof(float));
                    off += w;
                }
                break;
            }
        }
    }
}

// cpu.rs:188-214
inline void silu_mul_quant(const float* gb, const float* u, size_t m, size_t n, int8_t* hq, float* sh, uint16_t* mh) {
    const size_t g = n / spec::GROUP;
#pragma omp parallel for schedule(static)
    for (long t = 0; t < (long)m; t++) {
        std::vector<float> h(n);
        for (size_t i = 0; i < n; i++) h[i] = spec::silu_f(gb[t * n + i]) * u[t * n + i];
        sh[t] = spec::quant_act_i8g(h.data(), hq + t * n, mh + t * g, n);
    }
}

struct AttnLayer {
    const float *q_norm, *k_norm, *v_scale, *v_inv_scale, *rope_cos, *rope_sin;
};
struct KvCache {
    int8_t* kq;
    float* sk;
    int16_t* vq;
    size_t capacity;
};
struct Shape {
    size_t m, pos0, n_h, n_kv, hd, rot;
    float eps;
};
// cpu.rs:216-291 — token by token: KV rows of token t are written before its attention; keys 0..=pos.
inline void attention(const AttnLayer& l, const KvCache& kv, const Shape& s, const float* qg, const float* k,
                      const float* v, float* o) {
    const size_t n_h = s.n_h, n_kv = s.n_kv, hd = s.hd, half = s.rot / 2;
    const size_t rep = n_h / n_kv;
    const float qscale = 1.0f / std::sqrt((float)hd);
    if ((spec::f32_bits(qscale) & 0x007FFFFFu) != 0) throw std::runtime_error("qscale must be a power of two");
    for (size_t t = 0; t < s.m; t++) {
        const size_t pos = s.pos0 + t;
        const float* rc = l.rope_cos + pos * half;
        const float* rs = l.rope_sin + pos * half;
        for (size_t h = 0; h < n_kv; h++) {
            const float* kr = k + (t * n_kv + h) * hd;
            std::vector<float> kn(hd);
            spec::rmsnorm(kr, l.k_norm, s.eps, kn.data(), hd);
            spec::rope(kn.data(), rc, rs, half);
            const size_t row = (pos * n_kv + h) * hd;
            kv.sk[pos * n_kv + h] = spec::quant_act_i8(kn.data(), kv.kq + row, hd);
            spec::quant_v(v + (t * n_kv + h) * hd, l.v_inv_scale[h], kv.vq + row, hd);
        }
#pragma omp parallel for schedule(static)
        for (long h = 0; h < (long)n_h; h++) {
            const size_t base = (t * n_h + h) * 2 * hd;
            const float* qr = qg + base;
            const float* gate = qg + base + hd;
            std::vector<float> qn(hd);
            spec::rmsnorm(qr, l.q_norm, s.eps, qn.data(), hd);
            spec::rope(qn.data(), rc, rs, half);
            for (size_t i = 0; i < hd; i++) qn[i] = qn[i] * qscale;
            std::vector<int8_t> qq(hd);
            const float sq = spec::quant_act_i8(qn.data(), qq.data(), hd);
            const size_t kvh = h / rep;
            std::vector<spec::KvRow> keys(pos + 1);
            for (size_t j = 0; j <= pos; j++)
                keys[j] = spec::KvRow{kv.kq + (j * n_kv + kvh) * hd, kv.sk[j * n_kv + kvh], kv.vq + (j * n_kv + kvh) * hd};
            float* oh = o + (t * n_h + h) * hd;
            spec::attn_head(qq.data(), sq, keys.data(), keys.size(), l.v_scale[kvh], oh, hd);
            spec::attn_gate(oh, gate, hd);
        }
    }
}

struct GdnLayer {
    const float *conv, *a, *dt_bias, *norm;
};
struct GdnState {
    float* conv_state;   // [3][conv_dim]
    float* s;            // [n_v][dk][dv]
};
struct GdnShape {
    size_t m, n_k, n_v, dk, dv;
    float eps;
};
// cpu.rs:293-391
inline void gdn(const GdnLayer& l, const GdnState& st, const GdnShape& s, const float* qkv, const float* z,
                const float* a, const float* b, float* on, float* gin, float* gout) {
    const size_t n_k = s.n_k, n_v = s.n_v, dk = s.dk, dv = s.dv;
    const size_t conv_dim = 2 * n_k * dk + n_v * dv;
    const size_t kd = n_k * dk;
    const size_t rep = n_v / n_k;
    const size_t gw = 2 * dk + dv * rep + 2 * rep;
    float* conv_state = st.conv_state;
    for (size_t t = 0; t < s.m; t++) {
        const float* xt = qkv + t * conv_dim;
        std::vector<float> y(conv_dim);
#pragma omp parallel for schedule(static)
        for (long c = 0; c < (long)conv_dim; c++) {
            const float win[4] = {conv_state[c], conv_state[conv_dim + c], conv_state[2 * conv_dim + c], xt[c]};
            y[c] = spec::gdn_conv(win, l.conv + c * 4);
        }
        std::memmove(conv_state, conv_state + conv_dim, 2 * conv_dim * sizeof(float));
        std::memcpy(conv_state + 2 * conv_dim, xt, conv_dim * sizeof(float));
        std::vector<float> q(kd), k(kd);
        for (size_t h = 0; h < n_k; h++) {
            spec::l2norm(y.data() + h * dk, s.eps, q.data() + h * dk, dk);
            for (size_t i = 0; i < dk; i++) q[h * dk + i] = q[h * dk + i] * spec::qscale_gdn();
            spec::l2norm(y.data() + kd + h * dk, s.eps, k.data() + h * dk, dk);
        }
        const float* v = y.data() + 2 * kd;
        std::vector<float> beta(n_v), decay(n_v);
        for (size_t h = 0; h < n_v; h++) {
            beta[h] = spec::sigmoid_f(b[t * n_v + h]);
            decay[h] = spec::gdn_decay(a[t * n_v + h], l.dt_bias[h], l.a[h]);
        }
        if (gin) {
            float* g = gin + t * n_k * gw;
            for (size_t kh = 0; kh < n_k; kh++) {
                float* r = g + kh * gw;
                std::memcpy(r, q.data() + kh * dk, dk * sizeof(float));
                std::memcpy(r + dk, k.data() + kh * dk, dk * sizeof(float));
                std::memcpy(r + 2 * dk, v + kh * rep * dv, rep * dv * sizeof(float));
                std::memcpy(r + 2 * dk + rep * dv, beta.data() + kh * rep, rep * sizeof(float));
                std::memcpy(r + 2 * dk + rep * dv + rep, decay.data() + kh * rep, rep * sizeof(float));
            }
        }
        std::vector<float> outs(n_v * dv);
#pragma omp parallel for schedule(static)
        for (long h = 0; h < (long)n_v; h++) {
            const size_t kh = h / rep;
            spec::gdn_head_step(st.s + h * dk * dv, dk, dv, k.data() + kh * dk, q.data() + kh * dk, v + h * dv, beta[h],
                                decay[h], outs.data() + h * dv);
        }
        for (size_t h = 0; h < n_v; h++) {
            const size_t base = (t * n_v + h) * dv;
            if (gout) std::memcpy(gout + base, outs.data() + h * dv, dv * sizeof(float));
            std::vector<float> yn(dv);
            spec::rmsnorm(outs.data() + h * dv, l.norm, s.eps, yn.data(), dv);
            for (size_t j = 0; j < dv; j++) on[base + j] = yn[j] * spec::silu_f(z[base + j]);
        }
    }
}

}  // namespace refops
