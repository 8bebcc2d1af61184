// TEST INFRASTRUCTURE — not part of the product.  CPU restatement of det's executable spec
// (crates/det/src/spec/{prim,quant,layers,sample,tensor}.rs, normative text docs/SPEC.md), one function per
// function, every expression in the spec's operation order.  Only tests, the smoke check and the CPU-baseline leg of
// the benchmark may use this directory; the CUDA path never calls into it.
//
// Parity status: the reference ships no golden vectors (its tests are purely differential), so this oracle is pinned
// by (1) the literal constants of the spec, (2) an independent numpy restatement of the primitives
// (tests/golden/make_golden.py) whose outputs are committed as fixtures, and (3) the reference's own conformance cases
// re-run differentially.  Against the unbuildable Rust reference itself parity is unpinned.
//
// Build rules (part of the numerics contract, docs/SPEC.md §8): -ffp-contract=off, no fast math, SSE2 scalar math,
// default MXCSR (round to nearest even, denormals preserved).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <algorithm>
#include <numeric>
#include <stdexcept>

namespace spec {

static inline float f32_from_bits(uint32_t b) { float f; std::memcpy(&f, &b, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t b; std::memcpy(&b, &f, 4); return b; }

// ---------------------------------------------------------------------------------------------------------------
// Rust `as` casts: float -> int saturates and maps NaN to 0 (the spec relies on it, e.g. x86/glue.rs:87).
static inline int32_t as_i32(float v) {
    if (v != v) return 0;
    if (v >= 2147483648.0f) return INT32_MAX;
    if (v <= -2147483648.0f) return INT32_MIN;
    return (int32_t)v;
}
static inline int64_t as_i64(float v) {
    if (v != v) return 0;
    if (v >= 9223372036854775808.0f) return INT64_MAX;
    if (v <= -9223372036854775808.0f) return INT64_MIN;
    return (int64_t)v;
}
static inline uint64_t as_u64(float v) {
    if (v != v) return 0;
    if (v <= 0.0f) return 0;
    if (v >= 18446744073709551616.0f) return UINT64_MAX;
    return (uint64_t)v;
}
static inline int8_t as_i8(float v) {
    if (v != v) return 0;
    if (v >= 127.0f) return 127;
    if (v <= -128.0f) return -128;
    return (int8_t)(int32_t)v;
}
static inline uint16_t as_u16(float v) {
    if (v != v) return 0;
    if (v <= 0.0f) return 0;
    if (v >= 65535.0f) return 65535;
    return (uint16_t)(int32_t)v;
}
static inline int16_t as_i16(float v) {
    if (v != v) return 0;
    if (v >= 32767.0f) return 32767;
    if (v <= -32768.0f) return -32768;
    return (int16_t)(int32_t)v;
}

// ---------------------------------------------------------------------------------------------------------------
// spec/prim.rs:4-36 — constants are f64 literals rounded once to f32.
static const float LOG2E = (float)1.44269504088896341;
static const float EXP_C1 = (float)0.693359375;
static const float EXP_C2 = (float)-2.12194440e-4;
static const float EXP_P[6] = {(float)1.9875691500E-4, (float)1.3981999507E-3, (float)8.3334519073E-3,
                               (float)4.1665795894E-2, (float)1.6666665459E-1, (float)5.0000001201E-1};
static const float EXP_LO = -87.0f;
static const float EXP_HI = 88.0f;
static const float LOG_SQRTHF = (float)0.707106781186547524;
static const float LOG_P[9] = {(float)7.0376836292E-2,  (float)-1.1514610310E-1, (float)1.1676998740E-1,
                               (float)-1.2420140846E-1, (float)1.4249322787E-1,  (float)-1.6668057665E-1,
                               (float)2.0000714765E-1,  (float)-2.4999993993E-1, (float)3.3333331174E-1};
static const float LOG_Q1 = (float)-2.12194440e-4;
static const float LOG_Q2 = (float)0.693359375;
static const float SOFTPLUS_THRESH = 20.0f;
static const float SOFTPLUS_LO = -15.0f;
static const float SIGMOID_LO = -80.0f;

// spec/prim.rs:38-70 — -0 orders below +0; a NaN operand is returned.
static inline float fmin_(float a, float b) {
    if (a != a || b != b) return (a != a) ? a : b;
    if (a < b || (a == b && std::signbit(a))) return a;
    return b;
}
static inline float fmax_(float a, float b) {
    if (a != a || b != b) return (a != a) ? a : b;
    if (a > b || (a == b && std::signbit(b))) return a;
    return b;
}
// spec/prim.rs:72-76 — round half to even (default rounding mode).
static inline float rint_(float x) { return std::nearbyintf(x); }

// spec/prim.rs:78-100
static inline float exp_f(float x) {
    x = fmin_(x, EXP_HI);
    if (x < EXP_LO) return 0.0f;
    float n = std::floor((x * LOG2E) + 0.5f);
    float r = x - (n * EXP_C1);
    r = r - (n * EXP_C2);
    float z = r * r;
    float y = EXP_P[0];
    y = (y * r) + EXP_P[1];
    y = (y * r) + EXP_P[2];
    y = (y * r) + EXP_P[3];
    y = (y * r) + EXP_P[4];
    y = (y * r) + EXP_P[5];
    y = (y * z) + r;
    y = y + 1.0f;
    int32_t ni = as_i32(n);
    float scale = f32_from_bits((uint32_t)((ni + 127) << 23));
    return y * scale;
}

// spec/prim.rs:102-127
static inline float log_f(float x) {
    uint32_t b = f32_bits(x);
    int32_t e = (int32_t)((b >> 23) & 0xFF) - 126;
    float m = f32_from_bits((b & 0x007FFFFFu) | 0x3F000000u);
    if (m < LOG_SQRTHF) {
        e -= 1;
        m = (m + m) - 1.0f;
    } else {
        m = m - 1.0f;
    }
    float z = m * m;
    float y = LOG_P[0];
    for (int i = 1; i < 9; i++) y = (y * m) + LOG_P[i];
    y = y * m;
    y = y * z;
    float ef = (float)e;
    y = y + (LOG_Q1 * ef);
    y = y + (-0.5f * z);
    float r = m + y;
    r = r + (LOG_Q2 * ef);
    return r;
}

// spec/prim.rs:129-138
static inline float softplus_f(float x) {
    if (x > SOFTPLUS_THRESH) return x;
    if (x < SOFTPLUS_LO) return exp_f(x);
    float xs = fmin_(x, SOFTPLUS_THRESH);
    return log_f(1.0f + exp_f(xs));
}
// spec/prim.rs:140-146
static inline float sigmoid_f(float x) {
    if (x < SIGMOID_LO) return exp_f(x);
    float xs = fmax_(x, SIGMOID_LO);
    return 1.0f / (1.0f + exp_f(-xs));
}
// spec/prim.rs:148-150
static inline float silu_f(float x) { return x * sigmoid_f(x); }
// spec/prim.rs:152-154
static inline float rsqrt_f(float x) { return 1.0f / std::sqrt(x); }

// spec/prim.rs:156-174 — balanced tree over the input padded with +0.0 to the next power of two.
static inline float treesum(const float* x, size_t len) {
    if (len == 0) return 0.0f;
    size_t p = 1;
    while (p < len) p <<= 1;
    std::vector<float> s(p, 0.0f);
    std::memcpy(s.data(), x, len * sizeof(float));
    size_t n = p;
    while (n > 1) {
        n /= 2;
        for (size_t i = 0; i < n; i++) s[i] = s[2 * i] + s[2 * i + 1];
    }
    return s[0];
}

// spec/prim.rs:176-185
static inline void rmsnorm(const float* x, const float* w, float eps, float* y, size_t n) {
    std::vector<float> sq(n);
    for (size_t i = 0; i < n; i++) sq[i] = x[i] * x[i];
    float ss = treesum(sq.data(), n);
    float mean = ss / (float)n;
    float inv = rsqrt_f(mean + eps);
    for (size_t i = 0; i < n; i++) y[i] = (x[i] * inv) * w[i];
}
// spec/prim.rs:187-194
static inline void l2norm(const float* x, float eps, float* y, size_t n) {
    std::vector<float> sq(n);
    for (size_t i = 0; i < n; i++) sq[i] = x[i] * x[i];
    float inv = rsqrt_f(treesum(sq.data(), n) + eps);
    for (size_t i = 0; i < n; i++) y[i] = x[i] * inv;
}
// spec/prim.rs:196-199
static inline float absmax(const float* x, size_t n) {
    float m = 0.0f;
    for (size_t i = 0; i < n; i++) m = fmax_(m, std::fabs(x[i]));
    return m;
}
// spec/prim.rs:201-205
static inline float bf16_to_f32(uint16_t b) { return f32_from_bits((uint32_t)b << 16); }
// spec/prim.rs:207-215 — returns the output, advances the state in place.
static inline uint64_t splitmix64(uint64_t& state) {
    state += 0x9E3779B97F4A7C15ull;
    uint64_t z = state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z;
}

// ---------------------------------------------------------------------------------------------------------------
// spec/quant.rs
static const size_t GROUP = 128;

// spec/quant.rs:51-60
static inline int8_t clamp_i8(float v) {
    if (v < -127.0f) return -127;
    if (v > 127.0f) return 127;
    return as_i8(v);
}
// spec/quant.rs:7-16
static inline float quant_act_i8(const float* x, int8_t* q, size_t n) {
    float amax = absmax(x, n);
    float s = (amax == 0.0f) ? 1.0f : amax / 127.0f;
    float inv = 1.0f / s;
    for (size_t i = 0; i < n; i++) q[i] = clamp_i8(rint_(x[i] * inv));
    return s;
}
// spec/quant.rs:21-49
static inline float quant_act_i8g(const float* x, int8_t* q, uint16_t* mx, size_t n) {
    size_t g = n / GROUP;
    if (g * GROUP != n) throw std::runtime_error("quant_act_i8g: n is not a multiple of 128");
    std::vector<float> s_g(g);
    for (size_t i = 0; i < g; i++) s_g[i] = absmax(x + i * GROUP, GROUP) / 127.0f;
    float smax = 0.0f;
    for (size_t i = 0; i < g; i++) smax = fmax_(smax, s_g[i]);
    float sx = (smax == 0.0f) ? 1.0f : smax / 65535.0f;
    for (size_t i = 0; i < g; i++) {
        float m = rint_(s_g[i] / sx);
        m = (m < 1.0f) ? 1.0f : (m > 65535.0f ? 65535.0f : m);
        mx[i] = as_u16(m);
        float eff = sx * (float)mx[i];
        float inv = 1.0f / eff;
        for (size_t k = 0; k < GROUP; k++) q[i * GROUP + k] = clamp_i8(rint_(x[i * GROUP + k] * inv));
    }
    return sx;
}

// spec/tensor.rs:33-41
static inline size_t bytes_per_32(int bits) {
    switch (bits) {
        case 8: return 32;
        case 6: return 24;
        case 4: return 16;
    }
    throw std::runtime_error("unsupported bit width");
}
// spec/tensor.rs:49-55
static inline size_t det_row_bytes(int bits, size_t k) {
    if (k % GROUP) throw std::runtime_error("K is not a multiple of 128");
    return k / 32 * bytes_per_32(bits) + 4 + k / GROUP * 2;
}

// spec/quant.rs:62-97
static inline void unpack_row(const uint8_t* packed, int bits, size_t k, int8_t* out) {
    if (k % 32) throw std::runtime_error("unpack_row: k % 32");
    switch (bits) {
        case 8:
            for (size_t i = 0; i < k; i++) out[i] = (int8_t)packed[i];
            break;
        case 4:
            for (size_t blk = 0; blk < k / 32; blk++) {
                const uint8_t* b = packed + blk * 16;
                for (int i = 0; i < 16; i++) {
                    out[blk * 32 + i] = (int8_t)((int)(b[i] & 0xF) - 8);
                    out[blk * 32 + 16 + i] = (int8_t)((int)(b[i] >> 4) - 8);
                }
            }
            break;
        case 6:
            for (size_t blk = 0; blk < k / 32; blk++) {
                const uint8_t* ql = packed + blk * 24;
                const uint8_t* qh = ql + 16;
                for (int i = 0; i < 32; i++) {
                    uint8_t lo = (i < 16) ? (ql[i] & 0xF) : (ql[i - 16] >> 4);
                    uint8_t hi = (qh[i % 8] >> (2 * (i / 8))) & 3;
                    out[blk * 32 + i] = (int8_t)((int)(lo | (hi << 4)) - 32);
                }
            }
            break;
        default:
            throw std::runtime_error("unsupported bit width");
    }
}

// A det row `[codes][c fp32 LE][m u16 LE × k/128]` (spec/tensor.rs:43-70).
struct DetRow {
    const uint8_t* codes;
    float c;
    const uint8_t* m_bytes;
    uint16_t m(size_t g) const { return (uint16_t)(m_bytes[2 * g] | (m_bytes[2 * g + 1] << 8)); }
};
static inline DetRow det_row(int bits, size_t k, const uint8_t* row) {
    size_t nc = k / 32 * bytes_per_32(bits);
    DetRow r;
    r.codes = row;
    std::memcpy(&r.c, row + nc, 4);
    r.m_bytes = row + nc + 4;
    return r;
}

// spec/quant.rs:99-117 — one output element; mx == nullptr means all ones.
static inline float gemm_row(const int8_t* wq, float c, const uint16_t* m, const int8_t* xq, float sx,
                             const uint16_t* mx, size_t k) {
    size_t g = k / GROUP;
    int64_t acc = 0;
    for (size_t gi = 0; gi < g; gi++) {
        int64_t part = 0;
        for (size_t i = gi * GROUP; i < (gi + 1) * GROUP; i++) part += (int64_t)wq[i] * (int64_t)xq[i];
        int64_t mult = (int64_t)m[gi] * (mx ? (int64_t)mx[gi] : 1);
        acc += mult * part;
    }
    return ((float)acc * c) * sx;
}

// spec/tensor.rs:7-30
static inline float f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1F;
    uint32_t mant = h & 0x3FF;
    uint32_t bits;
    if (exp == 0) {
        if (mant == 0) {
            bits = sign;
        } else {
            uint32_t m = mant;
            int32_t e = 127 - 15 + 1;
            while ((m & 0x400) == 0) {
                m <<= 1;
                e -= 1;
            }
            bits = sign | ((uint32_t)e << 23) | ((m & 0x3FF) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (mant << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (mant << 13);
    }
    return f32_from_bits(bits);
}

// ---------------------------------------------------------------------------------------------------------------
// spec/layers.rs
// spec/layers.rs:5-13 — neox half-split rotation of the first 2*half dims.
static inline void rope(float* x, const float* cos, const float* sin, size_t half) {
    for (size_t i = 0; i < half; i++) {
        float a = x[i], b = x[i + half];
        x[i] = (a * cos[i]) - (b * sin[i]);
        x[i + half] = (b * cos[i]) + (a * sin[i]);
    }
}
static const float P_FIX = 16777216.0f;  // spec/layers.rs:16

struct KvRow {
    const int8_t* kq;
    float sk;
    const int16_t* vq;
};
// spec/layers.rs:25-33
static inline float attn_score(const int8_t* qq, float sq, const KvRow& key, size_t hd) {
    int32_t dot = 0;
    for (size_t i = 0; i < hd; i++) dot += (int32_t)qq[i] * (int32_t)key.kq[i];
    return ((float)dot * sq) * key.sk;
}
// spec/layers.rs:37-49
static inline int64_t attn_chunk(const int8_t* qq, float sq, const KvRow* keys, size_t nkeys, float mx, int64_t* num,
                                 size_t hd) {
    int64_t den = 0;
    for (size_t j = 0; j < nkeys; j++) {
        float s = attn_score(qq, sq, keys[j], hd);
        int64_t pq = as_i64(rint_(exp_f(s - mx) * P_FIX));
        den += pq;
        for (size_t i = 0; i < hd; i++) num[i] += pq * (int64_t)keys[j].vq[i];
    }
    return den;
}
// spec/layers.rs:52-56
static inline void attn_output(const int64_t* num, int64_t den, float v_scale, float* o, size_t hd) {
    for (size_t i = 0; i < hd; i++) o[i] = ((float)num[i] / (float)den) * v_scale;
}
// spec/layers.rs:59-66
static inline void attn_head(const int8_t* qq, float sq, const KvRow* keys, size_t nkeys, float v_scale, float* o,
                             size_t hd) {
    float mx = -INFINITY;
    for (size_t j = 0; j < nkeys; j++) mx = fmax_(mx, attn_score(qq, sq, keys[j], hd));
    std::vector<int64_t> num(hd, 0);
    int64_t den = attn_chunk(qq, sq, keys, nkeys, mx, num.data(), hd);
    attn_output(num.data(), den, v_scale, o, hd);
}
// spec/layers.rs:69-73
static inline void attn_gate(float* o, const float* gate, size_t hd) {
    for (size_t i = 0; i < hd; i++) o[i] = o[i] * sigmoid_f(gate[i]);
}
// spec/layers.rs:76-87
static inline void quant_v(const float* v, float v_inv_scale, int16_t* vq, size_t n) {
    for (size_t i = 0; i < n; i++) {
        float r = rint_(v[i] * v_inv_scale);
        vq[i] = (r < -32767.0f) ? (int16_t)-32767 : (r > 32767.0f ? (int16_t)32767 : as_i16(r));
    }
}
// spec/layers.rs:91-101
static inline void gdn_column_step(float* col, const float* k, float v_j, float beta, float decay, size_t dk) {
    for (size_t i = 0; i < dk; i++) col[i] = col[i] * decay;
    std::vector<float> prod(dk);
    for (size_t i = 0; i < dk; i++) prod[i] = col[i] * k[i];
    float kv_mem = treesum(prod.data(), dk);
    float delta = (v_j - kv_mem) * beta;
    for (size_t i = 0; i < dk; i++) col[i] = col[i] + (k[i] * delta);
}
// spec/layers.rs:104-107
static inline float gdn_column_out(const float* col, const float* q, size_t dk) {
    std::vector<float> prod(dk);
    for (size_t i = 0; i < dk; i++) prod[i] = col[i] * q[i];
    return treesum(prod.data(), dk);
}
// spec/layers.rs:110-132 — s is [dk][dv] row-major.
static inline void gdn_head_step(float* s, size_t dk, size_t dv, const float* k, const float* q, const float* v,
                                 float beta, float decay, float* o) {
    std::vector<float> col(dk);
    for (size_t j = 0; j < dv; j++) {
        for (size_t i = 0; i < dk; i++) col[i] = s[i * dv + j];
        gdn_column_step(col.data(), k, v[j], beta, decay, dk);
        for (size_t i = 0; i < dk; i++) s[i * dv + j] = col[i];
        o[j] = gdn_column_out(col.data(), q, dk);
    }
}
// spec/layers.rs:135-140 — win: 4 inputs oldest first, w: 4 taps.
static inline float gdn_conv(const float win[4], const float w[4]) {
    float y = (w[0] * win[0]) + (w[1] * win[1]);
    y = y + (w[2] * win[2]);
    y = y + (w[3] * win[3]);
    return silu_f(y);
}
// spec/layers.rs:143-145
static inline float gdn_decay(float a, float dt_bias, float a_coef) {
    return exp_f(-(a_coef * softplus_f(a + dt_bias)));
}
static const uint32_t QSCALE_GDN_BITS = 0x3DB504F3u;  // spec/layers.rs:147
static inline float qscale_gdn() { return f32_from_bits(QSCALE_GDN_BITS); }

// ---------------------------------------------------------------------------------------------------------------
// spec/sample.rs
// spec/sample.rs:6-14 — lowest index of the maximum.
static inline size_t argmax(const float* logits, size_t v) {
    size_t best = 0;
    for (size_t i = 1; i < v; i++)
        if (logits[i] > logits[best]) best = i;
    return best;
}
// spec/sample.rs:17-23
static inline void weights(const float* logits, size_t v, float inv_temp, uint64_t* w) {
    std::vector<float> l(v);
    for (size_t i = 0; i < v; i++) l[i] = logits[i] * inv_temp;
    float mx = -INFINITY;
    for (size_t i = 0; i < v; i++) mx = fmax_(mx, l[i]);
    for (size_t i = 0; i < v; i++) w[i] = as_u64(rint_(exp_f(l[i] - mx) * 4294967296.0f));
}
// spec/sample.rs:44-87
static inline size_t sample_with_draw(const float* logits, size_t v, float inv_temp, size_t top_k, float top_p,
                                      uint64_t z) {
    std::vector<uint64_t> w(v);
    weights(logits, v, inv_temp, w.data());
    std::vector<uint8_t> kept(v, 1);
    bool use_k = top_k > 0 && top_k < v;
    bool use_p = top_p < 1.0f;
    if (use_k || use_p) {
        std::vector<size_t> order(v);
        std::iota(order.begin(), order.end(), (size_t)0);
        std::sort(order.begin(), order.end(), [&](size_t a, size_t b) {
            if (w[a] != w[b]) return w[a] > w[b];
            return a < b;
        });
        if (use_k)
            for (size_t j = top_k; j < v; j++) kept[order[j]] = 0;
        if (use_p) {
            unsigned __int128 total = 0;
            for (size_t i = 0; i < v; i++) total += w[i];
            double pr = std::nearbyint((double)top_p * 16777216.0);
            // Rust `f64 as u128`: NaN and negatives map to 0.
            unsigned __int128 p24 = (pr != pr || pr <= 0.0) ? 0 : (unsigned __int128)pr;
            unsigned __int128 thresh = (total * p24 + (((unsigned __int128)1) << 24) - 1) >> 24;
            unsigned __int128 acc = 0;
            size_t cut = v;
            for (size_t j = 0; j < v; j++) {
                acc += w[order[j]];
                if (acc >= thresh) {
                    cut = j + 1;
                    break;
                }
            }
            for (size_t j = cut; j < v; j++) kept[order[j]] = 0;
        }
    }
    uint64_t total = 0;
    for (size_t i = 0; i < v; i++)
        if (kept[i]) total += w[i];
    uint64_t u = z % total;
    uint64_t acc = 0;
    for (size_t i = 0; i < v; i++) {
        if (kept[i]) {
            acc += w[i];
            if (acc > u) return i;
        }
    }
    throw std::runtime_error("sample_with_draw: prefix sum never exceeded the draw");
}

}  // namespace spec
