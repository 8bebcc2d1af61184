// Host twin of the synthetic-model generator and the reference weight quantizer (crates/det/src/quantize.rs).
#include "synth.hpp"
#include <algorithm>
#include <cmath>
#include <cstring>
#include <stdexcept>
#include <thread>

namespace det {

Config config_tiny() {
    Config c;
    c.name = "tiny";
    c.hidden = 1024; c.n_layers = 8; c.vocab = 32768;
    c.n_heads = 8; c.n_kv = 2; c.head_dim = 256;
    c.intermediate = 3072;
    c.gdn_k_heads = 8; c.gdn_v_heads = 16;
    return c;
}
Config config_4b() {
    Config c;
    c.name = "4b";
    c.hidden = 2560; c.n_layers = 32; c.vocab = 248320;
    c.n_heads = 16; c.n_kv = 4; c.head_dim = 256;
    c.intermediate = 9216;
    c.gdn_k_heads = 16; c.gdn_v_heads = 32;
    return c;
}
Config config_27b() {
    Config c;
    c.name = "27b";
    c.hidden = 5120; c.n_layers = 64; c.vocab = 248320;
    c.n_heads = 24; c.n_kv = 4; c.head_dim = 256;
    c.intermediate = 17408;
    c.gdn_k_heads = 16; c.gdn_v_heads = 48;
    return c;
}
Config config_by_name(const std::string& name, size_t layers) {
    Config c;
    if (name == "tiny") c = config_tiny();
    else if (name == "4b") c = config_4b();
    else if (name == "27b") c = config_27b();
    else throw std::runtime_error("unknown config '" + name + "' (tiny, 4b, 27b)");
    if (layers) {
        if (layers % c.full_attention_interval) throw std::runtime_error("layer override must be a multiple of 4");
        c.n_layers = layers;
    }
    return c;
}

size_t det_row_bytes(int bits, size_t k) {
    const size_t per32 = bits == 8 ? 32 : (bits == 6 ? 24 : 16);
    return k / 32 * per32 + 4 + k / 128 * 2;
}

// quantize.rs:8-31
void pack_codes(const int8_t* codes, size_t n, int bits, uint8_t* out) {
    for (size_t blk = 0; blk < n / 32; blk++) {
        const int8_t* q = codes + blk * 32;
        if (bits == 8) {
            for (int i = 0; i < 32; i++) *out++ = (uint8_t)q[i];
        } else if (bits == 4) {
            for (int i = 0; i < 16; i++) *out++ = (uint8_t)((q[i] + 8) | ((q[i + 16] + 8) << 4));
        } else {
            uint8_t u[32];
            for (int i = 0; i < 32; i++) u[i] = (uint8_t)(q[i] + 32);
            for (int i = 0; i < 16; i++) *out++ = (uint8_t)((u[i] & 0xF) | ((u[i + 16] & 0xF) << 4));
            for (int i = 0; i < 8; i++)
                *out++ = (uint8_t)((u[i] >> 4) | ((u[i + 8] >> 4) << 2) | ((u[i + 16] >> 4) << 4) | ((u[i + 24] >> 4) << 6));
        }
    }
}

// quantize.rs:33-56 — the scale with the least squared error among base * (0.80 + 0.02 * step), step = 0..10
static double group_scale(const double* w, double qmax) {
    double amax = 0.0;
    for (int i = 0; i < 128; i++) amax = std::max(amax, std::fabs(w[i]));
    if (amax == 0.0) return 1.0;
    const double base = amax / qmax;
    double best_err = INFINITY, best_s = base;
    for (int step = 0; step <= 10; step++) {
        const double s = base * (0.80 + 0.02 * (double)step);
        double err = 0.0;
        for (int i = 0; i < 128; i++) {
            double q = std::nearbyint(w[i] / s);
            q = q < -qmax ? -qmax : (q > qmax ? qmax : q);
            const double d = q * s - w[i];
            err += d * d;
        }
        if (err < best_err) {
            best_err = err;
            best_s = s;
        }
    }
    return best_s;
}

// quantize.rs:58-85
void quantize_row(const float* w, size_t k, int bits, uint8_t* out_row) {
    const size_t g = k / 128;
    const double qmax = (double)((1 << (bits - 1)) - 1);
    std::vector<double> wd(k), scales(g);
    for (size_t i = 0; i < k; i++) wd[i] = (double)w[i];
    double smax = 0.0;
    for (size_t gi = 0; gi < g; gi++) {
        scales[gi] = group_scale(wd.data() + gi * 128, qmax);
        smax = std::max(smax, scales[gi]);
    }
    const float c = (float)(smax / 65535.0);
    std::vector<uint16_t> m(g);
    std::vector<int8_t> codes(k);
    for (size_t gi = 0; gi < g; gi++) {
        double mv = std::nearbyint(scales[gi] / (double)c);
        mv = mv < 1.0 ? 1.0 : (mv > 65535.0 ? 65535.0 : mv);
        m[gi] = (uint16_t)mv;
        const double eff = (double)c * (double)m[gi];
        for (size_t i = gi * 128; i < (gi + 1) * 128; i++) {
            double q = std::nearbyint(wd[i] / eff);
            q = q < -qmax ? -qmax : (q > qmax ? qmax : q);
            codes[i] = (int8_t)q;
        }
    }
    const size_t per32 = bits == 8 ? 32 : (bits == 6 ? 24 : 16);
    pack_codes(codes.data(), k, bits, out_row);
    uint8_t* tail = out_row + k / 32 * per32;
    std::memcpy(tail, &c, 4);
    std::memcpy(tail + 4, m.data(), g * 2);
}

std::vector<uint8_t> synth_det_rows(uint64_t seed, uint64_t tid, size_t n, size_t k, int bits, size_t row0) {
    const size_t rb = det_row_bytes(bits, k);
    std::vector<uint8_t> out(n * rb);
    unsigned nt = std::max(1u, std::min(std::thread::hardware_concurrency(), 32u));
    if (n * k < (1u << 20)) nt = 1;
    std::vector<std::thread> pool;
    for (unsigned w = 0; w < nt; w++) {
        pool.emplace_back([&, w]() {
            std::vector<float> row(k);
            for (size_t r = w; r < n; r += nt) {
                for (size_t i = 0; i < k; i++) row[i] = synth_weight(seed, tid, (row0 + r) * k + i);
                quantize_row(row.data(), k, bits, out.data() + r * rb);
            }
        });
    }
    for (auto& t : pool) t.join();
    return out;
}

void rope_tables(const Config& c, size_t n_pos, std::vector<float>& cos, std::vector<float>& sin) {
    const size_t half = c.rot_dim / 2;
    cos.resize(n_pos * half);
    sin.resize(n_pos * half);
    std::vector<double> inv_freq(half);
    for (size_t i = 0; i < half; i++) inv_freq[i] = std::pow(c.rope_theta, -((double)(2 * i)) / (double)c.rot_dim);
    for (size_t pos = 0; pos < n_pos; pos++)
        for (size_t i = 0; i < half; i++) {
            const double a = (double)pos * inv_freq[i];
            cos[pos * half + i] = (float)std::cos(a);
            sin[pos * half + i] = (float)std::sin(a);
        }
}

std::vector<int32_t> synth_prompt(uint64_t seed, size_t n, size_t vocab) {
    std::vector<int32_t> ids(n);
    for (size_t i = 0; i < n; i++) ids[i] = (int32_t)(mix64(elem_key(seed, 0, i)) % vocab);
    return ids;
}

}  // namespace det
