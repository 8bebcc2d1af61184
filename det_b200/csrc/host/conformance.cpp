// See conformance.hpp.  Each suite follows the reference's case list, generators and seeds
// (crates/det/src/conformance.rs: Rng 35-59, same/same_i 63-92, fake_gguf 104-144, acts 147-160, primitives 180-345,
// gemm 348-449, norms 453-537, attention 552-660, gdn 664-805, sampling 809-876).
#include "conformance.hpp"
#include "synth.hpp"
#include <cmath>
#include <cstdio>
#include <limits>

namespace det {

namespace {

// conformance.rs:35-59 — xorshift64
struct Rng {
    uint64_t s;
    explicit Rng(uint64_t seed) : s(seed) {}
    uint64_t next() {
        uint64_t x = s;
        x ^= x << 13;
        x ^= x >> 7;
        x ^= x << 17;
        s = x;
        return x;
    }
    float unit() { return (float)((double)(next() >> 11) / (double)(1ull << 53) * 2.0 - 1.0); }
    uint8_t byte() { return (uint8_t)(next() >> 56); }
    uint64_t below(uint64_t n) { return next() % n; }
    float denorm() {   // a nonzero denormal of either sign
        uint32_t b = (uint32_t)next() & 0x807FFFFFu;
        if ((b & 0x7FFFFFFFu) == 0) b |= 1;
        float f;
        std::memcpy(&f, &b, 4);
        return f;
    }
};

uint32_t bits_of(float f) {
    uint32_t b;
    std::memcpy(&b, &f, 4);
    return b;
}
float from_bits(uint32_t b) {
    float f;
    std::memcpy(&f, &b, 4);
    return f;
}

// conformance.rs:61-78 — bit-exact, except that any two NaNs match
std::string same(const std::vector<float>& a, const std::vector<float>& b, size_t n = (size_t)-1) {
    if (n == (size_t)-1) n = a.size();
    size_t bad = 0, first = 0;
    for (size_t i = 0; i < n; i++) {
        if (bits_of(a[i]) != bits_of(b[i]) && !(std::isnan(a[i]) && std::isnan(b[i]))) {
            if (!bad) first = i;
            bad++;
        }
    }
    if (!bad) return "";
    char buf[256];
    snprintf(buf, sizeof buf, "%zu of %zu differ, first at %zu: ref %e (%#010x) dut %e (%#010x)", bad, n, first,
             a[first], bits_of(a[first]), b[first], bits_of(b[first]));
    return buf;
}
template <class T>
std::string same_i(const std::vector<T>& a, const std::vector<T>& b) {
    size_t bad = 0, first = 0;
    for (size_t i = 0; i < a.size(); i++)
        if (a[i] != b[i]) {
            if (!bad) first = i;
            bad++;
        }
    if (!bad) return "";
    char buf[256];
    snprintf(buf, sizeof buf, "%zu of %zu differ, first at %zu: ref %lld dut %lld", bad, a.size(), first,
             (long long)a[first], (long long)b[first]);
    return buf;
}

float pow10_neg(int k) {
    float p = 1.0f;
    for (int i = 0; i < k; i++) p *= 10.0f;
    return 1.0f / p;
}

// conformance.rs:104-144 — det rows of random codes and scales (the reference wraps them in a GGUF file)
std::vector<uint8_t> fake_rows(Rng& rng, int bits, size_t n, size_t k) {
    const size_t rb = det_row_bytes(bits, k);
    const size_t nc = rb - 4 - k / 128 * 2;
    std::vector<uint8_t> data(n * rb);
    for (size_t r = 0; r < n; r++) {
        uint8_t* row = data.data() + r * rb;
        for (size_t i = 0; i < nc; i++) row[i] = rng.byte();
        const float c = std::fabs(rng.unit()) * 1e-6f + 1e-8f;
        std::memcpy(row + nc, &c, 4);
        for (size_t g = 0; g < k / 128; g++) {
            const uint16_t m = (uint16_t)(1 + rng.below(65535));
            std::memcpy(row + nc + 4 + 2 * g, &m, 2);
        }
    }
    return data;
}

struct Acts {
    Buf<int8_t> xq;
    Buf<float> sx;
    Buf<uint16_t> mx;
};
// conformance.rs:147-160 — group-quantized activations with a scale that varies by group, through the reference quant
Acts acts(Rng& rng, Backend& ref, size_t m, size_t k) {
    std::vector<float> x(m * k);
    for (size_t t = 0; t < m; t++)
        for (size_t g = 0; g < k / 128; g++) {
            const float scale = pow10_neg((int)((g + t) % 5));
            for (size_t i = 0; i < 128; i++) x[t * k + g * 128 + i] = rng.unit() * scale;
        }
    Buf<float> xb = ref.upload(x);
    Acts a{ref.alloc<int8_t>(m * k), ref.alloc<float>(m), ref.alloc<uint16_t>(m * k / 128)};
    ref.quant(xb, m, k, a.xq, a.sx, a.mx);
    return a;
}
template <class T>
Buf<T> mirror(Backend& ref, Backend& dut, const Buf<T>& b) {
    return dut.upload(ref.download(b));
}

}  // namespace

Report conformance_run(Backend& ref, Backend& dut, const Prim* prim, const PrimRef* prim_ref) {
    Report r;
    if (prim && prim_ref) conformance_primitives(*prim, *prim_ref, r);
    conformance_gemm(ref, dut, r);
    conformance_norms(ref, dut, r);
    conformance_attention(ref, dut, r);
    conformance_gdn(ref, dut, r);
    conformance_sampling(ref, dut, r);
    return r;
}

// conformance.rs:180-345
void conformance_primitives(const Prim& prim, const PrimRef& ref, Report& r) {
    Rng rng(1);
    const size_t n = 1 << 16;
    std::vector<float> x(n);
    for (size_t i = 0; i < n; i++) x[i] = (i % 7 == 0) ? from_bits((uint32_t)rng.next() & 0x00FFFFFFu) : rng.unit() * 100.0f;
    const float inf = std::numeric_limits<float>::infinity();
    const float minpos = std::numeric_limits<float>::min();
    const float lhs[] = {1e-40f, inf, 0.0f, -1e-42f, -inf, 1e-39f, 0.0f, 1.0f, minpos, -1e-41f, 0.0f, -0.0f, 3e-39f, inf};
    const float rhs[] = {inf, 1e-40f, 1e-40f, 0.0f, -1e-39f, -inf, 0.0f, 1e-40f, inf, inf, -0.0f, 0.0f, 2e-39f, inf};
    const size_t np = sizeof(lhs) / sizeof(lhs[0]);
    for (size_t i = 0; i < np; i++) {
        x[i] = lhs[i];
        x[n - 1 - i] = rhs[i];
    }
    x[np] = minpos;
    x[np + 1] = -minpos / 2.0f;
    const std::pair<int, const char*> unary[] = {{0, "exp_f"}, {3, "sigmoid_f"}, {4, "silu_f"}, {6, "rint"}, {8, "sqrt"}};
    for (auto [op, name] : unary) {
        std::vector<float> input = x;
        if (op == 8)
            for (float& v : input) v = std::fabs(v);
        r.add(std::string("prim ") + name, same(ref(op, input, 1, n), prim(op, input, 1, n), n));
    }
    std::vector<float> pos(n);
    for (size_t i = 0; i < n; i++) pos[i] = std::fabs(x[i]) + 1e-30f;
    r.add("prim log_f", same(ref(1, pos, 1, n), prim(1, pos, 1, n), n));
    r.add("prim softplus_f", same(ref(2, x, 1, n), prim(2, x, 1, n), n));
    const std::pair<int, const char*> binary[] = {{9, "mul"}, {10, "add"}, {14, "div"}, {15, "sub"}, {16, "fmax"}};
    for (auto [op, name] : binary) r.add(std::string("prim ") + name, same(ref(op, x, 1, n), prim(op, x, 1, n), n));

    std::vector<float> rows(8 * 5120);
    for (float& v : rows) v = rng.unit();
    for (size_t i = 0; i < rows.size(); i += 97) rows[i] = rng.denorm();
    r.add("prim treesum", same(ref(11, rows, 8, 5120), prim(11, rows, 8, 5120), 8));

    // int64 -> fp32 on random values and on crafted round-half-even ties for shifts 1..39
    std::vector<int64_t> vals;
    for (size_t i = 0; i < n / 2; i++) {
        if (i % 3 == 0) {
            const int64_t v = (int64_t)rng.next();
            vals.push_back(v >> (uint32_t)rng.below(40));
        } else {
            vals.push_back((int64_t)rng.next() >> 20);
        }
    }
    for (uint32_t s = 1; s <= 39; s++)
        for (int rep = 0; rep < 300; rep++) {
            const int64_t m = (int64_t)((rng.next() & 0x7FFFFF) | 0x800000);
            const int64_t half = (int64_t)1 << (s - 1);
            const int64_t tails[] = {half, half + 1, half - 1, half | 1, 1, ((int64_t)1 << s) - 1};
            for (int64_t tail : tails) {
                const int64_t v = (m << s) + tail;
                vals.push_back(v);
                vals.push_back(-v);
            }
        }
    std::vector<float> bits(vals.size() * 2);
    for (size_t i = 0; i < vals.size(); i++) {
        bits[2 * i] = from_bits((uint32_t)(uint64_t)vals[i]);
        bits[2 * i + 1] = from_bits((uint32_t)((uint64_t)vals[i] >> 32));
    }
    for (auto [op, name] : {std::pair<int, const char*>{5, "i64_to_f"}, {12, "native int64 to fp32 cast"}}) {
        const std::vector<float> want = ref(op, bits, 1, bits.size()), got = prim(op, bits, 1, bits.size());
        std::vector<float> w(vals.size()), g(vals.size());
        for (size_t i = 0; i < vals.size(); i++) {
            w[i] = want[2 * i];
            g[i] = got[2 * i];
        }
        r.add(std::string("prim ") + name, same(w, g));
    }
    const std::vector<float> big = {3e9f, -3e9f, 2147483648.0f, 2147483520.0f, -2147483648.0f, -2147483904.0f, 1e20f, -1e20f,
                                    inf, -inf, 2.5f, -2.5f, 3.5f, 1e38f, -1e38f, 4294967296.0f};
    r.add("prim fp32 to int32 saturation", same(ref(13, big, 1, big.size()), prim(13, big, 1, big.size()), big.size()));
}

// conformance.rs:348-449
void conformance_gemm(Backend& ref, Backend& dut, Report& r) {
    Rng rng(11);
    const std::pair<int, const char*> types[] = {{8, "det8"}, {6, "det6"}, {4, "det4"}};
    const std::pair<size_t, size_t> shapes[] = {{96, 256}, {200, 384}, {640, 2560}, {2560, 1024}, {48, 128}};
    for (auto [bits, tname] : types)
        for (auto [n, k] : shapes) {
            const std::vector<uint8_t> rows = fake_rows(rng, bits, n, k);
            auto lc = ref.linear({LinearPart{rows.data(), n}}, k, bits);
            auto lg = dut.linear({LinearPart{rows.data(), n}}, k, bits);
            std::vector<size_t> ms = {1, 3, 8, 9, 16, 17, 32, 45, 64};
            if (n == 640 && k == 2560) ms.insert(ms.end(), {65, 100, 300});
            for (size_t m : ms) {
                Acts a = acts(rng, ref, m, k);
                Buf<float> yc = ref.alloc<float>(m * n);
                ref.gemm(*lc, a.xq, a.sx, a.mx, m, GemmOut::write(yc));
                Buf<int8_t> xqg = mirror(ref, dut, a.xq);
                Buf<float> sxg = mirror(ref, dut, a.sx);
                Buf<uint16_t> mxg = mirror(ref, dut, a.mx);
                Buf<float> yg = dut.alloc<float>(m * n);
                dut.gemm(*lg, xqg, sxg, mxg, m, GemmOut::write(yg));
                dut.sync();
                char name[128];
                snprintf(name, sizeof name, "gemm %s n=%zu k=%zu m=%zu", tname, n, k, m);
                r.add(name, same(ref.download(yc), dut.download(yg)));
                std::vector<float> acc0(m * n);
                for (float& v : acc0) v = rng.unit();
                Buf<float> acc_c = ref.upload(acc0), acc_g = dut.upload(acc0);
                ref.gemm(*lc, a.xq, a.sx, a.mx, m, GemmOut::accumulate(acc_c));
                dut.gemm(*lg, xqg, sxg, mxg, m, GemmOut::accumulate(acc_g));
                dut.sync();
                snprintf(name, sizeof name, "gemm accumulate %s n=%zu k=%zu m=%zu", tname, n, k, m);
                r.add(name, same(ref.download(acc_c), dut.download(acc_g)));
            }
        }
    // fused parts: 100 + 60 columns of W6, K = 512
    const size_t k = 512;
    const std::vector<uint8_t> r1 = fake_rows(rng, 6, 100, k), r2 = fake_rows(rng, 6, 60, k);
    auto lc = ref.linear({LinearPart{r1.data(), 100}, LinearPart{r2.data(), 60}}, k, 6);
    auto lg = dut.linear({LinearPart{r1.data(), 100}, LinearPart{r2.data(), 60}}, k, 6);
    for (size_t m : {1, 7, 20, 90}) {
        Acts a = acts(rng, ref, m, k);
        Buf<float> ac = ref.alloc<float>(m * 100), bc = ref.alloc<float>(m * 60);
        ref.gemm(*lc, a.xq, a.sx, a.mx, m, GemmOut::parts({&ac, &bc}));
        Buf<float> ag = dut.alloc<float>(m * 100), bg = dut.alloc<float>(m * 60);
        Buf<int8_t> xqg = mirror(ref, dut, a.xq);
        Buf<float> sxg = mirror(ref, dut, a.sx);
        Buf<uint16_t> mxg = mirror(ref, dut, a.mx);
        dut.gemm(*lg, xqg, sxg, mxg, m, GemmOut::parts({&ag, &bg}));
        dut.sync();
        r.add("gemm fused parts a m=" + std::to_string(m), same(ref.download(ac), dut.download(ag)));
        r.add("gemm fused parts b m=" + std::to_string(m), same(ref.download(bc), dut.download(bg)));
    }
}

// conformance.rs:453-537
void conformance_norms(Backend& ref, Backend& dut, Report& r) {
    Rng rng(3);
    const std::pair<size_t, size_t> shapes[] = {{1, 2560}, {6, 2560}, {33, 4096}, {9, 9216}, {4, 5120}, {3, 17408}};
    for (auto [m, n] : shapes) {
        std::vector<float> x(m * n), u(m * n), w(n);
        for (size_t i = 0; i < m * n; i++) {
            const size_t row = i / n, col = i % n;
            float v;
            switch (row % 6) {
                case 0: v = rng.denorm(); break;
                case 1: v = (col % 2 == 0) ? rng.denorm() : 0.0f; break;
                case 2:
                    switch (col % 8) {
                        case 0: v = rng.unit() * 1e-20f; break;
                        case 1: v = rng.unit() * 1e-23f; break;
                        case 2: v = rng.denorm(); break;
                        case 3: v = rng.unit(); break;
                        case 4: v = 0.0f; break;
                        case 5: v = rng.unit() * 1e-30f; break;
                        case 6: v = -0.0f; break;
                        default: v = rng.unit() * 1e3f; break;
                    }
                    break;
                case 3: v = (col % 5 == 0) ? rng.unit() * 1e-19f : rng.unit() * 1e-38f; break;
                default: v = rng.unit() * pow10_neg((int)((i / 128) % 4)); break;
            }
            x[i] = v;
        }
        for (size_t i = 0; i < m * n; i++) {
            switch ((i % n) % 3) {
                case 0: u[i] = rng.unit() * 1e-20f; break;
                case 1: u[i] = rng.denorm(); break;
                default: u[i] = rng.unit() * 3.0f; break;
            }
        }
        for (float& v : w) v = 1.0f + rng.unit();
        Buf<float> xc = ref.upload(x), uc = ref.upload(u), wc = ref.upload(w);
        Buf<float> xg = dut.upload(x), ug = dut.upload(u), wg = dut.upload(w);
        const size_t g = n / 128;
        Buf<int8_t> qc = ref.alloc<int8_t>(m * n), qg = dut.alloc<int8_t>(m * n);
        Buf<float> sc = ref.alloc<float>(m), sg = dut.alloc<float>(m);
        Buf<uint16_t> mc = ref.alloc<uint16_t>(m * g), mg = dut.alloc<uint16_t>(m * g);
        auto check = [&](const char* name) {
            dut.sync();
            char buf[128];
            snprintf(buf, sizeof buf, "%s codes m=%zu n=%zu", name, m, n);
            r.add(buf, same_i(ref.download(qc), dut.download(qg)));
            snprintf(buf, sizeof buf, "%s multipliers m=%zu n=%zu", name, m, n);
            r.add(buf, same_i(ref.download(mc), dut.download(mg)));
            snprintf(buf, sizeof buf, "%s scales m=%zu n=%zu", name, m, n);
            r.add(buf, same(ref.download(sc), dut.download(sg)));
        };
        // the reference skips rmsnorm_quant beyond 8192 columns (its CUDA kernel stops there); this port does not
        ref.rmsnorm_quant(xc, wc, 1e-6f, m, n, qc, sc, mc);
        dut.rmsnorm_quant(xg, wg, 1e-6f, m, n, qg, sg, mg);
        check("rmsnorm_quant");
        ref.quant(xc, m, n, qc, sc, mc);
        dut.quant(xg, m, n, qg, sg, mg);
        check("quant");
        ref.silu_mul_quant(xc, uc, m, n, qc, sc, mc);
        dut.silu_mul_quant(xg, ug, m, n, qg, sg, mg);
        check("silu_mul_quant");
    }
}

namespace {
KvCache make_kv(Backend& b, size_t ctx, size_t n_kv, size_t hd) {
    KvCache kv;
    kv.kq = b.alloc<int8_t>(ctx * n_kv * hd);
    kv.sk = b.alloc<float>(ctx * n_kv);
    kv.vq = b.alloc<int16_t>(ctx * n_kv * hd);
    kv.capacity = ctx;
    return kv;
}
}  // namespace

// conformance.rs:552-660
void conformance_attention(Backend& ref, Backend& dut, Report& r) {
    Rng rng(9);
    const size_t n_h = 16, n_kv = 4, hd = 256, rot = 64, ctx = 400;
    const size_t half = rot / 2;
    std::vector<float> cos(ctx * half), sin(ctx * half);
    for (size_t i = 0; i < ctx * half; i++) {
        cos[i] = (float)std::cos((double)i * 0.001);
        sin[i] = (float)std::sin((double)i * 0.001);
    }
    std::vector<float> q_norm(hd), k_norm(hd);
    for (float& v : q_norm) v = 1.0f + rng.unit() * 0.5f;
    for (float& v : k_norm) v = 1.0f + rng.unit() * 0.5f;
    std::vector<float> v_scale(n_kv), v_inv(n_kv);
    for (size_t i = 0; i < n_kv; i++) {
        v_scale[i] = 0.001f * (float)(i + 1);
        v_inv[i] = 1.0f / v_scale[i];
    }
    Buf<float> qn_c = ref.upload(q_norm), kn_c = ref.upload(k_norm), vs_c = ref.upload(v_scale), vi_c = ref.upload(v_inv),
               co_c = ref.upload(cos), si_c = ref.upload(sin);
    Buf<float> qn_g = dut.upload(q_norm), kn_g = dut.upload(k_norm), vs_g = dut.upload(v_scale), vi_g = dut.upload(v_inv),
               co_g = dut.upload(cos), si_g = dut.upload(sin);
    AttnLayer lc{&qn_c, &kn_c, &vs_c, &vi_c, &co_c, &si_c};
    AttnLayer lg{&qn_g, &kn_g, &vs_g, &vi_g, &co_g, &si_g};
    KvCache kvc = make_kv(ref, ctx, n_kv, hd), kvg = make_kv(dut, ctx, n_kv, hd);
    auto scale_of = [](size_t row) -> float {
        switch (row % 6) {
            case 0: return 1e-25f;
            case 1: return 1e-38f;
            case 2: return 2.0f;
            case 3: return 1e-10f;
            case 4: return 2.0f;
            default: return 1e3f;
        }
    };
    size_t pos0 = 0;
    for (size_t m : {40, 1, 7, 100, 3, 16, 200, 5, 1}) {
        std::vector<float> qg(m * n_h * 2 * hd), k(m * n_kv * hd), v(m * n_kv * hd);
        for (size_t i = 0; i < qg.size(); i++)
            qg[i] = (i % (2 * hd) < hd) ? rng.unit() * scale_of(i / (2 * hd)) : rng.unit() * 200.0f;
        for (size_t i = 0; i < k.size(); i++) k[i] = rng.unit() * scale_of(i / hd + 1);
        for (size_t i = 0; i < v.size(); i++) v[i] = ((i / hd) % 4 == 1) ? rng.denorm() : rng.unit() * scale_of(i / hd + 2);
        Buf<float> oc = ref.alloc<float>(m * n_h * hd), og = dut.alloc<float>(m * n_h * hd);
        Shape shape{m, pos0, n_h, n_kv, hd, rot, 1e-6f};
        Buf<float> qg_c = ref.upload(qg), k_c = ref.upload(k), v_c = ref.upload(v);
        Buf<float> qg_g = dut.upload(qg), k_g = dut.upload(k), v_g = dut.upload(v);
        ref.attention(lc, kvc, shape, qg_c, k_c, v_c, oc);
        dut.attention(lg, kvg, shape, qg_g, k_g, v_g, og);
        dut.sync();
        const std::string tag = " m=" + std::to_string(m);
        r.add("attention" + tag + " pos0=" + std::to_string(pos0), same(ref.download(oc), dut.download(og)));
        r.add("attention kq cache" + tag, same_i(ref.download(kvc.kq), dut.download(kvg.kq)));
        r.add("attention vq cache" + tag, same_i(ref.download(kvc.vq), dut.download(kvg.vq)));
        r.add("attention sk cache" + tag, same(ref.download(kvc.sk), dut.download(kvg.sk)));
        pos0 += m;
    }
}

// conformance.rs:664-805
void conformance_gdn(Backend& ref, Backend& dut, Report& r) {
    Rng rng(21);
    const size_t n_k = 16, n_v = 32, dk = 128, dv = 128;
    const size_t conv_dim = 2 * n_k * dk + n_v * dv;
    const size_t rep = n_v / n_k;
    const size_t gw = 2 * dk + rep * dv + 2 * rep;
    const size_t kd = n_k * dk;
    std::vector<float> conv(conv_dim * 4, 0.0f);
    for (size_t c = 0; c < conv_dim; c++) {
        conv[c * 4 + 3] = 1.0f;
        conv[c * 4 + 2] = 0.01f * rng.unit();
    }
    std::vector<float> a(n_v);
    for (size_t h = 0; h < n_v; h++)
        a[h] = h == 0 ? 4.35f : (h == 1 ? 4.6f : (h == 2 ? 0.5f : 0.03f + 0.02f * ((float)h / (float)n_v)));
    std::vector<float> dt_bias(n_v, 20.0f), norm(dv);
    for (float& v : norm) v = 1.0f + rng.unit() * 0.3f;
    Buf<float> cv_c = ref.upload(conv), a_c = ref.upload(a), dt_c = ref.upload(dt_bias), nm_c = ref.upload(norm);
    Buf<float> cv_g = dut.upload(conv), a_g = dut.upload(a), dt_g = dut.upload(dt_bias), nm_g = dut.upload(norm);
    GdnLayer lc{&cv_c, &a_c, &dt_c, &nm_c}, lg{&cv_g, &a_g, &dt_g, &nm_g};
    GdnState stc{ref.alloc<float>(3 * conv_dim), ref.alloc<float>(n_v * dk * dv)};
    GdnState stg{dut.alloc<float>(3 * conv_dim), dut.alloc<float>(n_v * dk * dv)};
    size_t t0 = 0, denormal_seen = 0;
    for (size_t m : {60, 20, 20, 20, 20, 1, 1, 1, 1, 1, 10, 10, 10, 10, 10, 10, 10, 10, 10, 100, 37, 1, 5}) {
        std::vector<float> qkv(m * conv_dim), z(m * n_v * dv), av(m * n_v), bv(m * n_v);
        for (size_t i = 0; i < qkv.size(); i++) {
            const size_t t = i / conv_dim, c = i % conv_dim;
            const size_t tg = t0 + t;
            if (c >= kd && c < 2 * kd && tg >= 20 && (c - kd) % dk >= 32 && tg % 97 != 0) qkv[i] = -200.0f;
            else qkv[i] = rng.unit();
        }
        for (float& v : z) v = rng.unit() * 2.0f;
        for (float& v : av) v = rng.unit() * 3.0f;
        for (float& v : bv) v = rng.unit() * 3.0f;
        GdnShape shape{m, n_k, n_v, dk, dv, 1e-6f};
        Buf<float> onc = ref.alloc<float>(m * n_v * dv), ginc = ref.alloc<float>(m * n_k * gw), goutc = ref.alloc<float>(m * n_v * dv);
        Buf<float> ong = dut.alloc<float>(m * n_v * dv), ging = dut.alloc<float>(m * n_k * gw), goutg = dut.alloc<float>(m * n_v * dv);
        Buf<float> qkv_c = ref.upload(qkv), z_c = ref.upload(z), av_c = ref.upload(av), bv_c = ref.upload(bv);
        Buf<float> qkv_g = dut.upload(qkv), z_g = dut.upload(z), av_g = dut.upload(av), bv_g = dut.upload(bv);
        ref.gdn(lc, stc, shape, qkv_c, z_c, av_c, bv_c, onc, GdnExport{&ginc, &goutc});
        dut.gdn(lg, stg, shape, qkv_g, z_g, av_g, bv_g, ong, GdnExport{&ging, &goutg});
        dut.sync();
        const std::vector<float> s_ref = ref.download(stc.s);
        for (float x : s_ref)
            if (x != 0.0f && std::fabs(x) < std::numeric_limits<float>::min()) denormal_seen++;
        const std::string tag = " m=" + std::to_string(m) + " t0=" + std::to_string(t0);
        r.add("gdn output" + tag, same(ref.download(onc), dut.download(ong)));
        r.add("gdn inputs" + tag, same(ref.download(ginc), dut.download(ging)));
        r.add("gdn mixer output" + tag, same(ref.download(goutc), dut.download(goutg)));
        r.add("gdn state" + tag, same(s_ref, dut.download(stg.s)));
        r.add("gdn conv state" + tag, same(ref.download(stc.conv_state), dut.download(stg.conv_state)));
        t0 += m;
    }
    r.add("gdn state reached the denormal range",
          denormal_seen == 0 ? "no denormal state entry was produced; the sequence no longer exercises the denormal path" : "");
}

// conformance.rs:809-876
void conformance_sampling(Backend& ref, Backend& dut, Report& r) {
    Rng rng(77);
    const size_t v = 248320;
    std::vector<float> random(v), ties(v), zeros(v);
    for (float& x : random) x = rng.unit() * 12.0f;
    for (size_t i = 0; i < v; i++) ties[i] = (float)(i % 7) - 3.0f;
    for (size_t i = 0; i < v; i++) zeros[i] = i == 7 ? 0.0f : (i == 11 ? -0.0f : (i == 100 ? 0.0f : -1.0f - (float)(i % 13)));
    const std::pair<const char*, const std::vector<float>*> sets[] = {{"random", &random}, {"ties", &ties}, {"zero maxima", &zeros}};
    for (auto [name, logits] : sets) {
        Buf<float> lc = ref.upload(*logits), lg = dut.upload(*logits);
        const int32_t c = ref.argmax(lc, v), g = dut.argmax(lg, v);
        r.add(std::string("argmax ") + name, c != g ? "ref " + std::to_string(c) + " dut " + std::to_string(g) : "");
        struct P { float inv_temp; size_t top_k; float top_p; };
        std::vector<P> params;
        for (int i = 0; i < 24; i++) {
            const float inv_temp = 1.0f / (0.3f + std::fabs(rng.unit()) * 1.5f);
            size_t top_k = 0;
            if (i % 4 == 1) top_k = 1 + (size_t)rng.below(100);
            else if (i % 4 == 2) top_k = 40;
            float top_p = 1.0f;
            if (i % 3 == 1) top_p = 0.5f + std::fabs(rng.unit()) * 0.49f;
            else if (i % 3 == 2) top_p = 0.95f;
            params.push_back({inv_temp, top_k, top_p});
        }
        const P degenerate[] = {{1.0f, 0, 1e-9f}, {1.0f, 0, 2e-8f}, {1.0f, 0, 0.0f}, {1.0f, 0, -0.5f}, {1.0f, 3, 1e-9f},
                                {1.0f, 1, 1.0f},  {1.0f, 0, 0.999999f}, {1.0f, v, 0.5f}, {1.0f, v + 5, 0.5f}, {1.0f, 5, 0.3f}};
        for (const P& p : degenerate) params.push_back(p);
        for (const P& p : params) {
            const uint64_t z = rng.next();
            const int32_t cs = ref.sample(lc, v, p.inv_temp, p.top_k, p.top_p, z);
            const int32_t gs = dut.sample(lg, v, p.inv_temp, p.top_k, p.top_p, z);
            char buf[160];
            snprintf(buf, sizeof buf, "sample %s inv_temp=%g top_k=%zu top_p=%g", name, p.inv_temp, p.top_k, p.top_p);
            r.add(buf, cs != gs ? "ref " + std::to_string(cs) + " dut " + std::to_string(gs) : "");
        }
    }
}

}  // namespace det
