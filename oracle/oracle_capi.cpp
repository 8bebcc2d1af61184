// TEST INFRASTRUCTURE — not part of the product.  C entry points (ctypes) onto the CPU oracle: the reference backend as a
// det::Backend object, the spec primitives under the test hook's op numbers, and a runner that feeds both a reference
// backend and a backend under test to the driver library's conformance suites.
#include "x86_backend.hpp"
#include "../det_b200/csrc/host/conformance.hpp"
#include <cstdio>
#include <string>
#include <omp.h>

namespace oracle {

std::vector<float> prim_ref(int op, const std::vector<float>& x, size_t m, size_t n) {
    const size_t total = x.size();
    std::vector<float> out(std::max(total, m), 0.0f);
    if (op == 11) {
        for (size_t r = 0; r < m; r++) out[r] = spec::treesum(x.data() + r * n, n);
        return out;
    }
    for (size_t i = 0; i < total; i++) {
        const float a = x[i], b = x[total - 1 - i];
        float r = a;
        switch (op) {
            case 0: r = spec::exp_f(a); break;
            case 1: r = spec::log_f(a); break;
            case 2: r = spec::softplus_f(a); break;
            case 3: r = spec::sigmoid_f(a); break;
            case 4: r = spec::silu_f(a); break;
            case 5:
            case 12:
                if (i % 2 == 0 && i + 1 < total) {
                    const uint64_t lo = spec::f32_bits(x[i]), hi = spec::f32_bits(x[i + 1]);
                    r = (float)(int64_t)((hi << 32) | lo);   // conformance.rs:312 `v as f32`
                } else {
                    r = 0.0f;
                }
                break;
            case 6: r = spec::rint_(a); break;
            case 7: r = 1.0f / a; break;
            case 8: r = std::sqrt(a); break;
            case 9: r = a * b; break;
            case 10: r = a + b; break;
            case 13: r = (float)spec::as_i32(spec::rint_(a)); break;   // conformance.rs:337-340
            case 14: r = a / b; break;
            case 15: r = a - b; break;
            case 16: r = spec::fmax_(a, b); break;
        }
        out[i] = r;
    }
    return out;
}

}  // namespace oracle

typedef void (*prim_hook_fn)(int op, const float* x, size_t len, size_t m, size_t n, float* out, size_t out_len);

extern "C" {

void* orc_ref_backend_new() { return static_cast<det::Backend*>(new oracle::RefBackend()); }
// The timed CPU baseline and large-model parity reference: the restated x86 backend (x86_backend.hpp).  vnni: 1 = the
// AVX-VNNI build, 0 = the plain AVX2 build, -1 = whichever this CPU has.  NULL when the CPU lacks the instructions.
void* orc_cpu_backend_new(int vnni) {
#if defined(__x86_64__)
    try {
        const bool v = vnni < 0 ? x86port::have_vnni() : vnni != 0;
        return static_cast<det::Backend*>(new oracle::X86Backend(v));
    } catch (const std::exception& e) {
        fprintf(stderr, "oracle: %s\n", e.what());
    }
#endif
    return nullptr;
}
// 2: AVX-VNNI available, 1: AVX2 only, 0: neither (no x86 port on this host)
int orc_cpu_simd_level() {
#if defined(__x86_64__)
    return x86port::have_vnni() ? 2 : x86port::have_avx2() ? 1 : 0;
#else
    return 0;
#endif
}
// Thread count of the OpenMP loops (a launcher may have exported OMP_NUM_THREADS=1: the timed baseline sets its own).
void orc_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }
int orc_max_threads() { return omp_get_max_threads(); }
void orc_ref_backend_free(void* b) { delete static_cast<det::Backend*>(b); }

// Element-wise spec primitives on host arrays (the oracle side of the det_test_prim comparison).
void orc_prim(int op, const float* x, size_t len, size_t m, size_t n, float* out, size_t out_len) {
    std::vector<float> r = oracle::prim_ref(op, std::vector<float>(x, x + len), m, n);
    std::memcpy(out, r.data(), std::min(out_len, r.size()) * sizeof(float));
}

// Runs one conformance suite ("primitives", "gemm", "norms", "attention", "gdn", "sampling" or "all") with `ref` as the
// reference and `dut` as the backend under test.  Writes one line per check ("ok <name>" / "FAIL <name>: <mismatch>")
// into `report` and returns the number of failed checks (-1 on an exception).
int orc_conformance(void* ref, void* dut, const char* suite, prim_hook_fn dut_prim, char* report, size_t cap) {
    det::Report r;
    try {
        det::Backend& rb = *static_cast<det::Backend*>(ref);
        det::Backend& db = *static_cast<det::Backend*>(dut);
        const std::string s = suite;
        det::Prim prim = [&](int op, const std::vector<float>& x, size_t m, size_t n) {
            std::vector<float> out(std::max(x.size(), m));
            dut_prim(op, x.data(), x.size(), m, n, out.data(), out.size());
            return out;
        };
        det::PrimRef pref = oracle::prim_ref;
        if ((s == "primitives" || s == "all") && dut_prim) det::conformance_primitives(prim, pref, r);
        if (s == "gemm" || s == "all") det::conformance_gemm(rb, db, r);
        if (s == "norms" || s == "all") det::conformance_norms(rb, db, r);
        if (s == "attention" || s == "all") det::conformance_attention(rb, db, r);
        if (s == "gdn" || s == "all") det::conformance_gdn(rb, db, r);
        if (s == "sampling" || s == "all") det::conformance_sampling(rb, db, r);
    } catch (const std::exception& e) {
        snprintf(report, cap, "EXCEPTION %s\n", e.what());
        return -1;
    }
    std::string text;
    int failed = 0;
    for (const auto& c : r.checks) {
        if (c.second.empty()) text += "ok " + c.first + "\n";
        else {
            text += "FAIL " + c.first + ": " + c.second + "\n";
            failed++;
        }
    }
    if (r.checks.empty()) {
        text = "EXCEPTION no checks ran for suite '" + std::string(suite) + "'\n";
        failed = -1;
    }
    snprintf(report, cap, "%s", text.c_str());
    return failed;
}

// ---- op-level entry points on host arrays (used by the golden-vector and C-ABI parity tests)
void orc_quant(const float* x, size_t m, size_t n, int8_t* xq, float* sx, uint16_t* mx) { refops::quant(x, m, n, xq, sx, mx); }
void orc_rmsnorm_quant(const float* x, const float* w, float eps, size_t m, size_t n, int8_t* xq, float* sx, uint16_t* mx) {
    refops::rmsnorm_quant(x, w, eps, m, n, xq, sx, mx);
}
void orc_silu_mul_quant(const float* g, const float* u, size_t m, size_t n, int8_t* hq, float* sh, uint16_t* mh) {
    refops::silu_mul_quant(g, u, m, n, hq, sh, mh);
}
// y[m][n] from `n` det rows (one part); accumulate != 0 adds into y
void orc_gemm(const uint8_t* rows, size_t n, size_t k, int bits, const int8_t* xq, const float* sx, const uint16_t* mx,
              size_t m, float* y, int accumulate) {
    refops::Linear l;
    l.parts = {rows};
    l.widths = {n};
    l.k = k;
    l.bits = bits;
    float* dsts[1] = {y};
    refops::gemm(l, xq, sx, mx, m, accumulate ? refops::Out::Accumulate : refops::Out::Write, dsts);
}
// The restated x86 GEMM (strip repack + blocked kernel) on det rows, for the check against gemm_row.
void orc_gemm_x86(const uint8_t* rows, size_t n, size_t k, int bits, const int8_t* xq, const float* sx, const uint16_t* mx,
                  size_t m, float* y, int vnni) {
#if defined(__x86_64__)
    refops::Linear l;
    l.parts = {rows};
    l.widths = {n};
    l.k = k;
    l.bits = bits;
    x86port::StripLinear strips;
    x86port::repack(l, strips);
    float* dsts[1] = {y};
    if (vnni) x86vnni::gemm(strips, xq, sx, mx, m, refops::Out::Write, dsts, l.widths);
    else x86avx2::gemm(strips, xq, sx, mx, m, refops::Out::Write, dsts, l.widths);
#else
    (void)rows; (void)n; (void)k; (void)bits; (void)xq; (void)sx; (void)mx; (void)m; (void)y; (void)vnni;
#endif
}
void orc_unpack_row(const uint8_t* packed, int bits, size_t k, int8_t* out) { spec::unpack_row(packed, bits, k, out); }
float orc_treesum(const float* x, size_t n) { return spec::treesum(x, n); }
int orc_argmax(const float* logits, size_t v) { return (int)spec::argmax(logits, v); }
int orc_sample(const float* logits, size_t v, float inv_temp, size_t top_k, float top_p, uint64_t z) {
    return (int)spec::sample_with_draw(logits, v, inv_temp, top_k, top_p, z);
}
void orc_weights(const float* logits, size_t v, float inv_temp, uint64_t* w) { spec::weights(logits, v, inv_temp, w); }
uint64_t orc_splitmix64(uint64_t* state) { return spec::splitmix64(*state); }

}  // extern "C"
