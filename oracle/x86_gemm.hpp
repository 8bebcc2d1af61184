// TEST AND CPU-BASELINE INFRASTRUCTURE — not part of the product.  The integer GEMM of the reference's x86 backend
// (`--backend cpu`, crates/det/src/x86/gemm.rs:1-372) restated for the timed CPU baseline: weights are expanded once at
// load to one signed byte per code (gemm.rs:59-134 repacks into unsigned-code strips; the arithmetic is the same), a
// 128-group's dot product runs on 256-bit integer SIMD — `vpdpbusd` on unsigned codes u = wq + OFF with the OFF * sum(xq)
// correction when the CPU has AVX-VNNI (gemm.rs:8, 226-243), else the AVX2 multiply-add pair on |wq| and sign-adjusted xq
// (x86/simd.rs `dp`) — and every group sum is multiplied by m * mx and added into int64 (gemm.rs:182-200, 244-255).
// All of it is exact integer arithmetic, so the result equals spec gemm_row bit for bit (tests/test_oracle_cpu.py).
// Rows are independent: OpenMP splits them over the host threads as rayon does in the reference (gemm.rs:299-372).
#pragma once
#include "spec.hpp"
#if defined(__x86_64__)
#include <immintrin.h>
#endif

namespace x86gemm {

inline bool have_avx2() {
#if defined(__x86_64__)
    return __builtin_cpu_supports("avx2");
#else
    return false;
#endif
}
inline bool have_vnni() {
#if defined(__x86_64__)
    return __builtin_cpu_supports("avxvnni");
#else
    return false;
#endif
}

#if defined(__x86_64__)
__attribute__((target("avx2"))) static inline int hsum8(__m256i v) {
    __m128i s = _mm_add_epi32(_mm256_castsi256_si128(v), _mm256_extracti128_si256(v, 1));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0x4E));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0xB1));
    return _mm_cvtsi128_si32(s);
}
// sum over one 128-group of wq * xq, AVX2: |wq| (unsigned) times sign-adjusted xq, pairs summed in s16 (at most
// 2 * 127 * 127 < 2^15), then widened
__attribute__((target("avx2"))) static inline int group_dot_avx2(const int8_t* w, const int8_t* x) {
    const __m256i ones = _mm256_set1_epi16(1);
    __m256i acc = _mm256_setzero_si256();
    for (int i = 0; i < 128; i += 32) {
        const __m256i wv = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(w + i));
        const __m256i xv = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(x + i));
        const __m256i p = _mm256_maddubs_epi16(_mm256_abs_epi8(wv), _mm256_sign_epi8(xv, wv));
        acc = _mm256_add_epi32(acc, _mm256_madd_epi16(p, ones));
    }
    return hsum8(acc);
}
// the same with vpdpbusd: unsigned codes u = wq + 128, corrected by 128 * sum(xq) of the group
__attribute__((target("avx2,avxvnni"))) static inline int group_dot_vnni(const int8_t* w, const int8_t* x, int xsum) {
    const __m256i off = _mm256_set1_epi8((char)0x80);
    __m256i acc = _mm256_setzero_si256();
    for (int i = 0; i < 128; i += 32) {
        const __m256i wv = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(w + i));
        const __m256i xv = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(x + i));
        acc = _mm256_dpbusd_avx_epi32(acc, _mm256_xor_si256(wv, off), xv);   // wq + 128 as an unsigned byte
    }
    return hsum8(acc) - 128 * xsum;
}
#endif

// y[t][j] for rows j of one expanded linear: w8[n][k] signed codes, c[n], m[n][k/128]; out[t * n + j].
inline void gemm(const int8_t* w8, const float* c, const uint16_t* m, size_t n, size_t k, const int8_t* xq, const float* sx,
                 const uint16_t* mx, size_t tokens, float* out) {
#if defined(__x86_64__)
    const size_t g = k / spec::GROUP;
    const bool vnni = have_vnni();
    std::vector<int> xsum;
    if (vnni) {
        xsum.resize(tokens * g);
        for (size_t t = 0; t < tokens; t++)
            for (size_t gi = 0; gi < g; gi++) {
                int s = 0;
                for (size_t i = 0; i < spec::GROUP; i++) s += xq[t * k + gi * spec::GROUP + i];
                xsum[t * g + gi] = s;
            }
    }
#pragma omp parallel for schedule(static)
    for (long j = 0; j < (long)n; j++) {
        const int8_t* wrow = w8 + (size_t)j * k;
        const uint16_t* mrow = m + (size_t)j * g;
        for (size_t t = 0; t < tokens; t++) {
            const int8_t* xrow = xq + t * k;
            int64_t acc = 0;
            for (size_t gi = 0; gi < g; gi++) {
                const int part = vnni ? group_dot_vnni(wrow + gi * spec::GROUP, xrow + gi * spec::GROUP, xsum[t * g + gi])
                                      : group_dot_avx2(wrow + gi * spec::GROUP, xrow + gi * spec::GROUP);
                const int64_t mult = (int64_t)mrow[gi] * (mx ? (int64_t)mx[t * g + gi] : 1);
                acc += mult * (int64_t)part;
            }
            out[t * n + j] = ((float)acc * c[j]) * sx[t];
        }
    }
#else
    (void)w8; (void)c; (void)m; (void)n; (void)k; (void)xq; (void)sx; (void)mx; (void)tokens; (void)out;
    throw std::runtime_error("x86gemm: not an x86-64 build");
#endif
}

}  // namespace x86gemm
