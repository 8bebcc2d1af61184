// Device twin of the synthetic-model generator and of the reference weight quantizer (crates/det/src/quantize.rs:33-85):
// builds the det rows of a seeded random-init linear directly in device memory, in the reference layout of
// det_qlinear (row-major codes, c, m).  Every value equals what the host twin (csrc/host/synth.cpp) produces: the draw
// is integer arithmetic plus two fp32 multiplies, the quantizer is binary64 add / mul / div / rint without contraction.
// A 27B-shape model has 2.7e10 weights; generating them here takes seconds instead of many CPU-minutes.
#include "runtime.cuh"

namespace detb {

__device__ __forceinline__ unsigned long long mix64(unsigned long long key) {
    unsigned long long z = key + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ float draw_normal(unsigned long long seed, unsigned long long tid, unsigned long long i,
                                             float stddev) {
    const unsigned long long z = mix64(seed ^ (tid << 40) ^ i);
    const int t = (int)(z & 0xFFFF) + (int)((z >> 16) & 0xFFFF) + (int)((z >> 32) & 0xFFFF) + (int)(z >> 48) - 131070;
    const float unit = (float)(1.0 / 37837.22676);
    return fmul(fmul((float)t, unit), stddev);
}
__device__ __forceinline__ unsigned short to_bf16(float f) {
    unsigned b = __float_as_uint(f);
    b += 0x7FFFu + ((b >> 16) & 1u);
    return (unsigned short)(b >> 16);
}
__device__ __forceinline__ double weight_f64(unsigned long long seed, unsigned long long tid, unsigned long long i) {
    return (double)__uint_as_float((unsigned)to_bf16(draw_normal(seed, tid, i, 0.02f)) << 16);
}

__device__ __forceinline__ double clampd(double q, double lim) { return q < -lim ? -lim : (q > lim ? lim : q); }

// quantize.rs:33-56 for one (row, 128-group)
__global__ void k_synth_scales(unsigned long long seed, unsigned long long tid, long long src0, int n, int K, double qmax,
                               double* __restrict__ scales) {
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int G = K >> 7;
    if (id >= (long long)n * G) return;
    const long long r = id / G;
    const int g = (int)(id % G);
    const unsigned long long e0 = (unsigned long long)(src0 + r) * K + (unsigned long long)g * 128;
    double amax = 0.0;
    for (int i = 0; i < 128; i++) {
        const double a = fabs(weight_f64(seed, tid, e0 + i));
        amax = a > amax ? a : amax;
    }
    double best_s = 1.0;
    if (amax != 0.0) {
        const double base = __ddiv_rn(amax, qmax);
        double best_err = INFINITY;
        best_s = base;
        for (int step = 0; step <= 10; step++) {
            const double s = __dmul_rn(base, __dadd_rn(0.80, __dmul_rn(0.02, (double)step)));
            double err = 0.0;
            for (int i = 0; i < 128; i++) {
                const double v = weight_f64(seed, tid, e0 + i);
                const double q = clampd(rint(__ddiv_rn(v, s)), qmax);
                const double d = __dsub_rn(__dmul_rn(q, s), v);
                err = __dadd_rn(err, __dmul_rn(d, d));
            }
            if (err < best_err) { best_err = err; best_s = s; }
        }
    }
    scales[id] = best_s;
}

// quantize.rs:58-85 for one (row, 128-group): c, m, codes, packing (quantize.rs:8-31) into the reference layout
__global__ void k_synth_rows(unsigned long long seed, unsigned long long tid, long long src0, int n, int K, int bits, double qmax,
                             const double* __restrict__ scales, int row0, uint8_t* __restrict__ wq,
                             float* __restrict__ c, uint16_t* __restrict__ m) {
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int G = K >> 7;
    if (id >= (long long)n * G) return;
    const long long r = id / G;
    const int g = (int)(id % G);
    double smax = 0.0;
    for (int i = 0; i < G; i++) {
        const double s = scales[r * G + i];
        smax = s > smax ? s : smax;
    }
    const float cf = (float)__ddiv_rn(smax, 65535.0);
    double mv = rint(__ddiv_rn(scales[id], (double)cf));
    mv = mv < 1.0 ? 1.0 : (mv > 65535.0 ? 65535.0 : mv);
    const unsigned mg = (unsigned)mv;
    const double eff = __dmul_rn((double)cf, (double)mg);
    const long long orow = row0 + r;
    if (g == 0) c[orow] = cf;
    m[orow * G + g] = (uint16_t)mg;
    const unsigned long long e0 = (unsigned long long)(src0 + r) * K + (unsigned long long)g * 128;
    const int bp32 = bits == 8 ? 32 : (bits == 6 ? 24 : 16);
    uint8_t* dst = wq + ((size_t)orow * (K >> 5) + (size_t)g * 4) * bp32;
    const int off = bits == 6 ? 32 : (bits == 4 ? 8 : 0);
    for (int blk = 0; blk < 4; blk++) {
        uint8_t u[32];
        for (int i = 0; i < 32; i++) {
            const double q = clampd(rint(__ddiv_rn(weight_f64(seed, tid, e0 + blk * 32 + i), eff)), qmax);
            u[i] = (uint8_t)((int)q + off);
        }
        uint8_t* b = dst + blk * bp32;
        if (bits == 8) {
            for (int i = 0; i < 32; i++) b[i] = u[i];
        } else {
            for (int i = 0; i < 16; i++) b[i] = (uint8_t)((u[i] & 0xF) | ((u[i + 16] & 0xF) << 4));
            if (bits == 6)
                for (int i = 0; i < 8; i++)
                    b[16 + i] = (uint8_t)((u[i] >> 4) | ((u[i + 8] >> 4) << 2) | ((u[i + 16] >> 4) << 4) | ((u[i + 24] >> 4) << 6));
        }
    }
}

__global__ void k_synth_bf16(unsigned long long seed, unsigned long long tid, long long count,
                             unsigned short* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) out[i] = to_bf16(draw_normal(seed, tid, (unsigned long long)i, 0.02f));
}

}  // namespace detb

using namespace detb;

extern "C" {

// Rows [src_row0, src_row0 + n) of synthetic tensor `tid` into rows [row0, row0 + n) of a reference-layout linear.
// `scratch` holds n * K/128 doubles.
void det_synth_linear(unsigned long long seed, unsigned long long tid, long long src_row0, int n, int K, int bits,
                      int row0, uint8_t* wq, float* c, uint16_t* m, double* scratch, cudaStream_t st) {
    DETB_REQUIRE((bits == 4 || bits == 6 || bits == 8) && K % 128 == 0 && n > 0, "bad synthetic linear shape");
    const double qmax = (double)((1 << (bits - 1)) - 1);
    const long long work = (long long)n * (K >> 7);
    const unsigned grid = (unsigned)((work + 127) / 128);
    cudaStream_t q = queue_of(st);
    k_synth_scales<<<grid, 128, 0, q>>>(seed, tid, src_row0, n, K, qmax, scratch);
    k_synth_rows<<<grid, 128, 0, q>>>(seed, tid, src_row0, n, K, bits, qmax, scratch, row0, wq, c, m);
    DETB_CUDA_OK(cudaGetLastError());
}

// count bf16 elements of synthetic tensor `tid` (the embedding table).
void det_synth_bf16(unsigned long long seed, unsigned long long tid, long long count, uint16_t* out, cudaStream_t st) {
    k_synth_bf16<<<(unsigned)((count + 255) / 256), 256, 0, queue_of(st)>>>(seed, tid, count, out);
    DETB_CUDA_OK(cudaGetLastError());
}

}  // extern "C"
