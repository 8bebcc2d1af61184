// Device-side numerics kit: the fixed IEEE binary32 operation sequences of det's spec
// (crates/det/src/spec/prim.rs, docs/SPEC.md §1, §4, §8) for sm_100a.
//
// Every arithmetic step goes through a round-to-nearest intrinsic (__fmul_rn, __fadd_rn, ...), which the compiler never
// contracts into an FMA and which keeps denormals; the build additionally passes -fmad=false.  Constants are written as
// (float)(double literal), the path the spec's `f64 literal as f32` takes.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#define DETB_CUDA_OK(call)                                                                              \
    do {                                                                                                \
        cudaError_t err__ = (call);                                                                     \
        if (err__ != cudaSuccess) {                                                                     \
            fprintf(stderr, "det_b200: CUDA error '%s' at %s:%d\n", cudaGetErrorString(err__), __FILE__, \
                    __LINE__);                                                                          \
            abort();                                                                                    \
        }                                                                                               \
    } while (0)

#define DETB_REQUIRE(cond, msg)                                                      \
    do {                                                                             \
        if (!(cond)) {                                                               \
            fprintf(stderr, "det_b200: %s (%s) at %s:%d\n", msg, #cond, __FILE__, __LINE__); \
            abort();                                                                 \
        }                                                                            \
    } while (0)

namespace detb {

constexpr unsigned FULL = 0xffffffffu;

// Programmatic dependent launch (PTX griddepcontrol).  A kernel launched with the programmatic-serialization attribute
// may start while its predecessor in the stream still runs: pdl_trigger() lets the successor's CTAs be scheduled,
// pdl_wait() blocks until the predecessor has completed and its writes are visible.  Every kernel here triggers first
// thing and waits before it touches anything an earlier kernel may write; only read-only weights are fetched before
// the wait.  Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- the five rounded operations and the conversions (docs/SPEC.md §1.2, §8 CUDA bullet)
__device__ __forceinline__ float fmul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float fadd(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float fsub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float fdiv(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ float fsqrt(float a) { return __fsqrt_rn(a); }
__device__ __forceinline__ float frint(float a) { return rintf(a); }                 // cvt.rni.f32.f32
__device__ __forceinline__ int f2i_sat(float a) { return __float2int_rn(a); }        // saturating, NaN -> 0
__device__ __forceinline__ float i64_to_f32(long long v) { return __ll2float_rn(v); }
// max with -0 < +0 (PTX max.f32 orders the zeros; spec/prim.rs:54-70)
__device__ __forceinline__ float fmax_ord(float a, float b) { return fmaxf(a, b); }

// Order-preserving map of fp32 bit patterns onto unsigned integers (so integer max == the spec's fmax, -0 < +0).
__device__ __forceinline__ unsigned f32_key(float f) {
    unsigned b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_f32(unsigned k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// ---- exp_f (spec/prim.rs:78-100)
__device__ __forceinline__ float exp_f(float x) {
    const float xc = fminf(x, 88.0f);
    const float n = floorf(fadd(fmul(xc, (float)1.44269504088896341), 0.5f));
    float r = fsub(xc, fmul(n, (float)0.693359375));
    r = fsub(r, fmul(n, (float)-2.12194440e-4));
    const float z = fmul(r, r);
    float y = (float)1.9875691500E-4;
    y = fadd(fmul(y, r), (float)1.3981999507E-3);
    y = fadd(fmul(y, r), (float)8.3334519073E-3);
    y = fadd(fmul(y, r), (float)4.1665795894E-2);
    y = fadd(fmul(y, r), (float)1.6666665459E-1);
    y = fadd(fmul(y, r), (float)5.0000001201E-1);
    y = fadd(fmul(y, z), r);
    y = fadd(y, 1.0f);
    const int e = __float2int_rz(n) + 127;
    const float res = fmul(y, __int_as_float(e << 23));
    return (xc < -87.0f) ? 0.0f : res;
}

// ---- log_f (spec/prim.rs:102-127); x > 0
__device__ __forceinline__ float log_f(float x) {
    const unsigned b = __float_as_uint(x);
    int e = (int)((b >> 23) & 0xffu) - 126;
    float m = __uint_as_float((b & 0x007fffffu) | 0x3f000000u);
    if (m < (float)0.707106781186547524) {
        e -= 1;
        m = fsub(fadd(m, m), 1.0f);
    } else {
        m = fsub(m, 1.0f);
    }
    const float z = fmul(m, m);
    float y = (float)7.0376836292E-2;
    y = fadd(fmul(y, m), (float)-1.1514610310E-1);
    y = fadd(fmul(y, m), (float)1.1676998740E-1);
    y = fadd(fmul(y, m), (float)-1.2420140846E-1);
    y = fadd(fmul(y, m), (float)1.4249322787E-1);
    y = fadd(fmul(y, m), (float)-1.6668057665E-1);
    y = fadd(fmul(y, m), (float)2.0000714765E-1);
    y = fadd(fmul(y, m), (float)-2.4999993993E-1);
    y = fadd(fmul(y, m), (float)3.3333331174E-1);
    y = fmul(y, m);
    y = fmul(y, z);
    const float ef = (float)e;
    y = fadd(y, fmul((float)-2.12194440e-4, ef));
    y = fadd(y, fmul(-0.5f, z));
    float r = fadd(m, y);
    r = fadd(r, fmul((float)0.693359375, ef));
    return r;
}

// spec/prim.rs:129-150
__device__ __forceinline__ float softplus_f(float x) {
    if (x > 20.0f) return x;
    if (x < -15.0f) return exp_f(x);
    return log_f(fadd(1.0f, exp_f(x)));
}
__device__ __forceinline__ float sigmoid_f(float x) {
    if (x < -80.0f) return exp_f(x);
    return fdiv(1.0f, fadd(1.0f, exp_f(-x)));
}
__device__ __forceinline__ float silu_f(float x) { return fmul(x, sigmoid_f(x)); }

// ---- treesum building blocks (docs/SPEC.md §1.3).  The spec tree over a power-of-two array pairs neighbours level
// by level.  A thread that owns an aligned contiguous run of 2^k inputs folds it in place; lanes then continue the same
// tree with xor offsets 1, 2, 4, ... (ascending), and warps continue it in warp order.
template <int N>
__device__ __forceinline__ float fold_run(float (&v)[N]) {
    static_assert((N & (N - 1)) == 0, "run length must be a power of two");
#pragma unroll
    for (int step = 1; step < N; step <<= 1) {
#pragma unroll
        for (int i = 0; i < N; i += 2 * step) v[i] = fadd(v[i], v[i + step]);
    }
    return v[0];
}
// Continues the tree across `width` consecutive lanes (width a power of two, lanes aligned to it).
template <int WIDTH = 32>
__device__ __forceinline__ float fold_lanes(float v) {
#pragma unroll
    for (int off = 1; off < WIDTH; off <<= 1) v = fadd(v, __shfl_xor_sync(FULL, v, off));
    return v;
}
// Continues the tree across the NW warps of a block (NW a power of two); every thread returns the total.
template <int NW>
__device__ __forceinline__ float fold_warps(float warp_total, float* sh /* [NW] */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) sh[warp] = warp_total;
    __syncthreads();
    float v = (lane < NW) ? sh[lane] : 0.0f;
    if (NW > 1) v = fold_lanes<(NW > 1 ? NW : 2)>(v);
    return __shfl_sync(FULL, v, 0);
}

// ---- order-free maxima
__device__ __forceinline__ float max_lanes(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(FULL, v, off));
    return v;
}
template <int NW>
__device__ __forceinline__ float max_block(float v, float* sh /* [NW] */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = max_lanes(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float r = (lane < NW) ? sh[lane] : sh[0];
    return max_lanes(r);
}

// ---- activation quantization pieces (spec/quant.rs:7-60)
__device__ __forceinline__ int quant_code(float x, float inv) {
    int q = __float2int_rn(fmul(x, inv));   // NaN -> 0, +-inf saturate: the Rust `as` semantics the spec relies on
    return max(-127, min(127, q));
}
// Group multiplier: clamp(rint(s_g / sx), 1, 65535) with NaN -> 0 (a NaN fails both clamps, then `as u16` gives 0).
__device__ __forceinline__ unsigned group_mult(float s_g, float sx) {
    const float m = frint(fdiv(s_g, sx));
    if (m != m) return 0u;
    if (m < 1.0f) return 1u;
    if (m > 65535.0f) return 65535u;
    return (unsigned)m;
}

}  // namespace detb
