// Device twin of the synthetic-model generator and of the reference weight quantizer (crates/det/src/quantize.rs:33-85):
// builds the det rows of a seeded random-init linear directly in device memory, in the reference layout of
// det_qlinear (row-major codes, c, m), and quantizes float tensors of a source checkpoint into det file rows (the device
// side of `det convert`, crates/det/src/convert.rs:346-369).  Every value equals what the host twin
// (csrc/host/synth.cpp) produces: the draw is integer arithmetic plus two fp32 multiplies, the quantizer is binary64
// add / mul / div / rint without contraction.  A 27B-shape model has 2.7e10 weights; quantizing them here takes seconds
// instead of many CPU-minutes.  Also here: the calibration fold (largest |v| per kv head) and the typed embedding lookup.
#include "runtime.cuh"
#include <cuda_fp16.h>

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

// Where the quantizer reads a weight from: element k of logical row r, widened to binary64.
struct SynthSrc {   // the seeded generator: rows [src0, src0 + n) of tensor tid
    unsigned long long seed, tid;
    long long src0;
    int K;
    __device__ __forceinline__ double at(long long r, int k) const {
        return weight_f64(seed, tid, (unsigned long long)(src0 + r) * K + (unsigned long long)k);
    }
};
struct TensorSrc {   // a float tensor in device memory, [rows][K] of F32 (0), F16 (1) or BF16 (30), with optional
    const void* p;   // row and column permutations (perm[new] = old; crates/det/src/convert.rs:352-367)
    int type, K;
    const int* row_perm;
    const int* col_perm;
    __device__ __forceinline__ double at(long long r, int k) const {
        const size_t i = (size_t)(row_perm ? row_perm[r] : r) * K + (col_perm ? col_perm[k] : k);
        if (type == 0) return (double)static_cast<const float*>(p)[i];
        if (type == 1) return (double)__half2float(__ushort_as_half(static_cast<const unsigned short*>(p)[i]));
        return (double)__uint_as_float((unsigned)static_cast<const unsigned short*>(p)[i] << 16);
    }
};
// Where a quantized row goes: codes, c and m each at base + row * stride (one struct covers the separate arrays of
// det_qlinear and the [codes][c][m] rows of a det file, spec/tensor.rs:43-55).
struct RowsOut {
    uint8_t *wq, *c, *m;
    size_t wq_stride, c_stride, m_stride;
};

// quantize.rs:33-56 for one (row, 128-group)
template <class Src>
__global__ void k_quant_scales(const Src src, int n, int K, double qmax, double* __restrict__ scales) {
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int G = K >> 7;
    if (id >= (long long)n * G) return;
    const long long r = id / G;
    const int g = (int)(id % G);
    double amax = 0.0;
    for (int i = 0; i < 128; i++) {
        const double a = fabs(src.at(r, g * 128 + i));
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
                const double v = src.at(r, g * 128 + i);
                const double q = clampd(rint(__ddiv_rn(v, s)), qmax);
                const double d = __dsub_rn(__dmul_rn(q, s), v);
                err = __dadd_rn(err, __dmul_rn(d, d));
            }
            if (err < best_err) { best_err = err; best_s = s; }
        }
    }
    scales[id] = best_s;
}

// quantize.rs:58-85 for one (row, 128-group): c, m, codes, packing (quantize.rs:8-31)
template <class Src>
__global__ void k_quant_rows(const Src src, int n, int K, int bits, double qmax, const double* __restrict__ scales,
                             int row0, const RowsOut out) {
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
    if (g == 0) {   // unaligned-safe stores: a det file row has no alignment beyond its own bytes
        const unsigned cb = __float_as_uint(cf);
        uint8_t* cp = out.c + (size_t)orow * out.c_stride;
        for (int i = 0; i < 4; i++) cp[i] = (uint8_t)(cb >> (8 * i));
    }
    uint8_t* mp = out.m + (size_t)orow * out.m_stride + (size_t)g * 2;
    mp[0] = (uint8_t)mg;
    mp[1] = (uint8_t)(mg >> 8);
    const int bp32 = bits == 8 ? 32 : (bits == 6 ? 24 : 16);
    uint8_t* dst = out.wq + (size_t)orow * out.wq_stride + (size_t)g * 4 * bp32;
    const int off = bits == 6 ? 32 : (bits == 4 ? 8 : 0);
    for (int blk = 0; blk < 4; blk++) {
        uint8_t u[32];
        for (int i = 0; i < 32; i++) {
            const double q = clampd(rint(__ddiv_rn(src.at(r, g * 128 + blk * 32 + i), eff)), qmax);
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

template <class Src>
static void quantize_launch(const Src& src, int n, int K, int bits, int row0, const RowsOut& out, double* scratch,
                            cudaStream_t q) {
    const double qmax = (double)((1 << (bits - 1)) - 1);
    const long long work = (long long)n * (K >> 7);
    const unsigned grid = (unsigned)((work + 127) / 128);
    k_quant_scales<Src><<<grid, 128, 0, q>>>(src, n, K, qmax, scratch);
    k_quant_rows<Src><<<grid, 128, 0, q>>>(src, n, K, bits, qmax, scratch, row0, out);
    DETB_CUDA_OK(cudaGetLastError());
}

// Largest |v| of each head over the rows of a batch, folded into slots[head] (crates/det/src/calibrate.rs:21-36).  The
// maximum of non-negative floats is order-free, so an integer atomic on their bit patterns gives the fold's value; a NaN
// is skipped as f32::max skips it.
__global__ void k_absmax_heads(const float* __restrict__ v, int t, int heads, int hd, float* __restrict__ slots) {
    const int head = blockIdx.x % heads, row = blockIdx.x / heads;
    if (row >= t) return;
    const float* p = v + ((size_t)row * heads + head) * hd;
    unsigned best = 0;
    for (int i = threadIdx.x; i < hd; i += blockDim.x) {
        const float a = fabsf(p[i]);
        if (a == a) best = max(best, __float_as_uint(a));
    }
    for (int o = 16; o; o >>= 1) best = max(best, __shfl_xor_sync(0xFFFFFFFFu, best, o));
    if ((threadIdx.x & 31) == 0 && best) atomicMax(reinterpret_cast<unsigned*>(slots) + head, best);
}

// Embedding rows out of a float table of any of the three types (crates/det/src/model.rs:389-413), exact.
__global__ void k_embed_table(const void* __restrict__ table, int type, const int* __restrict__ ids, int H,
                              float* __restrict__ x) {
    pdl_trigger();
    pdl_wait();
    const size_t base = (size_t)ids[blockIdx.x] * H;
    float* dst = x + (size_t)blockIdx.x * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float f;
        if (type == 0) f = static_cast<const float*>(table)[base + i];
        else if (type == 1) f = __half2float(__ushort_as_half(static_cast<const unsigned short*>(table)[base + i]));
        else f = __uint_as_float((unsigned)static_cast<const unsigned short*>(table)[base + i] << 16);
        dst[i] = f;
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
    const int bp32 = bits == 8 ? 32 : (bits == 6 ? 24 : 16);
    const RowsOut out{wq, reinterpret_cast<uint8_t*>(c), reinterpret_cast<uint8_t*>(m), (size_t)(K >> 5) * bp32, 4,
                      (size_t)(K >> 7) * 2};
    quantize_launch(SynthSrc{seed, tid, src_row0, K}, n, K, bits, row0, out, scratch, queue_of(st));
}

// The reference weight quantizer (crates/det/src/quantize.rs:33-100) on the device: `n` rows of K floats from a device
// tensor of ggml type 0 (F32), 1 (F16) or 30 (BF16) become det file rows ([codes][c][m], spec/tensor.rs:43-55) at
// rows_out.  Output row r reads source row row_perm[r] (NULL: r), element k reads column col_perm[k] (NULL: k).
// `scratch` holds n * K/128 doubles.  Bit-identical to the host quantizer: binary64 add / mul / div / rint, no contraction.
void det_quantize_rows(const void* src, int ggml_type, const int* row_perm, const int* col_perm, int n, int K, int bits,
                       uint8_t* rows_out, double* scratch, cudaStream_t st) {
    DETB_REQUIRE((bits == 4 || bits == 6 || bits == 8) && K % 128 == 0 && n > 0, "bad linear shape");
    DETB_REQUIRE(ggml_type == 0 || ggml_type == 1 || ggml_type == 30, "source tensors are F32, F16 or BF16");
    const size_t nc = (size_t)(K >> 5) * (bits == 8 ? 32 : (bits == 6 ? 24 : 16)), rb = nc + 4 + (size_t)(K >> 7) * 2;
    const RowsOut out{rows_out, rows_out + nc, rows_out + nc + 4, rb, rb, rb};
    quantize_launch(TensorSrc{src, ggml_type, K, row_perm, col_perm}, n, K, bits, 0, out, scratch, queue_of(st));
}

// slots[heads] = max(slots, largest |v[row][head][:]| over the t rows)  (crates/det/src/calibrate.rs:21-36)
void det_absmax_heads(const float* v, int t, int heads, int hd, float* slots, cudaStream_t st) {
    if (t <= 0) return;
    k_absmax_heads<<<(unsigned)(t * heads), 128, 0, queue_of(st)>>>(v, t, heads, hd, slots);
    DETB_CUDA_OK(cudaGetLastError());
}

// det_embed for a float table of ggml type 0 (F32), 1 (F16) or 30 (BF16).
void det_embed_table(const void* table, int ggml_type, const int* ids, int M, int H, float* x, cudaStream_t st) {
    DETB_REQUIRE(ggml_type == 0 || ggml_type == 1 || ggml_type == 30, "embedding tables are F32, F16 or BF16");
    if (M <= 0) return;
    launch_pdl(k_embed_table, dim3(M), dim3(256), 0, queue_of(st), 1, table, ggml_type, ids, H, x);
}

// count bf16 elements of synthetic tensor `tid` (the embedding table).
void det_synth_bf16(unsigned long long seed, unsigned long long tid, long long count, uint16_t* out, cudaStream_t st) {
    k_synth_bf16<<<(unsigned)((count + 255) / 256), 256, 0, queue_of(st)>>>(seed, tid, count, out);
    DETB_CUDA_OK(cudaGetLastError());
}

}  // extern "C"
