// Row-wise glue of the token loop: RMSNorm, activation quantization (quant_act_i8g / quant_act_i8), SwiGLU product,
// embedding lookup, residual add and greedy argmax.  Replaces kernels/cuda/norm.cu behind the same entry points
// (det_rmsnorm_quant, det_quant, det_silu_mul_quant, det_embed, det_add, det_argmax).
//
// One CTA owns one row.  The sum of squares follows the spec tree (docs/SPEC.md §1.3): the row is padded with +0.0 to
// P = next power of two, each thread folds an aligned run of P / blockDim values, lanes continue with ascending xor
// offsets and warps in warp order.  Quantization then re-reads the row with one warp per 128-group (4 values per lane),
// keeps the produced values in registers across the row-global max, and emits codes, multipliers and the row scale.
#include "runtime.cuh"

namespace detb {

enum RowMode : int { ROW_RMSNORM = 0, ROW_PLAIN = 1, ROW_SWIGLU = 2 };

struct RowArgs {
    const float* a;     // x (rmsnorm, plain) or gate (swiglu)
    const float* b;     // norm weight (rmsnorm) or up (swiglu)
    float eps;
    int n;
    float* y;           // optional fp32 copy of the produced row
    int8_t* q;          // optional codes
    float* sx;
    uint16_t* mx;       // NULL: per-row int8 (quant_act_i8)
};

// Continues the spec tree over the warps of a block whose warp count is a power of two known at run time.
__device__ __forceinline__ float fold_warps_rt(float warp_total, float* sh, int nw) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) sh[warp] = warp_total;
    __syncthreads();
    float v = (lane < nw) ? sh[lane] : 0.0f;
    for (int off = 1; off < nw; off <<= 1) v = fadd(v, __shfl_xor_sync(FULL, v, off));
    return __shfl_sync(FULL, v, 0);
}
__device__ __forceinline__ float max_block_rt(float v, float* sh, int nw) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = max_lanes(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    return max_lanes((lane < nw) ? sh[lane] : sh[0]);
}

template <int MODE, int RUN, int MAXG>
__global__ void __launch_bounds__(1024) k_row(RowArgs p) {
    __shared__ float sh[32];
    const int row = blockIdx.x;
    const int n = p.n;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const float* a = p.a + (size_t)row * n;
    const float* b = (MODE == ROW_SWIGLU) ? p.b + (size_t)row * n : p.b;

    float inv_rms = 0.0f;
    if (MODE == ROW_RMSNORM) {
        float sq[RUN];
#pragma unroll
        for (int i = 0; i < RUN; i++) {
            const int idx = threadIdx.x * RUN + i;
            const float v = idx < n ? a[idx] : 0.0f;
            sq[i] = fmul(v, v);
        }
        float ss = fold_lanes<32>(fold_run<RUN>(sq));
        ss = fold_warps_rt(ss, sh, nw);
        const float mean = fdiv(ss, (float)n);
        inv_rms = fdiv(1.0f, fsqrt(fadd(mean, p.eps)));
    }

    // ---- one warp per 128-wide slice, 4 consecutive values per lane
    const int slices = (n + 127) >> 7;
    float val[MAXG][4];
    float s_slice[MAXG];
    float local_max = 0.0f;
#pragma unroll
    for (int j = 0; j < MAXG; j++) {
        const int g = warp + j * nw;
        s_slice[j] = 0.0f;
#pragma unroll
        for (int e = 0; e < 4; e++) val[j][e] = 0.0f;
        if (g < slices) {
            const int base = g * 128 + lane * 4;
            float amax = 0.0f;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int idx = base + e;
                float v = 0.0f;
                if (idx < n) {
                    if (MODE == ROW_RMSNORM) v = fmul(fmul(a[idx], inv_rms), b[idx]);
                    else if (MODE == ROW_PLAIN) v = a[idx];
                    else v = fmul(silu_f(a[idx]), b[idx]);
                    if (p.y) p.y[(size_t)row * n + idx] = v;
                }
                val[j][e] = v;
                amax = fmaxf(amax, fabsf(v));
            }
            amax = max_lanes(amax);
            s_slice[j] = p.mx ? fdiv(amax, 127.0f) : amax;
            local_max = fmaxf(local_max, s_slice[j]);
        }
    }
    if (!p.q) return;
    const float top = max_block_rt(local_max, sh, nw);

    if (p.mx) {
        // quant_act_i8g: sx = smax / 65535 (1 when smax == 0); per group mult, eff = sx * mult, inv = 1 / eff
        const float sx = (top == 0.0f) ? 1.0f : fdiv(top, 65535.0f);
        if (threadIdx.x == 0) p.sx[row] = sx;
#pragma unroll
        for (int j = 0; j < MAXG; j++) {
            const int g = warp + j * nw;
            if (g < slices) {
                const unsigned mult = group_mult(s_slice[j], sx);
                const float inv = fdiv(1.0f, fmul(sx, (float)mult));
                char4 c;
                c.x = (signed char)quant_code(val[j][0], inv);
                c.y = (signed char)quant_code(val[j][1], inv);
                c.z = (signed char)quant_code(val[j][2], inv);
                c.w = (signed char)quant_code(val[j][3], inv);
                *reinterpret_cast<char4*>(p.q + (size_t)row * n + g * 128 + lane * 4) = c;
                if (lane == 0) p.mx[(size_t)row * (n >> 7) + g] = (uint16_t)mult;
            }
        }
    } else {
        // quant_act_i8: s = amax / 127 (1 when amax == 0)
        const float s = (top == 0.0f) ? 1.0f : fdiv(top, 127.0f);
        const float inv = fdiv(1.0f, s);
        if (threadIdx.x == 0) p.sx[row] = s;
#pragma unroll
        for (int j = 0; j < MAXG; j++) {
            const int g = warp + j * nw;
            if (g < slices) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int idx = g * 128 + lane * 4 + e;
                    if (idx < n) p.q[(size_t)row * n + idx] = (int8_t)quant_code(val[j][e], inv);
                }
            }
        }
    }
}

template <int MODE>
static void launch_row(const RowArgs& p, int M, cudaStream_t q) {
    const int n = p.n;
    DETB_REQUIRE(n >= 1 && n <= 32768, "row length must be 1..32768");
    if (p.q && p.mx) DETB_REQUIRE(n % 128 == 0, "grouped quantization needs n % 128 == 0");
    int P = 32;
    while (P < n) P <<= 1;
    const int threads = P < 1024 ? P : 1024;
    const int run = P / threads;                       // 1, 2, 4, ..., 32
    const int nw = threads / 32;
    const int maxg = (((n + 127) >> 7) + nw - 1) / nw;   // <= 8
#define DETB_ROW(RUN_, MAXG_) k_row<MODE, RUN_, MAXG_><<<M, threads, 0, q>>>(p)
    if (MODE != ROW_RMSNORM) {
        // no tree: only the slice mapping matters
        if (maxg <= 1) DETB_ROW(1, 1);
        else if (maxg <= 2) DETB_ROW(1, 2);
        else if (maxg <= 4) DETB_ROW(1, 4);
        else DETB_ROW(1, 8);
    } else {
        switch (run) {
            case 1: DETB_ROW(1, 1); break;
            case 2: DETB_ROW(2, 1); break;
            case 4: DETB_ROW(4, 1); break;
            case 8: DETB_ROW(8, 2); break;
            case 16: DETB_ROW(16, 4); break;
            default: DETB_ROW(32, 8); break;
        }
    }
#undef DETB_ROW
    DETB_CUDA_OK(cudaGetLastError());
}

// ---- embedding rows (bf16 table -> fp32, exact), residual add, argmax
__global__ void k_embed_rows(const uint16_t* __restrict__ table, const int* __restrict__ ids, int H,
                             float* __restrict__ x) {
    const uint16_t* src = table + (size_t)ids[blockIdx.x] * H;
    float* dst = x + (size_t)blockIdx.x * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = __uint_as_float((unsigned)src[i] << 16);
}
__global__ void k_residual_add(float* __restrict__ x, const float* __restrict__ y, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = fadd(x[i], y[i]);
}
// Lowest index of the maximum (spec/sample.rs:6-14): a strictly greater value replaces the running best, so +0 and -0
// tie and the lower index stays.
__global__ void __launch_bounds__(1024) k_argmax_rows(const float* __restrict__ logits, int V, int* __restrict__ out) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const float* row = logits + (size_t)blockIdx.x * V;
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > best || at == 0x7fffffff) { best = v; at = i; }
    }
    auto better = [](float v, int i, float w, int j) { return v > w || (v == w && i < j); };
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(FULL, best, off);
        const int oi = __shfl_xor_sync(FULL, at, off);
        if (oi != 0x7fffffff && (at == 0x7fffffff || better(ov, oi, best, at))) { best = ov; at = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) { bv[warp] = best; bi[warp] = at; }
    __syncthreads();
    if (warp == 0) {
        best = lane < nw ? bv[lane] : -INFINITY;
        at = lane < nw ? bi[lane] : 0x7fffffff;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(FULL, best, off);
            const int oi = __shfl_xor_sync(FULL, at, off);
            if (oi != 0x7fffffff && (at == 0x7fffffff || better(ov, oi, best, at))) { best = ov; at = oi; }
        }
        if (lane == 0) out[blockIdx.x] = at == 0x7fffffff ? 0 : at;
    }
}

}  // namespace detb

using namespace detb;

extern "C" {

void det_rmsnorm_quant(const float* x, const float* w, float eps, int M, int n, float* y, int8_t* xq, float* sx,
                       uint16_t* mx, cudaStream_t st) {
    if (M <= 0) return;
    RowArgs p{x, w, eps, n, y, xq, sx, mx};
    launch_row<ROW_RMSNORM>(p, M, queue_of(st));
}
void det_quant(const float* x, int M, int n, int8_t* xq, float* sx, uint16_t* mx, cudaStream_t st) {
    if (M <= 0) return;
    RowArgs p{x, nullptr, 0.0f, n, nullptr, xq, sx, mx};
    launch_row<ROW_PLAIN>(p, M, queue_of(st));
}
void det_silu_mul_quant(const float* g, const float* u, int M, int n, float* h, int8_t* hq, float* sh, uint16_t* mh,
                        cudaStream_t st) {
    if (M <= 0) return;
    RowArgs p{g, u, 0.0f, n, h, hq, sh, mh};
    launch_row<ROW_SWIGLU>(p, M, queue_of(st));
}
void det_embed(const uint16_t* table_bf16, const int* ids, int M, int H, float* x, cudaStream_t st) {
    if (M <= 0) return;
    k_embed_rows<<<M, 256, 0, queue_of(st)>>>(table_bf16, ids, H, x);
    DETB_CUDA_OK(cudaGetLastError());
}
void det_add(float* x, const float* y, long long n, cudaStream_t st) {
    if (n <= 0) return;
    k_residual_add<<<(unsigned)((n + 255) / 256), 256, 0, queue_of(st)>>>(x, y, n);
    DETB_CUDA_OK(cudaGetLastError());
}
void det_argmax(const float* logits, int M, int V, int* out, cudaStream_t st) {
    if (M <= 0) return;
    k_argmax_rows<<<M, 1024, 0, queue_of(st)>>>(logits, V, out);
    DETB_CUDA_OK(cudaGetLastError());
}

}  // extern "C"
