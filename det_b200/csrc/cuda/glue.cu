// Row-wise glue of the token loop: RMSNorm, activation quantization (quant_act_i8g / quant_act_i8), SwiGLU product,
// embedding lookup, residual add and greedy argmax.  Replaces kernels/cuda/norm.cu behind the same entry points
// (det_rmsnorm_quant, det_quant, det_silu_mul_quant, det_embed, det_add, det_argmax).
//
// A row is spread over a thread-block cluster (up to 8 CTAs, one warp per 128-wide slice) so that a single decode row
// of 5120 or 17408 values is not a one-SM job; the row-wide sum of squares (the spec tree, docs/SPEC.md §1.3) and the
// row-wide maximum are combined through distributed shared memory.
#include "exchange.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

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
    float* acc;         // optional (rmsnorm, plain): the row is acc + a, and acc is updated to it (residual add)
};

__device__ __forceinline__ float max_block_rt(float v, float* sh, int nw) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = max_lanes(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    return max_lanes((lane < nw) ? sh[lane] : sh[0]);
}

// One row is handled by a thread-block cluster of CS CTAs (1, 2, 4 or 8).  A warp owns one 128-wide slice of the row
// (4 consecutive values per lane); CTA `rank` of the cluster owns the slices [rank * spc, (rank + 1) * spc).
//   * sum of squares: a slice is an aligned subtree of the spec tree, so each warp folds its slice exactly; the slice
//     sums are exchanged through distributed shared memory and every CTA finishes the same tree over the P / 128 slice
//     sums (zero padded), so all CTAs hold the bit-identical row total;
//   * the row-global maximum of the group scales is order-free: per-CTA maxima are exchanged the same way.
// Values stay in registers between the two phases.
constexpr int MAX_SLICES = 256;   // rows up to 32768 values

__device__ __forceinline__ float* peer_smem(float* local, unsigned rank) {
    return cg::this_cluster().map_shared_rank(local, rank);
}
// The two halves of a cluster barrier; every thread of every CTA executes both, alternately.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// XCHG: the rows come out of the tensor-parallel exchange, which is this kernel's prologue: every CTA of the grid sends its
// share of the local slice to all ranks, then each lane polls the staging packets that hold its four values (the grid is
// at most 8 CTAs per row and 8 rows, all resident).  p.a is unused.
template <int MODE, bool XCHG>
__global__ void __launch_bounds__(1024) k_row(RowArgs p, int spc /* slices per CTA */, int pslices /* P / 128 */,
                                              const XchgArgs xa) {
    __shared__ float all_sums[MAX_SLICES];   // slice sums of the whole row: every CTA's are PUSHED into every peer's copy
    __shared__ float cta_maxes[8];           // largest group scale of every CTA of the cluster, pushed the same way
    __shared__ float shf[32];
    // Exchanges are stores into the peers' shared memory followed by one cluster barrier (arrive + wait): nobody reads
    // remote memory, so a round costs one barrier and no CTA has to stay alive for a late reader.  The first arrive
    // is posted at entry and waited for just before the first remote store (a peer's shared memory may only be touched
    // once that peer runs); by then it has usually completed.
    for (int i = threadIdx.x; i < pslices; i += blockDim.x) all_sums[i] = 0.0f;   // zero padding of the tree
    __syncthreads();
    cluster_arrive();
    pdl_trigger();
    pdl_wait();
    unsigned seq = 0;
    if (XCHG) {
        seq = xchg_seq(xa);
        xchg_push(xa, seq);
    }
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank(), cs = cluster.num_blocks();
    const int row = blockIdx.y;
    const int n = p.n;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const float* a = p.a + (size_t)row * n;
    const float* b = (MODE == ROW_SWIGLU) ? p.b + (size_t)row * n : p.b;
    const int slices = (n + 127) >> 7;
    const int g = (int)rank * spc + warp;           // this warp's slice
    const bool have = warp < spc && g < slices;
    const int base = g * 128 + lane * 4;

    float raw[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (have) {
        if (XCHG) {   // n is a multiple of 128 here
            const size_t pk = ((size_t)row * n + base) >> 1;
            const float2 lo = xchg_read(xa, seq, pk), hi = xchg_read(xa, seq, pk + 1);
            raw[0] = lo.x; raw[1] = lo.y; raw[2] = hi.x; raw[3] = hi.y;
        } else {
#pragma unroll
            for (int e = 0; e < 4; e++)
                if (base + e < n) raw[e] = a[base + e];
        }
        if (MODE != ROW_SWIGLU && p.acc) {
            float* acc = p.acc + (size_t)row * n;
#pragma unroll
            for (int e = 0; e < 4; e++)
                if (base + e < n) acc[base + e] = raw[e] = fadd(acc[base + e], raw[e]);
        }
    }
    float inv_rms = 0.0f;
    if (MODE == ROW_RMSNORM) {
        float sq[4];
#pragma unroll
        for (int e = 0; e < 4; e++) sq[e] = fmul(raw[e], raw[e]);
        const float ssum = fold_lanes<32>(fold_run<4>(sq));
        cluster_wait();                                   // every CTA of the cluster is running
        if (have && lane < (int)cs) peer_smem(all_sums, lane)[g] = ssum;   // lane r stores into CTA r's copy
        cluster_arrive();
        cluster_wait();                                   // all slice sums of the row have landed here
        // finish the tree: lane owns pslices / 32 consecutive slice sums (or one each when there are fewer than 32)
        float tot;
        if (pslices >= 32) {
            const int per = pslices >> 5;   // 1, 2, 4 or 8
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = i < per ? all_sums[lane * per + i] : 0.0f;
            // fold the first `per` entries pairwise (per is a power of two; entries past it are never touched)
#pragma unroll
            for (int step = 1; step < 8; step <<= 1) {
#pragma unroll
                for (int i = 0; i < 8; i += 2 * step)
                    if (step < per) v[i] = fadd(v[i], v[i + step]);
            }
            tot = fold_lanes<32>(v[0]);
        } else {
            float v = lane < pslices ? all_sums[lane] : 0.0f;
            for (int off = 1; off < pslices; off <<= 1) v = fadd(v, __shfl_xor_sync(FULL, v, off));
            tot = __shfl_sync(FULL, v, 0);
        }
        const float mean = fdiv(tot, (float)n);
        inv_rms = fdiv(1.0f, fsqrt(fadd(mean, p.eps)));
    }

    // ---- produce the row values of this warp's slice, the slice scale and the CTA maximum
    float val[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float s_slice = 0.0f;
    if (have) {
        float amax = 0.0f;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int idx = base + e;
            float v = 0.0f;
            if (idx < n) {
                if (MODE == ROW_RMSNORM) v = fmul(fmul(raw[e], inv_rms), b[idx]);
                else if (MODE == ROW_PLAIN) v = raw[e];
                else v = fmul(silu_f(raw[e]), b[idx]);
                if (p.y) p.y[(size_t)row * n + idx] = v;
            }
            val[e] = v;
            amax = fmaxf(amax, fabsf(v));
        }
        amax = max_lanes(amax);
        s_slice = p.mx ? fdiv(amax, 127.0f) : amax;
    }
    if (!p.q) {
        if (MODE != ROW_RMSNORM) cluster_wait();   // pair the arrive posted at entry
        return;
    }
    const float cmax = max_block_rt(s_slice, shf, nw);
    if (MODE != ROW_RMSNORM) cluster_wait();       // (the RMSNorm path has already waited for the start of its peers)
    if (threadIdx.x < cs) peer_smem(cta_maxes, threadIdx.x)[rank] = cmax;
    cluster_arrive();
    cluster_wait();
    float top = 0.0f;
    for (unsigned r = 0; r < cs; r++) top = fmaxf(top, cta_maxes[r]);

    if (p.mx) {
        // quant_act_i8g: sx = smax / 65535 (1 when smax == 0); per group mult, eff = sx * mult, inv = 1 / eff
        const float sx = (top == 0.0f) ? 1.0f : fdiv(top, 65535.0f);
        if (rank == 0 && threadIdx.x == 0) p.sx[row] = sx;
        if (have) {
            const unsigned mult = group_mult(s_slice, sx);
            const float inv = fdiv(1.0f, fmul(sx, (float)mult));
            char4 c;
            c.x = (signed char)quant_code(val[0], inv);
            c.y = (signed char)quant_code(val[1], inv);
            c.z = (signed char)quant_code(val[2], inv);
            c.w = (signed char)quant_code(val[3], inv);
            *reinterpret_cast<char4*>(p.q + (size_t)row * n + base) = c;
            if (lane == 0) p.mx[(size_t)row * (n >> 7) + g] = (uint16_t)mult;
        }
    } else {
        // quant_act_i8: s = amax / 127 (1 when amax == 0)
        const float s = (top == 0.0f) ? 1.0f : fdiv(top, 127.0f);
        const float inv = fdiv(1.0f, s);
        if (rank == 0 && threadIdx.x == 0) p.sx[row] = s;
        if (have) {
#pragma unroll
            for (int e = 0; e < 4; e++)
                if (base + e < n) p.q[(size_t)row * n + base + e] = (int8_t)quant_code(val[e], inv);
        }
    }
}

// The same row operations for MANY rows (prefill chunks): one CTA per row, each warp walks several 128-wide slices, no
// cluster.  A single row finishes later than in the cluster kernel, but hundreds of rows are in flight at once and
// nothing waits on a cluster barrier.  (At 32 rows the cluster kernel is still faster — measured 7.8 vs 18.6 us for the
// SwiGLU row of 17408 — so the switch-over is at 128 rows.)  The arithmetic per slice, the tree over the slice sums and the maxima are the
// same expressions as above, so the values are the same bits.
constexpr int WIDE_MAXK = 8;     // slices per warp: rows up to 32 * 8 * 128 = 32768 values

template <int MODE>
__global__ void __launch_bounds__(1024) k_row_wide(RowArgs p, int pslices /* P / 128 */) {
    __shared__ float all_sums[MAX_SLICES];
    __shared__ float shf[32];
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int n = p.n;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const float* a = p.a + (size_t)row * n;
    const float* b = (MODE == ROW_SWIGLU) ? p.b + (size_t)row * n : p.b;
    const int slices = (n + 127) >> 7;

    float raw[WIDE_MAXK][4];
#pragma unroll
    for (int k = 0; k < WIDE_MAXK; k++) {
        const int g = warp + k * nw, base = g * 128 + lane * 4;
#pragma unroll
        for (int e = 0; e < 4; e++) raw[k][e] = 0.0f;
        if (g < slices) {
#pragma unroll
            for (int e = 0; e < 4; e++)
                if (base + e < n) raw[k][e] = a[base + e];
            if (MODE != ROW_SWIGLU && p.acc) {
                float* acc = p.acc + (size_t)row * n;
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (base + e < n) acc[base + e] = raw[k][e] = fadd(acc[base + e], raw[k][e]);
            }
        }
    }
    float inv_rms = 0.0f;
    if (MODE == ROW_RMSNORM) {
        for (int i = threadIdx.x; i < pslices; i += blockDim.x) all_sums[i] = 0.0f;   // zero padding of the tree
        __syncthreads();
#pragma unroll
        for (int k = 0; k < WIDE_MAXK; k++) {
            const int g = warp + k * nw;
            float sq[4];
#pragma unroll
            for (int e = 0; e < 4; e++) sq[e] = fmul(raw[k][e], raw[k][e]);
            const float ssum = fold_lanes<32>(fold_run<4>(sq));
            if (lane == 0 && g < slices) all_sums[g] = ssum;
        }
        __syncthreads();
        float tot;
        if (pslices >= 32) {
            const int per = pslices >> 5;   // 1, 2, 4 or 8
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = i < per ? all_sums[lane * per + i] : 0.0f;
#pragma unroll
            for (int step = 1; step < 8; step <<= 1) {
#pragma unroll
                for (int i = 0; i < 8; i += 2 * step)
                    if (step < per) v[i] = fadd(v[i], v[i + step]);
            }
            tot = fold_lanes<32>(v[0]);
        } else {
            float v = lane < pslices ? all_sums[lane] : 0.0f;
            for (int off = 1; off < pslices; off <<= 1) v = fadd(v, __shfl_xor_sync(FULL, v, off));
            tot = __shfl_sync(FULL, v, 0);
        }
        const float mean = fdiv(tot, (float)n);
        inv_rms = fdiv(1.0f, fsqrt(fadd(mean, p.eps)));
    }
    float s_slice[WIDE_MAXK];
    float smax = 0.0f;
#pragma unroll
    for (int k = 0; k < WIDE_MAXK; k++) {
        const int g = warp + k * nw, base = g * 128 + lane * 4;
        s_slice[k] = 0.0f;
        if (g < slices) {
            float amax = 0.0f;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int idx = base + e;
                float v = 0.0f;
                if (idx < n) {
                    if (MODE == ROW_RMSNORM) v = fmul(fmul(raw[k][e], inv_rms), b[idx]);
                    else if (MODE == ROW_PLAIN) v = raw[k][e];
                    else v = fmul(silu_f(raw[k][e]), b[idx]);
                    if (p.y) p.y[(size_t)row * n + idx] = v;
                }
                raw[k][e] = v;                      // from here on the row values
                amax = fmaxf(amax, fabsf(v));
            }
            amax = max_lanes(amax);
            s_slice[k] = p.mx ? fdiv(amax, 127.0f) : amax;
            smax = fmaxf(smax, s_slice[k]);
        }
    }
    if (!p.q) return;
    const float top = max_block_rt(smax, shf, nw);
    if (p.mx) {
        const float sx = (top == 0.0f) ? 1.0f : fdiv(top, 65535.0f);
        if (threadIdx.x == 0) p.sx[row] = sx;
#pragma unroll
        for (int k = 0; k < WIDE_MAXK; k++) {
            const int g = warp + k * nw, base = g * 128 + lane * 4;
            if (g < slices) {
                const unsigned mult = group_mult(s_slice[k], sx);
                const float inv = fdiv(1.0f, fmul(sx, (float)mult));
                char4 c;
                c.x = (signed char)quant_code(raw[k][0], inv);
                c.y = (signed char)quant_code(raw[k][1], inv);
                c.z = (signed char)quant_code(raw[k][2], inv);
                c.w = (signed char)quant_code(raw[k][3], inv);
                *reinterpret_cast<char4*>(p.q + (size_t)row * n + base) = c;
                if (lane == 0) p.mx[(size_t)row * (n >> 7) + g] = (uint16_t)mult;
            }
        }
    } else {
        const float s = (top == 0.0f) ? 1.0f : fdiv(top, 127.0f);
        const float inv = fdiv(1.0f, s);
        if (threadIdx.x == 0) p.sx[row] = s;
#pragma unroll
        for (int k = 0; k < WIDE_MAXK; k++) {
            const int g = warp + k * nw, base = g * 128 + lane * 4;
            if (g < slices) {
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (base + e < n) p.q[(size_t)row * n + base + e] = (int8_t)quant_code(raw[k][e], inv);
            }
        }
    }
}

static int g_row_wide_min = 128;   // rows from which the one-CTA-per-row kernel is used (det_debug_set_rows; 0 = never)

template <int MODE, bool XCHG = false>
static void launch_row(const RowArgs& p, int M, cudaStream_t q, const XchgArgs* xa = nullptr) {
    const int n = p.n;
    DETB_REQUIRE(n >= 1 && n <= 32768, "row length must be 1..32768");
    if (p.q && p.mx) DETB_REQUIRE(n % 128 == 0, "grouped quantization needs n % 128 == 0");
    DETB_REQUIRE(M <= 65535, "at most 65535 rows per call");
    int P = 128;
    while (P < n) P <<= 1;
    const int slices = (n + 127) >> 7;
    if (!XCHG && g_row_wide_min > 0 && M >= g_row_wide_min) {   // many rows: one CTA per row (a choice by shape only)
        const int warps = slices < 32 ? slices : 32;
        launch_pdl(k_row_wide<MODE>, dim3(M), dim3(warps * 32), 0, q, 1, p, P / 128);
        return;
    }
    int cs = 8;                                   // cluster size: by shape only
    while (cs > 1 && slices / cs < 4) cs >>= 1;
    if (XCHG)                                     // every CTA of a fused exchange must be resident: at most 64 of them
        while (cs > 1 && cs * M > 64) cs >>= 1;
    const int spc = (slices + cs - 1) / cs;       // <= 32
    if (XCHG) DETB_REQUIRE(cs * M <= 64 && spc <= 32 && spc * 32 >= XCHG_MAX_RANKS, "fused exchange: rows too many or too long");
    launch_pdl(k_row<MODE, XCHG>, dim3(cs, M, 1), dim3(spc * 32, 1, 1), 0, q, cs, p, spc, P / 128,
               xa ? *xa : XchgArgs{});
}

// ---- embedding rows (bf16 table -> fp32, exact), residual add, argmax
__global__ void k_embed_rows(const uint16_t* __restrict__ table, const int* __restrict__ ids, int H,
                             float* __restrict__ x) {
    pdl_trigger();
    pdl_wait();
    const uint16_t* src = table + (size_t)ids[blockIdx.x] * H;
    float* dst = x + (size_t)blockIdx.x * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = __uint_as_float((unsigned)src[i] << 16);
}
__global__ void k_residual_add(float* __restrict__ x, const float* __restrict__ y, long long n) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = fadd(x[i], y[i]);
}
// Lowest index of the maximum (spec/sample.rs:6-14): a strictly greater value replaces the running best, so +0 and -0
// tie and the lower index stays.
__global__ void __launch_bounds__(1024) k_argmax_rows(const float* __restrict__ logits, int V, int* __restrict__ out) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    pdl_trigger();
    pdl_wait();
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

// The same result for few rows of a large vocabulary (decode): ARGMAX_SPLIT CTAs per row each reduce one contiguous
// chunk, the CTA that finishes last merges the chunk results.  (value, index) pairs merge exactly: greater value wins,
// equal values keep the lower index.
constexpr int ARGMAX_SPLIT = 32, ARGMAX_SPLIT_ROWS = 8;
static __device__ float g_argmax_val[ARGMAX_SPLIT_ROWS * ARGMAX_SPLIT];
static __device__ int g_argmax_idx[ARGMAX_SPLIT_ROWS * ARGMAX_SPLIT];
static __device__ unsigned g_argmax_done[ARGMAX_SPLIT_ROWS];

__global__ void __launch_bounds__(256) k_argmax_split(const float* __restrict__ logits, int V, int* __restrict__ out) {
    __shared__ float bv[8];
    __shared__ int bi[8];
    __shared__ bool last;
    pdl_trigger();
    pdl_wait();
    const int rowi = blockIdx.y;
    const float* row = logits + (size_t)rowi * V;
    const int chunk = (V + ARGMAX_SPLIT - 1) / ARGMAX_SPLIT;
    const int lo = blockIdx.x * chunk, hi = min(V, lo + chunk);
    auto better = [](float v, int i, float w, int j) { return v > w || (v == w && i < j); };
    auto merge = [&](float& best, int& at, float ov, int oi) {
        if (oi != 0x7fffffff && (at == 0x7fffffff || better(ov, oi, best, at))) { best = ov; at = oi; }
    };
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = row[i];
        if (v > best || at == 0x7fffffff) { best = v; at = i; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) merge(best, at, __shfl_xor_sync(FULL, best, off), __shfl_xor_sync(FULL, at, off));
    if (lane == 0) { bv[warp] = best; bi[warp] = at; }
    __syncthreads();
    if (warp == 0) {
        best = lane < 8 ? bv[lane] : -INFINITY;
        at = lane < 8 ? bi[lane] : 0x7fffffff;
#pragma unroll
        for (int off = 4; off > 0; off >>= 1) merge(best, at, __shfl_xor_sync(FULL, best, off), __shfl_xor_sync(FULL, at, off));
        if (lane == 0) {
            g_argmax_val[rowi * ARGMAX_SPLIT + blockIdx.x] = best;
            g_argmax_idx[rowi * ARGMAX_SPLIT + blockIdx.x] = at;
            __threadfence();
            last = atomicAdd(&g_argmax_done[rowi], 1u) == ARGMAX_SPLIT - 1;
        }
    }
    __syncthreads();
    if (!last || warp != 0) return;
    __threadfence();
    best = __ldcg(&g_argmax_val[rowi * ARGMAX_SPLIT + lane]);
    at = __ldcg(&g_argmax_idx[rowi * ARGMAX_SPLIT + lane]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) merge(best, at, __shfl_xor_sync(FULL, best, off), __shfl_xor_sync(FULL, at, off));
    if (lane == 0) {
        out[rowi] = at == 0x7fffffff ? 0 : at;
        g_argmax_done[rowi] = 0;
    }
}

// tmp[P][M][slice] -> full[M][P][slice]
__global__ void k_unshard(const float* __restrict__ tmp, float* __restrict__ full, int P, int M, int slice) {
    pdl_trigger();
    pdl_wait();
    const long long total = (long long)P * M * slice;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int e = (int)(i % slice);
        const long long rm = i / slice;
        const int t = (int)(rm % M), r = (int)(rm / M);
        full[((size_t)t * P + r) * slice + e] = tmp[i];
    }
}

}  // namespace detb

using namespace detb;

extern "C" {

void det_rmsnorm_quant(const float* x, const float* w, float eps, int M, int n, float* y, int8_t* xq, float* sx,
                       uint16_t* mx, cudaStream_t st) {
    if (M <= 0) return;
    RowArgs p{x, w, eps, n, y, xq, sx, mx, nullptr};
    launch_row<ROW_RMSNORM>(p, M, queue_of(st));
}
void det_quant(const float* x, int M, int n, int8_t* xq, float* sx, uint16_t* mx, cudaStream_t st) {
    if (M <= 0) return;
    RowArgs p{x, nullptr, 0.0f, n, nullptr, xq, sx, mx, nullptr};
    launch_row<ROW_PLAIN>(p, M, queue_of(st));
}
void det_silu_mul_quant(const float* g, const float* u, int M, int n, float* h, int8_t* hq, float* sh, uint16_t* mh,
                        cudaStream_t st) {
    if (M <= 0) return;
    RowArgs p{g, u, 0.0f, n, h, hq, sh, mh, nullptr};
    launch_row<ROW_SWIGLU>(p, M, queue_of(st));
}
// ---- tensor-parallel decode: the exchange that produces a gathered row, and the row operation that consumes it, as
// one launch; n = size * slice.   x[M][n] += gathered; then det_rmsnorm_quant of x.
// Whether M gathered rows of n values can go through the fused exchange kernels: all their CTAs (clusters of up to 8 per
// row, at most 32 slices of 128 values per CTA) have to be resident at once, which 64 CTAs always are.
static bool fused_shape(int M, int n) {
    if (M < 1 || M > 64 || n % 128 != 0) return false;
    const int slices = n >> 7;
    int cs = 8;
    while (cs > 1 && slices / cs < 4) cs >>= 1;
    while (cs > 1 && cs * M > 64) cs >>= 1;
    return cs * M <= 64 && (slices + cs - 1) / cs <= 32;
}
int det_xchg_fusable(int M, int n) { return fused_shape(M, n) ? 1 : 0; }
static void check_fused(const Xchg* xc, int M, int slice) {
    DETB_REQUIRE(slice % 2 == 0 && fused_shape(M, slice * xc->size),
                 "fused exchange: rows of whole 128-value groups, det_xchg_fusable(M, n) must hold");
    DETB_REQUIRE((size_t)M * xc->size * slice * 8 <= xc->slot_bytes, "exchange larger than the staging slot");
}
void det_xchg_add_rmsnorm_quant(void* h, const float* local, int slice, float* x, const float* w, float eps, int M,
                                int8_t* xq, float* sx, uint16_t* mx, cudaStream_t st) {
    const Xchg* xc = static_cast<const Xchg*>(h);
    check_fused(xc, M, slice);
    const XchgArgs xa = xchg_args(xc, local, nullptr, M, slice);
    RowArgs p{nullptr, w, eps, slice * xc->size, nullptr, xq, sx, mx, x};
    launch_row<ROW_RMSNORM, true>(p, M, queue_of(st), &xa);
}
// det_quant of the gathered rows; with local_b the sent values are silu(local) * local_b (det_silu_mul_quant's product
// over this rank's columns), so SwiGLU + exchange + quantization are one launch.
void det_xchg_quant(void* h, const float* local, const float* local_b, int slice, int M, int8_t* xq, float* sx,
                    uint16_t* mx, cudaStream_t st) {
    const Xchg* xc = static_cast<const Xchg*>(h);
    check_fused(xc, M, slice);
    const XchgArgs xa = xchg_args(xc, local, local_b, M, slice);
    RowArgs p{nullptr, nullptr, 0.0f, slice * xc->size, nullptr, xq, sx, mx, nullptr};
    launch_row<ROW_PLAIN, true>(p, M, queue_of(st), &xa);
}
// Measurement switch: the number of rows from which the one-CTA-per-row kernel is used (default 128; 0 = never).
void det_debug_set_rows(int min_rows) { g_row_wide_min = min_rows; }
void det_embed(const uint16_t* table_bf16, const int* ids, int M, int H, float* x, cudaStream_t st) {
    if (M <= 0) return;
    launch_pdl(k_embed_rows, dim3(M), dim3(256), 0, queue_of(st), 1, table_bf16, ids, H, x);
}
void det_add(float* x, const float* y, long long n, cudaStream_t st) {
    if (n <= 0) return;
    launch_pdl(k_residual_add, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, queue_of(st), 1, x, y, n);
}
void det_unshard(const float* tmp, float* full, int P, int M, int slice, cudaStream_t st) {
    const long long total = (long long)P * M * slice;
    if (total <= 0) return;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184);
    launch_pdl(k_unshard, dim3(blocks), dim3(256), 0, queue_of(st), 1, tmp, full, P, M, slice);
}
void det_argmax(const float* logits, int M, int V, int* out, cudaStream_t st) {
    if (M <= 0) return;
    if (M <= ARGMAX_SPLIT_ROWS && V >= 16384)
        launch_pdl(k_argmax_split, dim3(ARGMAX_SPLIT, M), dim3(256), 0, queue_of(st), 1, logits, V, out);
    else
        launch_pdl(k_argmax_rows, dim3(M), dim3(1024), 0, queue_of(st), 1, logits, V, out);
}

}  // extern "C"
