// Integer GEMM  y[t][n] = ((float)acc * c[n]) * sx[t],  acc = sum_g (m[n][g] * mx[t][g]) * sum_{k in g} wq[n][k] * xq[t][k]
// (docs/SPEC.md §3, spec/quant.rs:99-117).  Replaces kernels/cuda/gemm.cu behind det_gemm / det_gemm_ex.
//
// All sums are exact integers, so any split of K over lanes, warps or stages gives the same acc; the two fp32
// multiplies (and the optional residual add) run once per output element in the spec's order.
//
// Kernels here:
//   k_gemv_stream   decode (M <= 8 per pass): persistent warp-specialised CTAs.  One producer thread streams records of
//                   the repacked weight layout HBM -> shared memory with cp.async.bulk into a ring of stages guarded by
//                   mbarriers; consumer warps unpack 4/6/8-bit codes in registers from 128-bit shared loads and
//                   accumulate with dp4a.  HBM-bound: algorithmic bytes = N * (K*bits/8 + 4 + K/128*2).
//   k_repack_stream reference layout -> streaming layout (load time).
//   k_gemm_rowmajor any M on the reference row-major layout (fallback; one warp per output row, 8 tokens per pass).
#include "runtime.cuh"

namespace detb {

// ------------------------------------------------------------------------------------------------------------------
// Output routing shared by all kernels (Write / Accumulate / Parts of crates/det/src/backend.rs:136-142).
struct OutSpec {
    float* y;
    int N;
    int accumulate;
    int nparts;          // 0 or 1: plain y
    int offs[5];         // part i = columns [offs[i], offs[i+1])
    float* dsts[4];
};
__device__ __forceinline__ void emit(const OutSpec& o, int t, int n, float v) {
    if (o.nparts > 1) {
        int i = 0;
#pragma unroll
        for (int j = 1; j < 4; j++)
            if (j < o.nparts && n >= o.offs[j]) i = j;
        const int width = o.offs[i + 1] - o.offs[i];
        o.dsts[i][(size_t)t * width + (n - o.offs[i])] = v;
    } else {
        float* dst = o.y + (size_t)t * o.N + n;
        *dst = o.accumulate ? fadd(*dst, v) : v;
    }
}

__device__ __forceinline__ long long shfl_xor_i64(long long v, int off) {
    int lo = (int)(unsigned long long)v, hi = (int)((unsigned long long)v >> 32);
    lo = __shfl_xor_sync(FULL, lo, off);
    hi = __shfl_xor_sync(FULL, hi, off);
    return (long long)(((unsigned long long)(unsigned)hi << 32) | (unsigned)lo);
}

constexpr unsigned NIB = 0x0f0f0f0fu;   // low nibble of every byte
constexpr unsigned TOP2 = 0x30303030u;  // bits 4,5 of every byte

__host__ __device__ constexpr int code_offset(int bits) { return bits == 6 ? 32 : (bits == 4 ? 8 : 0); }
__host__ __device__ constexpr int bytes_per_32(int bits) { return bits == 8 ? 32 : (bits == 6 ? 24 : 16); }

// ------------------------------------------------------------------------------------------------------------------
// Reference layout: unpack one block of 32 codes (spec/quant.rs:62-97, quantize.rs:8-31) into eight words of four
// consecutive-k codes each.  W4 / W6 stay unsigned (code + offset); W8 is signed.
template <int BITS>
__device__ __forceinline__ void unpack_block32(const uint8_t* blk, unsigned (&o)[8]) {
    const unsigned* w = reinterpret_cast<const unsigned*>(blk);
    if (BITS == 8) {
#pragma unroll
        for (int i = 0; i < 8; i++) o[i] = __ldg(w + i);
    } else {
        unsigned q[4];
#pragma unroll
        for (int i = 0; i < 4; i++) q[i] = __ldg(w + i);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            o[i] = q[i] & NIB;
            o[i + 4] = (q[i] >> 4) & NIB;
        }
        if (BITS == 6) {
            const unsigned h0 = __ldg(w + 4), h1 = __ldg(w + 5);
            // code index c = 4*i + b sits in high-bit byte (c % 8), field (c / 8): word h[i & 1], field i >> 1
            o[0] |= (h0 << 4) & TOP2;
            o[1] |= (h1 << 4) & TOP2;
            o[2] |= (h0 << 2) & TOP2;
            o[3] |= (h1 << 2) & TOP2;
            o[4] |= h0 & TOP2;
            o[5] |= h1 & TOP2;
            o[6] |= (h0 >> 2) & TOP2;
            o[7] |= (h1 >> 2) & TOP2;
        }
    }
}

// Four byte products added to acc: signed x signed for W8, unsigned codes x signed activations for W4 / W6.
template <int BITS>
__device__ __forceinline__ int dot4(unsigned w, int x, int acc) {
    int r;
    if (BITS == 8) asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(x), "r"(acc));
    else asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(x), "r"(acc));
    return r;
}

// ------------------------------------------------------------------------------------------------------------------
// Fallback on the reference layout: one warp per output row, TM tokens per pass over the row.
template <int BITS, int TM>
__global__ void __launch_bounds__(256) k_gemm_rowmajor(const uint8_t* __restrict__ wq, const float* __restrict__ c,
                                                       const uint16_t* __restrict__ m, int N, int K,
                                                       const int8_t* __restrict__ xq, const float* __restrict__ sx,
                                                       const uint16_t* __restrict__ mx, int t0, int M, OutSpec out) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (n >= N) return;
    const int nblk = K >> 5, G = K >> 7;
    const uint8_t* row = wq + (size_t)n * nblk * bytes_per_32(BITS);
    long long acc[TM];
#pragma unroll
    for (int t = 0; t < TM; t++) acc[t] = 0;
    for (int b = lane; b < nblk; b += 32) {
        unsigned o[8];
        unpack_block32<BITS>(row + (size_t)b * bytes_per_32(BITS), o);
        const unsigned mw = __ldg(m + (size_t)n * G + (b >> 2));
#pragma unroll
        for (int t = 0; t < TM; t++) {
            if (t0 + t < M) {
                const int* xw = reinterpret_cast<const int*>(xq + (size_t)(t0 + t) * K + b * 32);
                int dot = 0, xs = 0;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int xv = __ldg(xw + i);
                    dot = dot4<BITS>(o[i], xv, dot);
                    if (BITS != 8) xs = __dp4a(xv, 0x01010101, xs);
                }
                dot -= code_offset(BITS) * xs;
                const unsigned mult = mw * (mx ? (unsigned)__ldg(mx + (size_t)(t0 + t) * G + (b >> 2)) : 1u);
                acc[t] += (long long)dot * (long long)mult;
            }
        }
    }
#pragma unroll
    for (int t = 0; t < TM; t++) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc[t] += shfl_xor_i64(acc[t], off);
    }
    if (lane == 0) {
        const float cn = c[n];
#pragma unroll
        for (int t = 0; t < TM; t++)
            if (t0 + t < M) emit(out, t0 + t, n, fmul(fmul(i64_to_f32(acc[t]), cn), sx[t0 + t]));
    }
}

// ------------------------------------------------------------------------------------------------------------------
// Streaming layout.  Rows are grouped four at a time into a record
//     [ codes row 0 | codes row 1 | codes row 2 | codes row 3 | c[4] fp32 | m[4][K/128] u16 | pad to 16 B ]
// and records are contiguous, so any run of records moves with ONE bulk copy.  Inside a row the codes are cut into
// units of 64 consecutive k (half a 128-group); a unit is NP = bits/2 pieces of 16 bytes, and piece p of unit u lives at
// byte (p * U + u) * 16 of the row (U = K / 64) so that neighbouring lanes, which own neighbouring units, read
// neighbouring 16-byte words of shared memory (no bank conflicts).
//   W8 unit: 64 signed bytes in k order (4 pieces).
//   W4 unit: words W[0..7]; byte b of W[i] = u[4i+b] | u[32+4i+b] << 4,  u = code + 8 (2 pieces).
//   W6 unit: words W[0..7] as W4 with the low nibbles of u = code + 32, then H[0..3]; byte b of H[j] holds, in bit
//            field f (bits 2f, 2f+1), the top two bits of u[4(j+4f) + b] (3 pieces).
// The consumer rebuilds sixteen words o[i] of four consecutive-k unsigned codes: o[i] = nibbles | shifted H field.
struct StreamGeom {
    int N, K, bits;
    int U;            // units per row
    int np;           // 16-byte pieces per unit
    int row_bytes;    // U * np * 16
    int G;
    int c_off;        // 4 * row_bytes
    int m_off;        // c_off + 16
    int rec_bytes;    // padded to 16
    int nrec;         // ceil(N / 4)
};
__host__ __device__ inline StreamGeom stream_geom(int N, int K, int bits) {
    StreamGeom g;
    g.N = N; g.K = K; g.bits = bits;
    g.U = K / 64;
    g.np = bits / 2;
    g.row_bytes = g.U * g.np * 16;
    g.G = K / 128;
    g.c_off = 4 * g.row_bytes;
    g.m_off = g.c_off + 16;
    g.rec_bytes = (g.m_off + 4 * g.G * 2 + 15) & ~15;
    g.nrec = (N + 3) / 4;
    return g;
}

// One thread per (row, unit): decode 64 codes from the reference layout, write the unit's pieces.
__global__ void k_repack_stream(const uint8_t* __restrict__ wq, const float* __restrict__ c,
                                const uint16_t* __restrict__ m, StreamGeom g, uint8_t* __restrict__ dst) {
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long rows_padded = (long long)g.nrec * 4;
    if (id >= rows_padded * g.U) return;
    const int n = (int)(id / g.U), u = (int)(id % g.U);
    uint8_t* rec = dst + (size_t)(n >> 2) * g.rec_bytes;
    uint8_t* row = rec + (size_t)(n & 3) * g.row_bytes;
    const bool live = n < g.N;
    uint8_t code[64];   // unsigned code (+offset) or raw signed byte for W8
    const int bp32 = bytes_per_32(g.bits);
    for (int h = 0; h < 2; h++) {
        const uint8_t* blk = wq + ((size_t)n * (g.K >> 5) + (size_t)(2 * u + h)) * bp32;
        for (int i = 0; i < 32; i++) {
            uint8_t v = 0;
            if (live) {
                if (g.bits == 8) v = blk[i];
                else {
                    const uint8_t lo = (i < 16) ? (blk[i] & 0xF) : (blk[i - 16] >> 4);
                    v = lo;
                    if (g.bits == 6) v |= ((blk[16 + (i & 7)] >> (2 * (i >> 3))) & 3) << 4;
                }
            }
            code[h * 32 + i] = v;
        }
    }
    uint8_t piece[64];
    if (g.bits == 8) {
        for (int i = 0; i < 64; i++) piece[i] = code[i];
    } else {
        for (int i = 0; i < 8; i++)
            for (int b = 0; b < 4; b++) piece[4 * i + b] = (code[4 * i + b] & 0xF) | ((code[32 + 4 * i + b] & 0xF) << 4);
        if (g.bits == 6)
            for (int j = 0; j < 4; j++)
                for (int b = 0; b < 4; b++) {
                    uint8_t v = 0;
                    for (int f = 0; f < 4; f++) v |= (code[4 * (j + 4 * f) + b] >> 4) << (2 * f);
                    piece[32 + 4 * j + b] = v;
                }
    }
    for (int p = 0; p < g.np; p++)
        *reinterpret_cast<uint4*>(row + ((size_t)p * g.U + u) * 16) = *reinterpret_cast<const uint4*>(piece + 16 * p);
    if (u == 0) {
        reinterpret_cast<float*>(rec + g.c_off)[n & 3] = live ? c[n] : 0.0f;
        uint16_t* mrow = reinterpret_cast<uint16_t*>(rec + g.m_off) + (n & 3) * g.G;
        for (int gi = 0; gi < g.G; gi++) mrow[gi] = live ? m[(size_t)n * g.G + gi] : (uint16_t)1;
    }
}

// ---- mbarrier / bulk-copy helpers (sm_90+ PTX; one CTA per cluster, so shared::cluster == shared::cta addresses)
__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: polls until the phase completes or about two seconds of SM clock have passed; returns false then.
constexpr long long WAIT_CYCLES = 4000000000ll;
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - start > WAIT_CYCLES) return false;
    }
}
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

constexpr int GEMV_CONSUMER_WARPS = 8;
constexpr int GEMV_THREADS = (GEMV_CONSUMER_WARPS + 1) * 32;
constexpr int GEMV_MAX_STAGES = 8;

struct GemvArgs {
    const uint8_t* w;         // streaming layout
    StreamGeom g;
    const int8_t* xq;         // [MT][K] rows t0 ..
    const float* sx;
    const uint16_t* mx;       // may be NULL
    int t0;                   // first token of this pass (for routing)
    int mt;                   // live tokens in this pass (<= MT)
    int rec_per_chunk;        // power of two, 1..16
    int stages;
    int stage_bytes;          // rec_per_chunk * rec_bytes
    int* error_flag;
    OutSpec out;
};

// Shared memory map: [stages x stage_bytes] [x pieces: MT*K] [xsum: MT*U int] [mx: MT*G u16 -> padded] [red] [barriers]
template <int BITS, int MT>
__global__ void __launch_bounds__(GEMV_THREADS, 1) k_gemv_stream(const GemvArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const StreamGeom& g = a.g;
    const int U = g.U, G = g.G;
    uint8_t* stage_base = smem;
    uint8_t* xs = stage_base + (size_t)a.stages * a.stage_bytes;                     // MT * K bytes, piece-transposed
    int* xsum = reinterpret_cast<int*>(xs + (size_t)MT * g.K);                       // MT * U
    unsigned* mxs = reinterpret_cast<unsigned*>(xsum + MT * U);                      // MT * G (as u32)
    long long* red = reinterpret_cast<long long*>(
        (reinterpret_cast<uintptr_t>(mxs + MT * G) + 15) & ~(uintptr_t)15);          // 2 * warps * MT
    unsigned long long* full = reinterpret_cast<unsigned long long*>(red + 2 * GEMV_CONSUMER_WARPS * MT);
    unsigned long long* empty = full + GEMV_MAX_STAGES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_chunks = (g.nrec + a.rec_per_chunk - 1) / a.rec_per_chunk;

    if (tid == 0) {
        for (int s = 0; s < a.stages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], GEMV_CONSUMER_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == GEMV_CONSUMER_WARPS) {
        // ---------------- producer: one elected thread keeps the ring full
        if (lane == 0) {
            bool ok = true;
            int issued = 0;
            for (int ch = blockIdx.x; ch < n_chunks && ok; ch += gridDim.x, issued++) {
                const int s = issued % a.stages;
                const unsigned round = (unsigned)(issued / a.stages);
                ok = mbar_wait(&empty[s], (round & 1u) ^ 1u);
                if (!ok) break;
                const int rec0 = ch * a.rec_per_chunk;
                const int nr = min(a.rec_per_chunk, g.nrec - rec0);
                const unsigned bytes = (unsigned)nr * (unsigned)g.rec_bytes;
                mbar_expect_tx(&full[s], bytes);
                bulk_g2s(stage_base + (size_t)s * a.stage_bytes, a.w + (size_t)rec0 * g.rec_bytes, bytes, &full[s]);
            }
            if (!ok) {
                atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
                // copies already issued still target this CTA's shared memory: wait (bounded) for each to land
                for (int k = 0; k < a.stages && k < issued; k++) {
                    const int i = issued - 1 - k;
                    (void)mbar_wait(&full[i % a.stages], (unsigned)(i / a.stages) & 1u);
                }
            }
        }
        return;
    }

    // ---------------- consumers: stage the activations once, then drain the ring
    {
        const int pieces_per_tok = g.K >> 4;
        const int total = MT * pieces_per_tok;
        const int span = GEMV_CONSUMER_WARPS * 32;
        for (int base = 0; base < total; base += span) {
            const int pid = base + tid;
            const bool live = pid < total;
            int t = 0, q = 0;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (live) {
                t = pid / pieces_per_tok;
                q = pid - t * pieces_per_tok;
                if (t < a.mt) v = *reinterpret_cast<const uint4*>(a.xq + (size_t)t * g.K + (size_t)q * 16);
                const int u = q >> 2, p = q & 3;
                *reinterpret_cast<uint4*>(xs + ((size_t)(t * 4 + p) * U + u) * 16) = v;
            }
            int s = __dp4a((int)v.x, 0x01010101, 0);
            s = __dp4a((int)v.y, 0x01010101, s);
            s = __dp4a((int)v.z, 0x01010101, s);
            s = __dp4a((int)v.w, 0x01010101, s);
            s += __shfl_xor_sync(FULL, s, 1);
            s += __shfl_xor_sync(FULL, s, 2);
            if (live && (q & 3) == 0) xsum[t * U + (q >> 2)] = s;
        }
        for (int i = tid; i < MT * G; i += span) {
            const int t = i / G;
            mxs[i] = (a.mx && t < a.mt) ? (unsigned)a.mx[(size_t)t * G + (i - t * G)] : 1u;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(GEMV_CONSUMER_WARPS * 32) : "memory");
    }

    const int R = a.rec_per_chunk * 4;                        // rows per chunk
    const int lpr = (GEMV_CONSUMER_WARPS * 32) / R;           // lanes per row: 4 .. 64
    const int r = tid / lpr, j = tid - r * lpr;
    const int rec_in_chunk = r >> 2, row_in_rec = r & 3;

    int consumed = 0;
    bool ok = true;
    for (int ch = blockIdx.x; ch < n_chunks; ch += gridDim.x, consumed++) {
        const int s = consumed % a.stages;
        const unsigned round = (unsigned)(consumed / a.stages);
        ok = mbar_wait(&full[s], round & 1u);
        if (!ok) break;
        const uint8_t* rec = stage_base + (size_t)s * a.stage_bytes + (size_t)rec_in_chunk * g.rec_bytes;
        const uint8_t* wrow = rec + (size_t)row_in_rec * g.row_bytes;
        const uint16_t* mrow = reinterpret_cast<const uint16_t*>(rec + g.m_off) + row_in_rec * G;
        const int n = (ch * a.rec_per_chunk + rec_in_chunk) * 4 + row_in_rec;

        long long acc[MT];
#pragma unroll
        for (int t = 0; t < MT; t++) acc[t] = 0;

        if (n < g.N) {
            for (int u = j; u < U; u += lpr) {
                unsigned o[16];
                if (BITS == 8) {
#pragma unroll
                    for (int p = 0; p < 4; p++) {
                        const uint4 v = *reinterpret_cast<const uint4*>(wrow + ((size_t)p * U + u) * 16);
                        o[4 * p] = v.x; o[4 * p + 1] = v.y; o[4 * p + 2] = v.z; o[4 * p + 3] = v.w;
                    }
                } else {
                    const uint4 w0 = *reinterpret_cast<const uint4*>(wrow + (size_t)u * 16);
                    const uint4 w1 = *reinterpret_cast<const uint4*>(wrow + ((size_t)U + u) * 16);
                    const unsigned w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        o[i] = w[i] & NIB;
                        o[i + 8] = (w[i] >> 4) & NIB;
                    }
                    if (BITS == 6) {
                        const uint4 hv = *reinterpret_cast<const uint4*>(wrow + ((size_t)2 * U + u) * 16);
                        const unsigned h[4] = {hv.x, hv.y, hv.z, hv.w};
#pragma unroll
                        for (int jj = 0; jj < 4; jj++) {
                            o[jj] |= (h[jj] << 4) & TOP2;
                            o[jj + 4] |= (h[jj] << 2) & TOP2;
                            o[jj + 8] |= h[jj] & TOP2;
                            o[jj + 12] |= (h[jj] >> 2) & TOP2;
                        }
                    }
                }
                const unsigned mw = mrow[u >> 1];
#pragma unroll
                for (int t = 0; t < MT; t++) {
                    int dot = 0;
#pragma unroll
                    for (int p = 0; p < 4; p++) {
                        const uint4 xv = *reinterpret_cast<const uint4*>(xs + ((size_t)(t * 4 + p) * U + u) * 16);
                        dot = dot4<BITS>(o[4 * p], (int)xv.x, dot);
                        dot = dot4<BITS>(o[4 * p + 1], (int)xv.y, dot);
                        dot = dot4<BITS>(o[4 * p + 2], (int)xv.z, dot);
                        dot = dot4<BITS>(o[4 * p + 3], (int)xv.w, dot);
                    }
                    if (BITS != 8) dot -= code_offset(BITS) * xsum[t * U + u];
                    const unsigned mult = mw * mxs[t * G + (u >> 1)];
                    acc[t] += (long long)dot * (long long)mult;
                }
            }
        }
        // this warp is done with the stage's bytes (c is read below, before the arrive)
        const float cn = reinterpret_cast<const float*>(rec + g.c_off)[row_in_rec];
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);

        // ---- reduce over the lanes of a row
        const int inwarp = lpr < 32 ? lpr : 32;
#pragma unroll
        for (int t = 0; t < MT; t++)
            for (int off = 1; off < inwarp; off <<= 1) acc[t] += shfl_xor_i64(acc[t], off);
        if (lpr > 32) {
            long long* rb = red + (size_t)(consumed & 1) * GEMV_CONSUMER_WARPS * MT;
            if (lane == 0) {
#pragma unroll
                for (int t = 0; t < MT; t++) rb[warp * MT + t] = acc[t];
            }
            asm volatile("bar.sync 1, %0;" ::"n"(GEMV_CONSUMER_WARPS * 32) : "memory");
            const int wpr = lpr >> 5;
            if (j == 0 && n < g.N) {
#pragma unroll
                for (int t = 0; t < MT; t++) {
                    long long sum = 0;
                    for (int k = 0; k < wpr; k++) sum += rb[(warp + k) * MT + t];
                    if (t < a.mt) emit(a.out, a.t0 + t, n, fmul(fmul(i64_to_f32(sum), cn), a.sx[t]));
                }
            }
        } else if (j == 0 && n < g.N) {
#pragma unroll
            for (int t = 0; t < MT; t++)
                if (t < a.mt) emit(a.out, a.t0 + t, n, fmul(fmul(i64_to_f32(acc[t]), cn), a.sx[t]));
        }
    }
    if (!ok && lane == 0) atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
}

// ------------------------------------------------------------------------------------------------------------------
// Host side

struct GemvPlan {
    int rec_per_chunk, stages, stage_bytes;
    size_t smem;
    int grid;
};
// Shape-only plan: stage size near 32 KB while leaving at least ~8 chunks per SM; ring as deep as shared memory allows.
static bool plan_gemv(const StreamGeom& g, int MT, GemvPlan& p) {
    const size_t budget = smem_optin() - 1024;
    const size_t fixed = (size_t)MT * g.K + (size_t)MT * g.U * 4 + (size_t)MT * g.G * 4 + 16 +
                         2 * GEMV_CONSUMER_WARPS * MT * 8 + 2 * GEMV_MAX_STAGES * 8;
    const int sms = sm_count();
    int rpc = 16;
    while (rpc > 1 && ((size_t)rpc * g.rec_bytes > 40 * 1024 || (g.nrec + rpc - 1) / rpc < 8 * sms)) rpc >>= 1;
    // rows per chunk may not exceed the consumer threads / 4 lanes
    p.rec_per_chunk = rpc;
    p.stage_bytes = rpc * g.rec_bytes;
    if (fixed + 2 * (size_t)p.stage_bytes > budget) return false;
    int stages = (int)((budget - fixed) / p.stage_bytes);
    if (stages > GEMV_MAX_STAGES) stages = GEMV_MAX_STAGES;
    p.stages = stages;
    p.smem = fixed + (size_t)stages * p.stage_bytes;
    const int n_chunks = (g.nrec + rpc - 1) / rpc;
    p.grid = n_chunks < sms ? n_chunks : sms;
    return true;
}

template <int BITS, int MT>
static void launch_gemv(const GemvArgs& a, const GemvPlan& p, cudaStream_t q) {
    static bool configured = false;
    if (!configured) {
        DETB_CUDA_OK(cudaFuncSetAttribute(k_gemv_stream<BITS, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)(smem_optin())));
        configured = true;
    }
    k_gemv_stream<BITS, MT><<<p.grid, GEMV_THREADS, p.smem, q>>>(a);
    DETB_CUDA_OK(cudaGetLastError());
}

template <int BITS>
static void gemv_stream_bits(const det_qlinear* L, const int8_t* xq, const float* sx, const uint16_t* mx, int M,
                             const OutSpec& out, cudaStream_t q) {
    const StreamGeom g = stream_geom(L->N, L->K, BITS);
    int t0 = 0;
    while (t0 < M) {
        int MT = (M - t0 >= 8) ? 8 : (M - t0 > 2 ? 4 : (M - t0 == 2 ? 2 : 1));
        if (M - t0 > 4 && M - t0 < 8) MT = 8;
        GemvPlan p;
        while (!plan_gemv(g, MT, p)) {
            DETB_REQUIRE(MT > 1, "K is too large for the streaming GEMV");
            MT >>= 1;
        }
        GemvArgs a;
        a.w = L->wq;
        a.g = g;
        a.xq = xq + (size_t)t0 * g.K;
        a.sx = sx + t0;
        a.mx = mx ? mx + (size_t)t0 * g.G : nullptr;
        a.t0 = t0;
        a.mt = (M - t0 < MT) ? (M - t0) : MT;
        a.rec_per_chunk = p.rec_per_chunk;
        a.stages = p.stages;
        a.stage_bytes = p.stage_bytes;
        a.error_flag = error_word();
        a.out = out;
        switch (MT) {
            case 1: launch_gemv<BITS, 1>(a, p, q); break;
            case 2: launch_gemv<BITS, 2>(a, p, q); break;
            case 4: launch_gemv<BITS, 4>(a, p, q); break;
            default: launch_gemv<BITS, 8>(a, p, q); break;
        }
        t0 += a.mt;
    }
}

template <int BITS>
static void gemm_rowmajor_bits(const det_qlinear* L, const int8_t* xq, const float* sx, const uint16_t* mx, int M,
                               const OutSpec& out, cudaStream_t q) {
    const unsigned grid = (unsigned)((L->N + 7) / 8);
    for (int t0 = 0; t0 < M; t0 += 8) {
        const int left = M - t0;
        if (left >= 5) k_gemm_rowmajor<BITS, 8><<<grid, 256, 0, q>>>(L->wq, L->c, L->m, L->N, L->K, xq, sx, mx, t0, M, out);
        else if (left >= 3) k_gemm_rowmajor<BITS, 4><<<grid, 256, 0, q>>>(L->wq, L->c, L->m, L->N, L->K, xq, sx, mx, t0, M, out);
        else if (left == 2) k_gemm_rowmajor<BITS, 2><<<grid, 256, 0, q>>>(L->wq, L->c, L->m, L->N, L->K, xq, sx, mx, t0, M, out);
        else k_gemm_rowmajor<BITS, 1><<<grid, 256, 0, q>>>(L->wq, L->c, L->m, L->N, L->K, xq, sx, mx, t0, M, out);
        DETB_CUDA_OK(cudaGetLastError());
    }
}

}  // namespace detb

using namespace detb;

extern "C" {

size_t det_linear_repack_bytes(int N, int K, int bits) {
    DETB_REQUIRE((bits == 4 || bits == 6 || bits == 8) && K > 0 && K % 128 == 0 && N > 0, "bad linear shape");
    const StreamGeom g = stream_geom(N, K, bits);
    return (size_t)g.nrec * g.rec_bytes;
}

void det_linear_repack(const det_qlinear* src, void* dst, cudaStream_t st) {
    DETB_REQUIRE((src->bits == 4 || src->bits == 6 || src->bits == 8) && src->K % 128 == 0, "bad linear shape");
    const StreamGeom g = stream_geom(src->N, src->K, src->bits);
    const long long work = (long long)g.nrec * 4 * g.U;
    k_repack_stream<<<(unsigned)((work + 127) / 128), 128, 0, queue_of(st)>>>(src->wq, src->c, src->m, g,
                                                                             (uint8_t*)dst);
    DETB_CUDA_OK(cudaGetLastError());
}

size_t det_gemm_scratch_bytes(int M, int K) { return (size_t)(M > 0 ? M : 1) * (size_t)(K / 128) * sizeof(int); }
void det_gemm_set_scratch(void* p, size_t bytes) { (void)p; (void)bytes; }

void det_gemm_ex(const det_qlinear* L, const int8_t* xq, const float* sx, const uint16_t* mx, int M, float* y,
                 int accumulate, int nparts, const int* offs, float* const* dsts, cudaStream_t st) {
    if (M <= 0) return;
    const int bits = L->bits & 0xff;
    const bool stream = (L->bits & DET_LAYOUT_STREAM) != 0;
    DETB_REQUIRE(bits == 4 || bits == 6 || bits == 8, "bits must be 4, 6 or 8");
    DETB_REQUIRE(L->K > 0 && L->K % 128 == 0 && L->N > 0, "K must be a positive multiple of 128");
    DETB_REQUIRE(nparts <= 4, "at most 4 fused parts");
    OutSpec out;
    out.y = y;
    out.N = L->N;
    out.accumulate = accumulate;
    out.nparts = nparts > 1 ? nparts : 0;
    for (int i = 0; i < 5; i++) out.offs[i] = L->N;
    for (int i = 0; i < 4; i++) out.dsts[i] = nullptr;
    if (nparts > 1) {
        DETB_REQUIRE(offs && dsts && offs[0] == 0, "fused parts need offs (offs[0] == 0) and dsts");
        for (int i = 0; i < nparts; i++) {
            out.offs[i] = offs[i];
            out.dsts[i] = dsts[i];
        }
    } else if (nparts == 1 && dsts && !y) {
        out.y = dsts[0];
    }
    cudaStream_t q = queue_of(st);
    if (stream) {
        if (bits == 8) gemv_stream_bits<8>(L, xq, sx, mx, M, out, q);
        else if (bits == 6) gemv_stream_bits<6>(L, xq, sx, mx, M, out, q);
        else gemv_stream_bits<4>(L, xq, sx, mx, M, out, q);
    } else {
        if (bits == 8) gemm_rowmajor_bits<8>(L, xq, sx, mx, M, out, q);
        else if (bits == 6) gemm_rowmajor_bits<6>(L, xq, sx, mx, M, out, q);
        else gemm_rowmajor_bits<4>(L, xq, sx, mx, M, out, q);
    }
}

void det_gemm(const det_qlinear* L, const int8_t* xq, const float* sx, const uint16_t* mx, int M, float* y,
              cudaStream_t st) {
    det_gemm_ex(L, xq, sx, mx, M, y, 0, 0, nullptr, nullptr, st);
}

}  // extern "C"
