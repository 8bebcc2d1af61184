// Decode GEMV (M <= 8 tokens per pass) on the streaming weight layout: the HBM-bound kernel of the token loop.
// Replaces the reference's k_decode (kernels/cuda/gemm.cu:201-337) with a B200 design:
//
//   * persistent CTAs (one per SM), warp-specialised: one producer thread streams weight records HBM -> shared memory
//     with cp.async.bulk into a ring of slots guarded by full/empty mbarriers; sixteen consumer warps each own whole
//     records, so consumers never synchronise with each other;
//   * a record holds TR complete output rows (TR chosen from K so a record is 8-20 KB); the 32 lanes of the owning warp
//     split into TR groups of 32/TR lanes, one group per row, and walk the row in units of 64 codes;
//   * codes are unpacked in registers from 128-bit shared loads (W6: 48 bytes per unit -> 16 words of four unsigned
//     codes), multiplied with dp4a against int8 activations staged once per CTA, and widened to int64 with the
//     group multiplier m * mx per unit;  sum(code * x) = sum(u * x) - offset * sum(x) for the unsigned W4/W6 codes.
//
// Algorithmic bytes per launch: N * (K*bits/8 + 4 + K/128*2) weights + M * (K + 4 + K/128*2) in + M * N * 4 out.
#include "gemm_common.cuh"

namespace detb {

// ------------------------------------------------------------------------------------------------------------------
// Streaming layout.  TR consecutive rows form a record
//     [ codes row 0 | ... | codes row TR-1 | c[TR] fp32 (padded to 16 B) | m[TR][K/128] u16 | pad to 16 B ]
// and records are contiguous.  Inside a row the codes are cut into units of 64 consecutive k (half a 128-group); a unit
// is NP = bits/2 pieces of 16 bytes, and piece p of unit u lives at byte (p * U + u) * 16 of the row (U = K / 64), so
// lanes that own neighbouring units read neighbouring 16-byte words of shared memory (no bank conflicts).
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
    int TR;           // rows per record: 1, 2, 4 or 8
    int c_off;        // TR * row_bytes
    int m_off;
    int rec_bytes;    // padded to 16
    int nrec;         // ceil(N / TR)
};
__host__ __device__ inline StreamGeom stream_geom(int N, int K, int bits) {
    StreamGeom g;
    g.N = N; g.K = K; g.bits = bits;
    g.U = K / 64;
    g.np = bits / 2;
    g.row_bytes = g.U * g.np * 16;
    g.G = K / 128;
    int tr = 8;
    while (tr > 1 && tr * g.row_bytes > 20 * 1024) tr >>= 1;   // a function of (K, bits) only
    g.TR = tr;
    g.c_off = tr * g.row_bytes;
    g.m_off = g.c_off + (tr * 4 + 15) / 16 * 16;
    g.rec_bytes = (g.m_off + tr * g.G * 2 + 15) & ~15;
    g.nrec = (N + tr - 1) / tr;
    return g;
}

// One thread per (row, unit): decode 64 codes from the reference layout (spec/quant.rs:62-97), write the unit's pieces.
__global__ void k_repack_stream(const uint8_t* __restrict__ wq, const float* __restrict__ c,
                                const uint16_t* __restrict__ m, StreamGeom g, uint8_t* __restrict__ dst) {
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long rows_padded = (long long)g.nrec * g.TR;
    if (id >= rows_padded * g.U) return;
    const int n = (int)(id / g.U), u = (int)(id % g.U);
    const int rr = n % g.TR;
    uint8_t* rec = dst + (size_t)(n / g.TR) * g.rec_bytes;
    uint8_t* row = rec + (size_t)rr * g.row_bytes;
    const bool live = n < g.N;
    __align__(16) uint8_t code[64];   // unsigned code (+offset), or the raw signed byte for W8
    const int bp32 = bytes_per_32(g.bits);
    for (int h = 0; h < 2; h++) {
        const uint8_t* blk = wq + ((size_t)n * (g.K >> 5) + (size_t)(2 * u + h)) * bp32;
        for (int i = 0; i < 32; i++) {
            uint8_t v = 0;
            if (live) {
                if (g.bits == 8) v = blk[i];
                else {
                    v = (i < 16) ? (blk[i] & 0xF) : (blk[i - 16] >> 4);
                    if (g.bits == 6) v |= ((blk[16 + (i & 7)] >> (2 * (i >> 3))) & 3) << 4;
                }
            }
            code[h * 32 + i] = v;
        }
    }
    __align__(16) uint8_t piece[64];
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
        reinterpret_cast<float*>(rec + g.c_off)[rr] = live ? c[n] : 0.0f;
        uint16_t* mrow = reinterpret_cast<uint16_t*>(rec + g.m_off) + rr * g.G;
        for (int gi = 0; gi < g.G; gi++) mrow[gi] = live ? m[(size_t)n * g.G + gi] : (uint16_t)1;
    }
}

// ------------------------------------------------------------------------------------------------------------------
constexpr int NCW = 16;                          // consumer warps
constexpr int GEMV_THREADS = (NCW + 1) * 32;     // + one producer warp
constexpr int MAX_SLOTS = 24;

struct GemvArgs {
    const uint8_t* w;         // streaming layout
    StreamGeom g;
    const int8_t* xq;         // rows of this pass
    const float* sx;
    const uint16_t* mx;       // may be NULL
    int t0;                   // first token of this pass (for routing)
    int mt;                   // live tokens in this pass (<= MT)
    int slots;                // ring depth, a multiple of `workers`
    int workers;              // consumer warps that take records (<= NCW); warp w owns slots w, w + workers, ...
    int* error_flag;
    OutSpec out;
    // Fused activation prologue (k_gemv_stream<.., FUSED = true>): the rows are produced from fp32 inputs inside the
    // kernel — the op sequences of RMSNorm + quant_act_i8g, plain quant_act_i8g or SwiGLU + quant_act_i8g — instead of
    // being read as codes.  CTA 0 also stores the codes / scale / multipliers for later consumers when asked to.
    int pro;                  // PRO_RMS, PRO_PLAIN, PRO_SWIGLU
    const float* pa;          // x, or the gate rows
    const float* pb;          // norm weight, or the up rows
    float eps;
    int pslices;              // next power of two >= K, over 128
    int8_t* xq_out;
    float* sx_out;
    uint16_t* mx_out;
};
enum : int { PRO_RMS = 1, PRO_PLAIN = 2, PRO_SWIGLU = 3 };
constexpr int FUSED_MAX_ROUNDS = 9;   // slices per consumer warp: K <= 9 * 16 * 128 = 18432

// Sixteen words of four consecutive-k codes from one unit; `pu` is the byte distance between pieces (U * 16).
template <int BITS>
__device__ __forceinline__ void unpack_unit(const uint8_t* wp, int pu, unsigned (&o)[16]) {
    if (BITS == 8) {
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const uint4 v = *reinterpret_cast<const uint4*>(wp + (size_t)p * pu);
            o[4 * p] = v.x; o[4 * p + 1] = v.y; o[4 * p + 2] = v.z; o[4 * p + 3] = v.w;
        }
    } else {
        const uint4 w0 = *reinterpret_cast<const uint4*>(wp);
        const uint4 w1 = *reinterpret_cast<const uint4*>(wp + pu);
        const unsigned w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; i++) {
            o[i] = w[i] & NIB;
            o[i + 8] = (w[i] >> 4) & NIB;
        }
        if (BITS == 6) {
            const uint4 hv = *reinterpret_cast<const uint4*>(wp + 2 * (size_t)pu);
            const unsigned h[4] = {hv.x, hv.y, hv.z, hv.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                o[j] |= (h[j] << 4) & TOP2;
                o[j + 4] |= (h[j] << 2) & TOP2;
                o[j + 8] |= h[j] & TOP2;
                o[j + 12] |= (h[j] >> 2) & TOP2;
            }
        }
    }
}


// Produces the int8 rows of this pass from fp32 inputs, straight into the staged (piece-transposed) layout.
// One warp owns one 128-wide slice at a time, 4 consecutive values per lane, values held in registers between phases;
// the row-wide sum of squares is the spec tree (slice sums are aligned subtrees; every warp finishes the same tree over
// them), the row-wide maximum is order-free.  Same fp32 operation sequence as k_row in glue.cu.
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory"); }

__device__ void fused_stage(const GemvArgs& a, uint8_t* xs, int2* xmeta, float* slice_sum, float* wmax, float* sxs) {
    const StreamGeom& g = a.g;
    const int K = g.K, U = g.U, G = g.G;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool keep = blockIdx.x == 0 && a.xq_out != nullptr;
    for (int t = 0; t < a.mt; t++) {
        const float* pa = a.pa + (size_t)t * K;
        const float* pb = a.pro == PRO_SWIGLU ? a.pb + (size_t)t * K : a.pb;
        float v[FUSED_MAX_ROUNDS][4];
#pragma unroll
        for (int r = 0; r < FUSED_MAX_ROUNDS; r++) {
            const int s = warp + r * NCW;
            float4 x4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (s < G) x4 = *reinterpret_cast<const float4*>(pa + s * 128 + lane * 4);
            v[r][0] = x4.x; v[r][1] = x4.y; v[r][2] = x4.z; v[r][3] = x4.w;
        }
        float inv_rms = 0.0f;
        if (a.pro == PRO_RMS) {
#pragma unroll
            for (int r = 0; r < FUSED_MAX_ROUNDS; r++) {
                const int s = warp + r * NCW;
                float sq[4];
#pragma unroll
                for (int e = 0; e < 4; e++) sq[e] = fmul(v[r][e], v[r][e]);
                const float ssum = fold_lanes<32>(fold_run<4>(sq));
                if (lane == 0 && s < G) slice_sum[s] = ssum;
            }
            for (int i = G + tid; i < a.pslices; i += NCW * 32) slice_sum[i] = 0.0f;
            consumer_barrier();
            float tot;
            if (a.pslices >= 32) {
                const int per = a.pslices >> 5;   // 1, 2, 4 or 8
                float w8[8];
#pragma unroll
                for (int i = 0; i < 8; i++) w8[i] = i < per ? slice_sum[lane * per + i] : 0.0f;
#pragma unroll
                for (int step = 1; step < 8; step <<= 1) {
#pragma unroll
                    for (int i = 0; i < 8; i += 2 * step)
                        if (step < per) w8[i] = fadd(w8[i], w8[i + step]);
                }
                tot = fold_lanes<32>(w8[0]);
            } else {
                float w1 = lane < a.pslices ? slice_sum[lane] : 0.0f;
                for (int off = 1; off < a.pslices; off <<= 1) w1 = fadd(w1, __shfl_xor_sync(FULL, w1, off));
                tot = __shfl_sync(FULL, w1, 0);
            }
            inv_rms = fdiv(1.0f, fsqrt(fadd(fdiv(tot, (float)K), a.eps)));
        }
        float s_slice[FUSED_MAX_ROUNDS];
        float local_max = 0.0f;
#pragma unroll
        for (int r = 0; r < FUSED_MAX_ROUNDS; r++) {
            const int s = warp + r * NCW;
            s_slice[r] = 0.0f;
            if (s < G) {
                float amax = 0.0f;
                float4 b4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (a.pro != PRO_PLAIN) b4 = *reinterpret_cast<const float4*>(pb + s * 128 + lane * 4);
                const float bb[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    float val = v[r][e];
                    if (a.pro == PRO_RMS) val = fmul(fmul(val, inv_rms), bb[e]);
                    else if (a.pro == PRO_SWIGLU) val = fmul(silu_f(val), bb[e]);
                    v[r][e] = val;
                    amax = fmaxf(amax, fabsf(val));
                }
                amax = max_lanes(amax);
                s_slice[r] = fdiv(amax, 127.0f);
                local_max = fmaxf(local_max, s_slice[r]);
            }
        }
        if (lane == 0) wmax[warp] = local_max;
        consumer_barrier();
        float top = 0.0f;
#pragma unroll
        for (int w = 0; w < NCW; w++) top = fmaxf(top, wmax[w]);
        const float sx = (top == 0.0f) ? 1.0f : fdiv(top, 65535.0f);
        if (tid == 0) {
            sxs[t] = sx;
            if (keep) a.sx_out[t] = sx;
        }
#pragma unroll
        for (int r = 0; r < FUSED_MAX_ROUNDS; r++) {
            const int s = warp + r * NCW;
            if (s < G) {
                const unsigned mult = group_mult(s_slice[r], sx);
                const float inv = fdiv(1.0f, fmul(sx, (float)mult));
                unsigned word = (unsigned)(quant_code(v[r][0], inv) & 0xff);
                word |= (unsigned)(quant_code(v[r][1], inv) & 0xff) << 8;
                word |= (unsigned)(quant_code(v[r][2], inv) & 0xff) << 16;
                word |= (unsigned)(quant_code(v[r][3], inv) & 0xff) << 24;
                // value index e = s * 128 + lane * 4: unit 2s + lane / 16, piece (lane % 16) / 4, word lane % 4
                const int u = 2 * s + (lane >> 4), pc = (lane & 15) >> 2;
                *reinterpret_cast<unsigned*>(xs + ((size_t)(t * 4 + pc) * U + u) * 16 + (lane & 3) * 4) = word;
                int sum = __dp4a((int)word, 0x01010101, 0);
#pragma unroll
                for (int off = 1; off < 16; off <<= 1) sum += __shfl_xor_sync(FULL, sum, off);
                if ((lane & 15) == 0) xmeta[t * U + u] = make_int2(sum, (int)mult);
                if (keep) {
                    *reinterpret_cast<unsigned*>(a.xq_out + (size_t)t * K + s * 128 + lane * 4) = word;
                    if (lane == 0) a.mx_out[(size_t)t * G + s] = (uint16_t)mult;
                }
            }
        }
        consumer_barrier();
    }
}

// Shared memory: [slots x rec_bytes] [x pieces: MT*K] [xmeta: MT*U int2 = (sum of x over the unit, mx of its group)]
//                [full[MAX_SLOTS]] [empty[MAX_SLOTS]] [slice sums: 256 f32] [warp maxima: NCW f32] [row scales: 8 f32]
template <int BITS, int MT, bool FUSED>
__global__ void __launch_bounds__(GEMV_THREADS, 1) k_gemv_stream(const GemvArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const StreamGeom& g = a.g;
    const int U = g.U, G = g.G;
    uint8_t* ring = smem;
    uint8_t* xs = ring + (size_t)a.slots * g.rec_bytes;
    int2* xmeta = reinterpret_cast<int2*>(xs + (size_t)MT * g.K);
    unsigned long long* full = reinterpret_cast<unsigned long long*>(xmeta + MT * U);
    unsigned long long* empty = full + MAX_SLOTS;
    float* slice_sum = reinterpret_cast<float*>(empty + MAX_SLOTS);
    float* wmax = slice_sum + 256;
    float* sxs = wmax + NCW;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const long long wl = wait_limit(a.error_flag);
    pdl_trigger();
    if (tid == 0) {
        for (int s = 0; s < a.slots; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == NCW) {
        // ---------------- producer: one thread keeps the ring full; weights do not depend on earlier kernels
        if (lane == 0) {
            bool ok = true;
            int issued = 0;
            for (int rec = blockIdx.x; rec < g.nrec; rec += gridDim.x, issued++) {
                const int s = issued % a.slots;
                ok = mbar_wait(&empty[s], ((unsigned)(issued / a.slots) & 1u) ^ 1u, wl);
                if (!ok) break;
                mbar_expect_tx(&full[s], (unsigned)g.rec_bytes);
                bulk_g2s(ring + (size_t)s * g.rec_bytes, a.w + (size_t)rec * g.rec_bytes, (unsigned)g.rec_bytes, &full[s]);
            }
            if (!ok) {
                atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
                // copies already issued still target this CTA's shared memory: wait (bounded) for each to land
                for (int k = 0; k < a.slots && k < issued; k++) {
                    const int i = issued - 1 - k;
                    (void)mbar_wait(&full[i % a.slots], (unsigned)(i / a.slots) & 1u, wl);
                }
            }
        }
        return;
    }

    // ---------------- consumers: stage the activations once (piece-transposed like the weights), then drain records.
    // The activations (and the output rows) belong to earlier kernels: wait for them here, while the producer is
    // already pulling weights.
    pdl_wait();
    if (FUSED) {
        fused_stage(a, xs, xmeta, slice_sum, wmax, sxs);
    } else {
        const int pieces_per_tok = g.K >> 4;
        const int total = MT * pieces_per_tok;
        for (int base = 0; base < total; base += NCW * 32) {
            const int pid = base + tid;
            const bool live = pid < total;
            int t = 0, q = 0;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (live) {
                t = pid / pieces_per_tok;
                q = pid - t * pieces_per_tok;
                if (t < a.mt) v = *reinterpret_cast<const uint4*>(a.xq + (size_t)t * g.K + (size_t)q * 16);
                *reinterpret_cast<uint4*>(xs + ((size_t)(t * 4 + (q & 3)) * U + (q >> 2)) * 16) = v;
            }
            int s = __dp4a((int)v.x, 0x01010101, 0);
            s = __dp4a((int)v.y, 0x01010101, s);
            s = __dp4a((int)v.z, 0x01010101, s);
            s = __dp4a((int)v.w, 0x01010101, s);
            s += __shfl_xor_sync(FULL, s, 1);
            s += __shfl_xor_sync(FULL, s, 2);
            if (live && (q & 3) == 0) {
                const int u = q >> 2;
                const int mxv = (a.mx && t < a.mt) ? (int)a.mx[(size_t)t * G + (u >> 1)] : 1;
                xmeta[t * U + u] = make_int2(s, mxv);
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
    }

    // Record i of this CTA lands in slot i % slots and belongs to warp i % workers.  slots is a multiple of workers, so
    // a warp meets the phases of each of its slots strictly in order (a parity wait can tell only two phases apart).
    if (warp >= a.workers) return;
    float sxr[MT];                               // row scales, fetched once (not once per record)
#pragma unroll
    for (int t = 0; t < MT; t++) sxr[t] = FUSED ? sxs[t] : (t < a.mt ? a.sx[t] : 0.0f);
    const int lpr = 32 / g.TR;                   // lanes per row
    const int r = lane / lpr, j = lane - r * lpr;
    const int pu = U * 16;
    bool ok = true;
    for (int i = warp;; i += a.workers) {
        const int rec_id = blockIdx.x + i * gridDim.x;   // i-th record of this CTA
        if (rec_id >= g.nrec) break;
        const int s = i % a.slots;
        ok = mbar_wait(&full[s], (unsigned)(i / a.slots) & 1u, wl);
        if (!ok) break;
        const uint8_t* rec = ring + (size_t)s * g.rec_bytes;
        const uint8_t* wp = rec + (size_t)r * g.row_bytes + j * 16;
        const uint8_t* xp = xs + j * 16;
        const uint16_t* mrow = reinterpret_cast<const uint16_t*>(rec + g.m_off) + r * G;
        const int n = rec_id * g.TR + r;

        long long acc[MT];
#pragma unroll
        for (int t = 0; t < MT; t++) acc[t] = 0;
        for (int u = j; u < U; u += lpr, wp += lpr * 16, xp += lpr * 16) {
            unsigned o[16];
            unpack_unit<BITS>(wp, pu, o);
            const unsigned mw = mrow[u >> 1];
#pragma unroll
            for (int t = 0; t < MT; t++) {
                int d0 = 0, d1 = 0, d2 = 0, d3 = 0;   // independent chains, summed below
                const uint8_t* xt = xp + (size_t)t * 4 * pu;
                const uint4 x0 = *reinterpret_cast<const uint4*>(xt);
                const uint4 x1 = *reinterpret_cast<const uint4*>(xt + pu);
                const uint4 x2 = *reinterpret_cast<const uint4*>(xt + 2 * (size_t)pu);
                const uint4 x3 = *reinterpret_cast<const uint4*>(xt + 3 * (size_t)pu);
                d0 = dot4<BITS>(o[0], (int)x0.x, d0); d1 = dot4<BITS>(o[1], (int)x0.y, d1);
                d2 = dot4<BITS>(o[2], (int)x0.z, d2); d3 = dot4<BITS>(o[3], (int)x0.w, d3);
                d0 = dot4<BITS>(o[4], (int)x1.x, d0); d1 = dot4<BITS>(o[5], (int)x1.y, d1);
                d2 = dot4<BITS>(o[6], (int)x1.z, d2); d3 = dot4<BITS>(o[7], (int)x1.w, d3);
                d0 = dot4<BITS>(o[8], (int)x2.x, d0); d1 = dot4<BITS>(o[9], (int)x2.y, d1);
                d2 = dot4<BITS>(o[10], (int)x2.z, d2); d3 = dot4<BITS>(o[11], (int)x2.w, d3);
                d0 = dot4<BITS>(o[12], (int)x3.x, d0); d1 = dot4<BITS>(o[13], (int)x3.y, d1);
                d2 = dot4<BITS>(o[14], (int)x3.z, d2); d3 = dot4<BITS>(o[15], (int)x3.w, d3);
                const int2 meta = xmeta[t * U + u];
                int dot = (d0 + d1) + (d2 + d3);
                if (BITS != 8) dot -= code_offset(BITS) * meta.x;
                const unsigned mult = mw * (unsigned)meta.y;
                acc[t] += (long long)dot * (long long)mult;
            }
        }
        const float cn = reinterpret_cast<const float*>(rec + g.c_off)[r];
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);   // the slot may be refilled

#pragma unroll
        for (int t = 0; t < MT; t++)
            for (int off = 1; off < lpr; off <<= 1) acc[t] += shfl_xor_i64(acc[t], off);
        if (j == 0 && n < g.N) {
#pragma unroll
            for (int t = 0; t < MT; t++)
                if (t < a.mt) emit(a.out, a.t0 + t, n, fmul(fmul(i64_to_f32(acc[t]), cn), sxr[t]));
        }
    }
    if (!ok && lane == 0) atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
}

// ------------------------------------------------------------------------------------------------------------------
struct GemvPlan {
    int slots, workers;
    size_t smem;
    int grid;
};
// A plan by shape only: the ring takes whatever shared memory the staged activations leave, up to MAX_SLOTS records.
static bool plan_gemv(const StreamGeom& g, int MT, GemvPlan& p) {
    const size_t budget = smem_optin() - 1024;
    const size_t fixed = (size_t)MT * g.K + (size_t)MT * g.U * 8 + 2 * MAX_SLOTS * 8 + (256 + NCW + 8) * 4;
    if (fixed + 2 * (size_t)g.rec_bytes > budget) return false;
    int slots = (int)((budget - fixed) / g.rec_bytes);
    if (slots > MAX_SLOTS) slots = MAX_SLOTS;
    p.workers = slots < NCW ? slots : NCW;
    slots -= slots % p.workers;
    p.slots = slots;
    p.smem = fixed + (size_t)slots * g.rec_bytes;
    const int sms = sm_count();
    p.grid = g.nrec < sms ? g.nrec : sms;
    return true;
}

template <int BITS, int MT, bool FUSED>
static void launch_gemv_one(const GemvArgs& a, const GemvPlan& p, cudaStream_t q) {
    static bool configured = false;
    if (!configured) {
        DETB_CUDA_OK(cudaFuncSetAttribute(k_gemv_stream<BITS, MT, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)(smem_optin())));
        configured = true;
    }
    launch_pdl(k_gemv_stream<BITS, MT, FUSED>, dim3(p.grid), dim3(GEMV_THREADS), p.smem, q, 1, a);
}
template <int BITS, int MT>
static void launch_gemv(const GemvArgs& a, const GemvPlan& p, cudaStream_t q) {
    if (a.pro) launch_gemv_one<BITS, MT, true>(a, p, q);
    else launch_gemv_one<BITS, MT, false>(a, p, q);
}

template <int BITS>
static void gemv_stream_bits(const det_qlinear* L, const int8_t* xq, const float* sx, const uint16_t* mx, int M,
                             const OutSpec& out, cudaStream_t q, const det_act_source* src) {
    const StreamGeom g = stream_geom(L->N, L->K, BITS);
    int t0 = 0;
    while (t0 < M) {
        const int left = M - t0;
        int MT = left >= 5 ? 8 : (left >= 3 ? 4 : left);
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
        a.mt = left < MT ? left : MT;
        a.slots = p.slots;
        a.workers = p.workers;
        a.error_flag = error_word();
        a.out = out;
        a.pro = 0;
        if (src) {
            DETB_REQUIRE(g.G <= FUSED_MAX_ROUNDS * NCW, "K is too large for the fused activation prologue");
            a.pro = src->kind;
            a.pa = src->a + (size_t)t0 * g.K;
            a.pb = src->kind == PRO_SWIGLU ? src->b + (size_t)t0 * g.K : src->b;
            a.eps = src->eps;
            int P = 128;
            while (P < g.K) P <<= 1;
            a.pslices = P / 128;
            a.xq_out = src->xq ? src->xq + (size_t)t0 * g.K : nullptr;
            a.sx_out = src->sx ? src->sx + t0 : nullptr;
            a.mx_out = src->mx ? src->mx + (size_t)t0 * g.G : nullptr;
        }
        switch (MT) {
            case 1: launch_gemv<BITS, 1>(a, p, q); break;
            case 2: launch_gemv<BITS, 2>(a, p, q); break;
            case 4: launch_gemv<BITS, 4>(a, p, q); break;
            default: launch_gemv<BITS, 8>(a, p, q); break;
        }
        t0 += a.mt;
    }
}

void gemv_stream_launch(const det_qlinear* L, int bits, const int8_t* xq, const float* sx, const uint16_t* mx, int M,
                        const OutSpec& out, cudaStream_t q, const det_act_source* src) {
    if (src) {
        DETB_REQUIRE(src->kind >= PRO_RMS && src->kind <= PRO_SWIGLU && src->a, "bad activation source");
        DETB_REQUIRE((src->xq != nullptr) == (src->sx != nullptr) && (src->xq != nullptr) == (src->mx != nullptr),
                     "the quantized-row outputs come all together or not at all");
    }
    if (bits == 8) gemv_stream_bits<8>(L, xq, sx, mx, M, out, q, src);
    else if (bits == 6) gemv_stream_bits<6>(L, xq, sx, mx, M, out, q, src);
    else gemv_stream_bits<4>(L, xq, sx, mx, M, out, q, src);
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
    const long long work = (long long)g.nrec * g.TR * g.U;
    k_repack_stream<<<(unsigned)((work + 127) / 128), 128, 0, queue_of(st)>>>(src->wq, src->c, src->m, g,
                                                                             (uint8_t*)dst);
    DETB_CUDA_OK(cudaGetLastError());
}

}  // extern "C"
