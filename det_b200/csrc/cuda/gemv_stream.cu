// Decode GEMV (M <= 8 tokens per pass) on the streaming weight layout: the HBM-bound kernel of the token loop.
// Replaces the reference's k_decode (kernels/cuda/gemm.cu:201-337) with a B200 design:
//
//   * persistent CTAs of sixteen worker warps.  A warp owns whole groups of four output rows and a private set of
//     shared-memory slots: it streams its own weight records HBM -> shared memory with cp.async.bulk (one elected lane
//     issues the copy of record i + SPW into the slot the warp has just finished reading, so no "empty" barrier and no
//     producer thread is needed) and waits on one mbarrier per slot, so warps never synchronise with each other;
//   * one CTA per SM with up to 150 KB of weight records in flight; with programmatic dependent launch every warp
//     requests its first records before it waits for the kernel's predecessor, so the slots fill while the row operation
//     in front of the GEMV (or its own prologue) still runs;
//   * a record is a 1024-wide K chunk of four rows: the 32 lanes of the owning warp are 4 rows x 8 lanes, and a lane
//     walks one whole 128-group of its row per record — unsigned codes unpacked in registers from 128-bit shared loads,
//     dp4a against int8 activations staged once per CTA, ONE exact 64-bit multiply-add per group;
//   * the activation quantization that feeds the GEMV (RMSNorm + quant_act_i8g, or plain quant_act_i8g) can run as the
//     kernel's prologue while the ring fills (the reference runs it as a separate kernel, qwen35.rs:33, 62, 121), a second
//     small W8 linear reading the same row (the GDN a|b projection) can ride in the same launch, and a gate|up linear
//     stored with interleaved rows can emit the SwiGLU product silu_f(gate) * up from its epilogue.
//
// Algorithmic bytes per launch: N * (K*bits/8 + 4 + K/128*2) weights + M * (K + 4 + K/128*2) in + M * N * 4 out.
#include "gemm_common.cuh"
#include "exchange.cuh"

namespace detb {

// ------------------------------------------------------------------------------------------------------------------
// Streaming layout.  Four consecutive rows ("quad") x one K chunk of UC units (a unit = 64 consecutive k = half a
// 128-group; UC = 16, or 8 when K is an odd multiple of 512) form one record
//     [ row 0: pieces | row 1 | row 2 | row 3 | m[4][UC/2] u16 ]                      (16-byte aligned)
// and the records of a quad follow each other in K order, quads in row order.  A unit is NP = bits/2 pieces of 16 bytes;
// piece pp of physical unit p of row r lives at byte ((r * NP + pp) * UC + p) * 16, so the 8 lanes of a row read
// neighbouring 16-byte words (no bank conflicts).  With UC = 16 the units of a chunk are stored permuted — physical unit
// p is logical unit (p & 7) * 2 + (p >> 3) — so that lane j, which reads physical units j and j + 8, owns exactly the
// group j of the chunk.  c stays in its own array (one load per row).
//   W8 unit: 64 signed bytes in k order (4 pieces).
//   W4 unit: words W[0..7]; byte b of W[i] = u[4i+b] | u[32+4i+b] << 4,  u = code + 8 (2 pieces).
//   W6 unit: words W[0..7] as W4 with the low nibbles of u = code + 32, then H[0..3]; byte b of H[j] holds, in bit
//            field f (bits 2f, 2f+1), the top two bits of u[4(j+4f) + b] (3 pieces).
// The consumer rebuilds sixteen words o[i] of four consecutive-k unsigned codes: o[i] = nibbles | shifted H field.
// Pairs layout (DET_LAYOUT_PAIRS): physical row 2i is row i of the linear's first half (gate), row 2i+1 row i of its
// second half (up), so a quad holds two complete (gate, up) pairs.
constexpr int QR = 4;     // rows per record
constexpr int LPR = 8;    // lanes per row

struct StreamGeom {
    int N, K, bits;
    int U, G, np;
    int UC;            // units per chunk
    int NCH;           // chunks per row
    int m_off;         // QR * np * UC * 16
    int rec_bytes;
    int nquads;
};
__host__ __device__ inline StreamGeom stream_geom(int N, int K, int bits) {
    StreamGeom g;
    g.N = N; g.K = K; g.bits = bits;
    g.U = K / 64;
    g.G = K / 128;
    g.np = bits / 2;
    g.UC = (g.U % 16 != 0 && g.U % 8 == 0) ? 8 : 16;     // a function of K only
    g.NCH = (g.U + g.UC - 1) / g.UC;
    g.m_off = QR * g.np * g.UC * 16;
    g.rec_bytes = (g.m_off + QR * (g.UC / 2) * 2 + 15) & ~15;
    g.nquads = (N + QR - 1) / QR;
    return g;
}
__host__ __device__ inline int phys_unit(int UC, int l) { return UC == 16 ? (l >> 1) + (l & 1) * 8 : l; }

// One thread per (padded row, unit slot of the padded K): decode 64 codes from the reference layout
// (spec/quant.rs:62-97), write the unit's pieces.  Padding (rows past N, units past K) holds the code of value 0.
__global__ void k_repack_stream(const uint8_t* __restrict__ wq, const uint16_t* __restrict__ m, StreamGeom g, int pairs,
                                uint8_t* __restrict__ dst) {
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int slots = g.NCH * g.UC;
    if (id >= (long long)g.nquads * QR * slots) return;
    const int n = (int)(id / slots), lu = (int)(id % slots);
    const int r = n % QR, c = lu / g.UC, l = lu % g.UC;
    const int src_row = pairs ? ((n & 1) ? g.N / 2 + (n >> 1) : (n >> 1)) : n;
    const bool live = n < g.N && lu < g.U;
    uint8_t* rec = dst + ((size_t)(n / QR) * g.NCH + c) * g.rec_bytes;
    __align__(16) uint8_t code[64];   // unsigned code (+offset), or the raw signed byte for W8
    const int bp32 = bytes_per_32(g.bits);
    for (int h = 0; h < 2; h++) {
        const uint8_t* blk = live ? wq + ((size_t)src_row * (g.K >> 5) + (size_t)(2 * lu + h)) * bp32 : nullptr;
        for (int i = 0; i < 32; i++) {
            uint8_t v = (uint8_t)code_offset(g.bits);
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
    const int p = phys_unit(g.UC, l);
    for (int pp = 0; pp < g.np; pp++)
        *reinterpret_cast<uint4*>(rec + ((size_t)(r * g.np + pp) * g.UC + p) * 16) = *reinterpret_cast<const uint4*>(piece + 16 * pp);
    if ((l & 1) == 0)
        reinterpret_cast<uint16_t*>(rec + g.m_off)[r * (g.UC / 2) + (l >> 1)] = live ? m[(size_t)src_row * g.G + (lu >> 1)] : (uint16_t)1;
}

// ------------------------------------------------------------------------------------------------------------------
constexpr int NCW = 16;                          // warps per CTA
constexpr int GEMV_THREADS = NCW * 32;
constexpr int MAX_SPW = 5;                       // slots per worker warp
constexpr int MAX_SLOTS = MAX_SPW * NCW;
constexpr int RREG = 4;                          // 128-slices per warp kept in registers by the prologue

struct GemvSeg {
    const uint8_t* w;         // streaming layout
    const float* c;           // [N]
    int N, nquads, rec_bytes, m_off;
    OutSpec out;
};
struct GemvArgs {
    GemvSeg seg[2];           // seg[1] (DUAL instantiations only) is a W8 linear over the same input row
    int K, U, G, UC, NCH;
    int slot_bytes;
    const int8_t* xq;         // rows of this pass
    const float* sx;
    const uint16_t* mx;       // may be NULL
    int t0;                   // first token of this pass (for routing)
    int mt;                   // live tokens in this pass (<= MT)
    int spw;                  // slots per worker warp; warp w owns slots [w * spw, (w + 1) * spw)
    int workers;              // warps that take quads (<= NCW); the others only help staging the activations
    int* error_flag;
    // Activation prologue: the rows are produced from fp32 inputs inside the kernel — the op sequences of RMSNorm +
    // quant_act_i8g or plain quant_act_i8g — instead of being read as codes.  CTA 0 also stores the codes / scale /
    // multipliers for later consumers when asked to.
    int pro;                  // 0, PRO_RMS, PRO_PLAIN
    const float* pa;          // x
    const float* pb;          // norm weight
    float eps;
    int pslices;              // next power of two >= K, over 128
    int8_t* xq_out;
    float* sx_out;
    uint16_t* mx_out;
    // SwiGLU epilogue (seg[0] in the pairs layout): h[t][i] = silu_f(y[2i]) * y[2i+1] instead of y
    float* h;
    int h_width;
    // Group maxima handed from a SwiGLU epilogue to the prologue of the GEMV that quantizes h: word 0 of the buffer counts
    // the CTAs that have read the maxima; from word 4 on, eight words per (row t, group g) — at 4 + (t * groups + g) * 8 —
    // hold max |h| over an eighth of the group's values each, as fp32 bit patterns (non-negative floats order like their
    // bits, so an integer atomic maximum folds them; the maximum is order-free; eight cells per group keep the number of
    // atomics that meet on one address small).
    // The producer folds into them; the consumer reads them instead of scanning the row — which is what lets a row longer
    // than 8192 values go through the prologue — and its last CTA leaves them zero for the next producer.
    unsigned* h_amax;         // producer side (NULL: none)
    unsigned* pamax;          // consumer side (NULL: the prologue scans the row)
    // Tensor-parallel prologue: the fp32 rows are not read from `pa` but gathered from every rank's slice through the
    // packet exchange of exchange.cuh — every CTA pushes its share of this rank's slice, then polls the packets of the
    // rows it stages.  With acc_in the staged value is acc_in + gathered (the residual add; CTA 0 stores the sums to
    // acc_out, a different buffer: the other CTAs still read acc_in).
    int xchg;
    XchgArgs xa;
    const float* acc_in;
    float* acc_out;
};
enum : int { PRO_RMS = 1, PRO_PLAIN = 2 };

// Sixteen words of four consecutive-k codes from one unit; `pu` is the byte distance between pieces (UC * 16).
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

__device__ __forceinline__ void consumer_barrier() { __syncthreads(); }

// Where the 16-byte piece holding activation codes k0 .. k0+15 of token row t lives in the staged copy: the same chunk /
// piece / physical-unit order as the weights.
template <int UC>
__device__ __forceinline__ int stage_piece(int NCH, int t, int q /* piece index k0 / 16 */) {
    const int lu = q >> 2, pp = q & 3;
    const int c = lu / UC, l = lu % UC;
    return (((t * NCH + c) * 4 + pp) * UC + phys_unit(UC, l)) * 16;
}
template <int UC>
__device__ __forceinline__ int stage_unit(int NCH, int t, int lu) {
    const int c = lu / UC, l = lu % UC;
    return (t * NCH + c) * UC + phys_unit(UC, l);
}

// Produces the int8 rows of this pass from fp32 inputs, straight into the staged layout (rows of at most RREG * NCW
// 128-slices = 8192 values).  One warp owns one 128-wide slice per round, 4 consecutive values per lane, values held in
// registers between the phases.  The per-slice scalars (group scale, multiplier, reciprocal) are computed for all of a
// warp's slices at once, one slice per lane, so the exact divisions run once per warp instead of once per slice.  The
// row-wide sum of squares is the spec tree (slice sums are aligned subtrees; every warp finishes the same tree over
// them), the row-wide maximum is order-free.  Same fp32 operation sequence per value as k_row in glue.cu.
template <int UC>
__device__ __forceinline__ void fused_stage(const GemvArgs& a, uint8_t* xs, int2* xmeta, float* slice_sum, float* wmax,
                                            float* sxs) {
    const int K = a.K, G = a.G, NCH = a.NCH;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool keep = blockIdx.x == 0 && a.xq_out != nullptr;
    const bool rms = a.pro == PRO_RMS;
    unsigned seq = 0;
    if (a.xchg) {               // this rank's slice goes out to every rank before anybody polls
        seq = xchg_seq(a.xa);
        xchg_push(a.xa, seq);
    }
    for (int t = 0; t < a.mt; t++) {
        const float* pa = a.pa + (size_t)t * K;
        float4 v[RREG], wv[RREG];
#pragma unroll
        for (int r = 0; r < RREG; r++) {
            const int s = warp + r * NCW;
            v[r] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            wv[r] = v[r];
            if (s < G) {
                if (a.xchg) {
                    const size_t e0 = (size_t)(a.t0 + t) * K + s * 128 + lane * 4;     // first of the lane's four values
                    const float2 lo = xchg_read(a.xa, seq, e0 >> 1), hi = xchg_read(a.xa, seq, (e0 >> 1) + 1);
                    v[r] = make_float4(lo.x, lo.y, hi.x, hi.y);
                    if (a.acc_in) {
                        const float4 x = *reinterpret_cast<const float4*>(a.acc_in + e0);
                        v[r] = make_float4(fadd(x.x, v[r].x), fadd(x.y, v[r].y), fadd(x.z, v[r].z), fadd(x.w, v[r].w));
                        if (blockIdx.x == 0) *reinterpret_cast<float4*>(a.acc_out + e0) = v[r];
                    }
                } else {
                    v[r] = *reinterpret_cast<const float4*>(pa + s * 128 + lane * 4);
                }
                if (rms) wv[r] = *reinterpret_cast<const float4*>(a.pb + s * 128 + lane * 4);
            }
        }
        if (rms) {
#pragma unroll
            for (int r = 0; r < RREG; r++) {
                const int s = warp + r * NCW;
                float sq[4] = {fmul(v[r].x, v[r].x), fmul(v[r].y, v[r].y), fmul(v[r].z, v[r].z), fmul(v[r].w, v[r].w)};
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
            const float inv_rms = fdiv(1.0f, fsqrt(fadd(fdiv(tot, (float)K), a.eps)));
#pragma unroll
            for (int r = 0; r < RREG; r++)
                v[r] = make_float4(fmul(fmul(v[r].x, inv_rms), wv[r].x), fmul(fmul(v[r].y, inv_rms), wv[r].y),
                                   fmul(fmul(v[r].z, inv_rms), wv[r].z), fmul(fmul(v[r].w, inv_rms), wv[r].w));
        }
        // group scales: lane r of the warp takes slice warp + r * NCW
        float amax_sel = 0.0f;
#pragma unroll
        for (int r = 0; r < RREG; r++) {
            float am = fmaxf(fmaxf(fabsf(v[r].x), fabsf(v[r].y)), fmaxf(fabsf(v[r].z), fabsf(v[r].w)));
            am = max_lanes(am);
            if (lane == r) amax_sel = am;
        }
        const bool have = lane < RREG && warp + lane * NCW < G;
        const float sg_sel = have ? fdiv(amax_sel, 127.0f) : 0.0f;
        const float local_max = max_lanes(sg_sel);
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
        const unsigned mult_sel = have ? group_mult(sg_sel, sx) : 1u;
        const float inv_sel = fdiv(1.0f, fmul(sx, (float)mult_sel));
#pragma unroll
        for (int r = 0; r < RREG; r++) {
            const int s = warp + r * NCW;
            const unsigned mult = __shfl_sync(FULL, mult_sel, r);
            const float inv = __shfl_sync(FULL, inv_sel, r);
            if (s < G) {
                unsigned word = (unsigned)(quant_code(v[r].x, inv) & 0xff);
                word |= (unsigned)(quant_code(v[r].y, inv) & 0xff) << 8;
                word |= (unsigned)(quant_code(v[r].z, inv) & 0xff) << 16;
                word |= (unsigned)(quant_code(v[r].w, inv) & 0xff) << 24;
                // value index e = s * 128 + lane * 4: 16-byte piece s * 8 + lane / 4, word lane % 4 of it
                *reinterpret_cast<unsigned*>(xs + stage_piece<UC>(NCH, t, s * 8 + (lane >> 2)) + (lane & 3) * 4) = word;
                int sum = __dp4a((int)word, 0x01010101, 0);
#pragma unroll
                for (int off = 1; off < 16; off <<= 1) sum += __shfl_xor_sync(FULL, sum, off);
                if ((lane & 15) == 0) xmeta[stage_unit<UC>(NCH, t, 2 * s + (lane >> 4))] = make_int2(sum, (int)mult);
                if (keep) {
                    *reinterpret_cast<unsigned*>(a.xq_out + (size_t)t * K + s * 128 + lane * 4) = word;
                    if (lane == 0) a.mx_out[(size_t)t * G + s] = (uint16_t)mult;
                }
            }
        }
        consumer_barrier();     // the tables are reused by the next row; the staged row is complete
    }
}

// The same staging for a plain row whose group maxima are already known (a.pamax): no scan of the row and no values held
// in registers, so any row length goes.  Every warp derives the row scale from the maxima on its own (order-free), lane r
// computes the multiplier and reciprocal of the warp's r-th slice, then the slices are quantized one after the other.
// Same fp32 operation sequence per value as quant_act_i8g (spec/quant.rs:21-49).  The last CTA of the grid to finish
// reading leaves the maxima zero.
template <int UC>
__device__ __forceinline__ void fused_stage_amax(const GemvArgs& a, uint8_t* xs, int2* xmeta, float* sxs) {
    const int K = a.K, G = a.G, NCH = a.NCH;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool keep = blockIdx.x == 0 && a.xq_out != nullptr;
    for (int t = 0; t < a.mt; t++) {
        const float* pa = a.pa + (size_t)t * K;
        const uint4* am4 = reinterpret_cast<const uint4*>(a.pamax + 4 + (size_t)(a.t0 + t) * G * 8);
        auto group_max = [&](int s) {
            const uint4 lo = am4[2 * s], hi = am4[2 * s + 1];
            return max(max(max(lo.x, lo.y), max(lo.z, lo.w)), max(max(hi.x, hi.y), max(hi.z, hi.w)));
        };
        // the largest group scale: x -> x / 127 is monotone, so it is the scale of the largest maximum (one division)
        unsigned topbits = 0u;
        for (int s = lane; s < G; s += 32) topbits = max(topbits, group_max(s));
#pragma unroll
        for (int off = 16; off; off >>= 1) topbits = max(topbits, __shfl_xor_sync(FULL, topbits, off));
        const float top = fdiv(__uint_as_float(topbits), 127.0f);
        const float sx = (top == 0.0f) ? 1.0f : fdiv(top, 65535.0f);
        if (tid == 0) {
            sxs[t] = sx;
            if (keep) a.sx_out[t] = sx;
        }
        for (int r0 = 0; warp + r0 * NCW < G; r0 += 32) {
            const int s_sel = warp + (r0 + lane) * NCW;
            const bool have = s_sel < G;
            const float sg_sel = have ? fdiv(__uint_as_float(group_max(s_sel)), 127.0f) : 0.0f;
            const unsigned mult_sel = have ? group_mult(sg_sel, sx) : 1u;
            const float inv_sel = fdiv(1.0f, fmul(sx, (float)mult_sel));
            for (int rb = 0; rb < 32 && warp + (r0 + rb) * NCW < G; rb += 4) {
                float4 v[4];           // four slices in flight
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int s = warp + (r0 + rb + u) * NCW;
                    v[u] = s < G ? *reinterpret_cast<const float4*>(pa + s * 128 + lane * 4) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int s = warp + (r0 + rb + u) * NCW;
                    const unsigned mult = __shfl_sync(FULL, mult_sel, (rb + u) & 31);
                    const float inv = __shfl_sync(FULL, inv_sel, (rb + u) & 31);
                    if (s < G) {
                        unsigned word = (unsigned)(quant_code(v[u].x, inv) & 0xff);
                        word |= (unsigned)(quant_code(v[u].y, inv) & 0xff) << 8;
                        word |= (unsigned)(quant_code(v[u].z, inv) & 0xff) << 16;
                        word |= (unsigned)(quant_code(v[u].w, inv) & 0xff) << 24;
                        *reinterpret_cast<unsigned*>(xs + stage_piece<UC>(NCH, t, s * 8 + (lane >> 2)) + (lane & 3) * 4) = word;
                        int sum = __dp4a((int)word, 0x01010101, 0);
#pragma unroll
                        for (int off = 1; off < 16; off <<= 1) sum += __shfl_xor_sync(FULL, sum, off);
                        if ((lane & 15) == 0) xmeta[stage_unit<UC>(NCH, t, 2 * s + (lane >> 4))] = make_int2(sum, (int)mult);
                        if (keep) {
                            *reinterpret_cast<unsigned*>(a.xq_out + (size_t)t * K + s * 128 + lane * 4) = word;
                            if (lane == 0) a.mx_out[(size_t)t * G + s] = (uint16_t)mult;
                        }
                    }
                }
            }
        }
    }
    consumer_barrier();     // the staged rows are complete; every read of the maxima by this CTA is done
    if (tid < 32) {
        unsigned last = 0;
        if (lane == 0) {
            __threadfence();
            last = atomicAdd(a.pamax, 1u) == gridDim.x - 1 ? 1u : 0u;
        }
        if (__shfl_sync(FULL, last, 0)) {
            for (int i = lane; i < a.mt * G * 8; i += 32) a.pamax[4 + (size_t)a.t0 * G * 8 + i] = 0u;
            if (lane == 0) a.pamax[0] = 0u;
        }
    }
}

// One record (a K chunk of the quad) for this lane's row: the lane's whole 128-group (two units; one unit = half a group
// when UC = 8), all MT tokens.  acc gathers dot * (m * mx - 2^31) exactly in 64 bits with ONE signed multiply-add per
// group and token, accs the plain sum of the dots: the caller adds accs * 2^31 back at the end of the row.
// wp: the lane's first piece in the record; xp / mp: the lane's first activation piece / unit entry of this chunk.
template <int BITS, int MT, int UC>
__device__ __forceinline__ void quad_chunk(const uint8_t* wp, unsigned mw, const uint8_t* xp, const int2* mp, int tok_bytes,
                                           int tok_units, long long (&acc)[MT], int (&accs)[MT]) {
    constexpr int PU = UC * 16;          // byte distance between the pieces of a unit
    constexpr int UPL = UC / 8;          // units per lane: 2 (a whole group) or 1
    int dots[MT], mxv[MT];
#pragma unroll
    for (int t = 0; t < MT; t++) { dots[t] = 0; mxv[t] = 1; }
#pragma unroll
    for (int uu = 0; uu < UPL; uu++) {
        unsigned o[16];
        unpack_unit<BITS>(wp + uu * (LPR * 16), PU, o);
#pragma unroll
        for (int t = 0; t < MT; t++) {
            int d0 = 0, d1 = 0, d2 = 0, d3 = 0;   // independent chains, summed below
            const uint8_t* xt = xp + (size_t)t * tok_bytes + uu * (LPR * 16);
            const uint4 x0 = *reinterpret_cast<const uint4*>(xt);
            const uint4 x1 = *reinterpret_cast<const uint4*>(xt + PU);
            const uint4 x2 = *reinterpret_cast<const uint4*>(xt + 2 * PU);
            const uint4 x3 = *reinterpret_cast<const uint4*>(xt + 3 * PU);
            d0 = dot4<BITS>(o[0], (int)x0.x, d0); d1 = dot4<BITS>(o[1], (int)x0.y, d1);
            d2 = dot4<BITS>(o[2], (int)x0.z, d2); d3 = dot4<BITS>(o[3], (int)x0.w, d3);
            d0 = dot4<BITS>(o[4], (int)x1.x, d0); d1 = dot4<BITS>(o[5], (int)x1.y, d1);
            d2 = dot4<BITS>(o[6], (int)x1.z, d2); d3 = dot4<BITS>(o[7], (int)x1.w, d3);
            d0 = dot4<BITS>(o[8], (int)x2.x, d0); d1 = dot4<BITS>(o[9], (int)x2.y, d1);
            d2 = dot4<BITS>(o[10], (int)x2.z, d2); d3 = dot4<BITS>(o[11], (int)x2.w, d3);
            d0 = dot4<BITS>(o[12], (int)x3.x, d0); d1 = dot4<BITS>(o[13], (int)x3.y, d1);
            d2 = dot4<BITS>(o[14], (int)x3.z, d2); d3 = dot4<BITS>(o[15], (int)x3.w, d3);
            const int2 meta = mp[t * tok_units + uu * LPR];
            int dot = (d0 + d1) + (d2 + d3);
            if (BITS != 8) dot -= code_offset(BITS) * meta.x;
            dots[t] += dot;
            mxv[t] = meta.y;
        }
    }
#pragma unroll
    for (int t = 0; t < MT; t++) {
        const int mults = (int)(mw * (unsigned)mxv[t] + 0x80000000u);     // m * mx - 2^31 as a signed word
        acc[t] += (long long)dots[t] * (long long)mults;
        accs[t] += dots[t];
    }
}

// Shared memory: [slots: workers * spw] [x pieces: MT * NCH * UC * 64] [xmeta: MT * NCH * UC int2 = (sum of x over
// the unit, mx of its group)] [full[MAX_SLOTS]] [slice sums: 256 f32] [warp maxima: NCW f32] [row scales: 8 f32]
template <int BITS, int MT, bool DUAL, int UC>
__global__ void __launch_bounds__(GEMV_THREADS, 1) k_gemv_stream(const GemvArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int NCH = a.NCH;
    const int upad = NCH * UC;
    uint8_t* ring = smem;
    uint8_t* xs = ring + (size_t)a.workers * a.spw * a.slot_bytes;
    int2* xmeta = reinterpret_cast<int2*>(xs + (size_t)MT * upad * 64);
    unsigned long long* full = reinterpret_cast<unsigned long long*>(xmeta + MT * upad);
    float* slice_sum = reinterpret_cast<float*>(full + MAX_SLOTS);
    float* wmax = slice_sum + 256;
    float* sxs = wmax + NCW;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const long long wl = wait_limit(a.error_flag);
    const int W = a.workers, SPW = a.spw;
    const int total = a.seg[0].nquads + (DUAL ? a.seg[1].nquads : 0);
    pdl_trigger();
    if (tid < W * SPW) {          // one barrier per thread (at most 80)
        mbar_init(&full[tid], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // Quad i of this CTA (global quad blockIdx.x + i * gridDim.x) belongs to warp i % workers.  The warp's records —
    // NCH per quad, quads in order — land in the warp's slots round-robin, so the warp meets the phases of each of its
    // slots strictly in sequence (a parity wait can tell only two phases apart).  (ili, ic, islot) = the next record to
    // request: quad number within the warp, chunk, slot.
    const long long qstep = (long long)W * gridDim.x;
    long long iq = (long long)blockIdx.x + (long long)warp * gridDim.x;     // global quad of the next request
    int ic = 0, islot = 0;
    auto issue = [&]() {        // one lane: request the warp's next record, if there is one
        if (iq >= total) return;
        const int sg = (DUAL && iq >= a.seg[0].nquads) ? 1 : 0;
        const long long q = sg ? iq - a.seg[0].nquads : iq;
        const int s = warp * SPW + islot;
        const unsigned bytes = (unsigned)a.seg[sg].rec_bytes;
        mbar_expect_tx(&full[s], bytes);
        bulk_g2s(ring + (size_t)s * a.slot_bytes, a.seg[sg].w + ((size_t)q * NCH + ic) * bytes, bytes, &full[s]);
        if (++islot == SPW) islot = 0;
        if (++ic == NCH) { ic = 0; iq += qstep; }
    };
    // weights do not depend on earlier kernels: every worker fills its slots before waiting for its predecessor
    if (warp < W && lane == 0)
        for (int i = 0; i < SPW; i++) issue();

    // ---------------- stage the activations once (same chunk / piece order as the weights).  The activations (and the
    // output rows) belong to earlier kernels: wait for them here, while the first weights are already on their way.
    pdl_wait();
    if (upad != a.U) {     // ragged last chunk: the padding units must read as zero
        for (int i = tid; i < MT * upad * 4; i += NCW * 32) reinterpret_cast<uint4*>(xs)[i] = make_uint4(0, 0, 0, 0);
        for (int i = tid; i < MT * upad; i += NCW * 32) xmeta[i] = make_int2(0, 1);
        consumer_barrier();
    }
    if (a.pro && a.pamax) {
        fused_stage_amax<UC>(a, xs, xmeta, sxs);
    } else if (a.pro) {
        fused_stage<UC>(a, xs, xmeta, slice_sum, wmax, sxs);
    } else {
        const int pieces_per_tok = a.K >> 4;
        const int total_pieces = MT * pieces_per_tok;
        for (int base = 0; base < total_pieces; base += NCW * 32) {
            const int pid = base + tid;
            const bool live = pid < total_pieces;
            int t = 0, q = 0;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (live) {
                t = pid / pieces_per_tok;
                q = pid - t * pieces_per_tok;
                if (t < a.mt) v = *reinterpret_cast<const uint4*>(a.xq + (size_t)t * a.K + (size_t)q * 16);
                *reinterpret_cast<uint4*>(xs + stage_piece<UC>(NCH, t, q)) = v;
            }
            int s = __dp4a((int)v.x, 0x01010101, 0);
            s = __dp4a((int)v.y, 0x01010101, s);
            s = __dp4a((int)v.z, 0x01010101, s);
            s = __dp4a((int)v.w, 0x01010101, s);
            s += __shfl_xor_sync(FULL, s, 1);
            s += __shfl_xor_sync(FULL, s, 2);
            if (live && (q & 3) == 0) {
                const int lu = q >> 2;
                const int mxv = (a.mx && t < a.mt) ? (int)a.mx[(size_t)t * a.G + (lu >> 1)] : 1;
                xmeta[stage_unit<UC>(NCH, t, lu)] = make_int2(s, mxv);
            }
        }
        consumer_barrier();
    }

    if (warp >= W) return;
    float sxr[MT];                               // row scales, fetched once (not once per record)
#pragma unroll
    for (int t = 0; t < MT; t++) sxr[t] = a.pro ? sxs[t] : (t < a.mt ? a.sx[t] : 0.0f);
    const int r = lane / LPR, j = lane - r * LPR;
    constexpr int NP = BITS / 2;
    const int tok_bytes = NCH * UC * 64, tok_units = NCH * UC;      // one token's staged row
    const int chunk_bytes = UC * 64;
    const uint8_t* xlane = xs + j * 16;
    const int2* mlane = xmeta + j;
    const int woff = (r * NP * UC + j) * 16, woff8 = (r * 4 * UC + j) * 16;   // the lane's first piece (W8 for a DUAL tail)
    const int moff = (r * (UC >> 1) + (UC == 16 ? j : (j >> 1))) * 2;
    int cslot = 0;
    unsigned cphase = 0;
    bool ok = true;
    for (long long Q = (long long)blockIdx.x + (long long)warp * gridDim.x; ok && Q < total; Q += qstep) {
        const int sg = (DUAL && Q >= a.seg[0].nquads) ? 1 : 0;
        const GemvSeg& S = a.seg[sg];
        const int n = (int)(sg ? Q - a.seg[0].nquads : Q) * QR + r;
        // the row's scale, in flight while the row is summed (c is indexed by the linear's own row order)
        const float cn = (j == 0 && n < S.N) ? S.c[S.out.pairs ? (n & 1) * (S.N >> 1) + (n >> 1) : n] : 0.0f;
        long long acc[MT];
        int accs[MT];
#pragma unroll
        for (int t = 0; t < MT; t++) { acc[t] = 0; accs[t] = 0; }
        const uint8_t* xp = xlane;
        const int2* mp = mlane;
        for (int c = 0; c < NCH; c++, xp += chunk_bytes, mp += UC) {
            const int s = warp * SPW + cslot;
            ok = mbar_wait(&full[s], cphase, wl);
            if (!ok) break;
            const uint8_t* rec = ring + (size_t)s * a.slot_bytes;
            const unsigned mw = *reinterpret_cast<const uint16_t*>(rec + S.m_off + moff);
            if (DUAL && sg) quad_chunk<8, MT, UC>(rec + woff8, mw, xp, mp, tok_bytes, tok_units, acc, accs);
            else quad_chunk<BITS, MT, UC>(rec + woff, mw, xp, mp, tok_bytes, tok_units, acc, accs);
            if (++cslot == SPW) { cslot = 0; cphase ^= 1u; }
            __syncwarp();                            // every lane has finished reading the slot
            if (lane == 0) issue();                  // refill it with the warp's record SPW ahead
        }
        if (!ok) break;
        float y[MT];
#pragma unroll
        for (int t = 0; t < MT; t++) {
            long long tot = acc[t] + ((long long)accs[t] << 31);
#pragma unroll
            for (int off = 1; off < LPR; off <<= 1) tot += shfl_xor_i64(tot, off);
            y[t] = fmul(fmul(i64_to_f32(tot), cn), sxr[t]);
        }
        if (a.h && !sg) {
            // pairs layout: rows r = 0, 2 are gate rows, r + 1 their up rows; lane (r, 0) fetches up from lane (r + 1, 0)
#pragma unroll
            for (int t = 0; t < MT; t++) {
                const float up = __shfl_down_sync(FULL, y[t], LPR);
                if (j == 0 && (r & 1) == 0 && n < S.N && t < a.mt) {
                    const float hv = fmul(silu_f(y[t]), up);
                    a.h[(size_t)(a.t0 + t) * a.h_width + (n >> 1)] = hv;
                    if (a.h_amax)
                        atomicMax(a.h_amax + 4 + ((size_t)(a.t0 + t) * (a.h_width >> 7) + (n >> 8)) * 8 + ((n >> 2) & 7),
                                  __float_as_uint(fabsf(hv)));
                }
            }
        } else if (j == 0 && n < S.N) {
#pragma unroll
            for (int t = 0; t < MT; t++)
                if (t < a.mt) emit(S.out, a.t0 + t, n, y[t]);
        }
    }
    if (!ok && lane == 0) {
        atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
        // copies this warp has requested still target this CTA's shared memory: give each slot a (bounded) chance to land
        for (int s = warp * SPW; s < (warp + 1) * SPW; s++) {
            (void)mbar_wait(&full[s], 0u, wl >> 5);
            (void)mbar_wait(&full[s], 1u, wl >> 5);
        }
    }
}

// ------------------------------------------------------------------------------------------------------------------
struct GemvPlan {
    int spw, workers;
    size_t smem;
    int grid;
};
// Measurement switch (det_debug_set_gemv): bits 4..8 = worker warps per CTA (0 = all sixteen); bits 9.. = slots per
// worker (0 = as many as fit, at most 5).  Results do not depend on it.
static int g_gemv_flags = 0;

// A plan by shape only: one CTA per SM, sixteen workers, as many slots per worker as the staged activations leave room
// for (bytes in flight per CTA = workers * (spw - 1) records).
static bool plan_gemv(int K, int slot_bytes, int MT, long long total_quads, GemvPlan& p) {
    const StreamGeom g = stream_geom(QR, K, 8);
    const int upad = g.NCH * g.UC;
    const size_t fixed = (size_t)MT * upad * 64 + (size_t)MT * upad * 8 + MAX_SLOTS * 8 + (256 + NCW + 8) * 4;
    const size_t budget = smem_optin() - 1024;
    if (fixed + 2 * (size_t)slot_bytes > budget) return false;
    const int slots = (int)((budget - fixed) / slot_bytes);
    int workers = (g_gemv_flags >> 4) & 31;
    if (workers < 1 || workers > NCW) workers = NCW;
    while (workers > 1 && slots / workers < 2) workers--;
    p.workers = workers;
    p.spw = slots / workers;
    const int cap_spw = (g_gemv_flags >> 9) > 0 ? (g_gemv_flags >> 9) : MAX_SPW;
    if (p.spw > cap_spw) p.spw = cap_spw;
    if (p.spw > MAX_SPW) p.spw = MAX_SPW;
    if (p.spw < 1) return false;
    p.smem = fixed + (size_t)p.workers * p.spw * slot_bytes;
    const long long cap = (long long)sm_count();
    p.grid = (int)(total_quads < cap ? total_quads : cap);
    return true;
}

template <int BITS, int MT, bool DUAL, int UC>
static void launch_gemv_one(const GemvArgs& a, const GemvPlan& p, cudaStream_t q) {
    static bool configured = false;
    if (!configured) {
        DETB_CUDA_OK(cudaFuncSetAttribute(k_gemv_stream<BITS, MT, DUAL, UC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)(smem_optin())));
        configured = true;
    }
    launch_pdl(k_gemv_stream<BITS, MT, DUAL, UC>, dim3(p.grid), dim3(GEMV_THREADS), p.smem, q, 1, a);
}
template <int BITS, int MT>
static void launch_gemv(const GemvArgs& a, const GemvPlan& p, bool dual, cudaStream_t q) {
    if (a.UC == 16) {
        if (dual) {
            if constexpr (MT <= 2) launch_gemv_one<BITS, MT, true, 16>(a, p, q);
        } else {
            launch_gemv_one<BITS, MT, false, 16>(a, p, q);
        }
    } else {
        if (dual) {
            if constexpr (MT <= 2) launch_gemv_one<BITS, MT, true, 8>(a, p, q);
        } else {
            launch_gemv_one<BITS, MT, false, 8>(a, p, q);
        }
    }
}

template <int BITS>
static void gemv_stream_bits(const GemvCall& call, cudaStream_t q) {
    const det_qlinear* L = call.lin;
    const StreamGeom g = stream_geom(L->N, L->K, BITS);
    DETB_REQUIRE(g.G <= 256, "K is too large for the streaming GEMV");
    if (call.lin2 && call.M > 2) {
        // more than two rows: the two linears go out as two launches (the second one reads the rows the first one's
        // prologue stored, or quantizes them again when nothing was stored: same values either way)
        GemvCall first = call, second = call;
        first.lin2 = nullptr;
        second.lin = call.lin2;
        second.lin2 = nullptr;
        second.out = call.out2;
        second.h = nullptr;
        if (call.src && call.src->xq) {
            second.src = nullptr;
            second.xq = call.src->xq; second.sx = call.src->sx; second.mx = call.src->mx;
        }
        gemv_stream_launch(first, q);
        gemv_stream_launch(second, q);
        return;
    }
    const bool dual = call.lin2 != nullptr;
    StreamGeom g2 = g;
    if (dual) {
        DETB_REQUIRE((call.lin2->bits & 0xff) == 8 && (call.lin2->bits & DET_LAYOUT_STREAM) && call.lin2->K == L->K,
                     "the second linear of a GEMV launch is a W8 streaming-layout linear over the same input");
        g2 = stream_geom(call.lin2->N, call.lin2->K, 8);
    }
    const det_act_source* src = call.src;
    int t0 = 0;
    while (t0 < call.M) {
        const int left = call.M - t0;
        int MT = left >= 5 ? 8 : (left >= 3 ? 4 : left);
        const int slot_bytes = dual && g2.rec_bytes > g.rec_bytes ? g2.rec_bytes : g.rec_bytes;
        GemvPlan p;
        while (!plan_gemv(L->K, slot_bytes, MT, (long long)g.nquads + (dual ? g2.nquads : 0), p)) {
            DETB_REQUIRE(MT > 1, "K is too large for the streaming GEMV");
            MT >>= 1;
        }
        GemvArgs a;
        a.seg[0] = GemvSeg{L->wq, L->c, L->N, g.nquads, g.rec_bytes, g.m_off, call.out};
        a.seg[1] = a.seg[0];
        if (dual) a.seg[1] = GemvSeg{call.lin2->wq, call.lin2->c, call.lin2->N, g2.nquads, g2.rec_bytes, g2.m_off, call.out2};
        a.K = g.K; a.U = g.U; a.G = g.G; a.UC = g.UC; a.NCH = g.NCH;
        a.slot_bytes = slot_bytes;
        a.xq = call.xq ? call.xq + (size_t)t0 * g.K : nullptr;
        a.sx = call.sx ? call.sx + t0 : nullptr;
        a.mx = call.mx ? call.mx + (size_t)t0 * g.G : nullptr;
        a.t0 = t0;
        a.mt = left < MT ? left : MT;
        a.spw = p.spw;
        a.workers = p.workers;
        a.error_flag = error_word();
        a.pro = 0;
        a.pa = a.pb = nullptr;
        a.eps = 0.0f;
        a.pslices = 0;
        a.xq_out = nullptr; a.sx_out = nullptr; a.mx_out = nullptr;
        a.pamax = nullptr;
        a.h_amax = call.h ? call.h_amax : nullptr;
        a.xchg = 0;
        a.acc_in = nullptr;
        a.acc_out = nullptr;
        if (src && src->xchg) {
            const Xchg* xc = static_cast<const Xchg*>(src->xchg);
            DETB_REQUIRE(xc->size * src->slice == g.K && src->slice % 2 == 0, "exchange prologue: size * slice must be K");
            DETB_REQUIRE((size_t)call.M * g.K * 8 <= xc->slot_bytes, "exchange larger than the staging slot");
            DETB_REQUIRE(t0 == 0 && call.M <= MT, "exchange prologue: all rows in one launch");
            a.xchg = 1;
            a.xa = xchg_args(xc, src->local, nullptr, call.M, src->slice);
            if (src->kind == PRO_RMS && src->acc_out) {
                DETB_REQUIRE(src->a && src->acc_out != src->a, "the summed rows need a buffer of their own");
                a.acc_in = src->a;
                a.acc_out = src->acc_out;
            }
        }
        if (src) {
            a.pamax = src->amax;
            a.pro = src->kind;
            a.pa = src->a + (size_t)t0 * g.K;
            a.pb = src->b;
            a.eps = src->eps;
            int P = 128;
            while (P < g.K) P <<= 1;
            a.pslices = P / 128;
            a.xq_out = src->xq ? src->xq + (size_t)t0 * g.K : nullptr;
            a.sx_out = src->sx ? src->sx + t0 : nullptr;
            a.mx_out = src->mx ? src->mx + (size_t)t0 * g.G : nullptr;
        }
        a.h = call.h;
        a.h_width = L->N / 2;
        switch (MT) {
            case 1: launch_gemv<BITS, 1>(a, p, dual, q); break;
            case 2: launch_gemv<BITS, 2>(a, p, dual, q); break;
            case 4: launch_gemv<BITS, 4>(a, p, dual, q); break;
            default: launch_gemv<BITS, 8>(a, p, dual, q); break;
        }
        t0 += a.mt;
    }
}

void gemv_stream_launch(const GemvCall& call, cudaStream_t q) {
    const int bits = call.lin->bits & 0xff;
    if (call.src) {
        DETB_REQUIRE(call.lin->K <= RREG * NCW * 128 || (call.src->kind == PRO_PLAIN && call.src->amax),
                     "the activation prologue takes rows of at most 8192 values unless their group maxima are given");
        DETB_REQUIRE(!call.src->amax || (call.src->kind == PRO_PLAIN && !call.lin2),
                     "group maxima go with the plain quantization of a single linear only");
        DETB_REQUIRE((call.src->kind == PRO_RMS || call.src->kind == PRO_PLAIN) && (call.src->a || call.src->xchg), "bad activation source");
        DETB_REQUIRE(!call.src->xchg || (call.src->local && !call.src->amax && (!call.lin2 || call.M <= 2)),
                     "exchange prologue: needs the local slice, no group maxima, one launch");
        DETB_REQUIRE(call.src->kind != PRO_RMS || call.src->b, "RMSNorm needs its weight");
        DETB_REQUIRE((call.src->xq != nullptr) == (call.src->sx != nullptr) && (call.src->xq != nullptr) == (call.src->mx != nullptr),
                     "the quantized-row outputs come all together or not at all");
    } else {
        DETB_REQUIRE(call.xq && call.sx, "a GEMV needs its quantized input rows");
    }
    if (call.h) DETB_REQUIRE((call.lin->bits & DET_LAYOUT_PAIRS) && call.lin->N % 2 == 0, "the SwiGLU epilogue needs the pairs layout");
    if (bits == 8) gemv_stream_bits<8>(call, q);
    else if (bits == 6) gemv_stream_bits<6>(call, q);
    else gemv_stream_bits<4>(call, q);
}

}  // namespace detb

using namespace detb;

extern "C" {

size_t det_linear_repack_bytes(int N, int K, int bits) {
    DETB_REQUIRE((bits == 4 || bits == 6 || bits == 8) && K > 0 && K % 128 == 0 && N > 0, "bad linear shape");
    const StreamGeom g = stream_geom(N, K, bits);
    return (size_t)g.nquads * g.NCH * g.rec_bytes;
}

static void repack(const det_qlinear* src, void* dst, int pairs, cudaStream_t st) {
    DETB_REQUIRE((src->bits == 4 || src->bits == 6 || src->bits == 8) && src->K % 128 == 0, "bad linear shape");
    DETB_REQUIRE(!pairs || src->N % 2 == 0, "the pairs layout needs an even number of rows");
    const StreamGeom g = stream_geom(src->N, src->K, src->bits);
    const long long work = (long long)g.nquads * QR * g.NCH * g.UC;
    k_repack_stream<<<(unsigned)((work + 127) / 128), 128, 0, queue_of(st)>>>(src->wq, src->m, g, pairs, (uint8_t*)dst);
    DETB_CUDA_OK(cudaGetLastError());
}
void det_linear_repack(const det_qlinear* src, void* dst, cudaStream_t st) { repack(src, dst, 0, st); }
void det_linear_repack_pairs(const det_qlinear* src, void* dst, cudaStream_t st) { repack(src, dst, 1, st); }

void det_debug_set_gemv(int flags) { g_gemv_flags = flags; }

}  // extern "C"
