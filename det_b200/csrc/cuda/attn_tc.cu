// Prefill attention on the 5th-generation tensor cores (tcgen05.mma kind::i8, TMA-fed operands, TMEM accumulators).
// Replaces the reference's mma.sync attention (kernels/cuda/attn.cu:405-852: tc::k_tc_max, tc::k_tc_acc, the byte slicing
// of 685-732) for batches of 16 tokens and more; the arithmetic is docs/SPEC.md §5.1 / spec/layers.rs:15-74, so every
// output equals the CUDA-core kernels of attn.cu bit for bit:
//
//   s[r][j]  = ((float) dot(qq[r], kq[j]) * sq[r]) * sk[j]                       dot: s8 x s8 -> s32, exact
//   max[r]   = max_j s[r][j]                                                    order-free
//   p[r][j]  = rint(exp_f(s - max) * 2^24)  in [0, 2^24]                         keys after the row's position: 0
//   den[r]   = sum_j p,   num[r][d] = sum_j p[r][j] * vq[j][d]                   int64, exact in any order
//   o[r][d]  = (((float) num / (float) den) * v_scale) * sigmoid_f(gate)
//
// A query row r is a (token, q head) pair; the rows of the q heads that share kv head g are laid out token-major
// ([g][token * rep + head]) so that a tile of 128 rows is one UMMA M and reads one K / V stream.
//
//   k_attn_vt      V of all keys of the call, split into its low (u8) and high (s8) bytes and transposed to
//                  [byte plane][g][d][key]: keys become the contraction dimension of a K-major UMMA operand.
//   k_attn_tc_s<1> scores of a (row tile, key tile) pair as 8 UMMA steps (K = 32 bytes of the 256-byte head) into a
//                  128 x 128 s32 TMEM tile, two tiles in flight; the epilogue warps fold the masked maxima.
//   k_attn_tc_s<2> the same scores again, then p and den; p = q + e with e = [p == 2^24] and q = p - e < 2^24, and the
//                  three byte slices of q plus e go out as four u8 planes [plane][g][row][key] into the workspace (keys
//                  contiguous: again a K-major operand).
//   k_attn_tc_pv   num as byte-sliced integer GEMMs over the keys: (q slice i, u8) x (V low byte, u8) carries weight
//                  2^(8i), (q slice i) x (V high byte, s8) weight 2^(8i+8), e x low / high byte weights 1 and 2^8.  The
//                  eight products go into four TMEM accumulators by weight (128 rows x 128 value dims each: all 512
//                  columns) that run over ALL key tiles of the CTA — an s32 sum grows by at most 255*255 + 255*128 + 128
//                  per key, so 16384 keys stay below 2^31 — and are widened to int64 once, at the end.
//
// No value ever depends on the tiling: integer sums and maxima only.  Waits are bounded (runtime.cuh); no multicast.
#include "attn_tc.cuh"
#include "umma.cuh"
#include <algorithm>

namespace detb {

constexpr int AQ = 128;            // query rows per tile (UMMA M)
constexpr int AK = 128;            // keys per tile
constexpr int AT_HD = 256;         // head dimension of the tensor path
constexpr int PV_DIMS = 128;       // value dimensions per k_attn_tc_pv CTA
constexpr int PV_MAX_TILES = 128;  // key tiles per k_attn_tc_pv CTA: 16384 keys keep every s32 accumulator below 2^31

struct AttnTc {
    int M, n_h, n_kv, rep, pos0, keys;
    int Rpad, Kpad;
    int rt0, rts;                  // this launch covers row tiles [rt0, rt0 + rts) of every kv head
    int kt_per_cta;
    const float* sq;               // [n_kv][Rpad]
    const float* sk;               // cache: [key][n_kv]
    unsigned* mxkey;               // [n_kv][Rpad]
    long long* den;                // [n_kv][Rpad]
    long long* num;                // [n_kv][Rpad][256] (key-split launches only)
    uint8_t* planes;               // [4][n_kv][rts * 128][Kpad]
    const float* qg;
    const float* v_scale;
    float* o;
    int* error_flag;
    int nz;                        // key splits of k_attn_tc_pv
};

__device__ __forceinline__ uint8_t* align_1k(uint8_t* p) {
    return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~(uintptr_t)1023);
}
// key tiles a row tile needs: its last row's token sits at position pos0 + token
__device__ __forceinline__ int tiles_needed(const AttnTc& a, int rt) {
    const int tok_max = min(a.M - 1, (rt * AQ + AQ - 1) / a.rep);
    return (a.pos0 + tok_max) / AK + 1;
}

// ---- V -> byte planes, transposed.  Block = 64 keys of one kv head; thread d gathers its dimension's 64 bytes per plane.
__global__ void __launch_bounds__(256) k_attn_vt(const int16_t* __restrict__ vq, int n_kv, int keys, int Kpad,
                                                 uint8_t* __restrict__ vt) {
    __shared__ __align__(16) int16_t tile[64][AT_HD];
    pdl_trigger();
    pdl_wait();
    const int g = blockIdx.y, k0 = blockIdx.x * 64;
    for (int i = threadIdx.x; i < 64 * (AT_HD / 8); i += 256) {
        const int kk = i / (AT_HD / 8), v = i % (AT_HD / 8);
        uint4 val = make_uint4(0, 0, 0, 0);
        if (k0 + kk < keys) val = *reinterpret_cast<const uint4*>(vq + ((size_t)(k0 + kk) * n_kv + g) * AT_HD + v * 8);
        *reinterpret_cast<uint4*>(&tile[kk][v * 8]) = val;
    }
    __syncthreads();
    const int d = threadIdx.x;
    unsigned lo[16], hi[16];
#pragma unroll
    for (int w = 0; w < 16; w++) {
        unsigned l = 0, h = 0;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const unsigned v = (unsigned short)tile[w * 4 + b][d];
            l |= (v & 0xffu) << (8 * b);
            h |= (v >> 8) << (8 * b);
        }
        lo[w] = l;
        hi[w] = h;
    }
    uint4* dlo = reinterpret_cast<uint4*>(vt + ((size_t)g * AT_HD + d) * Kpad + k0);
    uint4* dhi = reinterpret_cast<uint4*>(vt + ((size_t)(n_kv + g) * AT_HD + d) * Kpad + k0);
#pragma unroll
    for (int w = 0; w < 4; w++) {
        dlo[w] = make_uint4(lo[4 * w], lo[4 * w + 1], lo[4 * w + 2], lo[4 * w + 3]);
        dhi[w] = make_uint4(hi[4 * w], hi[4 * w + 1], hi[4 * w + 2], hi[4 * w + 3]);
    }
}

// ---- scores.  Warp 0: TMA producer, warp 1: TMEM + MMA issue, warps 2..9: epilogue (warp w reads TMEM lanes
// 32 * (w % 4) .. + 31 — one query row per thread — and 64 of the tile's 128 key columns).
constexpr int S_STAGES = 3;
constexpr int S_STAGE_BYTES = 2 * AK * 128;        // a key tile: two 128-byte halves of the head, 16 KB each
constexpr int S_THREADS = 320;
constexpr size_t S_SMEM = 1024 + 2 * AQ * 128 + S_STAGES * S_STAGE_BYTES + (2 * S_STAGES + 5) * 8 + 16;

template <int PASS>
__global__ void __launch_bounds__(S_THREADS, 1)
k_attn_tc_s(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const AttnTc a) {
    extern __shared__ __align__(1024) uint8_t s_raw[];
    uint8_t* smem = align_1k(s_raw);
    uint8_t* qt = smem;                                   // query tile: 2 x 16 KB
    uint8_t* stages = smem + 2 * AQ * 128;
    unsigned long long* full = reinterpret_cast<unsigned long long*>(stages + S_STAGES * S_STAGE_BYTES);
    unsigned long long* empty = full + S_STAGES;
    unsigned long long* tfull = empty + S_STAGES;         // [2] scores complete in TMEM buffer
    unsigned long long* tempty = tfull + 2;               // [2] epilogue drained the buffer
    unsigned long long* qfull = tempty + 2;
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(qfull + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = blockIdx.z, rt = a.rt0 + blockIdx.y;
    const int nkt = tiles_needed(a, rt);
    const int kt0 = blockIdx.x * a.kt_per_cta;
    const int n = min(nkt, kt0 + a.kt_per_cta) - kt0;    // key tiles of this CTA
    pdl_trigger();
    if (n <= 0) return;
    const long long wl = wait_limit(a.error_flag);

    if (threadIdx.x == 0) {
        for (int s = 0; s < S_STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], 8);
        }
        mbar_init(qfull, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, 256);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    pdl_wait();   // the query rows, their scales, the cache rows of this batch and the maxima come from earlier kernels
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(qfull, 2 * AQ * 128);
            tma_load_2d(qt, &map_q, 0, g * a.Rpad + rt * AQ, qfull);
            tma_load_2d(qt + AQ * 128, &map_q, 128, g * a.Rpad + rt * AQ, qfull);
            int issued = 0;
            for (int l = 0; l < n; l++, issued++) {
                const int s = l % S_STAGES;
                if (l >= S_STAGES) {
                    ok = mbar_wait(&empty[s], ((unsigned)(l / S_STAGES) & 1u) ^ 1u, wl);
                    if (!ok) break;
                }
                uint8_t* st = stages + (size_t)s * S_STAGE_BYTES;
                mbar_expect_tx(&full[s], S_STAGE_BYTES);
                tma_load_3d(st, &map_k, 0, g, (kt0 + l) * AK, &full[s]);
                tma_load_3d(st + AK * 128, &map_k, 128, g, (kt0 + l) * AK, &full[s]);
            }
            if (!ok) {
                atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
                for (int k = 0; k < S_STAGES && k < issued; k++) {   // let the copies in flight land before the CTA goes
                    const int i = issued - 1 - k;
                    (void)mbar_wait(&full[i % S_STAGES], (unsigned)(i / S_STAGES) & 1u, wl);
                }
                (void)mbar_wait(qfull, 0u, wl);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr unsigned IDESC = umma_idesc_i8(AK, true, true);
            ok = mbar_wait(qfull, 0u, wl);
            for (int l = 0; ok && l < n; l++) {
                const int s = l % S_STAGES, b = l & 1;
                ok = mbar_wait(&full[s], (unsigned)(l / S_STAGES) & 1u, wl) &&
                     mbar_wait(&tempty[b], ((unsigned)(l >> 1) & 1u) ^ 1u, wl);
                if (!ok) break;
                tc_fence_after();
                const uint8_t* st = stages + (size_t)s * S_STAGE_BYTES;
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const unsigned long long dq = umma_desc(qt + h * AQ * 128), dk = umma_desc(st + h * AK * 128);
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        umma_i8(tmem_base + b * AK, dq + 2 * k, dk + 2 * k, IDESC, (h | k) ? 1u : 0u);
                }
                umma_commit(&empty[s]);
                umma_commit(&tfull[b]);
            }
            if (!ok) atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
        }
    } else {
        const int q = warp & 3, ch = (warp - 2) >> 2;
        const int row_in = q * 32 + lane, row = rt * AQ + row_in;
        const bool valid = row < a.M * a.rep;
        const int pos = a.pos0 + row / a.rep;
        const size_t cell = (size_t)g * a.Rpad + row;
        const float sqv = valid ? a.sq[cell] : 0.0f;
        const float mx = (PASS == 2 && valid) ? key_f32(a.mxkey[cell]) : 0.0f;
        unsigned best = 0u;
        unsigned long long dsum = 0ull;
        for (int l = 0; l < n; l++) {
            const int b = l & 1, kt = kt0 + l;
            ok = mbar_wait(&tfull[b], (unsigned)(l >> 1) & 1u, wl);
            if (!ok) break;
            tc_fence_after();
            int r[2][32];
            const unsigned taddr = tmem_base + ((unsigned)(q * 32) << 16) + b * AK + ch * 64;
            tmem_ld(taddr, r[0]);
            tmem_ld(taddr + 32, r[1]);
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[b]);
#pragma unroll
            for (int c = 0; c < 2; c++) {
                const int key0 = kt * AK + ch * 64 + c * 32;
                const float skl = key0 + lane < a.keys ? a.sk[(size_t)(key0 + lane) * a.n_kv + g] : 0.0f;
                if (PASS == 1) {
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        const float s = fmul(fmul((float)r[c][i], sqv), __shfl_sync(FULL, skl, i));
                        if (valid && key0 + i <= pos) best = max(best, f32_key(s));
                    }
                } else {
                    unsigned words[4][8];
                    unsigned tsum = 0u;
#pragma unroll
                    for (int i4 = 0; i4 < 8; i4++) {
                        unsigned p[4];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int i = i4 * 4 + u;
                            const float s = fmul(fmul((float)r[c][i], sqv), __shfl_sync(FULL, skl, i));
                            const int pv = f2i_sat(fmul(exp_f(fsub(s, mx)), 16777216.0f));
                            p[u] = (valid && key0 + i <= pos) ? (unsigned)pv : 0u;
                            tsum += p[u];           // 32 values of at most 2^24
                            const unsigned e = p[u] >> 24;          // p = q + e, e = [p == 2^24]
                            p[u] = (p[u] - e) | (e << 24);          // three bytes of q, e in the fourth
                        }
#pragma unroll
                        for (int sl = 0; sl < 4; sl++) {   // byte sl of four consecutive keys into one word
                            const unsigned t01 = __byte_perm(p[0], p[1], sl | ((4 + sl) << 4));
                            const unsigned t23 = __byte_perm(p[2], p[3], sl | ((4 + sl) << 4));
                            words[sl][i4] = __byte_perm(t01, t23, 0x5410);
                        }
                    }
                    dsum += tsum;
#pragma unroll
                    for (int sl = 0; sl < 4; sl++) {
                        uint4* dst = reinterpret_cast<uint4*>(
                            a.planes + ((size_t)(sl * a.n_kv + g) * (a.rts * AQ) + (size_t)(rt - a.rt0) * AQ + row_in) * a.Kpad + key0);
                        dst[0] = make_uint4(words[sl][0], words[sl][1], words[sl][2], words[sl][3]);
                        dst[1] = make_uint4(words[sl][4], words[sl][5], words[sl][6], words[sl][7]);
                    }
                }
            }
        }
        if (!ok && lane == 0) atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
        if (ok && valid) {
            if (PASS == 1) {
                if (best) atomicMax(a.mxkey + cell, best);
            } else if (dsum) {
                atomicAdd(reinterpret_cast<unsigned long long*>(a.den + cell), dsum);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 256);
}

// ---- P.V.  Warp 0: TMA producer, warp 1: TMEM + MMA issue, warps 2..5: the final drain (one query row per thread).
constexpr int PV_STAGES = 2;
constexpr int PV_A_BYTES = AQ * 128;                          // one slice tile: 128 rows x 128 keys
constexpr int PV_B_BYTES = PV_DIMS * 128;                     // one V byte plane tile: 64 dims x 128 keys
constexpr int PV_STAGE_BYTES = 4 * PV_A_BYTES + 2 * PV_B_BYTES;
constexpr int PV_THREADS = 192;
constexpr size_t PV_SMEM = 1024 + PV_STAGES * PV_STAGE_BYTES + (2 * PV_STAGES + 1) * 8 + 16;

__global__ void __launch_bounds__(PV_THREADS, 1)
k_attn_tc_pv(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_v, const AttnTc a) {
    extern __shared__ __align__(1024) uint8_t pv_raw[];
    uint8_t* stages = align_1k(pv_raw);
    unsigned long long* full = reinterpret_cast<unsigned long long*>(stages + PV_STAGES * PV_STAGE_BYTES);
    unsigned long long* empty = full + PV_STAGES;
    unsigned long long* done = empty + PV_STAGES;
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(done + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int dc = blockIdx.x % (AT_HD / PV_DIMS), zs = blockIdx.x / (AT_HD / PV_DIMS);
    const int g = blockIdx.z, rt = a.rt0 + blockIdx.y;
    const int nkt = tiles_needed(a, rt);
    const int kt0 = zs * a.kt_per_cta;
    const int n = min(nkt, kt0 + a.kt_per_cta) - kt0;
    pdl_trigger();
    if (n <= 0) return;
    const long long wl = wait_limit(a.error_flag);

    if (threadIdx.x == 0) {
        for (int s = 0; s < PV_STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    pdl_wait();
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            int issued = 0;
            for (int l = 0; l < n; l++, issued++) {
                const int s = l % PV_STAGES;
                if (l >= PV_STAGES) {
                    ok = mbar_wait(&empty[s], ((unsigned)(l / PV_STAGES) & 1u) ^ 1u, wl);
                    if (!ok) break;
                }
                uint8_t* st = stages + (size_t)s * PV_STAGE_BYTES;
                const int key0 = (kt0 + l) * AK;
                mbar_expect_tx(&full[s], PV_STAGE_BYTES);
#pragma unroll
                for (int sl = 0; sl < 4; sl++)
                    tma_load_2d(st + sl * PV_A_BYTES, &map_p, key0, ((sl * a.n_kv + g) * a.rts + (rt - a.rt0)) * AQ, &full[s]);
                tma_load_2d(st + 4 * PV_A_BYTES, &map_v, key0, g * AT_HD + dc * PV_DIMS, &full[s]);
                tma_load_2d(st + 4 * PV_A_BYTES + PV_B_BYTES, &map_v, key0, (a.n_kv + g) * AT_HD + dc * PV_DIMS, &full[s]);
            }
            if (!ok) {
                atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
                for (int k = 0; k < PV_STAGES && k < issued; k++) {
                    const int i = issued - 1 - k;
                    (void)mbar_wait(&full[i % PV_STAGES], (unsigned)(i / PV_STAGES) & 1u, wl);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr unsigned UU = umma_idesc_i8(PV_DIMS, false, false), US = umma_idesc_i8(PV_DIMS, false, true);
            for (int l = 0; l < n; l++) {
                const int s = l % PV_STAGES;
                ok = mbar_wait(&full[s], (unsigned)(l / PV_STAGES) & 1u, wl);
                if (!ok) break;
                tc_fence_after();
                const uint8_t* st = stages + (size_t)s * PV_STAGE_BYTES;
                const unsigned long long dlo = umma_desc(st + 4 * PV_A_BYTES), dhi = umma_desc(st + 4 * PV_A_BYTES + PV_B_BYTES);
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const bool first = l == 0 && k == 0;
#pragma unroll
                    for (int sl = 0; sl < 4; sl++) {
                        // accumulator w (TMEM columns 128 w ..) holds weight 2^(8 w): q slice sl x low byte -> w = sl, x high
                        // byte -> w = sl + 1 (in the first step that product is what initialises w = sl + 1); e x low byte
                        // -> w = 0, e x high byte -> w = 1
                        const unsigned long long da = umma_desc(st + sl * PV_A_BYTES) + 2 * k;
                        const int wl_ = sl < 3 ? sl : 0, wh_ = sl < 3 ? sl + 1 : 1;
                        umma_i8(tmem_base + PV_DIMS * wl_, da, dlo + 2 * k, UU, (first && sl == 0) ? 0u : 1u);
                        umma_i8(tmem_base + PV_DIMS * wh_, da, dhi + 2 * k, US, (first && sl < 3) ? 0u : 1u);
                    }
                }
                umma_commit(&empty[s]);
            }
            if (ok) umma_commit(done);
            else atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
        }
    } else {
        const int q = warp & 3;
        const int row = rt * AQ + q * 32 + lane;
        const bool valid = row < a.M * a.rep;
        ok = mbar_wait(done, 0u, wl);
        if (ok) {
            tc_fence_after();
            const size_t cell = (size_t)g * a.Rpad + row;
            const int t = row / a.rep, h = g * a.rep + row % a.rep;
            const float vs = a.v_scale[g];
            const float denf = (valid && a.nz == 1) ? i64_to_f32(a.den[cell]) : 1.0f;
#pragma unroll 1
            for (int c = 0; c < PV_DIMS / 16; c++) {
                int w[4][16];
                const unsigned taddr = tmem_base + ((unsigned)(q * 32) << 16) + c * 16;
#pragma unroll
                for (int i = 0; i < 4; i++) tmem_ld(taddr + PV_DIMS * i, w[i]);
                tmem_wait_ld();
                if (!valid) continue;
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    long long num = (long long)w[0][i];
                    num += (long long)w[1][i] << 8;
                    num += (long long)w[2][i] << 16;
                    num += (long long)w[3][i] << 24;
                    const int d = dc * PV_DIMS + c * 16 + i;
                    if (a.nz == 1) {
                        const float gate = a.qg[((size_t)t * a.n_h + h) * 2 * AT_HD + AT_HD + d];
                        const float val = fmul(fdiv(i64_to_f32(num), denf), vs);
                        a.o[((size_t)t * a.n_h + h) * AT_HD + d] = fmul(val, sigmoid_f(gate));
                    } else if (num) {
                        atomicAdd(reinterpret_cast<unsigned long long*>(a.num + cell * AT_HD + d), (unsigned long long)num);
                    }
                }
            }
        } else if (lane == 0) {
            atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// Key-split launches: o from the summed cells.
__global__ void __launch_bounds__(AT_HD) k_attn_tc_fin(const AttnTc a) {
    pdl_trigger();
    pdl_wait();
    const int g = blockIdx.y, row = a.rt0 * AQ + blockIdx.x, d = threadIdx.x;
    if (row >= a.M * a.rep) return;
    const size_t cell = (size_t)g * a.Rpad + row;
    const int t = row / a.rep, h = g * a.rep + row % a.rep;
    const float gate = a.qg[((size_t)t * a.n_h + h) * 2 * AT_HD + AT_HD + d];
    const float val = fmul(fdiv(i64_to_f32(a.num[cell * AT_HD + d]), i64_to_f32(a.den[cell])), a.v_scale[g]);
    a.o[((size_t)t * a.n_h + h) * AT_HD + d] = fmul(val, sigmoid_f(gate));
}

static bool g_attn_tc = true;
static int g_attn_tc_min_m = 16;
void attn_tc_configure(int on, int min_m) {
    g_attn_tc = on != 0;
    if (min_m > 0) g_attn_tc_min_m = min_m;
}

bool attn_tc_applies(int M, int hd, bool rows_mode, bool device_pos, int n_kv, int keys) {
    if (!g_attn_tc || M < g_attn_tc_min_m || hd != AT_HD || rows_mode || device_pos) return false;
    size_t ws = 0;
    (void)attn_workspace(&ws);
    const size_t Kpad = (size_t)(keys + AK - 1) / AK * AK;
    const size_t vt = 2 * (size_t)n_kv * AT_HD * Kpad, per_tile = 4 * (size_t)n_kv * AQ * Kpad;
    return ws >= vt + per_tile;
}

void attn_tc_run(const AttnTcCall& c, cudaStream_t q) {
    size_t ws_bytes = 0;
    uint8_t* ws = static_cast<uint8_t*>(attn_workspace(&ws_bytes));
    DETB_REQUIRE((reinterpret_cast<uintptr_t>(ws) & 1023) == 0, "the attention workspace must be 1024-byte aligned");
    AttnTc a;
    a.M = c.M; a.n_h = c.n_h; a.n_kv = c.n_kv; a.rep = c.n_h / c.n_kv; a.pos0 = c.pos0; a.keys = c.pos0 + c.M;
    a.Rpad = c.Rpad;
    a.Kpad = (a.keys + AK - 1) / AK * AK;
    a.sq = c.sq; a.sk = c.sk; a.mxkey = c.mxkey; a.den = c.den; a.num = c.num;
    a.qg = c.qg; a.v_scale = c.v_scale; a.o = c.o;
    a.error_flag = error_word();
    const size_t vt_bytes = 2 * (size_t)a.n_kv * AT_HD * a.Kpad, per_tile = 4 * (size_t)a.n_kv * AQ * a.Kpad;
    const int row_tiles = (a.M * a.rep + AQ - 1) / AQ;
    const int fit = (int)std::min<size_t>((size_t)row_tiles, (ws_bytes - vt_bytes) / per_tile);
    DETB_REQUIRE(fit >= 1, "the attention workspace is too small");
    uint8_t* vt = ws;
    a.planes = ws + vt_bytes;

    static bool attrs = false;
    if (!attrs) {
        DETB_CUDA_OK(cudaFuncSetAttribute(k_attn_tc_s<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S_SMEM));
        DETB_CUDA_OK(cudaFuncSetAttribute(k_attn_tc_s<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S_SMEM));
        DETB_CUDA_OK(cudaFuncSetAttribute(k_attn_tc_pv, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PV_SMEM));
        attrs = true;
    }
    // operands as tensor maps (boxes of 128 bytes x rows, 128-byte swizzle = the K-major UMMA layout)
    const cuuint64_t qd[2] = {AT_HD, (cuuint64_t)a.n_kv * a.Rpad}, qs[1] = {AT_HD};
    const cuuint32_t qb[2] = {128, AQ};
    const CUtensorMap map_q = make_map_u8(c.qq, 2, qd, qs, qb);
    const cuuint64_t kd[3] = {AT_HD, (cuuint64_t)a.n_kv, (cuuint64_t)c.capacity};
    const cuuint64_t ks[2] = {AT_HD, (cuuint64_t)a.n_kv * AT_HD};
    const cuuint32_t kb[3] = {128, 1, AK};
    const CUtensorMap map_k = make_map_u8(c.kq, 3, kd, ks, kb);
    const cuuint64_t vd[2] = {(cuuint64_t)a.Kpad, (cuuint64_t)2 * a.n_kv * AT_HD}, vs[1] = {(cuuint64_t)a.Kpad};
    const cuuint32_t vb[2] = {128, PV_DIMS};
    const CUtensorMap map_v = make_map_u8(vt, 2, vd, vs, vb);

    launch_pdl(k_attn_vt, dim3(a.Kpad / 64, a.n_kv), dim3(256), 0, q, 1, c.vq, a.n_kv, a.keys, a.Kpad, vt);
    const int nkt_max = a.Kpad / AK;
    auto score_split = [&](int tiles_in_launch) {   // key tiles per CTA: about two CTAs per SM in total, by shape only
        const int want = std::max(1, 2 * sm_count() / std::max(1, tiles_in_launch * a.n_kv));
        const int splits = std::min(nkt_max, want);
        return (nkt_max + splits - 1) / splits;
    };
    // pass 1 over all row tiles (it needs no workspace)
    a.rt0 = 0; a.rts = row_tiles;
    a.kt_per_cta = score_split(row_tiles);
    a.nz = 1;
    launch_pdl(k_attn_tc_s<1>, dim3((nkt_max + a.kt_per_cta - 1) / a.kt_per_cta, row_tiles, a.n_kv), dim3(S_THREADS), S_SMEM, q, 1,
               map_q, map_k, a);
    for (int rt0 = 0; rt0 < row_tiles; rt0 += fit) {
        a.rt0 = rt0;
        a.rts = std::min(fit, row_tiles - rt0);
        const cuuint64_t pd[2] = {(cuuint64_t)a.Kpad, (cuuint64_t)4 * a.n_kv * a.rts * AQ}, ps[1] = {(cuuint64_t)a.Kpad};
        const cuuint32_t pb[2] = {128, AQ};
        const CUtensorMap map_p = make_map_u8(a.planes, 2, pd, ps, pb);
        a.kt_per_cta = score_split(a.rts);
        a.nz = 1;
        launch_pdl(k_attn_tc_s<2>, dim3((nkt_max + a.kt_per_cta - 1) / a.kt_per_cta, a.rts, a.n_kv), dim3(S_THREADS), S_SMEM, q, 1,
                   map_q, map_k, a);
        a.nz = (nkt_max + PV_MAX_TILES - 1) / PV_MAX_TILES;
        a.kt_per_cta = (nkt_max + a.nz - 1) / a.nz;
        launch_pdl(k_attn_tc_pv, dim3((AT_HD / PV_DIMS) * a.nz, a.rts, a.n_kv), dim3(PV_THREADS), PV_SMEM, q, 1, map_p, map_v, a);
        if (a.nz > 1) launch_pdl(k_attn_tc_fin, dim3(a.rts * AQ, a.n_kv), dim3(AT_HD), 0, q, 1, a);
    }
}

}  // namespace detb

extern "C" {
// Measurement switch: on = 0 keeps prefill attention on the CUDA-core kernels; min_m > 0 sets the batch size from which
// the tensor-core path is used (default 16).  Results do not depend on it.
void det_debug_set_attn_tc(int on, int min_m) { detb::attn_tc_configure(on, min_m); }
}
