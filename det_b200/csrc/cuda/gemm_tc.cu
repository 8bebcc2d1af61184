// Prefill integer GEMM on the 5th-generation tensor cores: tcgen05.mma kind::i8 (s8 x s8 -> s32) with TMA-fed operands
// and TMEM accumulators.  Replaces the reference's mma.sync kernels (kernels/cuda/gemm.cu:496-895) for M > 8.
//
//   acc[t][n] = sum_g (m[n][g] * mx[t][g]) * sum_{k in g} wq[n][k] * xq[t][k]        (docs/SPEC.md §3)
//
// The inner sum of one 128-wide group is four UMMA steps (K = 32 bytes each) into a TMEM tile; the group multiplier
// m * mx is a 32-bit integer that differs per (row, token, group), so every group's s32 tile is drained from TMEM and
// folded into int64 registers by the epilogue warps while the tensor core already works on the following groups in the
// other TMEM buffers.  CTA tile: 128 weight rows (UMMA M, one TMEM lane per row) x 32 / 64 / 128 tokens (UMMA N).
//
// The fold is ONE signed 32 x 32 + 64 multiply-add per (row, token, group): with S the group's s32 sum and u = m * mx
// (up to 2^32 - 2^17, so it does not fit a signed word), the kernel adds S * (u - 2^31), where u - 2^31 does fit, and
// repairs the difference at the end with 2^31 * (sum of S over all groups) — and that plain sum over the whole of K comes
// from the tensor core as well: every UMMA step is issued a second time into a TMEM tile that is never reset (|sum| <=
// K * 128 * 127 < 2^31 for K < 132096).  The tensor pipe has the room; the multiply pipe of the CUDA cores is what the
// fold is short of (measured: with the loads, the MMAs or the TMEM reads switched off the kernel is no faster; without the
// fold arithmetic it is).  The 32-token tile is the exception: its fold is short, the thread that issues the UMMAs sets
// the pace, and the plain sum is kept in registers of the epilogue threads instead (TcCfg::SUM_IN_REGS).
//
// Warp roles (320 threads): warp 0 = TMA producer (one thread), warp 1 = TMEM allocation + MMA issue (one thread),
// warps 2.. = epilogue (warp w reads TMEM lanes 32*(w%4) .. +31 and a block of the token columns).  Operands come from an
// int8-expanded tile-major copy of the weights (det_linear_expand) and from the int8 activations, both through
// 128-byte-swizzled TMA boxes, which is
// the canonical K-major SWIZZLE_128B layout the UMMA shared-memory descriptor names.  No multicast anywhere.
#include "umma.cuh"
#include <algorithm>

namespace detb {

constexpr int TC_ROWS = 128;      // weight rows per CTA (UMMA M)
constexpr int TC_KB = 128;        // bytes of K per stage = one quantization group
constexpr int TC_A_BYTES = TC_ROWS * TC_KB;   // 16 KB
// Per token-tile width TOK (UMMA N, 64 or 128): TOK / 32 epilogue warps per TMEM lane quarter, 32 token columns each;
// two TMEM accumulator buffers of TOK columns; as many stages as fit next to the multiplier table.
// EC = token columns per epilogue warp (8, 16 or 32): 4 * TOK / EC epilogue warps share a group's tile, so a narrower EC
// shortens the per-group drain (what bounds a CTA's K loop) at the price of more threads.
template <int TOK, int EC>
struct TcCfg {
    static constexpr int B_BYTES = TOK * TC_KB;
    static constexpr int STAGE_BYTES = TC_A_BYTES + B_BYTES;
    // The 32-token tile (the serving step) is sized for two CTAs per SM — four stages, half of TMEM: a launch of up to
    // 296 tiles is one wave, and the next launch's CTAs come up beside this launch's last ones.
    static constexpr int MIN_CTAS = TOK == 32 ? 2 : 1;
    static constexpr int STAGES = TOK == 32 ? 4 : (TOK == 64 ? 6 : 5);
    static constexpr int EPI_WARPS = 4 * (TOK / EC);
    static constexpr int THREADS = (2 + EPI_WARPS) * 32;
    // TMEM accumulator buffers: the MMA warp runs up to NBUF groups ahead of the epilogue, which hides the
    // commit -> mbarrier -> tcgen05.ld -> release round trip between the two
    static constexpr int NBUF = TOK == 32 ? 8 : (TOK == 64 ? 4 : 3);
    static constexpr int TOTAL_COL = NBUF * TOK;       // the running plain sum over K lives behind the group buffers
    static constexpr int TMEM_COLS = TOK == 32 ? 256 : 512;     // NBUF * TOK (+ TOK for the running sum) as a power of two
    // Where the plain sum over K is kept: in a TMEM tile fed by a second UMMA per step, or — for the 32-token tile, whose
    // K loop is paced by the MMA issue thread and not by the fold — in 32-bit registers of the epilogue threads (one add
    // per accumulator and group, half the UMMAs).
    static constexpr bool SUM_IN_REGS = TOK == 32;
    // UMMA instruction descriptor (kind::i8): D = s32, A = B = signed 8-bit, both K-major, N = TOK, M = 128.
    static constexpr unsigned IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(TOK >> 3) << 17) | ((TC_ROWS >> 4) << 24);
};

// acc += (s32) p * (s32) mult: one signed 32 x 32 + 64 multiply-add.
__device__ __forceinline__ void mad_s32_s32(long long& acc, int p, int mult) {
    asm("mad.wide.s32 %0, %1, %2, %0;" : "+l"(acc) : "r"(p), "r"(mult));
}

struct TcArgs {
    int N, K, G, M;
    const float* c;
    const uint16_t* m;
    const float* sx;
    const uint16_t* mx;   // may be NULL
    int* error_flag;
    OutSpec out;
    // split K (gridDim.z > 1): each CTA takes a run of groups and adds its exact int64 partial sums into `part`
    // ([tile][token][row]); the CTA that arrives last at the tile's counter converts and emits, and leaves both zeroed
    unsigned long long* part;
    unsigned* counters;
    // A second linear over the same input rows in the same launch (row tiles tiles1 .. of the grid; tiles1 = all of them
    // when there is none): a small linear next to a wide one — the a|b projection beside qkv|z — costs a launch of its own
    // about 10 us whatever its size.
    int tiles1, N2;
    const float* c2;
    const uint16_t* m2;
    OutSpec out2;
};

// Shared memory: [stages x (A 16 KB | B)] (1024-byte aligned) [mx table: G x TOK u16] [barriers] [tmem address]
template <int TOK, int ECW, bool PAIR>
__global__ void __launch_bounds__(TcCfg<TOK, ECW>::THREADS, TcCfg<TOK, ECW>::MIN_CTAS)
k_gemm_tc(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
          const __grid_constant__ CUtensorMap map_x, const TcArgs a) {
    using Cfg = TcCfg<TOK, ECW>;
    constexpr int TC_TOK = TOK, TC_STAGES = Cfg::STAGES, TC_STAGE_BYTES = Cfg::STAGE_BYTES;
    constexpr int TC_EPI_WARPS = Cfg::EPI_WARPS, TC_TMEM_COLS = Cfg::TMEM_COLS, NBUF = Cfg::NBUF;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* stages = smem;
    uint16_t* mxs = reinterpret_cast<uint16_t*>(stages + TC_STAGES * TC_STAGE_BYTES);   // [G][TOK] token multipliers
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(
        (reinterpret_cast<uintptr_t>(mxs + (size_t)a.G * TC_TOK) + 15) & ~(uintptr_t)15);
    unsigned long long* full = bars;                       // [TC_STAGES]  TMA bytes landed
    unsigned long long* empty = bars + TC_STAGES;          // [TC_STAGES]  MMAs that read the stage are done
    unsigned long long* tfull = bars + 2 * TC_STAGES;      // [NBUF]       group result complete in TMEM buffer
    unsigned long long* tempty = tfull + NBUF;             // [NBUF]       epilogue drained the buffer
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(tempty + NBUF);
    float* sxs = reinterpret_cast<float*>(tmem_slot + 4);     // [TOK] token scales, staged with the multipliers

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool second = PAIR && (int)blockIdx.y >= a.tiles1;  // this CTA's row tile belongs to the second linear
    const int ty = second ? (int)blockIdx.y - a.tiles1 : (int)blockIdx.y;
    const CUtensorMap* mapw = second ? &map_w2 : &map_w;
    const int t0 = blockIdx.x * TC_TOK, n0 = ty * TC_ROWS;
    const int G = a.G;
    const long long wl = wait_limit(a.error_flag);
    // this CTA's run of groups: [g0, g0 + GL)
    const int gper = (G + gridDim.z - 1) / gridDim.z;
    const int g0 = blockIdx.z * gper;
    const int GL = max(0, min(G, g0 + gper) - g0);
    pdl_trigger();

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < NBUF; b++) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], TC_EPI_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)),
                     "r"(TC_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        // ---------------- TMA producer.  Weights do not depend on the previous kernel: the first stages' weight boxes are
        // requested before griddepcontrol.wait, the activation boxes after it.
        if (lane == 0) {
            const int lead = GL < TC_STAGES ? GL : TC_STAGES;
            for (int l = 0; l < lead; l++) {
                uint8_t* st = stages + (size_t)l * TC_STAGE_BYTES;
                mbar_expect_tx(&full[l], TC_STAGE_BYTES);
                tma_load_2d(st, mapw, 0, (ty * G + g0 + l) * TC_ROWS, &full[l]);
            }
            pdl_wait();
            for (int l = 0; l < lead; l++)
                tma_load_2d(stages + (size_t)l * TC_STAGE_BYTES + TC_A_BYTES, &map_x, (g0 + l) * TC_KB, t0, &full[l]);
            int issued = lead;
            for (int l = lead; l < GL; l++, issued++) {
                const int s = l % TC_STAGES;
                ok = mbar_wait(&empty[s], ((unsigned)(l / TC_STAGES) & 1u) ^ 1u, wl);
                if (!ok) break;
                uint8_t* st = stages + (size_t)s * TC_STAGE_BYTES;
                mbar_expect_tx(&full[s], TC_STAGE_BYTES);
                tma_load_2d(st, mapw, 0, (ty * G + g0 + l) * TC_ROWS, &full[s]);
                tma_load_2d(st + TC_A_BYTES, &map_x, (g0 + l) * TC_KB, t0, &full[s]);
            }
            if (!ok) {
                atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
                for (int k = 0; k < TC_STAGES && k < issued; k++) {
                    const int i = issued - 1 - k;
                    (void)mbar_wait(&full[i % TC_STAGES], (unsigned)(i / TC_STAGES) & 1u, wl);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue: four K = 32 steps per group into TMEM buffer g & 1
        if (lane == 0) {
            for (int g = 0; g < GL; g++) {          // local group index
                const int s = g % TC_STAGES, b = g % NBUF;
                ok = mbar_wait(&full[s], (unsigned)(g / TC_STAGES) & 1u, wl) &&
                     mbar_wait(&tempty[b], ((unsigned)(g / NBUF) & 1u) ^ 1u, wl);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint8_t* st = stages + (size_t)s * TC_STAGE_BYTES;
                const unsigned long long da = umma_desc(st), db = umma_desc(st + TC_A_BYTES);
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    umma_i8(tmem_base + b * TC_TOK, da + 2 * k, db + 2 * k, Cfg::IDESC, k > 0 ? 1u : 0u);
                    if (!Cfg::SUM_IN_REGS)
                        umma_i8(tmem_base + Cfg::TOTAL_COL, da + 2 * k, db + 2 * k, Cfg::IDESC, (g | k) ? 1u : 0u);
                }
                umma_commit(&empty[s]);
                umma_commit(&tfull[b]);
            }
            if (!ok) atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
        }
    } else {
        // ---------------- epilogue: thread = one weight row x EC tokens, int64 accumulators in registers
        constexpr int EC = ECW;                        // token columns per epilogue warp
        const int q = warp & 3;                        // TMEM lane quarter this warp may read
        const int half = (warp - 2) >> 2;              // which block of 32 token columns
        const int n = n0 + q * 32 + lane;
        const int et = threadIdx.x - 64;
        // the row's scale belongs to the weights: on its way before the previous kernel is waited for
        const int N = second ? a.N2 : a.N;
        // (the 128-token tile has no register to spare for it and fetches the scale when it emits)
        float cn = 0.0f;
        if constexpr (TOK <= 64) cn = n < N ? (second ? a.c2 : a.c)[n] : 0.0f;
        pdl_wait();   // activations, their multipliers and the output rows belong to the previous kernels
        // token multipliers of this CTA's groups only (a split launch walks a fraction of K)
        for (int i = et; i < GL * TC_TOK; i += TC_EPI_WARPS * 32) {
            const int gl = i / TC_TOK, t = i - gl * TC_TOK;
            mxs[(g0 + gl) * TC_TOK + t] = (a.mx && t0 + t < a.M) ? a.mx[(size_t)(t0 + t) * G + g0 + gl] : (uint16_t)1;
        }
        if (et < TC_TOK) sxs[et] = t0 + et < a.M ? a.sx[t0 + et] : 0.0f;
        asm volatile("bar.sync 1, %0;" ::"n"(TC_EPI_WARPS * 32) : "memory");
        long long acc[EC];
        int plain[Cfg::SUM_IN_REGS ? EC : 1];
#pragma unroll
        for (int t = 0; t < EC; t++) acc[t] = 0;
#pragma unroll
        for (int t = 0; t < (Cfg::SUM_IN_REGS ? EC : 1); t++) plain[t] = 0;
        const uint16_t* mrow = (second ? a.m2 : a.m) + (size_t)(n < N ? n : 0) * G;
        unsigned mw_next = GL > 0 ? mrow[g0] : 0u;          // the row's multiplier, fetched one group ahead
        for (int l = 0; l < GL; l++) {
            const int b = l % NBUF, g = g0 + l;
            const unsigned mw = mw_next;
            if (l + 1 < GL) mw_next = mrow[g + 1];
            ok = mbar_wait(&tfull[b], (unsigned)(l / NBUF) & 1u, wl);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            int r[EC];
            tmem_ld(tmem_base + ((unsigned)(q * 32) << 16) + b * TC_TOK + half * EC, r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[b]);
            const unsigned* mxg = reinterpret_cast<const unsigned*>(mxs + g * TC_TOK + half * EC);
#pragma unroll
            for (int t = 0; t < EC; t += 2) {
                const unsigned pair = mxg[t >> 1];     // two u16 multipliers
                mad_s32_s32(acc[t], r[t], (int)(mw * (pair & 0xffffu) + 0x80000000u));
                mad_s32_s32(acc[t + 1], r[t + 1], (int)(mw * (pair >> 16) + 0x80000000u));
            }
            if constexpr (Cfg::SUM_IN_REGS) {
#pragma unroll
                for (int t = 0; t < EC; t++) plain[t] += r[t];
            }
        }
        if constexpr (Cfg::SUM_IN_REGS) {
#pragma unroll
            for (int t = 0; t < EC; t++) acc[t] += (long long)plain[t] << 31;
        } else if (ok && GL > 0) {
            // the last group's commit also covers every step into the running total: add 2^31 * (sum of S) back
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            int r[EC];
            tmem_ld(tmem_base + ((unsigned)(q * 32) << 16) + Cfg::TOTAL_COL + half * EC, r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int t = 0; t < EC; t++) acc[t] += (long long)r[t] << 31;
        }
        if (!ok && lane == 0) atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
        if (gridDim.z > 1) {
            // split K: add this CTA's partial sums to the tile's cells; the last of the tile's CTAs takes the totals
            __shared__ unsigned last_cta;
            const unsigned tile = blockIdx.y * gridDim.x + blockIdx.x;
            unsigned long long* cell = a.part + ((size_t)tile * TC_TOK + half * EC) * TC_ROWS + (q * 32 + lane);
#pragma unroll
            for (int t = 0; t < EC; t++) atomicAdd(cell + (size_t)t * TC_ROWS, (unsigned long long)acc[t]);
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"n"(TC_EPI_WARPS * 32) : "memory");
            if (et == 0) last_cta = atomicAdd(a.counters + tile, 1u) == gridDim.z - 1;
            asm volatile("bar.sync 1, %0;" ::"n"(TC_EPI_WARPS * 32) : "memory");
            if (last_cta) {
                __threadfence();
#pragma unroll
                for (int t = 0; t < EC; t++) acc[t] = (long long)atomicExch(cell + (size_t)t * TC_ROWS, 0ull);
                if (et == 0) a.counters[tile] = 0;
            } else {
                ok = false;        // nothing to emit from this CTA
            }
        }
        if (ok && n < N) {
            const OutSpec& out = second ? a.out2 : a.out;
            if constexpr (TOK > 64) cn = (second ? a.c2 : a.c)[n];
#pragma unroll
            for (int t = 0; t < EC; t++) {
                const int tt = t0 + half * EC + t;
                if (tt < a.M) emit(out, tt, n, fmul(fmul(i64_to_f32(acc[t]), cn), sxs[half * EC + t]));
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_TMEM_COLS)
                     : "memory");
}

// ---- tensor-pipe ceiling: tcgen05.mma kind::i8 issued back to back on resident shared-memory tiles (128 x 256 x 32 per
// instruction, one CTA per SM, no loads, no epilogue).  The measured rate is the denominator for "tensor-pipe
// utilisation" of the GEMM above.  Operand contents are irrelevant (zeros).
__global__ void __launch_bounds__(64, 1) k_umma_peak(int iters, int* error_flag) {
    extern __shared__ __align__(1024) uint8_t peak_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(peak_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* ta = smem;                    // 128 rows x 128 bytes
    uint8_t* tb = smem + 16384;            // 256 rows x 128 bytes
    unsigned long long* bar = reinterpret_cast<unsigned long long*>(smem + 16384 + 32768);
    unsigned* slot = reinterpret_cast<unsigned*>(bar + 1);
    for (int i = threadIdx.x; i < (16384 + 32768) / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long wl = wait_limit(error_flag);
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(slot)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = *slot;
    if (warp == 1 && lane == 0) {
        constexpr unsigned IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);
        const unsigned long long da = umma_desc(ta), db = umma_desc(tb);
        for (int i = 0; i < iters; i++) {
#pragma unroll
            for (int k = 0; k < 4; k++) umma_i8(tmem, da + 2 * k, db + 2 * k, IDESC, (i | k) ? 1u : 0u);
        }
        umma_commit(bar);
        if (!mbar_wait(bar, 0, wl)) atomicExch(error_flag, DETB_ERR_WAIT_EXPIRED);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256) : "memory");
}

// One thread per 32-code block: reference layout -> signed int8 codes in tile-major order
// [N / 128 row tiles][K / 128 groups][128 rows][128 codes], so that the (row tile, group) box one TMA load fetches is 16 KB
// of consecutive memory (whole DRAM pages, whole L2 lines) and a CTA's K loop streams forward.  The last row tile is
// padded with zero rows.
__global__ void k_expand_int8(const uint8_t* __restrict__ wq, int bits, int N, int K, int8_t* __restrict__ dst) {
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int bpr = K / 32;                                  // 32-code blocks per row
    const long long rows_padded = (long long)((N + TC_ROWS - 1) / TC_ROWS) * TC_ROWS;
    if (id >= rows_padded * bpr) return;
    const int n = (int)(id / bpr), kb = (int)(id % bpr);
    __align__(16) int8_t out[32];
    if (n < N) {
        const uint8_t* blk = wq + ((size_t)n * bpr + kb) * bytes_per_32(bits);
        for (int i = 0; i < 32; i++) {
            int v;
            if (bits == 8) v = (int8_t)blk[i];
            else {
                v = (i < 16) ? (blk[i] & 0xF) : (blk[i - 16] >> 4);
                if (bits == 6) v |= ((blk[16 + (i & 7)] >> (2 * (i >> 3))) & 3) << 4;
                v -= code_offset(bits);
            }
            out[i] = (int8_t)v;
        }
    } else {
        for (int i = 0; i < 32; i++) out[i] = 0;
    }
    const int G = K / 128, g = kb >> 2, part = kb & 3;
    const size_t off = ((((size_t)(n / TC_ROWS) * G + g) * TC_ROWS) + (n % TC_ROWS)) * TC_KB + part * 32;
    uint4* d4 = reinterpret_cast<uint4*>(dst + off);
    d4[0] = reinterpret_cast<const uint4*>(out)[0];
    d4[1] = reinterpret_cast<const uint4*>(out)[1];
}

// A [rows][K] int8 matrix as a 2-D tensor map with a (128 bytes x box_rows) box, 128-byte swizzle, zero fill.
static CUtensorMap make_map(const void* base, int rows, int K, int box_rows) {
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K};
    const cuuint32_t box[2] = {(cuuint32_t)TC_KB, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    DETB_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed");
    return map;
}

// Split K for narrow linears at a small batch (switched through det_debug_set_tc_variant: 0x100 on, 0x200 off).
static bool g_tc_splitk = true;

template <int TOK, int EC, bool PAIR>
static void gemm_tc_launch_tok(const det_qlinear* L, const int8_t* xq, const float* sx, const uint16_t* mx, int M,
                               const OutSpec& out, const det_qlinear* L2, const OutSpec* out2, cudaStream_t q) {
    using Cfg = TcCfg<TOK, EC>;
    constexpr int TC_TOK = TOK, TC_STAGES = Cfg::STAGES, TC_STAGE_BYTES = Cfg::STAGE_BYTES;
    const int N = L->N, K = L->K, G = K / 128;
    DETB_REQUIRE((reinterpret_cast<uintptr_t>(L->wq) & 15) == 0 && (reinterpret_cast<uintptr_t>(xq) & 15) == 0,
                 "tensor-core GEMM operands must be 16-byte aligned");
    const int row_tiles = (N + TC_ROWS - 1) / TC_ROWS;
    const CUtensorMap map_w = make_map(L->wq, row_tiles * G * TC_ROWS, TC_KB, TC_ROWS);   // tile-major: one box = 16 KB in a row
    const CUtensorMap map_x = make_map(xq, M, K, TC_TOK);
    TcArgs a;
    a.N = N; a.K = K; a.G = G; a.M = M;
    a.c = L->c; a.m = L->m; a.sx = sx; a.mx = mx;
    a.tiles1 = row_tiles;
    a.N2 = 0; a.c2 = nullptr; a.m2 = nullptr; a.out2 = out;
    CUtensorMap map_w2 = map_w;
    int row_tiles2 = 0;
    if (L2) {
        DETB_REQUIRE(L2->K == K && (reinterpret_cast<uintptr_t>(L2->wq) & 15) == 0, "the second linear shares the input rows");
        row_tiles2 = (L2->N + TC_ROWS - 1) / TC_ROWS;
        map_w2 = make_map(L2->wq, row_tiles2 * G * TC_ROWS, TC_KB, TC_ROWS);
        a.N2 = L2->N; a.c2 = L2->c; a.m2 = L2->m; a.out2 = *out2;
    }
    a.error_flag = error_word();
    a.out = out;
    const size_t smem = 1024 + (size_t)TC_STAGES * TC_STAGE_BYTES + (size_t)G * TC_TOK * 2 + 16 + (2 * TC_STAGES + 2 * Cfg::NBUF) * 8 + 16 +
                        (size_t)TC_TOK * 4;
    DETB_REQUIRE(smem + 64 <= smem_optin(), "K is too large for the tensor-core GEMM's multiplier table");
    static size_t configured = 0;     // the kernel also has a few bytes of static shared memory
    if (smem > configured) {
        DETB_CUDA_OK(cudaFuncSetAttribute(k_gemm_tc<TOK, EC, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    dim3 grid((M + TC_TOK - 1) / TC_TOK, row_tiles + row_tiles2);
    // Few tiles (a narrow linear at a small batch) leave most SMs idle: split K over up to 16 CTAs per tile.  The partial
    // sums are exact integers, so the split cannot change a result.  By shape only.
    a.part = nullptr;
    a.counters = nullptr;
    const int tiles = (int)(grid.x * grid.y);
    int ksplit = 1;
    // A CTA walks its groups one after the other (about 0.6 us each), so with few tiles the launch time is the K loop of one
    // CTA: split it over as many CTAs as there are idle SMs, down to three groups per CTA.
    // (the runtime's cells hold sm_count()/2 + 1 tiles of 128 x 128: four times as many 32-token tiles)
    if (g_tc_splitk && tiles * 2 <= Cfg::MIN_CTAS * sm_count() && G >= 16)
        ksplit = std::min(16, std::min(Cfg::MIN_CTAS * sm_count() / tiles, G / 3));
    if (ksplit > 1) {
        a.part = splitk_cells();          // (sm_count()/2 + 1) tiles of 128 x 128 int64, owned by the runtime
        a.counters = splitk_counters();
        grid.z = ksplit;
    }
    launch_pdl(k_gemm_tc<TOK, EC, PAIR>, grid, dim3(Cfg::THREADS), smem, q, 1, map_w, map_w2, map_x, a);
}

// Tile choice, by shape only: 32 tokens per CTA up to 32 rows (the serving step), 64 up to 64, else 128.  variant 1 / 2 /
// 3 pins the 32 / 64 / 128-token tile (measurement switch).
static int g_tc_variant = 0;
void gemm_tc_launch(const det_qlinear* L, const int8_t* xq, const float* sx, const uint16_t* mx, int M,
                    const OutSpec& out, cudaStream_t q, const det_qlinear* L2, const OutSpec* out2) {
    int v = g_tc_variant;
    if (v == 0) v = M <= 32 ? 1 : (M <= 64 ? 2 : 3);
    if (L2 && v == 3) {
        // the 128-token tile is short of registers as it is: two launches
        gemm_tc_launch_tok<128, 32, false>(L, xq, sx, mx, M, out, nullptr, nullptr, q);
        gemm_tc_launch_tok<128, 32, false>(L2, xq, sx, mx, M, *out2, nullptr, nullptr, q);
        return;
    }
    switch (v) {
        case 1:
            if (L2) gemm_tc_launch_tok<32, 16, true>(L, xq, sx, mx, M, out, L2, out2, q);
            else gemm_tc_launch_tok<32, 16, false>(L, xq, sx, mx, M, out, nullptr, nullptr, q);
            break;
        case 2:
            if (L2) gemm_tc_launch_tok<64, 32, true>(L, xq, sx, mx, M, out, L2, out2, q);
            else gemm_tc_launch_tok<64, 32, false>(L, xq, sx, mx, M, out, nullptr, nullptr, q);
            break;
        case 3: gemm_tc_launch_tok<128, 32, false>(L, xq, sx, mx, M, out, nullptr, nullptr, q); break;
        default: DETB_REQUIRE(false, "unknown tensor-core GEMM variant");
    }
}

}  // namespace detb

using namespace detb;

extern "C" {

// Measurement switch: 0 = tile chosen by shape; 1 / 2 / 3 pin the 32 / 64 / 128-token tile.  Results do not depend on it.
void det_debug_set_tc_variant(int v) {
    g_tc_variant = v & 0xff;
    if (v & 0x300) g_tc_splitk = (v & 0x100) != 0;   // 0x100: split K on, 0x200: off
}

// Runs the tensor-pipe ceiling kernel (one CTA per SM, `iters` x 4 MMAs of 128 x 256 x 32 each) and returns its int8
// rate in TOPS (2 * M * N * K per MMA), timed with events on the library queue; < 0 when a wait expired.
double det_debug_umma_peak(int iters) {
    cudaStream_t q = queue_of(nullptr);
    const size_t smem = 1024 + 16384 + 32768 + 64;
    DETB_CUDA_OK(cudaFuncSetAttribute(k_umma_peak, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaEvent_t e0, e1;
    DETB_CUDA_OK(cudaEventCreate(&e0));
    DETB_CUDA_OK(cudaEventCreate(&e1));
    k_umma_peak<<<sm_count(), 64, smem, q>>>(iters > 64 ? 64 : iters, error_word());     // warm-up
    DETB_CUDA_OK(cudaEventRecord(e0, q));
    k_umma_peak<<<sm_count(), 64, smem, q>>>(iters, error_word());
    DETB_CUDA_OK(cudaEventRecord(e1, q));
    DETB_CUDA_OK(cudaEventSynchronize(e1));
    DETB_CUDA_OK(cudaGetLastError());
    float ms = 0.0f;
    DETB_CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    const double ops = 2.0 * 128 * 256 * 32 * 4.0 * (double)iters * sm_count();
    return ops / (ms * 1e-3) / 1e12;
}

size_t det_linear_expand_bytes(int N, int K) { return (size_t)((N + TC_ROWS - 1) / TC_ROWS) * TC_ROWS * (size_t)K; }

void det_linear_expand(const det_qlinear* src, void* dst, cudaStream_t st) {
    DETB_REQUIRE((src->bits == 4 || src->bits == 6 || src->bits == 8) && src->K % 128 == 0, "bad linear shape");
    const long long nblocks = (long long)((src->N + TC_ROWS - 1) / TC_ROWS) * TC_ROWS * (src->K / 32);
    k_expand_int8<<<(unsigned)((nblocks + 255) / 256), 256, 0, queue_of(st)>>>(src->wq, src->bits, src->N, src->K,
                                                                              static_cast<int8_t*>(dst));
    DETB_CUDA_OK(cudaGetLastError());
}

}  // extern "C"
