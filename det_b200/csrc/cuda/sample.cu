// Deterministic sampling (docs/SPEC.md §5.5, spec/sample.rs:16-87).  Replaces kernels/cuda/sample.cu behind
// det_sample / det_sample_topkp / det_sample_scratch_bytes.
//
// After w_i = rint(exp_f(l_i * inv_temp - max) * 2^32) everything is exact integer arithmetic, so any parallel
// decomposition is legal.  The candidate order (weight descending, index ascending) is never materialised: the kept set
// is a prefix of that order, i.e. "w > w*" plus the first e elements (by index) with w == w*.  (w*, e) comes from a
// three-pass radix select on the 33-bit weights with per-digit (count, sum) histograms in shared memory, which finds the
// element where the first of the two prefix conditions — k elements taken, or the integer mass reaching
// ceil(p24 * total / 2^24) — becomes true.  The draw then walks the kept weights in index order.
// One CTA of 1024 threads per row.
#include "runtime.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace detb {

constexpr int ST = 1024;
constexpr int SW = ST / 32;
constexpr int DIGITS = 2048;
typedef unsigned long long u64;

__device__ __forceinline__ u64 shfl_u64(u64 v, int src) {
    unsigned lo = (unsigned)v, hi = (unsigned)(v >> 32);
    lo = __shfl_sync(FULL, lo, src);
    hi = __shfl_sync(FULL, hi, src);
    return ((u64)hi << 32) | lo;
}
__device__ __forceinline__ u64 shfl_up_u64(u64 v, int d) {
    unsigned lo = (unsigned)v, hi = (unsigned)(v >> 32);
    lo = __shfl_up_sync(FULL, lo, d);
    hi = __shfl_up_sync(FULL, hi, d);
    return ((u64)hi << 32) | lo;
}
__device__ __forceinline__ u64 warp_sum_u64(u64 v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        unsigned lo = (unsigned)v, hi = (unsigned)(v >> 32);
        lo = __shfl_xor_sync(FULL, lo, off);
        hi = __shfl_xor_sync(FULL, hi, off);
        v += ((u64)hi << 32) | lo;
    }
    return v;
}
__device__ __forceinline__ u64 warp_incl_scan_u64(u64 v, int lane) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const u64 o = shfl_up_u64(v, d);
        if (lane >= d) v += o;
    }
    return v;
}
// block-wide sum; every thread returns the total
__device__ u64 block_sum_u64(u64 v, u64* sh /* [SW] */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum_u64(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    u64 t = sh[lane];   // SW == 32
    return warp_sum_u64(t);
}

__device__ __forceinline__ u64 weight_of(float logit, float inv_temp, float mx) {
    return __float2ull_rn(fmul(exp_f(fsub(fmul(logit, inv_temp), mx)), 4294967296.0f));
}

struct Cut {
    int filtered;   // 0: every token kept
    u64 wstar;      // kept: w > wstar, plus the first `e` (by index) with w == wstar
    u64 e;
    u64 total;      // sum of kept weights
};

// The draw: smallest kept index whose inclusive prefix of kept weights exceeds u = z % total.  It runs over a
// contiguous index range [lo, hi) owned by one CTA (the whole row, or one eighth of it in the cluster kernel) in three
// steps, so that several CTAs can chain their ranges: count the elements equal to the cut weight, then the kept mass
// given how many equal elements precede the range, then the walk inside the range that contains the draw.
// Warp w owns [lo + w * wseg, lo + (w + 1) * wseg); W(i) returns the weight of index i.
struct WalkRange {
    int lo, hi, wseg;
    __device__ WalkRange(int lo_, int hi_) : lo(lo_), hi(hi_) {
        const int len = hi_ > lo_ ? hi_ - lo_ : 0;
        wseg = (((len + SW - 1) / SW) + 31) & ~31;
        if (wseg == 0) wseg = 32;
    }
    __device__ int wlo() const { return lo + (threadIdx.x >> 5) * wseg; }
    __device__ int whi() const { return min(hi, wlo() + wseg); }
};

// elements of the range equal to the cut weight: per warp into sh32[], returns the range's total
template <class WF>
__device__ unsigned range_eq(const WF& W, const WalkRange& r, const Cut& cut, unsigned* sh32) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned eq = 0;
    if (cut.filtered)
        for (int i = r.wlo() + lane; i < r.whi(); i += 32) eq += (W(i) == cut.wstar) ? 1u : 0u;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) eq += __shfl_xor_sync(FULL, eq, off);
    __syncthreads();
    if (lane == 0) sh32[warp] = eq;
    __syncthreads();
    unsigned tot = 0;
    for (int w = 0; w < SW; w++) tot += sh32[w];
    return tot;
}

// kept weight of index base + lane (all lanes of the warp in lockstep); eq_seen counts the equal elements before it
template <class WF>
__device__ __forceinline__ u64 kept_weight(const WF& W, const Cut& cut, int i, int hi, u64& eq_seen) {
    const int lane = threadIdx.x & 31;
    const bool in = i < hi;
    const u64 wv = in ? W(i) : 0;
    if (!cut.filtered) return wv;
    const bool is_eq = in && wv == cut.wstar;
    const unsigned mask = __ballot_sync(FULL, is_eq);
    const u64 rank = eq_seen + __popc(mask & ((1u << lane) - 1u));
    eq_seen += __popc(mask);
    if (!in) return 0;
    if (wv > cut.wstar) return wv;
    return (is_eq && rank < cut.e) ? wv : 0;
}

// kept mass of the range given `eq_before` equal elements in front of it: per warp into sh64[], returns the total.
// sh32[] must still hold range_eq's per-warp counts.
template <class WF>
__device__ u64 range_mass(const WF& W, const WalkRange& r, const Cut& cut, u64 eq_before, const unsigned* sh32, u64* sh64) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    u64 seen = eq_before;
    for (int w = 0; w < warp; w++) seen += sh32[w];
    u64 mass = 0;
    for (int b = r.wlo(); b < r.wlo() + r.wseg; b += 32) mass += kept_weight(W, cut, b + lane, r.whi(), seen);
    mass = warp_sum_u64(mass);
    __syncthreads();
    if (lane == 0) sh64[warp] = mass;
    __syncthreads();
    u64 tot = 0;
    for (int w = 0; w < SW; w++) tot += sh64[w];
    return tot;
}

// the walk inside the range that holds the draw: `before` is the kept mass in front of the range.  Returns the index
// in every thread (through sh32[0]).
template <class WF>
__device__ int range_pick(const WF& W, const WalkRange& r, const Cut& cut, u64 eq_before, u64 before, u64 u,
                          unsigned* sh32, const u64* sh64) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    u64 eq_base = eq_before;
    for (int w = 0; w < warp; w++) eq_base += sh32[w];
    int target = -1;
    for (int w = 0; w < SW; w++) {
        const u64 m = sh64[w];
        if (target < 0 && before + m > u) target = w;
        if (target < 0) before += m;
    }
    __syncthreads();
    int result = -1;
    if (warp == target) {
        u64 run = before, seen = eq_base;
        for (int b = r.wlo(); b < r.wlo() + r.wseg && result < 0; b += 32) {
            const u64 kw = kept_weight(W, cut, b + lane, r.whi(), seen);
            const u64 incl = warp_incl_scan_u64(kw, lane) + run;
            const unsigned hit = __ballot_sync(FULL, kw != 0 && incl > u);
            if (hit) result = b + __ffs(hit) - 1;
            run = shfl_u64(incl, 31);
        }
        if (lane == 0) sh32[0] = (unsigned)result;
    }
    __syncthreads();
    return (int)sh32[0];
}

// one CTA owns the whole row
template <class WF>
__device__ int walk(const WF& W, int V, const Cut& cut, u64 z, u64* sh64, unsigned* sh32) {
    const WalkRange r(0, V);
    (void)range_eq(W, r, cut, sh32);
    (void)range_mass(W, r, cut, 0, sh32, sh64);
    return range_pick(W, r, cut, 0, 0, z % cut.total, sh32, sh64);
}

__global__ void __launch_bounds__(ST) k_sample_plain(const float* __restrict__ logits, int V, float inv_temp,
                                                     const u64* __restrict__ z, int* __restrict__ out) {
    __shared__ float shf[32];
    __shared__ u64 sh64[SW];
    __shared__ unsigned sh32[SW];
    const float* row = logits + (size_t)blockIdx.x * V;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += ST) mx = fmaxf(mx, fmul(row[i], inv_temp));
    mx = max_block<SW>(mx, shf);
    u64 part = 0;
    for (int i = threadIdx.x; i < V; i += ST) part += weight_of(row[i], inv_temp, mx);
    Cut cut;
    cut.filtered = 0; cut.wstar = 0; cut.e = 0;
    cut.total = block_sum_u64(part, sh64);
    auto W = [&](int i) { return weight_of(row[i], inv_temp, mx); };
    const int r = walk(W, V, cut, z[blockIdx.x], sh64, sh32);
    if (threadIdx.x == 0) out[blockIdx.x] = r;
}

__global__ void __launch_bounds__(ST) k_sample_topkp(const float* __restrict__ logits, int V, float inv_temp,
                                                     int use_k, u64 top_k, int use_p, u64 p24,
                                                     const u64* __restrict__ z, int* __restrict__ out,
                                                     u64* __restrict__ wbuf_all) {
    __shared__ float shf[32];
    __shared__ u64 sh64[SW];
    __shared__ unsigned sh32[SW];
    __shared__ unsigned cnt[DIGITS];
    __shared__ u64 sum[DIGITS];
    __shared__ u64 sel[6];   // prefix value, k_left, s_left, sum_gt, cnt_sel, found
    const float* row = logits + (size_t)blockIdx.x * V;
    u64* wbuf = wbuf_all + (size_t)blockIdx.x * V;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += ST) mx = fmaxf(mx, fmul(row[i], inv_temp));
    mx = max_block<SW>(mx, shf);
    u64 part = 0;
    for (int i = threadIdx.x; i < V; i += ST) {
        const u64 wv = weight_of(row[i], inv_temp, mx);
        wbuf[i] = wv;
        part += wv;
    }
    const u64 total = block_sum_u64(part, sh64);
    if (threadIdx.x == 0) {
        // thresh = ceil(total * p24 / 2^24)  (spec/sample.rs:60-62), 128-bit intermediate
        const unsigned __int128 prod = (unsigned __int128)total * p24 + ((((unsigned __int128)1) << 24) - 1);
        sel[0] = 0;
        sel[1] = use_k ? top_k : (u64)V;
        sel[2] = (u64)(prod >> 24);
        sel[3] = 0;
    }
    __syncthreads();
    // three 11-bit digits, most significant first: bits [32:22], [21:11], [10:0]
    for (int pass = 0; pass < 3; pass++) {
        const int shift = 22 - 11 * pass;
        for (int i = threadIdx.x; i < DIGITS; i += ST) { cnt[i] = 0; sum[i] = 0; }
        __syncthreads();
        const u64 prefix = sel[0];
        // Most weights of a peaked distribution share one digit (the smallest): a thread keeps the running (count, sum)
        // of its current digit in registers and touches shared memory only when the digit changes.
        unsigned run_d = 0, run_c = 0;
        u64 run_s = 0;
        for (int i = threadIdx.x; i < V; i += ST) {
            const u64 wv = wbuf[i];
            if (pass == 0 || (wv >> (shift + 11)) == prefix) {
                const unsigned d = (unsigned)(wv >> shift) & (DIGITS - 1);
                if (d != run_d && run_c) {
                    atomicAdd(&cnt[run_d], run_c);
                    atomicAdd(&sum[run_d], run_s);
                    run_c = 0;
                    run_s = 0;
                }
                run_d = d;
                run_c++;
                run_s += wv;
            }
        }
        if (run_c) {
            atomicAdd(&cnt[run_d], run_c);
            atomicAdd(&sum[run_d], run_s);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            u64 k_left = sel[1], s_left = sel[2], sum_gt = sel[3];
            int chosen = 0;
            for (int d = DIGITS - 1; d >= 0; d--) {
                const unsigned c = cnt[d];
                if (!c) continue;
                if ((u64)c >= k_left || (use_p && sum[d] >= s_left)) { chosen = d; break; }
                k_left -= c;
                s_left -= sum[d];
                sum_gt += sum[d];
                chosen = d;   // stays the lowest non-empty digit when nothing triggers (cannot happen for valid input)
            }
            sel[0] = (prefix << 11) | (u64)chosen;
            sel[1] = k_left; sel[2] = s_left; sel[3] = sum_gt;
            sel[4] = cnt[chosen];
        }
        __syncthreads();
    }
    Cut cut;
    cut.filtered = 1;
    cut.wstar = sel[0];
    {
        const u64 k_left = sel[1], s_left = sel[2], n_eq = sel[4];
        u64 e = n_eq;
        if (use_k && k_left < e) e = k_left;
        if (use_p) {
            u64 ep;
            if (s_left == 0) ep = 1;
            else if (cut.wstar == 0) ep = n_eq;
            else ep = (s_left + cut.wstar - 1) / cut.wstar;
            if (ep < e) e = ep;
        }
        cut.e = e;
        cut.total = sel[3] + e * cut.wstar;
    }
    auto W = [&](int i) { return wbuf[i]; };
    const int r = walk(W, V, cut, z[blockIdx.x], sh64, sh32);
    if (threadIdx.x == 0) out[blockIdx.x] = r;
}

// ---- the sampler for vocabularies up to 262144: a thread-block cluster per row (8 CTAs above 32768 tokens, else 1), each
// CTA owning a contiguous index range of at most 32768 weights that it keeps in shared memory (low 32 bits + one bit
// plane for 2^32).  The cut weight w* is found by an 11-step radix select on 3-bit digits, most significant first: every
// thread bins its elements that match the prefix so far into eight (count, sum) pairs held in REGISTERS — no atomics,
// which is what bounded the histogram version — the pairs are reduced over the CTA by shuffles and over the cluster
// through distributed shared memory (integer sums: order-free), and every CTA takes the same decision from the same
// totals.  One cluster barrier per step (the exchange slots alternate).  The draw then walks the kept weights in index
// order, range by range (WalkRange).
constexpr int SCL = 8;
constexpr int SEL_RANGE = 32768;                  // weights per CTA
constexpr int SEL_SMEM = SEL_RANGE * 4 + SEL_RANGE / 8;

__device__ __forceinline__ u64 cluster_sum(cg::cluster_group& cluster, u64* slot, u64 mine, unsigned upto, u64* total) {
    // publishes `mine`, returns the sum over ranks < upto; *total = sum over all ranks.  Two cluster barriers.
    if (threadIdx.x == 0) *slot = mine;
    cluster.sync();
    u64 before = 0, all = 0;
    for (unsigned r = 0; r < cluster.num_blocks(); r++) {
        const u64 v = *cluster.map_shared_rank(slot, r);
        if (r < upto) before += v;
        all += v;
    }
    cluster.sync();
    if (total) *total = all;
    return before;
}

__global__ void __launch_bounds__(ST) k_sample_topkp_sel(const float* __restrict__ logits, int V, float inv_temp,
                                                         int use_k, u64 top_k, int use_p, u64 p24,
                                                         const u64* __restrict__ z, int* __restrict__ out,
                                                         u64* __restrict__ wbuf_all) {
    extern __shared__ __align__(16) unsigned sel_smem[];
    unsigned* wlo = sel_smem;                     // low 32 bits of the range's weights
    unsigned* whi = sel_smem + SEL_RANGE;         // bit 32, one bit per weight
    __shared__ float shf[32];
    __shared__ u64 sh64[SW];
    __shared__ unsigned sh32[SW];
    __shared__ unsigned red_c[SW][8];
    __shared__ u64 red_s[SW][8];
    __shared__ unsigned slot_c[2][8];             // this CTA's digit counts / sums of a step (read by the cluster)
    __shared__ u64 slot_s[2][8];
    __shared__ unsigned tot_c[8];
    __shared__ u64 tot_s[8];
    __shared__ u64 sel[6];                        // prefix value, k_left, s_left, sum_gt, cnt_sel
    __shared__ u64 slot;
    __shared__ float fslot;
    pdl_trigger();
    pdl_wait();
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank(), nranks = cluster.num_blocks();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rowi = blockIdx.y;
    const float* row = logits + (size_t)rowi * V;
    u64* wbuf = wbuf_all + (size_t)rowi * V;
    const int seg = (((V + (int)nranks - 1) / (int)nranks) + 1023) & ~1023;      // <= SEL_RANGE by the launcher's rule
    const int lo = min(V, (int)rank * seg), hi = min(V, lo + seg), len = hi - lo;

    float mx = -INFINITY;
    for (int i = lo + threadIdx.x; i < hi; i += ST) mx = fmaxf(mx, fmul(row[i], inv_temp));
    mx = max_block<SW>(mx, shf);
    if (threadIdx.x == 0) fslot = mx;
    cluster.sync();
    for (unsigned r = 0; r < nranks; r++) mx = fmaxf(mx, *cluster.map_shared_rank(&fslot, r));
    cluster.sync();

    u64 part = 0;
    for (int j = threadIdx.x; j < seg; j += ST) {          // whole warps: the ballot needs every lane
        u64 wv = 0;
        if (j < len) {
            wv = weight_of(row[lo + j], inv_temp, mx);
            wbuf[lo + j] = wv;
            wlo[j] = (unsigned)wv;
            part += wv;
        }
        const unsigned top = __ballot_sync(FULL, (wv >> 32) != 0);
        if (lane == 0 && j < len) whi[j >> 5] = top;
    }
    u64 total = 0;
    (void)cluster_sum(cluster, &slot, block_sum_u64(part, sh64), 0, &total);
    if (threadIdx.x == 0) {
        // thresh = ceil(total * p24 / 2^24)  (spec/sample.rs:60-62), 128-bit intermediate
        const unsigned __int128 prod = (unsigned __int128)total * p24 + ((((unsigned __int128)1) << 24) - 1);
        sel[0] = 0;
        sel[1] = use_k ? top_k : (u64)V;
        sel[2] = (u64)(prod >> 24);
        sel[3] = 0;
    }
    __syncthreads();
    // eleven 3-bit digits, most significant first: bits [32:30], [29:27], ..., [2:0]
    for (int pass = 0; pass < 11; pass++) {
        const int shift = 30 - 3 * pass;
        const u64 prefix = sel[0];
        unsigned c[8];
        u64 sm[8];
#pragma unroll
        for (int b = 0; b < 8; b++) { c[b] = 0; sm[b] = 0; }
        for (int j = threadIdx.x; j < len; j += ST) {
            const u64 wv = (u64)wlo[j] | ((u64)((whi[j >> 5] >> (j & 31)) & 1u) << 32);
            if (pass == 0 || (wv >> (shift + 3)) == prefix) {
                const unsigned d = (unsigned)(wv >> shift) & 7u;
#pragma unroll
                for (int b = 0; b < 8; b++) {
                    const bool hit = d == (unsigned)b;
                    c[b] += hit ? 1u : 0u;
                    sm[b] += hit ? wv : 0ull;
                }
            }
        }
#pragma unroll
        for (int b = 0; b < 8; b++) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) c[b] += __shfl_xor_sync(FULL, c[b], off);
            sm[b] = warp_sum_u64(sm[b]);
        }
        if (lane == 0) {
#pragma unroll
            for (int b = 0; b < 8; b++) { red_c[warp][b] = c[b]; red_s[warp][b] = sm[b]; }
        }
        __syncthreads();
        const int par = pass & 1;
        if (threadIdx.x < 8) {
            unsigned cc = 0;
            u64 ss = 0;
            for (int w = 0; w < SW; w++) { cc += red_c[w][threadIdx.x]; ss += red_s[w][threadIdx.x]; }
            slot_c[par][threadIdx.x] = cc;
            slot_s[par][threadIdx.x] = ss;
        }
        cluster.sync();                 // every range's digit sums of this step are published
        if (threadIdx.x < 8) {
            unsigned cc = 0;
            u64 ss = 0;
            for (unsigned r = 0; r < nranks; r++) {
                cc += cluster.map_shared_rank(&slot_c[par][0], r)[threadIdx.x];
                ss += cluster.map_shared_rank(&slot_s[par][0], r)[threadIdx.x];
            }
            tot_c[threadIdx.x] = cc;
            tot_s[threadIdx.x] = ss;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            u64 k_left = sel[1], s_left = sel[2], sum_gt = sel[3];
            int chosen = 0;
            for (int d = 7; d >= 0; d--) {
                const unsigned cd = tot_c[d];
                if (!cd) continue;
                if ((u64)cd >= k_left || (use_p && tot_s[d] >= s_left)) { chosen = d; break; }
                k_left -= cd;
                s_left -= tot_s[d];
                sum_gt += tot_s[d];
                chosen = d;   // stays the lowest non-empty digit when nothing triggers (cannot happen for valid input)
            }
            sel[0] = (prefix << 3) | (u64)chosen;
            sel[1] = k_left; sel[2] = s_left; sel[3] = sum_gt;
            sel[4] = tot_c[chosen];
        }
        __syncthreads();
    }
    Cut cut;
    cut.filtered = 1;
    cut.wstar = sel[0];
    {
        const u64 k_left = sel[1], s_left = sel[2], n_eq = sel[4];
        u64 e = n_eq;
        if (use_k && k_left < e) e = k_left;
        if (use_p) {
            u64 ep;
            if (s_left == 0) ep = 1;
            else if (cut.wstar == 0) ep = n_eq;
            else ep = (s_left + cut.wstar - 1) / cut.wstar;
            if (ep < e) e = ep;
        }
        cut.e = e;
        cut.total = sel[3] + e * cut.wstar;
    }
    auto W = [&](int i) { return wbuf[i]; };
    const WalkRange r(lo, hi);
    const u64 eq_before = cluster_sum(cluster, &slot, (u64)range_eq(W, r, cut, sh32), rank, nullptr);
    const u64 mass = range_mass(W, r, cut, eq_before, sh32, sh64);
    const u64 before = cluster_sum(cluster, &slot, mass, rank, nullptr);
    const u64 u = z[rowi] % cut.total;
    if (before <= u && u < before + mass) {          // exactly one range holds the draw
        const int pick = range_pick(W, r, cut, eq_before, before, u, sh32, sh64);
        if (threadIdx.x == 0) out[rowi] = pick;
    }
}

// Launches the top-k / top-p kernel for a shape: the register-binned cluster kernel up to 262144 tokens, the
// shared-memory histogram kernel (one CTA per row) above.
static cudaError_t launch_topkp(const float* logits, int M, int V, float inv_temp, int use_k, u64 top_k, int use_p, u64 p24,
                                const u64* z, int* out, u64* wbuf, cudaStream_t q) {
    if (V <= SCL * SEL_RANGE) {
        const int cl = V > SEL_RANGE ? SCL : 1;
        // the opt-in shared-memory size is a per-device property of the function: set it once on every device used
        static bool attr[64] = {};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev < 0 || dev >= 64 || !attr[dev]) {
            e = cudaFuncSetAttribute(k_sample_topkp_sel, cudaFuncAttributeMaxDynamicSharedMemorySize, SEL_SMEM);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) attr[dev] = true;
        }
        return launch_pdl_try(k_sample_topkp_sel, dim3(cl, M), dim3(ST), SEL_SMEM, q, cl, logits, V, inv_temp, use_k, top_k,
                              use_p, p24, z, out, wbuf);
    }
    k_sample_topkp<<<M, ST, 0, q>>>(logits, V, inv_temp, use_k, top_k, use_p, p24, z, out, wbuf);
    return cudaGetLastError();
}

// ---- scratch that lives in the library image, for det_sample_topkp_static
constexpr long long STATIC_SAMPLE_MAX = 1ll << 19;   // M * V weights of 8 bytes: 4 MiB per GPU that loads the library
static __device__ __align__(256) unsigned long long g_static_weights[STATIC_SAMPLE_MAX];

}  // namespace detb

using namespace detb;

extern "C" {

size_t det_sample_scratch_bytes(int M, int V) { return (size_t)(M > 0 ? M : 1) * (size_t)V * sizeof(u64); }

void det_sample(const float* logits, int M, int V, float inv_temp, const unsigned long long* z, int* out,
                cudaStream_t st) {
    if (M <= 0) return;
    k_sample_plain<<<M, ST, 0, queue_of(st)>>>(logits, V, inv_temp, z, out);
    DETB_CUDA_OK(cudaGetLastError());
}

void det_sample_topkp(const float* logits, int M, int V, float inv_temp, int top_k, float top_p,
                      const unsigned long long* z, int* out, void* scratch, cudaStream_t st) {
    if (M <= 0) return;
    const int use_k = top_k > 0 && top_k < V;
    const int use_p = top_p < 1.0f;
    if (!use_k && !use_p) {
        det_sample(logits, M, V, inv_temp, z, out, st);
        return;
    }
    // p24 = rint(top_p * 2^24) in binary64; negative values (and NaN) become 0, as Rust's `as u128` does
    double pr = __builtin_nearbyint((double)top_p * 16777216.0);
    const u64 p24 = (pr != pr || pr <= 0.0) ? 0 : (u64)pr;
    DETB_CUDA_OK(launch_topkp(logits, M, V, inv_temp, use_k, (u64)(top_k > 0 ? top_k : 0), use_p, p24, z, out,
                              static_cast<u64*>(scratch), queue_of(st)));
}

// Top-k / top-p sampling for callers that must not allocate.  Same result as det_sample_topkp, but the weight buffer is
// a fixed array inside the library image instead of a caller-provided scratch, and the call itself never reaches an
// allocator: no cudaMalloc, no cudaFree, no allocating library routine.  That is for hosts that fix their device-memory
// budget at start-up and ban allocation afterwards (an allocation can stall on the driver lock or fail once the KV cache
// owns the rest of HBM), and for plug-ins that only ever receive pointers and own no allocator.
//
// Limits and rules:
//   * M * V <= 524288 weights (4 MiB; one row of a 248320-token vocabulary fits twice over) whenever a top-k or top-p
//     filter is active.  Larger filtered requests are refused: the function prints the reason, launches nothing and
//     returns 1.  A request without an active filter (top_k <= 0 or >= V, top_p >= 1) needs no scratch and is taken at
//     any size.  0 means the work was queued; a launch the runtime rejects also returns 1 (it never aborts).
//   * det_init() must have succeeded earlier (this call does not bring the runtime up, since that allocates).
//   * The first call on a device looks the array's device address up (cudaGetSymbolAddress, with that device current),
//     which is also when the driver loads the module that holds the array; make that first call at start-up, outside any
//     stream capture.
//   * Every call uses the same array and finds the previous call's weights in it.  Nothing has to be cleared: the kernel
//     writes every weight of its rows before it reads any.  Two calls that overlap on the GPU (different streams) race
//     on the array; keep them on one stream or order them yourself.
int det_sample_topkp_static(const float* logits, int M, int V, float inv_temp, int top_k, float top_p,
                            const unsigned long long* z, int* out, cudaStream_t st) {
    if (M <= 0) return 0;
    if (V <= 0) {
        fprintf(stderr, "det_b200: det_sample_topkp_static: V = %d is not a vocabulary size\n", V);
        return 1;
    }
    const int use_k = top_k > 0 && top_k < V;
    const int use_p = top_p < 1.0f;
    if ((use_k || use_p) && (long long)M * V > STATIC_SAMPLE_MAX) {
        fprintf(stderr, "det_b200: det_sample_topkp_static: M * V = %lld exceeds the built-in scratch of %lld weights\n",
                (long long)M * V, STATIC_SAMPLE_MAX);
        return 1;
    }
    if (!runtime_is_up()) {
        fprintf(stderr, "det_b200: det_sample_topkp_static: call det_init() first\n");
        return 1;
    }
    // one address per device: in host code the array's name is only a handle, never a device pointer
    static unsigned long long* addr[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        fprintf(stderr, "det_b200: det_sample_topkp_static: no current device\n");
        return 1;
    }
    if (!addr[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_weights);
        if (e != cudaSuccess || !p) {
            fprintf(stderr, "det_b200: det_sample_topkp_static: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
            return 1;
        }
        addr[dev] = static_cast<unsigned long long*>(p);
    }
    if (!use_k && !use_p) {
        k_sample_plain<<<M, ST, 0, queue_of(st)>>>(logits, V, inv_temp, z, out);
    } else {
        double pr = __builtin_nearbyint((double)top_p * 16777216.0);
        const u64 p24 = (pr != pr || pr <= 0.0) ? 0 : (u64)pr;
        const cudaError_t le = launch_topkp(logits, M, V, inv_temp, use_k, (u64)(top_k > 0 ? top_k : 0), use_p, p24, z, out,
                                            addr[dev], queue_of(st));
        if (le != cudaSuccess) {
            fprintf(stderr, "det_b200: det_sample_topkp_static: launch failed: %s\n", cudaGetErrorString(le));
            return 1;
        }
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        fprintf(stderr, "det_b200: det_sample_topkp_static: launch failed: %s\n", cudaGetErrorString(e));
        return 1;
    }
    return 0;
}

}  // extern "C"
