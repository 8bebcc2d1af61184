// Gated full attention with an int8 K / int16 V cache (docs/SPEC.md §5.1, spec/layers.rs:5-87, cpu.rs:216-291).
// Replaces kernels/cuda/attn.cu behind det_attention / det_attention_dev / det_attn_scratch_bytes.
//
//   prep   one warp per (token, head) row: RMSNorm -> RoPE -> (q: * 1/sqrt(hd)) -> per-row int8; k rows and int16 v rows
//          go straight into the cache at position pos0 + t, q rows into scratch.
//   max    pass 1 over the keys: the largest score ((float)dot * sq) * sk per (token, q head), order-free, merged across
//          key splits with an integer atomicMax on an order-preserving key.
//   acc    pass 2: pq = rint(exp_f(s - max) * 2^24), den = sum pq, num[d] = sum pq * vq[d] in int64.  Integer sums are
//          exact in any order, so key ranges are split over CTAs and merged with 64-bit atomic adds.
//   fin    o = (((float)num / (float)den) * v_scale) * sigmoid_f(gate)
// All query heads that share a kv head are handled by the same CTA so K and V tiles are read once per group.
#include "attn_tc.cuh"

namespace detb {

constexpr int KT = 64;           // keys per shared-memory tile
constexpr int ATT_THREADS = 256;
constexpr int MAX_REP = 8;       // q heads per kv head

struct AttnArgs {
    // layer / cache
    const float *q_norm, *k_norm, *v_scale, *v_inv;
    int8_t* kq;
    float* sk;
    int16_t* vq;
    // inputs
    const float *qg, *k, *v, *rope_cos, *rope_sin;
    int rot;
    float eps, qscale;
    int M, n_h, n_kv, rep;
    int pos0;                // used when pos0_dev == NULL
    const int* pos0_dev;
    // batched decode: token row t belongs to its own sequence with cache rows[t] at position pos_rows[t]
    const det_kv_cache* rows;
    const int* pos_rows;
    float* o;
    // scratch
    int8_t* qq;              // [M][n_h][HD]
    float* sq;               // [M][n_h]
    unsigned* mxkey;         // [M][n_h]
    long long* den;          // [M][n_h]
    long long* num;          // [M][n_h][HD]
    unsigned* bar;           // [M][n_kv] CTAs of a (token, kv head) that have published their maxima (fused decode kernel)
    unsigned* done;          // [M][n_kv] CTAs that have added their partial sums
    int* error_flag;
    int nsplit, keys_per_split;
    int tc_rpad;             // > 0: the tile layout of the tensor-core path (attn_tc.cuh), rows per kv head
};
// scratch cell of query row (token t, head h)
__device__ __forceinline__ size_t q_cell(const AttnArgs& a, int t, int h) {
    if (a.tc_rpad) {
        const int g = h / a.rep;
        return (size_t)g * a.tc_rpad + (size_t)t * a.rep + (h - g * a.rep);
    }
    return (size_t)t * a.n_h + h;
}
// cache and position of token row t
struct RowCache {
    int8_t* kq;
    float* sk;
    int16_t* vq;
    int pos;
};
__device__ __forceinline__ RowCache row_cache(const AttnArgs& a, int t) {
    if (a.rows) {
        const det_kv_cache c = a.rows[t];
        return RowCache{c.kq, c.sk, c.vq, a.pos_rows[t]};
    }
    return RowCache{a.kq, a.sk, a.vq, (a.pos0_dev ? *a.pos0_dev : a.pos0) + t};
}

template <int HD>
__global__ void __launch_bounds__(256) k_attn_prep(const AttnArgs a) {
    constexpr int PER = HD / 32;
    __shared__ float rowbuf[8][HD];
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const long long row = (long long)blockIdx.x * 8 + wib;
    const long long n_q = (long long)a.M * a.n_h, n_kvrows = (long long)a.M * a.n_kv;
    if (row >= n_q + 2 * n_kvrows) return;
    if (row >= n_q + n_kvrows) {
        // ---- v row -> int16 cache (spec/layers.rs:76-87)
        const long long r = row - n_q - n_kvrows;
        const int t = (int)(r / a.n_kv), h = (int)(r % a.n_kv);
        const RowCache rc = row_cache(a, t);
        const float inv = a.v_inv[h];
        const float* src = a.v + ((size_t)t * a.n_kv + h) * HD;
        int16_t* dst = rc.vq + ((size_t)rc.pos * a.n_kv + h) * HD;
#pragma unroll
        for (int i = 0; i < PER; i++) {
            const int idx = lane * PER + i;
            int q = f2i_sat(fmul(src[idx], inv));
            dst[idx] = (int16_t)max(-32767, min(32767, q));
        }
        return;
    }
    const bool is_q = row < n_q;
    if (is_q) {
        // this (token, head)'s reduction cells start from zero (0 is below every order-preserving score key)
        const size_t cell = q_cell(a, (int)(row / a.n_h), (int)(row % a.n_h));
        if (lane == 0) {
            a.mxkey[cell] = 0u;
            a.den[cell] = 0;
            a.bar[row] = 0u;     // indexed by (token, kv head) <= (token, q head)
            a.done[row] = 0u;
        }
#pragma unroll
        for (int i = 0; i < PER; i++) a.num[cell * HD + lane * PER + i] = 0;
    }
    int t, h;
    const float *src, *wn;
    if (is_q) {
        t = (int)(row / a.n_h); h = (int)(row % a.n_h);
        src = a.qg + ((size_t)t * a.n_h + h) * 2 * HD;
        wn = a.q_norm;
    } else {
        const long long r = row - n_q;
        t = (int)(r / a.n_kv); h = (int)(r % a.n_kv);
        src = a.k + ((size_t)t * a.n_kv + h) * HD;
        wn = a.k_norm;
    }
    // rmsnorm over hd (spec/prim.rs:176-185): lane owns PER consecutive values
    float x[PER], sq[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) {
        x[i] = src[lane * PER + i];
        sq[i] = fmul(x[i], x[i]);
    }
    const float ss = fold_lanes<32>(fold_run<PER>(sq));
    const float inv_rms = fdiv(1.0f, fsqrt(fadd(fdiv(ss, (float)HD), a.eps)));
    float* buf = rowbuf[wib];
#pragma unroll
    for (int i = 0; i < PER; i++) buf[lane * PER + i] = fmul(fmul(x[i], inv_rms), wn[lane * PER + i]);
    __syncwarp();
    // rope on the first `rot` dims, neox pairing (spec/layers.rs:5-13)
    const int half = a.rot >> 1;
    const RowCache cache = row_cache(a, t);
    const float* rc = a.rope_cos + (size_t)cache.pos * half;
    const float* rs = a.rope_sin + (size_t)cache.pos * half;
    for (int p = lane; p < half; p += 32) {
        const float u = buf[p], w = buf[p + half];
        const float c = rc[p], s = rs[p];
        buf[p] = fsub(fmul(u, c), fmul(w, s));
        buf[p + half] = fadd(fmul(w, c), fmul(u, s));
    }
    __syncwarp();
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; i++) {
        float v = buf[lane * PER + i];
        if (is_q) v = fmul(v, a.qscale);
        x[i] = v;
        amax = fmaxf(amax, fabsf(v));
    }
    amax = max_lanes(amax);
    const float s = (amax == 0.0f) ? 1.0f : fdiv(amax, 127.0f);   // spec/quant.rs:7-16
    const float inv = fdiv(1.0f, s);
    int8_t* dst = is_q ? a.qq + q_cell(a, t, h) * HD : cache.kq + ((size_t)cache.pos * a.n_kv + h) * HD;
#pragma unroll
    for (int i = 0; i < PER; i++) dst[lane * PER + i] = (int8_t)quant_code(x[i], inv);
    if (lane == 0) {
        if (is_q) a.sq[q_cell(a, t, h)] = s;
        else cache.sk[(size_t)cache.pos * a.n_kv + h] = s;
    }
}

// Shared tile of KT keys with rows padded by 16 bytes: 128-bit reads by threads that own consecutive keys then fall into
// distinct banks.
template <int HD>
struct KTile {
    static constexpr int STRIDE = HD + 16;
    __device__ static void load(int8_t* tile, float* sks, const AttnArgs& a, const RowCache& c, int kvh, int key0, int nkeys) {
        constexpr int VEC = HD / 16;
        for (int i = threadIdx.x; i < KT * VEC; i += ATT_THREADS) {
            const int j = i / VEC, v = i % VEC;
            uint4 val = make_uint4(0, 0, 0, 0);
            if (j < nkeys)
                val = *reinterpret_cast<const uint4*>(c.kq + ((size_t)(key0 + j) * a.n_kv + kvh) * HD + v * 16);
            *reinterpret_cast<uint4*>(tile + j * STRIDE + v * 16) = val;
        }
        for (int j = threadIdx.x; j < KT; j += ATT_THREADS) sks[j] = j < nkeys ? c.sk[(size_t)(key0 + j) * a.n_kv + kvh] : 0.0f;
    }
    __device__ __forceinline__ static int dot(const int8_t* tile, int j, const int8_t* q) {
        int acc = 0;
#pragma unroll
        for (int v = 0; v < HD / 16; v++) {
            const uint4 kk = *reinterpret_cast<const uint4*>(tile + j * STRIDE + v * 16);
            const uint4 qv = *reinterpret_cast<const uint4*>(q + v * 16);
            acc = __dp4a((int)kk.x, (int)qv.x, acc);
            acc = __dp4a((int)kk.y, (int)qv.y, acc);
            acc = __dp4a((int)kk.z, (int)qv.z, acc);
            acc = __dp4a((int)kk.w, (int)qv.w, acc);
        }
        return acc;
    }
};

// acc += (s32) a * (s32) b as ONE 32 x 32 + 64 multiply-add (written out: the compiler otherwise widens both factors and
// multiplies 64-bit values, several instructions per product).
__device__ __forceinline__ void mad_wide(long long& acc, int a, int b) {
    asm("mad.wide.s32 %0, %1, %2, %0;" : "+l"(acc) : "r"(a), "r"(b));
}

// P.V of one tile for value dimension d: num[r] += sum_q pq[r][q] * v[q][d], exact in int64.  Four keys per turn (one
// 128-bit load of four p values per head, REP a compile-time count so nothing is predicated); rows of pq past the tile's
// keys hold p = 0, so the turn may run over the end of a short tile.
template <int HD, int REP>
__device__ __forceinline__ void pv_tile_n(const int (*pq)[KT], const int16_t* vtile, int nkeys, int d, long long (&num)[MAX_REP]) {
    const int n4 = (nkeys + 3) & ~3;
    for (int q = 0; q < n4; q += 4) {
        const int v0 = vtile[(q + 0) * HD + d], v1 = vtile[(q + 1) * HD + d];
        const int v2 = vtile[(q + 2) * HD + d], v3 = vtile[(q + 3) * HD + d];
#pragma unroll
        for (int r = 0; r < REP; r++) {
            const int4 p = *reinterpret_cast<const int4*>(&pq[r][q]);
            mad_wide(num[r], p.x, v0);
            mad_wide(num[r], p.y, v1);
            mad_wide(num[r], p.z, v2);
            mad_wide(num[r], p.w, v3);
        }
    }
}
template <int HD>
__device__ __forceinline__ void pv_tile(const int (*pq)[KT], const int16_t* vtile, int nkeys, int d, int rep,
                                        long long (&num)[MAX_REP]) {
    switch (rep) {
        case 1: pv_tile_n<HD, 1>(pq, vtile, nkeys, d, num); break;
        case 2: pv_tile_n<HD, 2>(pq, vtile, nkeys, d, num); break;
        case 3: pv_tile_n<HD, 3>(pq, vtile, nkeys, d, num); break;
        case 4: pv_tile_n<HD, 4>(pq, vtile, nkeys, d, num); break;
        case 5: pv_tile_n<HD, 5>(pq, vtile, nkeys, d, num); break;
        case 6: pv_tile_n<HD, 6>(pq, vtile, nkeys, d, num); break;
        case 7: pv_tile_n<HD, 7>(pq, vtile, nkeys, d, num); break;
        default: pv_tile_n<HD, 8>(pq, vtile, nkeys, d, num); break;
    }
}

// key range of this CTA for a token at position pos: [k0, k1) within [0, pos]
__device__ __forceinline__ void key_range(const AttnArgs& a, int pos, int& k0, int& k1) {
    const int total = pos + 1;
    k0 = blockIdx.x * a.keys_per_split;
    k1 = min(total, k0 + a.keys_per_split);
}

template <int HD>
__device__ __forceinline__ void fetch_k_async(int8_t* ktile, float* sks, const AttnArgs& a, const RowCache& c, int kvh,
                                              int key0, int nkeys);

template <int HD>
__global__ void __launch_bounds__(ATT_THREADS) k_attn_max(const AttnArgs a) {
    __shared__ __align__(16) int8_t ktiles[2][KT * KTile<HD>::STRIDE];   // the next K tile is in flight while this one is used
    __shared__ __align__(16) int8_t qs[MAX_REP * HD];
    __shared__ float sks2[2][KT];
    __shared__ float sqs[MAX_REP];
    __shared__ unsigned best[MAX_REP];
    pdl_trigger();
    pdl_wait();
    const int kvh = blockIdx.y, t = blockIdx.z;
    const RowCache cache = row_cache(a, t);
    int k0, k1;
    key_range(a, cache.pos, k0, k1);
    if (k0 >= k1) return;
    const int rep = a.rep;
    for (int i = threadIdx.x; i < rep * HD / 16; i += ATT_THREADS)
        reinterpret_cast<uint4*>(qs)[i] =
            reinterpret_cast<const uint4*>(a.qq + ((size_t)t * a.n_h + (size_t)kvh * rep) * HD)[i];
    if (threadIdx.x < rep) {
        sqs[threadIdx.x] = a.sq[(size_t)t * a.n_h + kvh * rep + threadIdx.x];
        best[threadIdx.x] = 0u;
    }
    const int j = threadIdx.x % KT, part = threadIdx.x / KT;   // 4 parts share the heads
    unsigned mine[MAX_REP / 4 + 1];
#pragma unroll
    for (int i = 0; i < MAX_REP / 4 + 1; i++) mine[i] = 0u;
    auto fetch = [&](int key0, int st) {
        fetch_k_async<HD>(ktiles[st], sks2[st], a, cache, kvh, key0, min(KT, k1 - key0));
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(k0, 0);
    int st = 0;
    for (int key0 = k0; key0 < k1; key0 += KT, st ^= 1) {
        const int nkeys = min(KT, k1 - key0);
        const bool more = key0 + KT < k1;
        if (more) fetch(key0 + KT, st ^ 1);
        if (more) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const int8_t* ktile = ktiles[st];
        const float* sks = sks2[st];
        if (j < nkeys) {
#pragma unroll
            for (int i = 0; i < MAX_REP / 4 + 1; i++) {
                const int r = part + 4 * i;
                if (r < rep) {
                    const int d = KTile<HD>::dot(ktile, j, qs + r * HD);
                    const float s = fmul(fmul((float)d, sqs[r]), sks[j]);
                    mine[i] = max(mine[i], f32_key(s));
                }
            }
        }
        __syncthreads();                                   // this stage may be refilled
    }
#pragma unroll
    for (int i = 0; i < MAX_REP / 4 + 1; i++) {
        const int r = part + 4 * i;
        if (r < rep && mine[i]) atomicMax(&best[r], mine[i]);
    }
    __syncthreads();
    if (threadIdx.x < rep && best[threadIdx.x])
        atomicMax(a.mxkey + (size_t)t * a.n_h + kvh * rep + threadIdx.x, best[threadIdx.x]);
}

template <int HD>
struct AccSmem {
    static constexpr int KTILE = KT * KTile<HD>::STRIDE;
    static constexpr int VTILE = KT * HD * 2;
    static constexpr int STAGE = KTILE + VTILE;
    static constexpr int TOTAL = 2 * STAGE;          // two stages: the next tile is in flight while this one is consumed
};

// V tile (KT keys x HD int16) into shared memory with asynchronous 16-byte copies; rows past nkeys are not touched.
template <int HD>
__device__ __forceinline__ void fetch_v_async(int16_t* vtile, const AttnArgs& a, const RowCache& c, int kvh, int key0, int nkeys) {
    constexpr int VEC = HD / 8;                          // 16-byte pieces per row
    for (int i = threadIdx.x; i < nkeys * VEC; i += ATT_THREADS) {
        const int q = i / VEC, v = i % VEC;
        const int16_t* src = c.vq + ((size_t)(key0 + q) * a.n_kv + kvh) * HD + v * 8;
        const unsigned dst = (unsigned)__cvta_generic_to_shared(vtile + q * HD + v * 8);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}
// K tile (padded rows) and the keys' scales, asynchronously; the caller commits.  Rows past nkeys are not touched.
template <int HD>
__device__ __forceinline__ void fetch_k_async(int8_t* ktile, float* sks, const AttnArgs& a, const RowCache& c, int kvh,
                                              int key0, int nkeys) {
    constexpr int VEC = HD / 16;
    for (int i = threadIdx.x; i < nkeys * VEC; i += ATT_THREADS) {
        const int j = i / VEC, v = i % VEC;
        const int8_t* src = c.kq + ((size_t)(key0 + j) * a.n_kv + kvh) * HD + v * 16;
        const unsigned dst = (unsigned)__cvta_generic_to_shared(ktile + j * KTile<HD>::STRIDE + v * 16);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
    }
    for (int j = threadIdx.x; j < nkeys; j += ATT_THREADS) {
        const unsigned dst = (unsigned)__cvta_generic_to_shared(sks + j);
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(c.sk + (size_t)(key0 + j) * a.n_kv + kvh) : "memory");
    }
}

template <int HD>
__global__ void __launch_bounds__(ATT_THREADS) k_attn_acc(const AttnArgs a) {
    static_assert(HD <= ATT_THREADS, "one thread per value dimension");
    extern __shared__ __align__(16) uint8_t asm_[];
    int8_t* ktile = reinterpret_cast<int8_t*>(asm_);
    int16_t* vtile = reinterpret_cast<int16_t*>(asm_ + AccSmem<HD>::KTILE);
    __shared__ __align__(16) int8_t qs[MAX_REP * HD];
    __shared__ float sks[KT];
    __shared__ float sqs[MAX_REP];
    __shared__ float mxs[MAX_REP];
    __shared__ __align__(16) int pq[MAX_REP][KT];
    __shared__ long long den_sh[MAX_REP];
    pdl_trigger();
    pdl_wait();
    const int kvh = blockIdx.y, t = blockIdx.z;
    const RowCache cache = row_cache(a, t);
    int k0, k1;
    key_range(a, cache.pos, k0, k1);
    if (k0 >= k1) return;
    const int rep = a.rep;
    for (int i = threadIdx.x; i < rep * HD / 16; i += ATT_THREADS)
        reinterpret_cast<uint4*>(qs)[i] =
            reinterpret_cast<const uint4*>(a.qq + ((size_t)t * a.n_h + (size_t)kvh * rep) * HD)[i];
    if (threadIdx.x < rep) {
        const size_t hh = (size_t)t * a.n_h + kvh * rep + threadIdx.x;
        sqs[threadIdx.x] = a.sq[hh];
        mxs[threadIdx.x] = key_f32(a.mxkey[hh]);
        den_sh[threadIdx.x] = 0;
    }
    const int j = threadIdx.x % KT, part = threadIdx.x / KT;
    const int d = threadIdx.x;   // value dimension owned in the P.V phase
    long long num[MAX_REP];
#pragma unroll
    for (int r = 0; r < MAX_REP; r++) num[r] = 0;
    for (int key0 = k0; key0 < k1; key0 += KT) {
        const int nkeys = min(KT, k1 - key0);
        __syncthreads();                                   // the previous tile's K, V and pq are no longer read
        fetch_v_async<HD>(vtile, a, cache, kvh, key0, nkeys);   // in flight while the scores are computed
        KTile<HD>::load(ktile, sks, a, cache, kvh, key0, nkeys);
        __syncthreads();
#pragma unroll
        for (int i = 0; i < MAX_REP / 4 + 1; i++) {
            const int r = part + 4 * i;
            if (r < rep) {
                int p = 0;
                if (j < nkeys) {
                    const int dt = KTile<HD>::dot(ktile, j, qs + r * HD);
                    const float s = fmul(fmul((float)dt, sqs[r]), sks[j]);
                    p = f2i_sat(fmul(exp_f(fsub(s, mxs[r])), 16777216.0f));
                }
                pq[r][j] = p;
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (threadIdx.x < rep) {
            long long s = 0;
            for (int q = 0; q < nkeys; q++) s += pq[threadIdx.x][q];
            den_sh[threadIdx.x] += s;
        }
        if (d < HD) pv_tile<HD>(pq, vtile, nkeys, d, rep, num);
    }
    __syncthreads();
    if (a.nsplit == 1) {
        if (d < HD) {
            const float vs = a.v_scale[kvh];
#pragma unroll
            for (int r = 0; r < MAX_REP; r++) {
                if (r < rep) {
                    const int h = kvh * rep + r;
                    const float gate = a.qg[((size_t)t * a.n_h + h) * 2 * HD + HD + d];
                    const float val = fmul(fdiv(i64_to_f32(num[r]), i64_to_f32(den_sh[r])), vs);
                    a.o[((size_t)t * a.n_h + h) * HD + d] = fmul(val, sigmoid_f(gate));
                }
            }
        }
    } else {
        if (d < HD) {
#pragma unroll
            for (int r = 0; r < MAX_REP; r++)
                if (r < rep)
                    atomicAdd(reinterpret_cast<unsigned long long*>(a.num + ((size_t)t * a.n_h + kvh * rep + r) * HD + d),
                              (unsigned long long)num[r]);
        }
        if (threadIdx.x < rep)
            atomicAdd(reinterpret_cast<unsigned long long*>(a.den + (size_t)t * a.n_h + kvh * rep + threadIdx.x),
                      (unsigned long long)den_sh[threadIdx.x]);
    }
}

template <int HD>
__global__ void k_attn_fin(const AttnArgs a) {
    pdl_trigger();
    pdl_wait();
    const size_t row = blockIdx.x;   // t * n_h + h
    const int d = threadIdx.x;
    const int t = (int)(row / a.n_h), h = (int)(row % a.n_h);
    const float vs = a.v_scale[h / a.rep];
    const float gate = a.qg[((size_t)t * a.n_h + h) * 2 * HD + HD + d];
    const float val = fmul(fdiv(i64_to_f32(a.num[row * HD + d]), i64_to_f32(a.den[row])), vs);
    a.o[row * HD + d] = fmul(val, sigmoid_f(gate));
}

// ---- decode-sized attention as one launch after prep: max, acc and fin of the same key range in one CTA.  The scores of
// the CTA's keys stay in shared memory between the two passes (K is read and multiplied once); the CTAs of one
// (token, kv head) meet at a counter after publishing their maxima (all CTAs of the grid are resident: the launcher asks
// for at most one per SM; the wait is bounded), V tiles are staged in shared memory (the first one is fetched
// asynchronously while the scores are computed), and the CTA that adds its partial sums last finishes the heads.
constexpr int DEC_MAX_KEYS = 512;   // keys per CTA whose scores fit the shared buffer

template <int HD>
struct DecSmem {
    static constexpr int KTILE = KT * KTile<HD>::STRIDE;
    static constexpr int VTILE = KT * HD * 2;
    static constexpr int SBUF = MAX_REP * DEC_MAX_KEYS * 4;
    static constexpr int QS = MAX_REP * HD;
    static constexpr int PQ = MAX_REP * KT * 4;
    static constexpr int TOTAL = KTILE + VTILE + SBUF + QS + PQ;
};

template <int HD>
__global__ void __launch_bounds__(ATT_THREADS) k_attn_dec(const AttnArgs a) {
    static_assert(HD <= ATT_THREADS, "one thread per value dimension");
    extern __shared__ __align__(16) uint8_t dsm[];
    int8_t* ktile = reinterpret_cast<int8_t*>(dsm);
    int16_t* vtile = reinterpret_cast<int16_t*>(dsm + DecSmem<HD>::KTILE);
    float* sbuf = reinterpret_cast<float*>(dsm + DecSmem<HD>::KTILE + DecSmem<HD>::VTILE);
    int8_t* qs = reinterpret_cast<int8_t*>(dsm + DecSmem<HD>::KTILE + DecSmem<HD>::VTILE + DecSmem<HD>::SBUF);
    int (*pq)[KT] = reinterpret_cast<int (*)[KT]>(dsm + DecSmem<HD>::KTILE + DecSmem<HD>::VTILE + DecSmem<HD>::SBUF + DecSmem<HD>::QS);
    __shared__ float sks[KT];
    __shared__ float sqs[MAX_REP];
    __shared__ float mxs[MAX_REP];
    __shared__ unsigned best[MAX_REP];
    __shared__ long long den_sh[MAX_REP];
    __shared__ bool last;
    pdl_trigger();
    pdl_wait();
    const int kvh = blockIdx.y, t = blockIdx.z;
    const RowCache cache = row_cache(a, t);
    const int total = cache.pos + 1;
    const int k0 = blockIdx.x * a.keys_per_split;
    const int k1 = min(total, k0 + a.keys_per_split);
    if (k0 >= k1) return;
    const unsigned active = (unsigned)((total + a.keys_per_split - 1) / a.keys_per_split);
    const int rep = a.rep;
    const size_t vstride = (size_t)a.n_kv * HD;            // int16 elements between consecutive keys

    // first V tile: asynchronous copies, consumed in pass 2
    fetch_v_async<HD>(vtile, a, cache, kvh, k0, min(KT, k1 - k0));

    for (int i = threadIdx.x; i < rep * HD / 16; i += ATT_THREADS)
        reinterpret_cast<uint4*>(qs)[i] =
            reinterpret_cast<const uint4*>(a.qq + ((size_t)t * a.n_h + (size_t)kvh * rep) * HD)[i];
    if (threadIdx.x < rep) {
        sqs[threadIdx.x] = a.sq[(size_t)t * a.n_h + kvh * rep + threadIdx.x];
        best[threadIdx.x] = 0u;
        den_sh[threadIdx.x] = 0;
    }
    const int j = threadIdx.x % KT, part = threadIdx.x / KT;   // 4 parts share the heads
    const int d = threadIdx.x;                                  // value dimension owned in the P.V phase

    // ---- pass 1: scores of this CTA's keys into sbuf, their maxima into best[]
    unsigned mine[MAX_REP / 4 + 1];
#pragma unroll
    for (int i = 0; i < MAX_REP / 4 + 1; i++) mine[i] = 0u;
    for (int key0 = k0; key0 < k1; key0 += KT) {
        const int nkeys = min(KT, k1 - key0);
        __syncthreads();
        KTile<HD>::load(ktile, sks, a, cache, kvh, key0, nkeys);
        __syncthreads();
        if (j < nkeys) {
#pragma unroll
            for (int i = 0; i < MAX_REP / 4 + 1; i++) {
                const int r = part + 4 * i;
                if (r < rep) {
                    const int dt = KTile<HD>::dot(ktile, j, qs + r * HD);
                    const float sc = fmul(fmul((float)dt, sqs[r]), sks[j]);
                    sbuf[r * DEC_MAX_KEYS + (key0 - k0) + j] = sc;
                    mine[i] = max(mine[i], f32_key(sc));
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < MAX_REP / 4 + 1; i++) {
        const int r = part + 4 * i;
        if (r < rep && mine[i]) atomicMax(&best[r], mine[i]);
    }
    __syncthreads();
    const unsigned cell = (unsigned)t * a.n_kv + kvh;
    if (active > 1) {
        if (threadIdx.x < rep && best[threadIdx.x])
            atomicMax(a.mxkey + (size_t)t * a.n_h + kvh * rep + threadIdx.x, best[threadIdx.x]);
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            atomicAdd(a.bar + cell, 1u);
            const long long start = clock64();
            bool ok = *reinterpret_cast<volatile int*>(a.error_flag) != 0;
            while (!ok) {
                if (*reinterpret_cast<volatile unsigned*>(a.bar + cell) >= active) { ok = true; break; }
                if (clock64() - start > wait_limit(a.error_flag)) break;      // about two seconds by default: report and carry on
            }
            if (!ok) atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
            __threadfence();
        }
        __syncthreads();
        if (threadIdx.x < rep)
            mxs[threadIdx.x] = key_f32(*reinterpret_cast<volatile unsigned*>(a.mxkey + (size_t)t * a.n_h + kvh * rep + threadIdx.x));
    } else if (threadIdx.x < rep) {
        mxs[threadIdx.x] = key_f32(best[threadIdx.x]);
    }

    // ---- pass 2: pq from the stored scores, den and num in int64
    long long num[MAX_REP];
#pragma unroll
    for (int r = 0; r < MAX_REP; r++) num[r] = 0;
    for (int key0 = k0; key0 < k1; key0 += KT) {
        const int nkeys = min(KT, k1 - key0);
        __syncthreads();            // mxs visible; the previous tile's pq and vtile are no longer read
        if (key0 == k0) {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        } else {
            constexpr int VEC = HD / 8;
            for (int i = threadIdx.x; i < nkeys * VEC; i += ATT_THREADS) {
                const int q = i / VEC, v = i % VEC;
                *reinterpret_cast<uint4*>(vtile + q * HD + v * 8) =
                    *reinterpret_cast<const uint4*>(cache.vq + ((size_t)(key0 + q) * a.n_kv + kvh) * HD + v * 8);
            }
        }
#pragma unroll
        for (int i = 0; i < MAX_REP / 4 + 1; i++) {
            const int r = part + 4 * i;
            if (r < rep) {
                int p = 0;
                if (j < nkeys)
                    p = f2i_sat(fmul(exp_f(fsub(sbuf[r * DEC_MAX_KEYS + (key0 - k0) + j], mxs[r])), 16777216.0f));
                pq[r][j] = p;
            }
        }
        __syncthreads();
        if (threadIdx.x < rep) {
            long long sum = 0;
            for (int q = 0; q < nkeys; q++) sum += pq[threadIdx.x][q];
            den_sh[threadIdx.x] += sum;
        }
        if (d < HD) pv_tile<HD>(pq, vtile, nkeys, d, rep, num);
    }
    __syncthreads();
    (void)vstride;
    // ---- finish: alone, or through the global cells with the last CTA converting
    if (active == 1) {
        if (d < HD) {
            const float vs = a.v_scale[kvh];
#pragma unroll
            for (int r = 0; r < MAX_REP; r++) {
                if (r < rep) {
                    const int h = kvh * rep + r;
                    const float gate = a.qg[((size_t)t * a.n_h + h) * 2 * HD + HD + d];
                    const float val = fmul(fdiv(i64_to_f32(num[r]), i64_to_f32(den_sh[r])), vs);
                    a.o[((size_t)t * a.n_h + h) * HD + d] = fmul(val, sigmoid_f(gate));
                }
            }
        }
        return;
    }
    if (d < HD) {
#pragma unroll
        for (int r = 0; r < MAX_REP; r++)
            if (r < rep)
                atomicAdd(reinterpret_cast<unsigned long long*>(a.num + ((size_t)t * a.n_h + kvh * rep + r) * HD + d),
                          (unsigned long long)num[r]);
    }
    if (threadIdx.x < rep)
        atomicAdd(reinterpret_cast<unsigned long long*>(a.den + (size_t)t * a.n_h + kvh * rep + threadIdx.x),
                  (unsigned long long)den_sh[threadIdx.x]);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(a.done + cell, 1u) == active - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (d < HD) {
        const float vs = a.v_scale[kvh];
        for (int r = 0; r < rep; r++) {
            const size_t row = (size_t)t * a.n_h + kvh * rep + r;
            const float gate = a.qg[row * 2 * HD + HD + d];
            const float val = fmul(fdiv(i64_to_f32(__ldcg(a.num + row * HD + d)), i64_to_f32(__ldcg(a.den + row))), vs);
            a.o[row * HD + d] = fmul(val, sigmoid_f(gate));
        }
    }
}

// Token tiling measured no faster on B200 (27B, 2048- and 8192-token prompts: the accumulate kernel is bound by its
// integer multiply-adds, not by K/V traffic), so it is off unless switched on.

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }
struct ScratchMap {
    size_t qq, sq, mx, den, num, bar, done, total;
};
static ScratchMap scratch_map(int M, int n_h, int hd) {
    ScratchMap s;
    const size_t rows = (size_t)(M + 128) * n_h;   // room for the tile layout: every kv head's rows padded to 128
    s.qq = 0;
    s.sq = align256(rows * hd);
    s.mx = s.sq + align256(rows * 4);
    s.den = s.mx + align256(rows * 4);
    s.num = s.den + align256(rows * 8);
    s.bar = s.num + align256(rows * hd * 8);
    s.done = s.bar + align256(rows * 4);
    s.total = s.done + align256(rows * 4);
    return s;
}

template <int HD>
static void run_attention(AttnArgs a, void* scratch, int max_total_keys, int capacity, cudaStream_t q) {
    const ScratchMap sm = scratch_map(a.M, a.n_h, HD);
    uint8_t* base = static_cast<uint8_t*>(scratch);
    a.qq = reinterpret_cast<int8_t*>(base + sm.qq);
    a.sq = reinterpret_cast<float*>(base + sm.sq);
    a.mxkey = reinterpret_cast<unsigned*>(base + sm.mx);
    a.den = reinterpret_cast<long long*>(base + sm.den);
    a.num = reinterpret_cast<long long*>(base + sm.num);
    a.bar = reinterpret_cast<unsigned*>(base + sm.bar);
    a.done = reinterpret_cast<unsigned*>(base + sm.done);
    a.error_flag = error_word();
    // key split: aim at ~4 CTAs per SM in total, whole tiles per split (a choice by shape only)
    const int tiles = (max_total_keys + KT - 1) / KT;
    int want = (4 * sm_count()) / (a.n_kv * a.M);
    int nsplit = want < 1 ? 1 : (want > tiles ? tiles : want);
    const int tiles_per_split = (tiles + nsplit - 1) / nsplit;
    nsplit = (tiles + tiles_per_split - 1) / tiles_per_split;
    a.nsplit = nsplit;
    a.keys_per_split = tiles_per_split * KT;

    const long long rows = (long long)a.M * (a.n_h + 2 * a.n_kv);
    a.tc_rpad = 0;
    if (attn_tc_applies(a.M, HD, a.rows != nullptr, a.pos0_dev != nullptr, a.n_kv, max_total_keys)) {
        // prefill on the tensor cores: prep writes the query rows in the tile layout, the rest is attn_tc.cu
        a.tc_rpad = (a.M * a.rep + 127) / 128 * 128;
        launch_pdl(k_attn_prep<HD>, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, q, 1, a);
        AttnTcCall c;
        c.M = a.M; c.n_h = a.n_h; c.n_kv = a.n_kv; c.pos0 = a.pos0; c.capacity = capacity; c.Rpad = a.tc_rpad;
        c.qq = a.qq; c.sq = a.sq; c.mxkey = a.mxkey; c.den = a.den; c.num = a.num;
        c.kq = a.kq; c.sk = a.sk; c.vq = a.vq; c.qg = a.qg; c.v_scale = a.v_scale; c.o = a.o;
        attn_tc_run(c, q);
        return;
    }
    launch_pdl(k_attn_prep<HD>, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, q, 1, a);
    // decode-sized calls: one fused launch, at most one CTA per SM so that all of them are resident at the counter
    const int fit = sm_count() / (a.n_kv * a.M);
    if (fit >= 1) {
        const int tps = (tiles + fit - 1) / fit;
        if (tps * KT <= DEC_MAX_KEYS) {
            a.nsplit = (tiles + tps - 1) / tps;
            a.keys_per_split = tps * KT;
            static bool attr_set = false;
            if (!attr_set) {
                DETB_CUDA_OK(cudaFuncSetAttribute(k_attn_dec<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecSmem<HD>::TOTAL));
                attr_set = true;
            }
            launch_pdl(k_attn_dec<HD>, dim3(a.nsplit, a.n_kv, a.M), dim3(ATT_THREADS), DecSmem<HD>::TOTAL, q, 1, a);
            return;
        }
    }
    if (a.rows) {
        // batched step: the sequences' lengths differ (only their maximum is known here), so cut fixed 512-key ranges
        // and let the CTAs past a sequence's end return at once
        const int tps = 8;
        nsplit = (tiles + tps - 1) / tps;
        a.nsplit = nsplit;
        a.keys_per_split = tps * KT;
    }
    const dim3 grid(nsplit, a.n_kv, a.M);
    static bool acc_attr = false;
    if (!acc_attr) {
        DETB_CUDA_OK(cudaFuncSetAttribute(k_attn_acc<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, AccSmem<HD>::STAGE));
        acc_attr = true;
    }
    launch_pdl(k_attn_max<HD>, grid, dim3(ATT_THREADS), 0, q, 1, a);
    launch_pdl(k_attn_acc<HD>, grid, dim3(ATT_THREADS), AccSmem<HD>::STAGE, q, 1, a);
    if (nsplit > 1) launch_pdl(k_attn_fin<HD>, dim3(a.M * a.n_h), dim3(HD), 0, q, 1, a);
}

static void attention_entry(const det_attn_layer* L, const det_kv_cache* kv, const float* qg, const float* k,
                            const float* v, const float* rope_cos, const float* rope_sin, int rot, float eps, int M,
                            int pos0, const int* pos0_dev, int max_pos, int n_h, int n_kv, int hd, float* o,
                            void* scratch, cudaStream_t st, const det_kv_cache* rows = nullptr,
                            const int* pos_rows = nullptr) {
    if (M <= 0) return;
    DETB_REQUIRE(n_kv > 0 && n_h % n_kv == 0 && n_h / n_kv <= MAX_REP, "n_h / n_kv must be an integer <= 8");
    DETB_REQUIRE(hd == 64 || hd == 256, "head_dim must be 64 or 256 (1/sqrt(hd) has to be a power of two, cpu.rs:225-230)");
    DETB_REQUIRE(rot >= 0 && rot <= hd && rot % 2 == 0, "bad rotary dimension");
    if (!rows) DETB_REQUIRE(max_pos + M <= kv->capacity, "positions exceed the cache capacity");
    AttnArgs a;
    a.rows = rows; a.pos_rows = pos_rows;
    a.q_norm = L->q_norm; a.k_norm = L->k_norm; a.v_scale = L->v_scale; a.v_inv = L->v_inv_scale;
    if (kv) { a.kq = kv->kq; a.sk = kv->sk; a.vq = kv->vq; }
    else { a.kq = nullptr; a.sk = nullptr; a.vq = nullptr; }
    a.qg = qg; a.k = k; a.v = v; a.rope_cos = rope_cos; a.rope_sin = rope_sin;
    a.rot = rot; a.eps = eps;
    a.qscale = hd == 256 ? 0.0625f : 0.125f;   // fp32(1/sqrt(hd)), exact
    a.M = M; a.n_h = n_h; a.n_kv = n_kv; a.rep = n_h / n_kv;
    a.pos0 = pos0; a.pos0_dev = pos0_dev; a.o = o;
    cudaStream_t q = queue_of(st);
    const int keys = rows ? max_pos + 1 : max_pos + M;
    const int capacity = kv ? kv->capacity : 0;
    if (hd == 256) run_attention<256>(a, scratch, keys, capacity, q);
    else run_attention<64>(a, scratch, keys, capacity, q);
}

}  // namespace detb

using namespace detb;

extern "C" {

size_t det_attn_scratch_bytes(int M, int n_h, int hd) { return scratch_map(M > 0 ? M : 1, n_h, hd).total; }

void det_attention(const det_attn_layer* L, const det_kv_cache* kv, const float* qg, const float* k, const float* v,
                   const float* rope_cos, const float* rope_sin, int rot, float eps, int M, int pos0, int n_h,
                   int n_kv, int hd, float* o, void* scratch, cudaStream_t st) {
    attention_entry(L, kv, qg, k, v, rope_cos, rope_sin, rot, eps, M, pos0, nullptr, pos0, n_h, n_kv, hd, o, scratch, st);
}

void det_attention_dev(const det_attn_layer* L, const det_kv_cache* kv, const float* qg, const float* k,
                       const float* v, const float* rope_cos, const float* rope_sin, int rot, float eps, int M,
                       const int* pos0_dev, int max_pos, int n_h, int n_kv, int hd, float* o, void* scratch,
                       cudaStream_t st) {
    attention_entry(L, kv, qg, k, v, rope_cos, rope_sin, rot, eps, M, 0, pos0_dev, max_pos, n_h, n_kv, hd, o, scratch, st);
}


// Batched decode (no reference counterpart): M sequences advance one token each.  Row t of qg / k / v / o belongs to the
// sequence whose cache is rows[t] (a DEVICE array of M det_kv_cache) at position pos[t] (device array); max_pos is a host
// bound on the positions.  Each row equals det_attention(M = 1, pos0 = pos[t]) on that cache.
void det_attention_rows(const det_attn_layer* L, const det_kv_cache* rows, const int* pos, int max_pos, const float* qg,
                        const float* k, const float* v, const float* rope_cos, const float* rope_sin, int rot, float eps,
                        int M, int n_h, int n_kv, int hd, float* o, void* scratch, cudaStream_t st) {
    attention_entry(L, nullptr, qg, k, v, rope_cos, rope_sin, rot, eps, M, 0, nullptr, max_pos, n_h, n_kv, hd, o, scratch, st,
                    rows, pos);
}

}  // extern "C"
