// Gated DeltaNet (docs/SPEC.md §5.2, spec/layers.rs:88-147, cpu.rs:293-391).  Replaces kernels/cuda/gdn.cu behind
// det_gdn / det_gdn_ex / det_gdn_scratch_bytes.
//
//   prep    causal conv (4 taps) + silu per channel, l2norm of q and k per k head (q scaled by QSCALE),
//           beta = sigmoid(b), decay = exp_f(-(A * softplus_f(a + dt_bias))); one warp per (token, 128-channel head).
//   recur   the strictly sequential state update.  A CTA owns 16 columns of one v head's S[dk][dv]; a column's 128
//           rows are spread over 8 consecutive lanes (16 rows each) and stay in registers for the whole call.  Both
//           contractions over dk are the spec tree: fold of the lane's aligned run, then xor offsets 1, 2, 4 across the
//           8 lanes.  State enters and leaves through a shared-memory slab so global traffic stays coalesced.
//   out     on = rmsnorm(o, norm) * silu_f(z) per (token, v head); the last three raw inputs become the conv state.
//   step    decode (one token per sequence): all three in ONE launch.  The 8 CTAs of a v head form a thread-block
//           cluster; each prepares its own operands, advances its 16 state columns, and the head-wide RMSNorm of the
//           outputs is finished over distributed shared memory (every CTA stores the spec-tree sum of its 16 squares
//           into its peers' shared memory, one cluster barrier).  The conv state is shifted by whoever read it last.
#include "runtime.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace detb {

constexpr int DK = 128, DV = 128;          // fixed by the model family (asserted at the entry points)
constexpr unsigned QSCALE_BITS = 0x3DB504F3u;   // fp32(1/sqrt(128)), spec/layers.rs:147

struct GdnArgs {
    const float *conv, *A, *dt_bias, *norm;
    float *conv_state, *S;
    const float *qkv, *z, *a, *b;
    float eps;
    int M, n_k, n_v, rep, conv_dim;
    float* on;
    // scratch
    float* y;        // [M][conv_dim]: q (normalised, scaled) | k (normalised) | v
    float* beta;     // [M][n_v]
    float* decay;    // [M][n_v]
    float* o;        // [M][n_v][DV] mixer output (gout when exported)
    float* gin;      // optional
    const det_gdn_state* rows;   // batched decode: token row t is the next token of the sequence with state rows[t]
};

// input of channel c `back` steps before token row t (times before the call reach into the conv state, which holds the
// three inputs before the call's first token; in a batched step every row is the first token of its own sequence)
__device__ __forceinline__ float conv_in(const GdnArgs& g, int t, int back, int c) {
    if (g.rows)
        return back == 0 ? g.qkv[(size_t)t * g.conv_dim + c] : g.rows[t].conv_state[(size_t)(3 - back) * g.conv_dim + c];
    const int tau = t - back;
    return tau < 0 ? g.conv_state[(size_t)(3 + tau) * g.conv_dim + c] : g.qkv[(size_t)tau * g.conv_dim + c];
}

// silu(causal conv) of channel c at token row t: ((w0*x[t-3] + w1*x[t-2]) + w2*x[t-1]) + w3*x[t]   (spec/layers.rs:135-140)
__device__ __forceinline__ float conv_silu(const GdnArgs& g, int t, int c) {
    const float4 w = *reinterpret_cast<const float4*>(g.conv + (size_t)c * 4);
    float acc = fadd(fmul(w.x, conv_in(g, t, 3, c)), fmul(w.y, conv_in(g, t, 2, c)));
    acc = fadd(acc, fmul(w.z, conv_in(g, t, 1, c)));
    acc = fadd(acc, fmul(w.w, conv_in(g, t, 0, c)));
    return silu_f(acc);
}

__global__ void __launch_bounds__(128) k_gdn_prep(const GdnArgs g) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int t = blockIdx.y;
    const int heads = 2 * g.n_k + g.n_v;     // 128-channel slices of conv_dim
    const int head = blockIdx.x * 4 + wib;
    if (head < heads) {
        const int c0 = head * 128 + lane * 4;
        float v[4], sq[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int c = c0 + e;
            const float4 w = *reinterpret_cast<const float4*>(g.conv + (size_t)c * 4);
            // ((w0*x[t-3] + w1*x[t-2]) + w2*x[t-1]) + w3*x[t]   (spec/layers.rs:135-140)
            float acc = fadd(fmul(w.x, conv_in(g, t, 3, c)), fmul(w.y, conv_in(g, t, 2, c)));
            acc = fadd(acc, fmul(w.z, conv_in(g, t, 1, c)));
            acc = fadd(acc, fmul(w.w, conv_in(g, t, 0, c)));
            v[e] = silu_f(acc);
            sq[e] = fmul(v[e], v[e]);
        }
        if (head < 2 * g.n_k) {
            // l2norm over the head's 128 channels (spec/prim.rs:187-194)
            const float ss = fold_lanes<32>(fold_run<4>(sq));
            const float inv = fdiv(1.0f, fsqrt(fadd(ss, g.eps)));
            const bool is_q = head < g.n_k;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                v[e] = fmul(v[e], inv);
                if (is_q) v[e] = fmul(v[e], __uint_as_float(QSCALE_BITS));
            }
        }
        *reinterpret_cast<float4*>(g.y + (size_t)t * g.conv_dim + c0) = make_float4(v[0], v[1], v[2], v[3]);
        if (g.gin) {
            // gin[t][kh]: q[128] | k[128] | v[rep][128] | beta[rep] | decay[rep]   (cpu.rs:345-357)
            const int gw = 2 * DK + g.rep * DV + 2 * g.rep;
            float* row;
            if (head < g.n_k) row = g.gin + ((size_t)t * g.n_k + head) * gw;
            else if (head < 2 * g.n_k) row = g.gin + ((size_t)t * g.n_k + (head - g.n_k)) * gw + DK;
            else {
                const int vh = head - 2 * g.n_k;
                row = g.gin + ((size_t)t * g.n_k + vh / g.rep) * gw + 2 * DK + (vh % g.rep) * DV;
            }
#pragma unroll
            for (int e = 0; e < 4; e++) row[lane * 4 + e] = v[e];
        }
    }
    // the last CTA row of the grid also produces beta and decay for this token
    if (blockIdx.x == gridDim.x - 1) {
        for (int h = threadIdx.x; h < g.n_v; h += blockDim.x) {
            const float be = sigmoid_f(g.b[(size_t)t * g.n_v + h]);
            const float sp = softplus_f(fadd(g.a[(size_t)t * g.n_v + h], g.dt_bias[h]));
            const float de = exp_f(-fmul(g.A[h], sp));
            g.beta[(size_t)t * g.n_v + h] = be;
            g.decay[(size_t)t * g.n_v + h] = de;
            if (g.gin) {
                const int gw = 2 * DK + g.rep * DV + 2 * g.rep;
                float* row = g.gin + ((size_t)t * g.n_k + h / g.rep) * gw + 2 * DK + g.rep * DV;
                row[h % g.rep] = be;
                row[g.rep + h % g.rep] = de;
            }
        }
    }
}

constexpr int RC = 16;    // columns per CTA
constexpr int RL = 8;     // lanes per column
constexpr int RR = DK / RL;   // rows per lane (16)

// The CTA's 128 x 16 slab of the state in shared memory.  A thread (p = row block, jj = column) reads rows p * 16 + i of
// column jj, so the 32 lanes of a warp touch 8 row blocks x 4 columns at once: element (r, c) lives at
// r * STRIDE + c + 4 * (r / 16) (any stride of 20 words or more that is a multiple of 4 leaves room for that shift: a
// block of 16 rows starts 4 words later than the one before), which puts those 32 words into 32 different banks (a plain padded row-major slab
// is an 8-way conflict), and keeps every 4-column piece 16-byte aligned for the asynchronous copies.
// The decode step and the sequence form keep rows 44 words apart (measured: the one-launch decode step is 0.8 % of a token
// faster with it than with 20); the batched recurrence, which wants two buffers and as many resident CTAs as it can get,
// uses 20.
constexpr int SLAB_STRIDE = 44;
constexpr int SLAB_STRIDE_DEC = 20;
constexpr int SLAB_FLOATS = DK * SLAB_STRIDE + 4 * (DK / 16);
constexpr int SLAB_FLOATS_DEC = DK * SLAB_STRIDE_DEC + 4 * (DK / 16);
template <int STRIDE = SLAB_STRIDE>
__device__ __forceinline__ int slab_at(int r, int c) { return r * STRIDE + c + 4 * (r >> 4); }
constexpr int RUN_STRIDE = RR + 4;      // a lane's 16-row run, padded: the 8 runs of a token fall into distinct banks

// One token of the recurrence for the thread's 16 rows of one state column (spec/layers.rs:104-131): decay, the
// k-contraction (spec tree: the lane's aligned run, then xor 1, 2, 4 over the column's 8 lanes), the delta update, the
// q-contraction.  Returns the output of the column.
__device__ __forceinline__ float recur_step(float (&s)[RR], const float* k, const float* q, float v, float beta, float decay) {
    float prod[RR];
#pragma unroll
    for (int i = 0; i < RR; i++) {
        s[i] = fmul(s[i], decay);
        prod[i] = fmul(s[i], k[i]);
    }
    const float kv_mem = fold_lanes<RL>(fold_run<RR>(prod));
    const float delta = fmul(fsub(v, kv_mem), beta);
#pragma unroll
    for (int i = 0; i < RR; i++) {
        s[i] = fadd(s[i], fmul(k[i], delta));
        prod[i] = fmul(s[i], q[i]);
    }
    return fold_lanes<RL>(fold_run<RR>(prod));
}

// the CTA's 128 x 16 slab of the state <-> shared memory, 16-byte pieces (4 per thread)
template <int STRIDE = SLAB_STRIDE>
__device__ __forceinline__ void slab_load_async(float* slab, const float* Sh, int j0) {
    for (int i = threadIdx.x; i < DK * (RC / 4); i += RC * RL) {
        const int row = i / (RC / 4), v = i % (RC / 4);
        const unsigned dst = (unsigned)__cvta_generic_to_shared(slab + slab_at<STRIDE>(row, v * 4));
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(Sh + (size_t)row * DV + j0 + v * 4) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int STRIDE = SLAB_STRIDE>
__device__ __forceinline__ void slab_store(const float* slab, float* Sh, int j0) {
    for (int i = threadIdx.x; i < DK * (RC / 4); i += RC * RL) {
        const int row = i / (RC / 4), v = i % (RC / 4);
        *reinterpret_cast<float4*>(Sh + (size_t)row * DV + j0 + v * 4) = *reinterpret_cast<const float4*>(slab + slab_at<STRIDE>(row, v * 4));
    }
}

// Batched decode with many sequences: every CTA advances one token of row blockIdx.y's sequence with the operands that
// k_gdn_prep left in scratch (preparing them once per head is less work than in each of a head's column CTAs).  A CTA
// walks DEC_SLABS neighbouring 16-column slabs of its head: the next slab is in flight (asynchronous copies into the other
// shared-memory buffer) while the current one is advanced and written back, and the head's k and q stay in registers.
// The launch moves every state once in and once out and is bound by how many bytes its CTAs keep in flight; a CTA with
// a single slab spends more than half of its life not loading.
constexpr int DEC_SLABS = 4;
__global__ void __launch_bounds__(RC * RL) k_gdn_recur_dec(const GdnArgs g) {
    constexpr int ST = SLAB_STRIDE_DEC;
    __shared__ __align__(16) float slabs[2][SLAB_FLOATS_DEC];
    pdl_trigger();
    pdl_wait();
    constexpr int CPH = DV / RC / DEC_SLABS;                     // CTAs per head
    const int h = blockIdx.x / CPH;
    const int c0 = (blockIdx.x % CPH) * DEC_SLABS;               // first slab of this CTA
    const int kh = h / g.rep;
    const int p = threadIdx.x % RL, jj = threadIdx.x / RL;
    const int t = g.rows ? blockIdx.y : 0;
    float* Sh = (g.rows ? g.rows[blockIdx.y].S : g.S) + (size_t)h * DK * DV;
    slab_load_async<ST>(slabs[0], Sh, c0 * RC);     // in flight while the operands are fetched
    const float* qrow = g.y + (size_t)t * g.conv_dim + (size_t)kh * DK + p * RR;
    const float* krow = g.y + (size_t)t * g.conv_dim + (size_t)g.n_k * DK + (size_t)kh * DK + p * RR;
    float k[RR], q[RR];
#pragma unroll
    for (int i = 0; i < RR; i += 4) {
        const float4 kk = *reinterpret_cast<const float4*>(krow + i);
        const float4 qq = *reinterpret_cast<const float4*>(qrow + i);
        k[i] = kk.x; k[i + 1] = kk.y; k[i + 2] = kk.z; k[i + 3] = kk.w;
        q[i] = qq.x; q[i + 1] = qq.y; q[i + 2] = qq.z; q[i + 3] = qq.w;
    }
    const float be = g.beta[(size_t)t * g.n_v + h], de = g.decay[(size_t)t * g.n_v + h];
    for (int c = 0; c < DEC_SLABS; c++) {
        const int j0 = (c0 + c) * RC;
        float* slab = slabs[c & 1];
        // the other buffer was written back in the last turn (the barrier at its end is behind every thread)
        if (c + 1 < DEC_SLABS) slab_load_async<ST>(slabs[(c + 1) & 1], Sh, j0 + RC);
        const float vv = g.y[(size_t)t * g.conv_dim + (size_t)2 * g.n_k * DK + (size_t)h * DV + j0 + jj];
        if (c + 1 < DEC_SLABS) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        float s[RR];
#pragma unroll
        for (int i = 0; i < RR; i++) s[i] = slab[slab_at<ST>(p * RR + i, jj)];
        const float ov = recur_step(s, k, q, vv, be, de);
        if (p == 0) g.o[((size_t)t * g.n_v + h) * DV + j0 + jj] = ov;
        __syncthreads();
#pragma unroll
        for (int i = 0; i < RR; i++) slab[slab_at<ST>(p * RR + i, jj)] = s[i];
        __syncthreads();
        slab_store<ST>(slab, Sh, j0);
        __syncthreads();
    }
}

// Decode step in one launch: conv + silu + l2norm + gates, the recurrence, the gated output norm and the conv-state
// shift.  Grid (n_v * 8, sequences), cluster (8, 1, 1): the 8 CTAs of a cluster own the 8 x 16 state columns of one v head.
// Every CTA computes what k_gdn_prep would have left in scratch for it — q and k of its k head (conv, silu, l2norm with
// the same per-lane runs and xor order), its 16 v channels, beta and decay — then advances its columns.  The RMSNorm over
// the head's 128 outputs is the spec tree: a CTA's 16 squares are an aligned subtree (xor 1, 2, 4, 8 over 16 lanes), the 8
// subtree sums are stored into every peer's shared memory and each CTA finishes the same tree over them (xor 1, 2, 4).
// Conv state: a CTA alone reads its 16 v channels and shifts them itself; the q / k channels of a k head are read by all
// CTAs of its rep heads — each counts itself in when it has read them, and the one that arrives last does the shift and
// resets the counter (nobody waits on the counter).
constexpr int GDN_CL = DV / RC;            // CTAs per head = cluster size
constexpr int CONV_COUNTERS = 4096;        // (sequence, k head) pairs of one launch
static __device__ unsigned g_conv_done[CONV_COUNTERS];

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

__global__ void __launch_bounds__(RC * RL) k_gdn_step(const GdnArgs g) {
    __shared__ __align__(16) float slab[SLAB_FLOATS];
    __shared__ __align__(16) float pq[RL][RUN_STRIDE], pk[RL][RUN_STRIDE];   // runs of 16 rows, padded against conflicts
    __shared__ float pv[RC], pbd[2], so[RC];
    __shared__ float peer_ss[GDN_CL];          // subtree sums of the head's 8 CTAs, stored here by the peers
    __shared__ bool last_reader;
    cluster_arrive();                          // paired with the wait before the first store into a peer
    pdl_trigger();
    pdl_wait();
    const int h = blockIdx.x / GDN_CL;
    const unsigned rank = blockIdx.x % GDN_CL;
    const int j0 = (int)rank * RC;
    const int kh = h / g.rep;
    const int p = threadIdx.x % RL, jj = threadIdx.x / RL;
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int t = g.rows ? blockIdx.y : 0;
    float* Sh = (g.rows ? g.rows[blockIdx.y].S : g.S) + (size_t)h * DK * DV;
    float* cstate = g.rows ? g.rows[blockIdx.y].conv_state : g.conv_state;
    slab_load_async(slab, Sh, j0);     // in flight while the operands are prepared
    // the gate input and the norm weight of this CTA's 16 outputs, fetched early
    float zv = 0.0f, nw = 0.0f;
    if (threadIdx.x < RC) {
        zv = g.z[((size_t)t * g.n_v + h) * DV + j0 + threadIdx.x];
        nw = g.norm[j0 + threadIdx.x];
    }
    if (wib < 2) {
        // warp 0: q of k head kh, warp 1: k — lane owns four consecutive channels, as in k_gdn_prep
        const int c0 = (wib == 0 ? kh : g.n_k + kh) * DK + lane * 4;
        float v[4], sq[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            v[e] = conv_silu(g, t, c0 + e);
            sq[e] = fmul(v[e], v[e]);
        }
        const float ss = fold_lanes<32>(fold_run<4>(sq));
        const float inv = fdiv(1.0f, fsqrt(fadd(ss, g.eps)));
        float (*dst)[RUN_STRIDE] = wib == 0 ? pq : pk;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            v[e] = fmul(v[e], inv);
            if (wib == 0) v[e] = fmul(v[e], __uint_as_float(QSCALE_BITS));
            dst[(lane * 4 + e) / RR][(lane * 4 + e) % RR] = v[e];
        }
    } else if (wib == 2) {
        if (lane < RC) pv[lane] = conv_silu(g, t, 2 * g.n_k * DK + h * DV + j0 + lane);
        if (lane == 0) pbd[0] = sigmoid_f(g.b[(size_t)t * g.n_v + h]);
    } else {
        if (lane == 0) {
            const float sp = softplus_f(fadd(g.a[(size_t)t * g.n_v + h], g.dt_bias[h]));
            pbd[1] = exp_f(-fmul(g.A[h], sp));
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    float s[RR], k[RR], q[RR];
#pragma unroll
    for (int i = 0; i < RR; i++) {
        s[i] = slab[slab_at(p * RR + i, jj)];
        k[i] = pk[p][i];
        q[i] = pq[p][i];
    }
    const float ov = recur_step(s, k, q, pv[jj], pbd[0], pbd[1]);
    if (p == 0) so[jj] = ov;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < RR; i++) slab[slab_at(p * RR + i, jj)] = s[i];
    // ---- gated output norm of the head: this CTA's subtree sum to every peer, then the tree over the 8 sums
    float mine = 0.0f, ss16 = 0.0f;
    if (wib == 0) {
        mine = lane < RC ? so[lane] : 0.0f;
        ss16 = fold_lanes<RC>(fmul(mine, mine));                 // lanes 0..15: the subtree over this CTA's 16 squares
    }
    cluster_wait();                                               // every CTA of the cluster is running
    if (wib == 0 && lane < GDN_CL) cg::this_cluster().map_shared_rank(peer_ss, lane)[rank] = ss16;
    cluster_arrive();
    cluster_wait();                                               // all eight sums have landed here
    if (wib == 0) {
        const float part = lane < GDN_CL ? peer_ss[lane] : 0.0f;
        const float tot = __shfl_sync(FULL, fold_lanes<GDN_CL>(part), 0);
        const float inv = fdiv(1.0f, fsqrt(fadd(fdiv(tot, (float)DV), g.eps)));
        if (lane < RC) {
            const float yn = fmul(fmul(mine, inv), nw);
            g.on[((size_t)t * g.n_v + h) * DV + j0 + lane] = fmul(yn, silu_f(zv));
        }
    }
    __syncthreads();
    slab_store(slab, Sh, j0);
    // ---- conv state <- the last three raw inputs.  Every read of it by this CTA is behind the barriers above.
    if (threadIdx.x < RC) {
        const size_t c = (size_t)2 * g.n_k * DK + (size_t)h * DV + j0 + threadIdx.x;
        const float s1 = cstate[(size_t)g.conv_dim + c], s2 = cstate[(size_t)2 * g.conv_dim + c];
        const float x0 = g.qkv[(size_t)t * g.conv_dim + c];
        cstate[c] = s1;
        cstate[(size_t)g.conv_dim + c] = s2;
        cstate[(size_t)2 * g.conv_dim + c] = x0;
    }
    if (threadIdx.x == 0) {
        unsigned* cnt = &g_conv_done[t * g.n_k + kh];
        __threadfence();
        last_reader = atomicAdd(cnt, 1u) == (unsigned)(g.rep * GDN_CL) - 1u;
        if (last_reader) *cnt = 0;
    }
    __syncthreads();
    if (last_reader) {
        __threadfence();
        // q channels kh * 128 .. and k channels (n_k + kh) * 128 ..: 256 channels, two per thread
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const size_t c = (size_t)(e == 0 ? kh : g.n_k + kh) * DK + threadIdx.x;
            const float s1 = __ldcg(cstate + (size_t)g.conv_dim + c), s2 = __ldcg(cstate + (size_t)2 * g.conv_dim + c);
            const float x0 = g.qkv[(size_t)t * g.conv_dim + c];
            cstate[c] = s1;
            cstate[(size_t)g.conv_dim + c] = s2;
            cstate[(size_t)2 * g.conv_dim + c] = x0;
        }
    }
}

// Sequence form (prefill): the CTA walks all M tokens of one sequence.  The recurrence is strictly sequential, so its
// speed is the latency of one step; the per-token operands that k_gdn_prep left in scratch (k and q of the k head, the
// 16 v values, beta, decay) are staged through shared memory in blocks of TB tokens, the next block in flight
// (cp.async) while the current one is consumed, so no step waits for global memory.
constexpr int TB = 8;
struct TokOps {
    float k[RL][RUN_STRIDE];
    float q[RL][RUN_STRIDE];
    float v[RC];
    float beta, decay, pad0, pad1;
};
static_assert(sizeof(TokOps) % 16 == 0, "token operands stay 16-byte aligned");

__global__ void __launch_bounds__(RC * RL) k_gdn_recur_seq(const GdnArgs g) {
    __shared__ __align__(16) float slab[SLAB_FLOATS];
    __shared__ __align__(16) TokOps ops[2][TB];
    pdl_trigger();
    pdl_wait();
    const int h = blockIdx.x / (DV / RC);
    const int j0 = (blockIdx.x % (DV / RC)) * RC;
    const int kh = h / g.rep;
    const int p = threadIdx.x % RL, jj = threadIdx.x / RL;
    float* Sh = g.S + (size_t)h * DK * DV;
    slab_load_async(slab, Sh, j0);
    const size_t ystride = g.conv_dim;
    const float* qbase = g.y + (size_t)kh * DK;
    const float* kbase = g.y + (size_t)g.n_k * DK + (size_t)kh * DK;
    const float* vbase = g.y + (size_t)2 * g.n_k * DK + (size_t)h * DV + j0;
    constexpr int CH = 2 * (DK / 4) + RC / 4;          // 16-byte pieces per token: k, q, v
    auto stage = [&](int t0, int buf) {
        const int n = min(TB, g.M - t0);
        for (int i = threadIdx.x; i < n * CH; i += RC * RL) {
            const int tok = i / CH, c = i % CH;
            const float* src;
            float* dst;
            if (c < DK / 4) { src = kbase + (size_t)(t0 + tok) * ystride + c * 4; dst = &ops[buf][tok].k[c >> 2][(c & 3) * 4]; }
            else if (c < 2 * (DK / 4)) { const int cc = c - DK / 4; src = qbase + (size_t)(t0 + tok) * ystride + cc * 4; dst = &ops[buf][tok].q[cc >> 2][(cc & 3) * 4]; }
            else { const int cc = c - 2 * (DK / 4); src = vbase + (size_t)(t0 + tok) * ystride + cc * 4; dst = &ops[buf][tok].v[cc * 4]; }
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
        }
        if ((int)threadIdx.x < 2 * n) {
            const int tok = threadIdx.x >> 1;
            const float* src = ((threadIdx.x & 1) ? g.decay : g.beta) + (size_t)(t0 + tok) * g.n_v + h;
            float* dst = (threadIdx.x & 1) ? &ops[buf][tok].decay : &ops[buf][tok].beta;
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(0, 0);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    float s[RR];
#pragma unroll
    for (int i = 0; i < RR; i++) s[i] = slab[slab_at(p * RR + i, jj)];
    int buf = 0;
    for (int t0 = 0; t0 < g.M; t0 += TB, buf ^= 1) {
        if (t0 + TB < g.M) stage(t0 + TB, buf ^ 1);        // next block in flight
        const int n = min(TB, g.M - t0);
        // two register sets: the next token's operands come out of shared memory while this token's step runs
        float kr[2][RR], qr[2][RR], vr[2], br[2], dr[2];
        auto take = [&](int tok, int b) {
            const TokOps& o = ops[buf][tok];
#pragma unroll
            for (int i = 0; i < RR; i += 4) {
                const float4 kk = *reinterpret_cast<const float4*>(&o.k[p][i]);
                const float4 qq = *reinterpret_cast<const float4*>(&o.q[p][i]);
                kr[b][i] = kk.x; kr[b][i + 1] = kk.y; kr[b][i + 2] = kk.z; kr[b][i + 3] = kk.w;
                qr[b][i] = qq.x; qr[b][i + 1] = qq.y; qr[b][i + 2] = qq.z; qr[b][i + 3] = qq.w;
            }
            vr[b] = o.v[jj];
            br[b] = o.beta;
            dr[b] = o.decay;
        };
        take(0, 0);
#pragma unroll 1
        for (int tok = 0; tok < n; tok += 2) {
#pragma unroll
            for (int b = 0; b < 2; b++) {
                const int tk = tok + b;
                if (tk < n) {
                    if (tk + 1 < n) take(tk + 1, b ^ 1);
                    const float ov = recur_step(s, kr[b], qr[b], vr[b], br[b], dr[b]);
                    if (p == 0) g.o[((size_t)(t0 + tk) * g.n_v + h) * DV + j0 + jj] = ov;
                }
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                   // the next block has landed; this one may be overwritten
    }
#pragma unroll
    for (int i = 0; i < RR; i++) slab[slab_at(p * RR + i, jj)] = s[i];
    __syncthreads();
    slab_store(slab, Sh, j0);
}

// on = rmsnorm(o, norm, eps) * silu_f(z): one warp per (token, v head).  Extra CTAs past the rows move the conv state.
__global__ void __launch_bounds__(128) k_gdn_out(const GdnArgs g, int row_blocks) {
    pdl_trigger();
    pdl_wait();
    if ((int)blockIdx.x >= row_blocks) {
        // conv state <- the last three raw inputs (times M-3 .. M-1); each channel is read fully before it is written
        const int cblocks = (g.conv_dim + 127) / 128;
        const int idx = blockIdx.x - row_blocks;
        const int seq = idx / cblocks;                       // 0 unless this is a batched step
        const int c = (idx % cblocks) * 128 + threadIdx.x;
        if (c < g.conv_dim) {
            const int t_last = g.rows ? seq : g.M - 1;       // the newest input of the sequence
            float* state = g.rows ? g.rows[seq].conv_state : g.conv_state;
            float keep[3];
#pragma unroll
            for (int r = 0; r < 3; r++) keep[r] = conv_in(g, t_last, 2 - r, c);
#pragma unroll
            for (int r = 0; r < 3; r++) state[(size_t)r * g.conv_dim + c] = keep[r];
        }
        return;
    }
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const long long row = (long long)blockIdx.x * 4 + wib;   // t * n_v + h
    if (row < (long long)g.M * g.n_v) {
        const float* o = g.o + row * DV + lane * 4;
        float v[4], sq[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            v[e] = o[e];
            sq[e] = fmul(v[e], v[e]);
        }
        const float ss = fold_lanes<32>(fold_run<4>(sq));
        const float inv = fdiv(1.0f, fsqrt(fadd(fdiv(ss, (float)DV), g.eps)));
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float yn = fmul(fmul(v[e], inv), g.norm[lane * 4 + e]);
            g.on[row * DV + lane * 4 + e] = fmul(yn, silu_f(g.z[row * DV + lane * 4 + e]));
        }
    }
}

static size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }
struct GdnScratch {
    size_t done, y, beta, decay, o, total;
};
static GdnScratch gdn_scratch(int M, int n_k, int n_v) {
    GdnScratch s;
    const size_t conv_dim = (size_t)2 * n_k * DK + (size_t)n_v * DV;
    s.done = 0;          // a counter at a fixed place (it must stay zero between calls whatever M is)
    s.y = 256;
    s.beta = s.y + up256((size_t)M * conv_dim * 4);
    s.decay = s.beta + up256((size_t)M * n_v * 4);
    s.o = s.decay + up256((size_t)M * n_v * 4);
    s.total = s.o + up256((size_t)M * n_v * DV * 4);
    return s;
}

}  // namespace detb

using namespace detb;

extern "C" {

size_t det_gdn_scratch_bytes(int M, int n_k, int n_v, int dk, int dv) {
    (void)dk; (void)dv;
    return gdn_scratch(M > 0 ? M : 1, n_k, n_v).total;
}

static void gdn_entry(const det_gdn_layer* L, det_gdn_state* S, const det_gdn_state* rows, const float* qkv, const float* z,
                      const float* a, const float* b, float eps, int M, int n_k, int n_v, int dk, int dv, float* on,
                      void* scratch, float* gin, float* gout, cudaStream_t st) {
    if (M <= 0) return;
    DETB_REQUIRE(dk == DK && dv == DV, "Gated DeltaNet kernels are built for dk = dv = 128");
    DETB_REQUIRE(n_k > 0 && n_v % n_k == 0, "n_v must be a multiple of n_k");
    const GdnScratch sm = gdn_scratch(M, n_k, n_v);
    uint8_t* base = static_cast<uint8_t*>(scratch);
    GdnArgs g;
    g.conv = L->conv; g.A = L->A; g.dt_bias = L->dt_bias; g.norm = L->norm;
    g.rows = rows;
    g.conv_state = S ? S->conv_state : nullptr;
    g.S = S ? S->S : nullptr;
    g.qkv = qkv; g.z = z; g.a = a; g.b = b;
    g.eps = eps; g.M = M; g.n_k = n_k; g.n_v = n_v; g.rep = n_v / n_k;
    g.conv_dim = 2 * n_k * DK + n_v * DV;
    g.on = on;
    g.y = reinterpret_cast<float*>(base + sm.y);
    g.beta = reinterpret_cast<float*>(base + sm.beta);
    g.decay = reinterpret_cast<float*>(base + sm.decay);
    g.o = gout ? gout : reinterpret_cast<float*>(base + sm.o);
    g.gin = gin;
    cudaStream_t q = queue_of(st);
    const int heads = 2 * n_k + n_v;
    // decode form (one token per sequence, nothing exported): the whole mixer in one launch, a cluster per v head.  With
    // many sequences the shared prep kernel is less work than preparing inside every recurrence CTA.
    const int seqs = rows ? M : 1;
    const bool one_launch = (rows ? M < 8 : M == 1) && gin == nullptr && gout == nullptr && seqs * n_k <= CONV_COUNTERS;
    if (one_launch) {
        launch_pdl(k_gdn_step, dim3(n_v * GDN_CL, seqs), dim3(RC * RL), 0, q, GDN_CL, g);
        return;
    }
    launch_pdl(k_gdn_prep, dim3((heads + 3) / 4, M), dim3(128), 0, q, 1, g);
    if (rows) launch_pdl(k_gdn_recur_dec, dim3(n_v * (DV / RC / DEC_SLABS), M), dim3(RC * RL), 0, q, 1, g);
    else launch_pdl(k_gdn_recur_seq, dim3(n_v * (DV / RC)), dim3(RC * RL), 0, q, 1, g);
    const int row_blocks = (int)(((long long)M * n_v + 3) / 4);
    const int state_blocks = ((g.conv_dim + 127) / 128) * (rows ? M : 1);
    launch_pdl(k_gdn_out, dim3(row_blocks + state_blocks), dim3(128), 0, q, 1, g, row_blocks);
}

void det_gdn_ex(const det_gdn_layer* L, det_gdn_state* S, const float* qkv, const float* z, const float* a,
                const float* b, float eps, int M, int n_k, int n_v, int dk, int dv, float* on, void* scratch,
                float* gin, float* gout, cudaStream_t st) {
    gdn_entry(L, S, nullptr, qkv, z, a, b, eps, M, n_k, n_v, dk, dv, on, scratch, gin, gout, st);
}
// Batched decode (no reference counterpart): M sequences advance one token each; row t of the inputs belongs to the
// sequence with state rows[t] (a DEVICE array of M det_gdn_state).  Each row equals det_gdn(M = 1) on that state.
void det_gdn_rows(const det_gdn_layer* L, const det_gdn_state* rows, const float* qkv, const float* z, const float* a,
                  const float* b, float eps, int M, int n_k, int n_v, int dk, int dv, float* on, void* scratch,
                  cudaStream_t st) {
    gdn_entry(L, nullptr, rows, qkv, z, a, b, eps, M, n_k, n_v, dk, dv, on, scratch, nullptr, nullptr, st);
}

void det_gdn(const det_gdn_layer* L, det_gdn_state* S, const float* qkv, const float* z, const float* a,
             const float* b, float eps, int M, int n_k, int n_v, int dk, int dv, float* on, void* scratch,
             cudaStream_t st) {
    det_gdn_ex(L, S, qkv, z, a, b, eps, M, n_k, n_v, dk, dv, on, scratch, nullptr, nullptr, st);
}

}  // extern "C"
