// Shared between the stand-alone exchange kernel (exchange.cu) and the row kernels that carry an exchange as their
// prologue (glue.cu): the region handle and the device side of the flag-in-data protocol.
//
// A gathered row travels as 16-byte packets {value, seq, value, seq}: two fp32 values, each with the number of the
// exchange they belong to.  A sender stores packets straight into every rank's staging area (plain 16-byte peer stores,
// each 8-byte half self-validating); a receiver polls the packet it needs until both numbers match.  No fence, no
// separate flag, no second trip: the cost of an exchange is one NVLink store latency.  Staging has two slots used
// alternately (seq & 1): a rank can only start exchange g+2 after it received every peer's part of g+1, and a peer sends
// that only after its kernel of exchange g — which does all its reading of slot g — has finished.
#pragma once
#include "runtime.cuh"

namespace detb {

constexpr int XCHG_MAX_RANKS = 8;

struct Xchg {
    uint8_t* base = nullptr;      // this rank's staging: two slots of slot_bytes
    size_t slot_bytes = 0;
    int rank = 0, size = 1;
    bool loopback = false;        // timing aid: every "peer" is this rank's own staging (one process stands in for a rank of `size`)
    int drop = -1;                // test aid (loopback only): packets of this rank's column block are never sent
    uint8_t* peer[XCHG_MAX_RANKS] = {};   // every rank's staging as seen from here (peer[rank] == base)
    unsigned* words = nullptr;    // device words: [0] exchanges completed so far, [1] CTAs of the running launch that have pushed
};

struct XchgArgs {
    const float* local;           // [M][slice]
    const float* local_b;         // optional: the pushed value is silu(local) * local_b (SwiGLU product of the local columns)
    int M, slice, rank, size, loopback, drop;
    size_t slot_bytes;
    uint8_t* peer[XCHG_MAX_RANKS];
    unsigned* words;
    int* error_flag;
};

inline XchgArgs xchg_args(const Xchg* x, const float* local, const float* local_b, int M, int slice) {
    XchgArgs a;
    a.local = local;
    a.local_b = local_b;
    a.M = M; a.slice = slice; a.rank = x->rank; a.size = x->size; a.loopback = x->loopback; a.drop = x->loopback ? x->drop : -1;
    a.slot_bytes = x->slot_bytes;
    for (int r = 0; r < XCHG_MAX_RANKS; r++) a.peer[r] = x->peer[r];
    a.words = x->words;
    a.error_flag = error_word();
    return a;
}

// Number of the exchange this launch performs.  Every CTA reads it before it pushes; the CTA that pushes last bumps it.
__device__ __forceinline__ unsigned xchg_seq(const XchgArgs& a) { return *reinterpret_cast<volatile unsigned*>(a.words) + 1; }

// Every thread of the grid sends its share of local[M][slice] as packets into column block `rank` of the gathered
// [M][size*slice] row in EVERY rank's staging slot.  Call from all threads of all CTAs.
__device__ __forceinline__ void xchg_push(const XchgArgs& a, unsigned seq) {
    const unsigned ctas = gridDim.x * gridDim.y;
    const unsigned cta = blockIdx.y * gridDim.x + blockIdx.x;
    const int half = a.slice >> 1;                      // packets per local row
    const size_t slot = (size_t)(seq & 1u) * a.slot_bytes;
    for (int j = cta * blockDim.x + threadIdx.x; j < a.M * half; j += ctas * blockDim.x) {
        const int t = j / half, v = j - t * half;
        float2 val = reinterpret_cast<const float2*>(a.local + (size_t)t * a.slice)[v];
        if (a.local_b) {
            const float2 u = reinterpret_cast<const float2*>(a.local_b + (size_t)t * a.slice)[v];
            val.x = fmul(silu_f(val.x), u.x);
            val.y = fmul(silu_f(val.y), u.y);
        }
        const unsigned d0 = __float_as_uint(val.x), d1 = __float_as_uint(val.y);
        for (int p = 0; p < a.size; p++) {
            if (p == a.drop) continue;
            const int col = a.loopback ? p : a.rank;
            uint8_t* dst = a.peer[p] + slot + (((size_t)t * a.size + col) * half + v) * 16;
            asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(d0), "r"(seq), "r"(d1), "r"(seq)
                         : "memory");
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned done = atomicAdd(a.words + 1, 1u);
        if (done == ctas - 1) {
            a.words[1] = 0;
            *reinterpret_cast<volatile unsigned*>(a.words) = seq;
        }
    }
}

// Values 2*pk and 2*pk+1 of the gathered data in this rank's staging slot (pk counts packets over [M][size*slice]).
// Polls until the packet of this exchange has arrived; bounded (wait_limit cycles, about two seconds by default; then
// the error word is set and zeros come back; while the error word is set nothing spins again — det_clear_error resets it).
__device__ __forceinline__ float2 xchg_read(const XchgArgs& a, unsigned seq, size_t pk) {
    const uint8_t* src = a.peer[a.rank] + (size_t)(seq & 1u) * a.slot_bytes + pk * 16;
    unsigned d0, f0, d1, f1;
    long long start = 0;
    for (unsigned spins = 0;; spins++) {
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(d0), "=r"(f0), "=r"(d1), "=r"(f1) : "l"(src) : "memory");
        if (f0 == seq && f1 == seq) break;
        if ((spins & 63u) == 63u) {
            if (start == 0) start = clock64();
            if (*reinterpret_cast<volatile int*>(a.error_flag) != 0 || clock64() - start > wait_limit(a.error_flag)) {
                atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
                d0 = d1 = 0;
                break;
            }
        }
    }
    return make_float2(__uint_as_float(d0), __uint_as_float(d1));
}

}  // namespace detb
