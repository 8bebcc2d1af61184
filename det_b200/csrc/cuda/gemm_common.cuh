// Pieces shared by the GEMM translation units: output routing (Write / Accumulate / Parts), 64-bit shuffles, the
// mixed-sign byte dot product, and the mbarrier / bulk-copy PTX wrappers.
#pragma once
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
    int pairs;           // rows come in the pairs layout: physical row n is column (n & 1) * N / 2 + n / 2
};
__device__ __forceinline__ void emit(const OutSpec& o, int t, int n, float v) {
    if (o.pairs) n = (n & 1) * (o.N >> 1) + (n >> 1);
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

// Four byte products added to acc: signed x signed for W8, unsigned codes x signed activations for W4 / W6.
template <int BITS>
__device__ __forceinline__ int dot4(unsigned w, int x, int acc) {
    int r;
    if (BITS == 8) asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(x), "r"(acc));
    else asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(x), "r"(acc));
    return r;
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
// Bounded wait: polls until the phase completes or `limit` SM clock cycles have passed (wait_limit(error_flag): about two
// seconds by default); returns false then.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, long long limit) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - start > limit) return false;
    }
}
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}


// Entry of the streaming GEMV (gemv_stream.cu): M tokens against a det_linear_repack layout.
struct GemvCall {
    const det_qlinear* lin = nullptr;      // streaming layout
    const det_qlinear* lin2 = nullptr;     // optional W8 streaming-layout linear over the same input rows
    const det_act_source* src = nullptr;   // activation prologue; otherwise xq / sx / mx
    const int8_t* xq = nullptr;
    const float* sx = nullptr;
    const uint16_t* mx = nullptr;
    int M = 0;
    OutSpec out{}, out2{};
    float* h = nullptr;                    // SwiGLU product instead of `out` (pairs layout)
    unsigned* h_amax = nullptr;            // with h: the buffer the epilogue folds the group maxima of h into
};
void gemv_stream_launch(const GemvCall& call, cudaStream_t q);

// Entry of the tensor-core GEMM (gemm_tc.cu): L->wq is the int8-expanded layout.
// L2 / out2 (optional): a second int8-layout linear over the same rows, taken into the same launch.
void gemm_tc_launch(const det_qlinear* L, const int8_t* xq, const float* sx, const uint16_t* mx, int M,
                    const OutSpec& out, cudaStream_t q, const det_qlinear* L2 = nullptr, const OutSpec* out2 = nullptr);

}  // namespace detb
