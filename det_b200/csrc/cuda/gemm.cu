// Integer GEMM  y[t][n] = ((float)acc * c[n]) * sx[t],  acc = sum_g (m[n][g] * mx[t][g]) * sum_{k in g} wq[n][k] * xq[t][k]
// (docs/SPEC.md §3, spec/quant.rs:99-117).  Replaces kernels/cuda/gemm.cu behind det_gemm / det_gemm_ex.
//
// All sums are exact integers, so any split of K over lanes, warps or stages gives the same acc; the two fp32
// multiplies (and the optional residual add) run once per output element in the spec's order.
//
// This file: the entry points and k_gemm_rowmajor, which serves any M on the reference row-major layout (one warp per
// output row, 8 tokens per pass over the row).  The decode path (M <= 8 on the repacked layout) is gemv_stream.cu.
#include "gemm_common.cuh"

namespace detb {

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

size_t det_gemm_scratch_bytes(int M, int K) { return (size_t)(M > 0 ? M : 1) * (size_t)(K / 128) * sizeof(int); }
void det_gemm_set_scratch(void* p, size_t bytes) { (void)p; (void)bytes; }

static OutSpec make_out(const det_qlinear* L, float* y, int accumulate, int nparts, const int* offs, float* const* dsts) {
    DETB_REQUIRE(nparts <= 4, "at most 4 fused parts");
    OutSpec out;
    out.y = y;
    out.N = L->N;
    out.accumulate = accumulate;
    out.nparts = nparts > 1 ? nparts : 0;
    out.pairs = (L->bits & DET_LAYOUT_PAIRS) ? 1 : 0;
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
    return out;
}
static void check_linear(const det_qlinear* L) {
    const int bits = L->bits & 0xff;
    DETB_REQUIRE(bits == 4 || bits == 6 || bits == 8, "bits must be 4, 6 or 8");
    DETB_REQUIRE(L->K > 0 && L->K % 128 == 0 && L->N > 0, "K must be a positive multiple of 128");
    DETB_REQUIRE(!(L->bits & DET_LAYOUT_PAIRS) || (L->bits & DET_LAYOUT_STREAM), "the pairs layout is a streaming layout");
}

void det_gemm_ex(const det_qlinear* L, const int8_t* xq, const float* sx, const uint16_t* mx, int M, float* y,
                 int accumulate, int nparts, const int* offs, float* const* dsts, cudaStream_t st) {
    if (M <= 0) return;
    check_linear(L);
    const int bits = L->bits & 0xff;
    const OutSpec out = make_out(L, y, accumulate, nparts, offs, dsts);
    cudaStream_t q = queue_of(st);
    if (L->bits & DET_LAYOUT_INT8) {
        gemm_tc_launch(L, xq, sx, mx, M, out, q);
    } else if (L->bits & DET_LAYOUT_STREAM) {
        GemvCall call;
        call.lin = L;
        call.xq = xq; call.sx = sx; call.mx = mx;
        call.M = M;
        call.out = out;
        gemv_stream_launch(call, q);
    } else {
        if (bits == 8) gemm_rowmajor_bits<8>(L, xq, sx, mx, M, out, q);
        else if (bits == 6) gemm_rowmajor_bits<6>(L, xq, sx, mx, M, out, q);
        else gemm_rowmajor_bits<4>(L, xq, sx, mx, M, out, q);
    }
}

void det_gemm_pair(const det_qlinear* L1, const det_qlinear* L2, const int8_t* xq, const float* sx, const uint16_t* mx, int M,
                   int nparts1, const int* offs1, float* const* dsts1, int nparts2, const int* offs2, float* const* dsts2,
                   cudaStream_t st) {
    if (M <= 0) return;
    DETB_REQUIRE(L1 && L2 && nparts1 >= 1 && nparts2 >= 1 && dsts1 && dsts2, "det_gemm_pair needs two linears and their outputs");
    if ((L1->bits & DET_LAYOUT_INT8) && (L2->bits & DET_LAYOUT_INT8) && L1->K == L2->K) {
        check_linear(L1);
        check_linear(L2);
        const OutSpec out1 = make_out(L1, nullptr, 0, nparts1, offs1, dsts1);
        const OutSpec out2 = make_out(L2, nullptr, 0, nparts2, offs2, dsts2);
        gemm_tc_launch(L1, xq, sx, mx, M, out1, queue_of(st), L2, &out2);
        return;
    }
    det_gemm_ex(L1, xq, sx, mx, M, nullptr, 0, nparts1, offs1, dsts1, st);
    det_gemm_ex(L2, xq, sx, mx, M, nullptr, 0, nparts2, offs2, dsts2, st);
}

void det_gemv(const det_gemv_op* op, cudaStream_t st) {
    DETB_REQUIRE(op && op->lin, "det_gemv needs a linear");
    if (op->M <= 0) return;
    check_linear(op->lin);
    DETB_REQUIRE(op->lin->bits & DET_LAYOUT_STREAM, "det_gemv needs the streaming weight layout");
    GemvCall call;
    call.lin = op->lin;
    call.lin2 = op->lin2;
    call.src = op->src;
    call.xq = op->xq; call.sx = op->sx; call.mx = op->mx;
    call.M = op->M;
    call.out = make_out(op->lin, op->y, op->accumulate, op->nparts, op->offs, op->dsts);
    if (op->lin2) {
        check_linear(op->lin2);
        call.out2 = make_out(op->lin2, op->y2, 0, op->nparts2, op->offs2, op->dsts2);
    }
    call.h = op->h;
    call.h_amax = op->h_amax;
    gemv_stream_launch(call, queue_of(st));
}

void det_gemm(const det_qlinear* L, const int8_t* xq, const float* sx, const uint16_t* mx, int M, float* y,
              cudaStream_t st) {
    det_gemm_ex(L, xq, sx, mx, M, y, 0, 0, nullptr, nullptr, st);
}

}  // extern "C"
