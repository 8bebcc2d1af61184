// Measurement aid: how fast does a B200 hand a large buffer to its SMs when there is nothing to compute?  The decode GEMV
// is a weight stream, so its ceiling is whatever the memory system gives to the GEMV's own access pattern; these kernels
// move bytes the same ways and do nothing else.  No result of the library depends on this file.
//
//   mode 0: plain loads.  Every thread reads 16 bytes at a time, grid-stride, four loads in flight (the pattern of the
//           copy that the HBM peak figure is measured with, without its store half).
//   mode 1: the GEMV's transport.  One CTA per SM; every warp owns `slots` shared-memory slots and streams records of
//           `rec_bytes` into them with cp.async.bulk, one mbarrier per slot; records are dealt out the way the GEMV deals
//           out its quads: `nch` consecutive records form a quad, quad i goes to CTA i % grid, warp (i / grid) % warps.
//   mode 2: the same ring, but every CTA streams one contiguous span of the buffer (its warps take consecutive records).
// A CTA has `warps` warps; a ring of less than half an SM's shared memory lets the CTA of the next launch come up beside
// it and fill its own ring while this one drains.
// The buffer holds `regions` pieces of `bytes`; launch r reads piece r % regions, so that launches the size of one GEMV
// (tens of MB, less than the L2 holds) still read from HBM.  Launches are chained with programmatic dependent launch the
// way the decode step chains its GEMVs: a launch fills its slots before it waits for its predecessor.
#include "gemm_common.cuh"

namespace detb {

__global__ void __launch_bounds__(1024) k_stream_loads(const uint4* __restrict__ p, size_t n16, unsigned* sink) {
    pdl_trigger();
    pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    unsigned acc = 0;
    for (; i + 3 * stride < n16; i += 4 * stride) {
        const uint4 a = __ldg(p + i), b = __ldg(p + i + stride), c = __ldg(p + i + 2 * stride), d = __ldg(p + i + 3 * stride);
        acc ^= a.x ^ b.y ^ c.z ^ d.w;
    }
    for (; i < n16; i += stride) acc ^= __ldg(p + i).x;
    if (acc == 0x9e3779b9u) *sink = acc;      // keeps the loads alive
}

struct RingArgs {
    const uint8_t* p;
    long long records;      // whole records in the buffer
    int rec_bytes, warps, slots, nch, contiguous;
    int* error_flag;
    unsigned* sink;
};

__global__ void __launch_bounds__(512) k_stream_ring(const RingArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int W = a.warps, S = a.slots;
    unsigned long long* full = reinterpret_cast<unsigned long long*>(smem);          // [W * S]
    uint8_t* ring = smem + ((W * S * 8 + 127) & ~127);
    const long long wl = wait_limit(a.error_flag);
    pdl_trigger();
    for (int i = threadIdx.x; i < W * S; i += blockDim.x) mbar_init(&full[i], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();
    // record number of this warp's i-th request
    const long long quads = a.records / a.nch;
    const long long span = (a.records + gridDim.x - 1) / gridDim.x;      // contiguous mode: records per CTA
    auto record = [&](long long i) -> long long {
        if (a.contiguous) {
            const long long r = (long long)blockIdx.x * span + i * W + warp;
            return (r < a.records && i * W + warp < span) ? r : -1;
        }
        const long long q = (long long)blockIdx.x + ((long long)warp + (i / a.nch) * W) * gridDim.x;
        return q < quads ? q * a.nch + i % a.nch : -1;
    };
    long long next = 0;        // next request
    int islot = 0;
    auto issue = [&]() {
        const long long r = record(next);
        if (r < 0) return;
        const int s = warp * S + islot;
        mbar_expect_tx(&full[s], (unsigned)a.rec_bytes);
        bulk_g2s(ring + (size_t)s * a.rec_bytes, a.p + (size_t)r * a.rec_bytes, (unsigned)a.rec_bytes, &full[s]);
        next++;
        if (++islot == S) islot = 0;
    };
    if (lane == 0)
        for (int i = 0; i < S; i++) issue();
    pdl_wait();
    unsigned acc = 0, phase = 0;
    int cslot = 0;
    bool ok = true;
    for (long long i = 0; record(i) >= 0; i++) {
        const int s = warp * S + cslot;
        ok = mbar_wait(&full[s], phase, wl);
        if (!ok) break;
        acc ^= *reinterpret_cast<const unsigned*>(ring + (size_t)s * a.rec_bytes + lane * 16);
        if (++cslot == S) { cslot = 0; phase ^= 1u; }
        __syncwarp();
        if (lane == 0) issue();
    }
    if (!ok && lane == 0) {
        atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
        for (int s = warp * S; s < (warp + 1) * S; s++) {      // copies still in flight target this CTA's shared memory
            (void)mbar_wait(&full[s], 0u, wl >> 5);
            (void)mbar_wait(&full[s], 1u, wl >> 5);
        }
    }
    if (acc == 0x9e3779b9u) *a.sink = acc;
}

}  // namespace detb

using namespace detb;

extern "C" double det_debug_stream_peak(const void* p, size_t bytes, int regions, int mode, int rec_bytes, int warps,
                                        int slots, int nch, int reps) {
    DETB_REQUIRE(p && bytes >= (1u << 20) && bytes % 256 == 0 && regions >= 1 && reps > 0 &&
                     (reinterpret_cast<uintptr_t>(p) & 255) == 0, "bad buffer");
    cudaStream_t q = queue_of(nullptr);
    static unsigned* sink = nullptr;
    if (!sink) DETB_CUDA_OK(cudaMalloc(&sink, 16));
    RingArgs a{};
    size_t smem = 0, moved = bytes & ~(size_t)15;
    if (mode != 0) {
        DETB_REQUIRE(rec_bytes >= 512 && rec_bytes % 16 == 0 && warps >= 1 && warps <= 16 && slots >= 1 && nch >= 1, "bad ring");
        smem = ((size_t)warps * slots * 8 + 127) / 128 * 128 + (size_t)warps * slots * rec_bytes;
        DETB_REQUIRE(smem <= smem_optin() - 1024, "the ring does not fit shared memory");
        DETB_CUDA_OK(cudaFuncSetAttribute(k_stream_ring, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        a.p = static_cast<const uint8_t*>(p);
        a.records = (long long)(bytes / rec_bytes);
        if (mode == 1) a.records = a.records / nch * nch;
        a.rec_bytes = rec_bytes; a.warps = warps; a.slots = slots; a.nch = nch; a.contiguous = mode == 2;
        a.error_flag = error_word();
        a.sink = sink;
        moved = (size_t)a.records * rec_bytes;
    }
    int turn = 0;
    auto launch = [&]() {
        const uint8_t* piece = static_cast<const uint8_t*>(p) + (size_t)(turn++ % regions) * bytes;
        if (mode == 0) {
            launch_pdl(k_stream_loads, dim3(sm_count() * 2), dim3(1024), 0, q, 1, reinterpret_cast<const uint4*>(piece),
                       bytes / 16, sink);
        } else {
            a.p = piece;
            // a ring of at most half an SM's shared memory leaves room for the next launch's CTA beside this one
            launch_pdl(k_stream_ring, dim3(sm_count()), dim3(warps * 32), smem, q, 1, a);
        }
    };
    cudaEvent_t e0, e1;
    DETB_CUDA_OK(cudaEventCreate(&e0));
    DETB_CUDA_OK(cudaEventCreate(&e1));
    launch();
    DETB_CUDA_OK(cudaEventRecord(e0, q));
    for (int r = 0; r < reps; r++) launch();
    DETB_CUDA_OK(cudaEventRecord(e1, q));
    DETB_CUDA_OK(cudaEventSynchronize(e1));
    DETB_CUDA_OK(cudaGetLastError());
    float ms = 0.0f;
    DETB_CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return (double)moved * reps / (ms * 1e-3) / 1e9;
}
