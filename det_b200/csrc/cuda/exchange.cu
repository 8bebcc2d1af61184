// One-shot all-gather over NVLink peer memory for the tensor-parallel decode step (latency-bound: a 27B token needs 257
// exchanges of a few KB each, so the cost of an exchange is its latency, not its bytes).  The reference has no
// multi-GPU code at all.
//
// Every rank owns a staging area of the same size, mapped into every other rank's address space through CUDA IPC
// handles.  One kernel launch per rank does the whole exchange: wait for the producer kernel (griddepcontrol.wait), send
// the local slice as self-validating packets into every rank's staging (plain peer stores — no multicast, no remote
// loads), then read the gathered row out of the local staging as the packets arrive.  All waits are bounded; a timeout
// sets the library's error word and the kernel returns.  The protocol is in exchange.cuh.
#include "exchange.cuh"
#include <algorithm>
#include <cstring>

namespace detb {

// full[M][size*slice] (ordinary local memory) <- the gathered rows
__global__ void __launch_bounds__(1024) k_xchg_gather(const XchgArgs a, float* __restrict__ full) {
    pdl_trigger();
    pdl_wait();
    const unsigned seq = xchg_seq(a);
    xchg_push(a, seq);
    const size_t packets = (size_t)a.M * a.size * (a.slice >> 1);
    for (size_t pk = (size_t)blockIdx.x * blockDim.x + threadIdx.x; pk < packets; pk += (size_t)gridDim.x * blockDim.x)
        reinterpret_cast<float2*>(full)[pk] = xchg_read(a, seq, pk);
}

}  // namespace detb

using namespace detb;

extern "C" {

void* det_xchg_create(size_t bytes, int rank, int size) {
    DETB_REQUIRE(size >= 1 && size <= XCHG_MAX_RANKS && rank >= 0 && rank < size, "bad exchange group");
    Xchg* x = new Xchg();
    x->slot_bytes = ((bytes + 1) / 2 + 255) & ~(size_t)255;
    x->rank = rank;
    x->size = size;
    (void)queue_of(nullptr);   // runtime up
    DETB_CUDA_OK(cudaMalloc(&x->base, 2 * x->slot_bytes));
    DETB_CUDA_OK(cudaMemset(x->base, 0, 2 * x->slot_bytes));
    DETB_CUDA_OK(cudaMalloc(&x->words, 2 * sizeof(unsigned)));
    DETB_CUDA_OK(cudaMemset(x->words, 0, 2 * sizeof(unsigned)));
    x->peer[rank] = x->base;
    return x;
}
void det_xchg_ipc_handle(void* h, uint8_t out[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t mh;
    DETB_CUDA_OK(cudaIpcGetMemHandle(&mh, static_cast<Xchg*>(h)->base));
    memcpy(out, &mh, 64);
}
// handles: size x 64 bytes, rank order (this rank's own entry is ignored).
void det_xchg_open(void* h, const uint8_t* handles) {
    Xchg* x = static_cast<Xchg*>(h);
    for (int r = 0; r < x->size; r++) {
        if (r == x->rank) continue;
        cudaIpcMemHandle_t mh;
        memcpy(&mh, handles + (size_t)r * 64, 64);
        void* p = nullptr;
        DETB_CUDA_OK(cudaIpcOpenMemHandle(&p, mh, cudaIpcMemLazyEnablePeerAccess));
        x->peer[r] = static_cast<uint8_t*>(p);
    }
}
// Timing aid: no peers are opened; every rank slot maps to this rank's own staging, so one process can run the launch
// sequence of one rank of `size` (the gathered values are meaningless).
void det_xchg_open_loopback(void* h) {
    Xchg* x = static_cast<Xchg*>(h);
    for (int r = 0; r < x->size; r++) x->peer[r] = x->base;
    x->loopback = true;
}
// Test aid for the bounded wait (loopback handles only): the packets of column block `rank` are not sent from now on, so
// a receiver's wait for them runs out; rank < 0 sends everything again.  Nothing faults or hangs: the wait gives up after
// the wait limit, sets the error word and the kernel returns zeros for the missing packets.
void det_debug_xchg_drop(void* h, int rank) {
    Xchg* x = static_cast<Xchg*>(h);
    DETB_REQUIRE(x->loopback, "det_debug_xchg_drop works on loopback handles only");
    x->drop = rank;
}
// Largest exchange the staging takes, in gathered fp32 values (M * size * slice).
size_t det_xchg_capacity(void* h) { return static_cast<Xchg*>(h)->slot_bytes / 8; }

void det_xchg_all_gather(void* h, const float* local, float* full, int M, int slice, cudaStream_t st) {
    Xchg* x = static_cast<Xchg*>(h);
    DETB_REQUIRE(slice % 2 == 0 && M > 0, "exchange slices are whole packets (two values)");
    DETB_REQUIRE((size_t)M * x->size * slice * 8 <= x->slot_bytes, "exchange larger than the staging slot");
    const XchgArgs a = xchg_args(x, local, nullptr, M, slice);
    const size_t packets = (size_t)M * x->size * (slice >> 1);
    const unsigned grid = (unsigned)std::min<size_t>(64, std::max<size_t>(1, packets / 1024));
    launch_pdl(k_xchg_gather, dim3(grid), dim3(1024), 0, queue_of(st), 1, a, full);
}
void det_xchg_destroy(void* h) {
    Xchg* x = static_cast<Xchg*>(h);
    if (!x) return;
    cudaDeviceSynchronize();
    for (int r = 0; r < x->size; r++)
        if (r != x->rank && x->peer[r] && !x->loopback) cudaIpcCloseMemHandle(x->peer[r]);
    cudaFree(x->base);
    cudaFree(x->words);
    delete x;
}

}  // extern "C"
