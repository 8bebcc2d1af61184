// One-shot all-gather over NVLink peer memory for the tensor-parallel decode step (latency-bound: a 27B token needs 257
// exchanges of a few KB each, so the cost of an exchange is its latency, not its bytes).  The reference has no
// multi-GPU code at all.
//
// Every rank owns one "exchange region" with the same layout: gathered buffers at identical offsets, then a flag word
// per peer.  Regions are mapped into every other rank's address space through CUDA IPC handles.  One kernel launch per
// rank does the whole exchange: wait for the producer kernel (griddepcontrol.wait), store the local slice straight into
// every peer's gathered buffer (plain peer stores — no multicast, no remote loads), fence, write this exchange's
// sequence number into every peer's flag slot, then poll the local flags until every peer's number has arrived.
// Reuse is safe without a second handshake as long as consecutive exchanges use different gathered buffers: a rank that
// starts exchange g+2 has seen every peer start exchange g+1, and a peer starts g+1 only after it consumed the result of
// g.  All waits are bounded; a timeout sets the library's error word and the kernel returns.
#include "runtime.cuh"
#include <algorithm>
#include <cstring>

namespace detb {

constexpr int XCHG_MAX_RANKS = 8;

struct Xchg {
    uint8_t* base = nullptr;      // this rank's region
    size_t bytes = 0;             // data bytes (flags follow)
    int rank = 0, size = 1;
    uint8_t* peer[XCHG_MAX_RANKS] = {};   // every rank's region as seen from here (peer[rank] == base)
    unsigned* words = nullptr;    // device words: [0] exchanges issued so far, [1] CTAs of the running launch that are done
};

struct XchgArgs {
    const float* local;           // [M][slice]
    size_t full_off;              // byte offset of the gathered [M][size*slice] buffer inside the region
    int M, slice, rank, size;
    size_t flag_off;              // byte offset of the flag array (XCHG_MAX_RANKS words)
    uint8_t* peer[XCHG_MAX_RANKS];
    unsigned* words;
    int* error_flag;
};

__global__ void __launch_bounds__(1024) k_xchg_gather(const XchgArgs a) {
    __shared__ unsigned last_s, seq_s;
    pdl_trigger();
    pdl_wait();
    // ---- push the local slice into every rank's gathered buffer (row t, column block `rank`)
    const int vec = a.slice >> 2;                       // float4 per row
    const int per_peer = a.M * vec;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < per_peer * a.size; i += gridDim.x * blockDim.x) {
        const int p = i / per_peer, j = i - p * per_peer;
        const int t = j / vec, v = j - t * vec;
        const float4 val = reinterpret_cast<const float4*>(a.local + (size_t)t * a.slice)[v];
        float* dst = reinterpret_cast<float*>(a.peer[p] + a.full_off) + ((size_t)t * a.size + a.rank) * a.slice;
        reinterpret_cast<float4*>(dst)[v] = val;
    }
    __threadfence_system();
    __syncthreads();
    // ---- the CTA that finishes last publishes and waits; the others are done
    if (threadIdx.x == 0) {
        const unsigned done = atomicAdd(a.words + 1, 1u);
        last_s = done == gridDim.x - 1;
        if (last_s) {
            a.words[1] = 0;
            seq_s = ++a.words[0];
            __threadfence_system();
        }
    }
    __syncthreads();
    if (!last_s) return;
    const unsigned seq = seq_s;
    // this rank's sequence number into every peer's flag slot, then poll the local slots for everybody's
    if ((int)threadIdx.x < a.size) {
        unsigned* remote = reinterpret_cast<unsigned*>(a.peer[threadIdx.x] + a.flag_off) + a.rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(seq) : "memory");
        const unsigned* mine = reinterpret_cast<const unsigned*>(a.peer[a.rank] + a.flag_off) + threadIdx.x;
        const long long start = clock64();
        bool ok = *reinterpret_cast<volatile int*>(a.error_flag) != 0;   // an earlier wait already gave up: do not wait again
        while (!ok) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if ((int)(v - seq) >= 0) { ok = true; break; }
            if (clock64() - start > 4000000000ll) break;     // about two seconds: give up, report, return
        }
        if (!ok) atomicExch(a.error_flag, DETB_ERR_WAIT_EXPIRED);
    }
    __syncthreads();
}

}  // namespace detb

using namespace detb;

extern "C" {

void* det_xchg_create(size_t bytes, int rank, int size) {
    DETB_REQUIRE(size >= 1 && size <= XCHG_MAX_RANKS && rank >= 0 && rank < size, "bad exchange group");
    Xchg* x = new Xchg();
    x->bytes = (bytes + 255) & ~(size_t)255;
    x->rank = rank;
    x->size = size;
    (void)queue_of(nullptr);   // runtime up
    DETB_CUDA_OK(cudaMalloc(&x->base, x->bytes + 256));
    DETB_CUDA_OK(cudaMemset(x->base, 0, x->bytes + 256));
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
void* det_xchg_base(void* h) { return static_cast<Xchg*>(h)->base; }
size_t det_xchg_bytes(void* h) { return static_cast<Xchg*>(h)->bytes; }

// full = base + full_off must lie inside the region; slice % 4 == 0.  Meant for decode-sized exchanges (KBs to a MB).
void det_xchg_all_gather(void* h, const float* local, size_t full_off, int M, int slice, cudaStream_t st) {
    Xchg* x = static_cast<Xchg*>(h);
    DETB_REQUIRE(slice % 4 == 0 && M > 0, "exchange slices are whole float4s");
    DETB_REQUIRE(full_off % 16 == 0 && full_off + (size_t)M * x->size * slice * 4 <= x->bytes, "gathered buffer outside the region");
    XchgArgs a;
    a.local = local;
    a.full_off = full_off;
    a.M = M; a.slice = slice; a.rank = x->rank; a.size = x->size;
    a.flag_off = x->bytes;
    for (int r = 0; r < XCHG_MAX_RANKS; r++) a.peer[r] = x->peer[r];
    a.words = x->words;
    a.error_flag = error_word();
    const size_t vecs = (size_t)M * (slice >> 2) * x->size;
    const unsigned grid = (unsigned)std::min<size_t>(32, std::max<size_t>(1, vecs / 4096));
    launch_pdl(k_xchg_gather, dim3(grid), dim3(1024), 0, queue_of(st), 1, a);
}
void det_xchg_destroy(void* h) {
    Xchg* x = static_cast<Xchg*>(h);
    if (!x) return;
    cudaDeviceSynchronize();
    for (int r = 0; r < x->size; r++)
        if (r != x->rank && x->peer[r]) cudaIpcCloseMemHandle(x->peer[r]);
    cudaFree(x->base);
    cudaFree(x->words);
    delete x;
}

}  // extern "C"
