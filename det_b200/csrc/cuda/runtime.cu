// Runtime of the B200 backend: device selection, the one in-order queue, tracked zero-filled allocations, copies, and
// the primitive test hook.  Replaces kernels/cuda/runtime.cu:83-127 behind the same symbols.
//
// The reference issues everything on the legacy default stream.  Here a stream argument of 0 maps to one private
// non-blocking stream instead, which keeps the same program-order semantics for every det_* call while allowing the
// decode step to be captured into a CUDA graph (the legacy stream cannot be captured).
#include "runtime.cuh"
#include <cstdlib>
#include <mutex>
#include <unordered_map>

namespace detb {

namespace {
struct Runtime {
    int device = 0;
    int sm_count = 0;
    size_t smem_optin = 0;
    char name[384] = {0};
    cudaStream_t queue = nullptr;
    std::mutex mu;
    std::unordered_map<void*, size_t> live;
    size_t live_bytes = 0;
    int* error_word = nullptr;
    // scratch owned by the library, allocated once here so that no call path ever allocates:
    unsigned long long* splitk_cells = nullptr;   // split-K partial sums of the tensor-core GEMM, zero between calls
    unsigned* splitk_counters = nullptr;
    void* attn_ws = nullptr;                      // workspace of the tensor-core prefill attention
    size_t attn_ws_bytes = 0;
    bool attn_ws_owned = false;
};
Runtime* g_rt = nullptr;
std::once_flag g_once;

void bring_up() {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        fprintf(stderr, "det_b200: no CUDA device is visible\n");
        return;
    }
    Runtime* rt = new Runtime();
    if (cudaGetDevice(&rt->device) != cudaSuccess) { delete rt; return; }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, rt->device) != cudaSuccess) { delete rt; return; }
    if (prop.major != 10) {
        fprintf(stderr, "det_b200: device '%s' is sm_%d%d; this library carries sm_100a code only\n", prop.name,
                prop.major, prop.minor);
        delete rt;
        return;
    }
    snprintf(rt->name, sizeof rt->name, "%s (sm_%d%d, %d SMs) det_b200", prop.name, prop.major, prop.minor,
             prop.multiProcessorCount);
    rt->sm_count = prop.multiProcessorCount;
    rt->smem_optin = prop.sharedMemPerBlockOptin;
    if (cudaStreamCreateWithFlags(&rt->queue, cudaStreamNonBlocking) != cudaSuccess) { delete rt; return; }
    if (cudaMalloc(&rt->error_word, 4 * sizeof(int)) != cudaSuccess) { delete rt; return; }
    if (cudaMemset(rt->error_word, 0, 4 * sizeof(int)) != cudaSuccess) { delete rt; return; }
    const long long limit = DEFAULT_WAIT_CYCLES;
    if (cudaMemcpy(rt->error_word + 2, &limit, sizeof limit, cudaMemcpyHostToDevice) != cudaSuccess) { delete rt; return; }
    const size_t tiles = (size_t)rt->sm_count / 2 + 1, ncell = tiles * 128 * 128;
    if (cudaMalloc(&rt->splitk_cells, ncell * 8) != cudaSuccess || cudaMemset(rt->splitk_cells, 0, ncell * 8) != cudaSuccess ||
        cudaMalloc(&rt->splitk_counters, 4 * tiles * sizeof(unsigned)) != cudaSuccess ||      // tiles as narrow as 32 tokens
        cudaMemset(rt->splitk_counters, 0, 4 * tiles * sizeof(unsigned)) != cudaSuccess) { delete rt; return; }
    // DET_B200_ATTN_WS_MB sizes the attention workspace (default 256; 0: none, prefill attention then stays on the CUDA cores
    // until det_attn_set_workspace provides one)
    size_t ws_mb = 256;
    if (const char* e = getenv("DET_B200_ATTN_WS_MB")) ws_mb = (size_t)strtoull(e, nullptr, 10);
    if (ws_mb) {
        if (cudaMalloc(&rt->attn_ws, ws_mb << 20) == cudaSuccess) {
            rt->attn_ws_bytes = ws_mb << 20;
            rt->attn_ws_owned = true;
        } else {
            (void)cudaGetLastError();
            fprintf(stderr, "det_b200: no room for a %zu MB attention workspace; prefill attention stays on the CUDA cores\n", ws_mb);
        }
    }
    g_rt = rt;
}
}  // namespace

bool runtime_ready() {
    std::call_once(g_once, bring_up);
    return g_rt != nullptr;
}
bool runtime_is_up() { return g_rt != nullptr; }
static Runtime& rt() {
    if (!runtime_ready()) {
        fprintf(stderr, "det_b200: the CUDA runtime could not be initialised\n");
        abort();
    }
    return *g_rt;
}
cudaStream_t queue_of(cudaStream_t st) { return st ? st : rt().queue; }
int sm_count() { return rt().sm_count; }
size_t smem_optin() { return rt().smem_optin; }
int* error_word() { return rt().error_word; }
unsigned long long* splitk_cells() { return rt().splitk_cells; }
unsigned* splitk_counters() { return rt().splitk_counters; }
void* attn_workspace(size_t* bytes) {
    *bytes = rt().attn_ws_bytes;
    return rt().attn_ws;
}
static bool g_pdl = true;
bool pdl_enabled() { return g_pdl; }

// ---- primitive test hook kernels
__global__ void k_unary_binary(int op, const float* __restrict__ x, int n, float* __restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float a = x[i];
    const float b = x[n - 1 - i];
    float r;
    switch (op) {
        case 0: r = exp_f(a); break;
        case 1: r = log_f(a); break;
        case 2: r = softplus_f(a); break;
        case 3: r = sigmoid_f(a); break;
        case 4: r = silu_f(a); break;
        case 6: r = frint(a); break;
        case 7: r = fdiv(1.0f, a); break;
        case 8: r = fsqrt(a); break;
        case 9: r = fmul(a, b); break;
        case 10: r = fadd(a, b); break;
        case 13: r = (float)f2i_sat(a); break;
        case 14: r = fdiv(a, b); break;
        case 15: r = fsub(a, b); break;
        case 16: r = fmax_ord(a, b); break;
        default: r = a;
    }
    out[i] = r;
}
// ops 5 and 12: pairs of fp32 bit patterns are the low and high words of an int64
__global__ void k_i64_to_f32(int op, const float* __restrict__ x, int n, float* __restrict__ out) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (2 * p + 1 >= n) return;
    const unsigned long long lo = __float_as_uint(x[2 * p]), hi = __float_as_uint(x[2 * p + 1]);
    const long long v = (long long)((hi << 32) | lo);
    out[2 * p] = (op == 5) ? i64_to_f32(v) : (float)v;
}
// op 11: spec tree over rows of n <= 8192.  P = the next power of two >= n; P threads-worth of inputs are spread as
// aligned contiguous runs of RUN values per thread, so the fold order equals the spec's pairwise levels exactly.
template <int RUN>
__global__ void __launch_bounds__(1024) k_row_treesum(const float* __restrict__ x, int n, float* __restrict__ out) {
    __shared__ float sh[32];
    const float* row = x + (size_t)blockIdx.x * n;
    float v[RUN];
#pragma unroll
    for (int i = 0; i < RUN; i++) {
        const int idx = threadIdx.x * RUN + i;
        v[i] = idx < n ? row[idx] : 0.0f;
    }
    float s = fold_lanes<32>(fold_run<RUN>(v));
    s = fold_warps<32>(s, sh);
    if (threadIdx.x == 0) out[blockIdx.x] = s;
}
// rows shorter than 1024 after padding: one thread per padded element, P/32 warps
template <int NW>
__global__ void k_row_treesum_small(const float* __restrict__ x, int n, float* __restrict__ out) {
    __shared__ float sh[32];
    const float* row = x + (size_t)blockIdx.x * n;
    float s = (int)threadIdx.x < n ? row[threadIdx.x] : 0.0f;
    s = fold_lanes<32>(s);
    s = fold_warps<NW>(s, sh);
    if (threadIdx.x == 0) out[blockIdx.x] = s;
}

}  // namespace detb

using namespace detb;

extern "C" {

int det_init(void) { return runtime_ready() ? 0 : 1; }
const char* det_device_name(void) { return rt().name; }
void* det_cuda_stream(void) { return (void*)rt().queue; }
int det_last_error(void) {
    if (!runtime_ready()) return 0;
    int code = 0;
    DETB_CUDA_OK(cudaDeviceSynchronize());
    DETB_CUDA_OK(cudaMemcpy(&code, g_rt->error_word, sizeof(int), cudaMemcpyDeviceToHost));
    return code;
}

// Replaces the attention workspace with caller memory (device, 1024-byte aligned); p == NULL returns to none.  Waits for
// pending work first.  The tensor-core prefill attention processes as many query rows per round as the workspace holds.
void det_attn_set_workspace(void* p, size_t bytes) {
    Runtime& r = rt();
    DETB_REQUIRE((reinterpret_cast<uintptr_t>(p) & 1023) == 0, "the attention workspace must be 1024-byte aligned");
    DETB_CUDA_OK(cudaDeviceSynchronize());
    if (r.attn_ws_owned) cudaFree(r.attn_ws);
    r.attn_ws_owned = false;
    r.attn_ws = p;
    r.attn_ws_bytes = p ? bytes : 0;
}

// Clears the error word after the caller has dealt with the error (waits for pending work first).
void det_clear_error(void) {
    if (!runtime_ready()) return;
    DETB_CUDA_OK(cudaDeviceSynchronize());
    DETB_CUDA_OK(cudaMemset(g_rt->error_word, 0, sizeof(int)));
}
// Limit of every bounded device-side wait, in SM clock cycles; <= 0 restores the default (about two seconds).
void det_debug_set_wait_limit(long long cycles) {
    if (!runtime_ready()) return;
    const long long limit = cycles > 0 ? cycles : DEFAULT_WAIT_CYCLES;
    DETB_CUDA_OK(cudaDeviceSynchronize());
    DETB_CUDA_OK(cudaMemcpy(g_rt->error_word + 2, &limit, sizeof limit, cudaMemcpyHostToDevice));
}

void* det_malloc(size_t bytes) {
    Runtime& r = rt();
    if (bytes == 0) bytes = 16;
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        (void)cudaGetLastError();
        fprintf(stderr, "det_b200: det_malloc(%zu) failed\n", bytes);
        return nullptr;
    }
    DETB_CUDA_OK(cudaMemsetAsync(p, 0, bytes, r.queue));
    std::lock_guard<std::mutex> lock(r.mu);
    r.live[p] = bytes;
    r.live_bytes += bytes;
    return p;
}

void det_free(void* p) {
    if (!p || !g_rt) return;
    Runtime& r = *g_rt;
    {
        std::lock_guard<std::mutex> lock(r.mu);
        auto it = r.live.find(p);
        if (it == r.live.end()) {
            fprintf(stderr, "det_b200: det_free(%p): not a det_malloc pointer\n", p);
            abort();
        }
        r.live_bytes -= it->second;
        r.live.erase(it);
    }
    DETB_CUDA_OK(cudaDeviceSynchronize());
    DETB_CUDA_OK(cudaFree(p));
}

size_t det_allocated_bytes(void) { return g_rt ? g_rt->live_bytes : 0; }

void det_sync(void) {
    rt();
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        fprintf(stderr, "det_b200: fatal: %s\n", cudaGetErrorString(e));
        abort();
    }
}
void det_flush(void) {}
// Debug switch for A/B measurements: programmatic dependent launch on (default) or off.
void det_debug_set_pdl(int on) { g_pdl = on != 0; }

void det_memset(void* p, int value, size_t bytes, cudaStream_t st) {
    DETB_CUDA_OK(cudaMemsetAsync(p, value, bytes, queue_of(st)));
}
void det_memcpy(void* dst, const void* src, size_t bytes, cudaStream_t st) {
    DETB_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, queue_of(st)));
}

void det_test_prim(int op, const float* x, int M, int n, float* out, cudaStream_t st) {
    cudaStream_t q = queue_of(st);
    if (op == 11) {
        DETB_REQUIRE(n >= 1 && n <= 8192, "treesum hook supports rows of 1..8192");
        int P = 32;
        while (P < n) P <<= 1;
        switch (P) {
            case 32: k_row_treesum_small<1><<<M, 32, 0, q>>>(x, n, out); break;
            case 64: k_row_treesum_small<2><<<M, 64, 0, q>>>(x, n, out); break;
            case 128: k_row_treesum_small<4><<<M, 128, 0, q>>>(x, n, out); break;
            case 256: k_row_treesum_small<8><<<M, 256, 0, q>>>(x, n, out); break;
            case 512: k_row_treesum_small<16><<<M, 512, 0, q>>>(x, n, out); break;
            case 1024: k_row_treesum<1><<<M, 1024, 0, q>>>(x, n, out); break;
            case 2048: k_row_treesum<2><<<M, 1024, 0, q>>>(x, n, out); break;
            case 4096: k_row_treesum<4><<<M, 1024, 0, q>>>(x, n, out); break;
            default: k_row_treesum<8><<<M, 1024, 0, q>>>(x, n, out); break;
        }
    } else if (op == 5 || op == 12) {
        const size_t total = (size_t)M * n;
        k_i64_to_f32<<<(unsigned)((total / 2 + 255) / 256), 256, 0, q>>>(op, x, (int)total, out);
    } else {
        const size_t total = (size_t)M * n;
        k_unary_binary<<<(unsigned)((total + 255) / 256), 256, 0, q>>>(op, x, (int)total, out);
    }
    DETB_CUDA_OK(cudaGetLastError());
}

}  // extern "C"
