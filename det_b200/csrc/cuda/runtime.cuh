// Internal interface of the runtime shared by the kernel translation units.
#pragma once
#include "../../../include/det_b200.h"
#include "prims.cuh"

namespace detb {
bool runtime_ready();
bool runtime_is_up();   // true once det_init (or any earlier call) has brought the runtime up; never initialises
cudaStream_t queue_of(cudaStream_t st);   // maps the ABI's stream 0 onto the library's queue
int sm_count();
size_t smem_optin();
// Device words that bounded waits use: [0] the error code they report into, [2..3] (one 64-bit word) the wait limit in
// SM clock cycles (about two seconds unless det_debug_set_wait_limit changed it).
int* error_word();
constexpr long long DEFAULT_WAIT_CYCLES = 4000000000ll;
#ifdef __CUDACC__
__device__ __forceinline__ long long wait_limit(const int* error_flag) {
    return *reinterpret_cast<const volatile long long*>(error_flag + 2);
}
#endif

// Scratch the library owns from the moment the runtime comes up (no call path allocates): the split-K cells of the
// tensor-core GEMM ((sm_count()/2 + 1) tiles of 128 x 128 int64, zero between calls) with their counters, and the workspace
// of the tensor-core prefill attention (may be absent: bytes == 0).
unsigned long long* splitk_cells();
unsigned* splitk_counters();
void* attn_workspace(size_t* bytes);

bool pdl_enabled();

// Launches `kernel` on `q` with the programmatic-dependent-launch attribute (and an optional cluster width) and returns
// the runtime's verdict on the launch.
template <class... KArgs, class... Args>
inline cudaError_t launch_pdl_try(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t q,
                                  int cluster_x, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = q;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pdl_enabled()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    if (cluster_x > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = cluster_x;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        na++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
// Same; a failed launch is fatal (the reference's error convention, kernels/cuda/common.cuh:8-9).
template <class... KArgs, class... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t q, int cluster_x,
                       Args&&... args) {
    DETB_CUDA_OK(launch_pdl_try(kernel, grid, block, smem, q, cluster_x, static_cast<Args&&>(args)...));
}

// Error codes reported by det_last_error().
enum : int { DETB_ERR_NONE = 0, DETB_ERR_WAIT_EXPIRED = 1, DETB_ERR_SIZE = 2 };
}  // namespace detb
