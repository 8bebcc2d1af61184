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
int* error_word();   // device word that bounded waits report into

bool pdl_enabled();

// Launches `kernel` on `q` with the programmatic-dependent-launch attribute (and an optional cluster width).
template <class... KArgs, class... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t q, int cluster_x,
                       Args&&... args) {
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
    DETB_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
}

// Error codes reported by det_last_error().
enum : int { DETB_ERR_NONE = 0, DETB_ERR_WAIT_EXPIRED = 1, DETB_ERR_SIZE = 2 };
}  // namespace detb
