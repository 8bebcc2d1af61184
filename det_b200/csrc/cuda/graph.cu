// Capture and replay of the decode step as a CUDA graph, and the device-side token feedback that lets a replayed step
// feed the next one without a host round trip.  The reference has no graph code (README.md:115 lists it as future
// work); the replayed kernels are the same ones the eager path launches, so results are identical by construction.
#include "runtime.cuh"

namespace detb {
__global__ void k_token_feedback(const int* __restrict__ pick, int* __restrict__ pos, int* __restrict__ log,
                                 int log_base, int log_cap) {
    pdl_trigger();
    pdl_wait();
    const int p = *pos;
    const int slot = p - log_base;
    if (log && slot >= 0 && slot < log_cap) log[slot] = *pick;
    *pos = p + 1;
}
}  // namespace detb

using namespace detb;

extern "C" {

void det_graph_begin(void) {
    DETB_CUDA_OK(cudaStreamBeginCapture(queue_of(nullptr), cudaStreamCaptureModeThreadLocal));
}

void* det_graph_end(void) {
    cudaGraph_t graph = nullptr;
    if (cudaStreamEndCapture(queue_of(nullptr), &graph) != cudaSuccess || !graph) {
        fprintf(stderr, "det_b200: graph capture failed: %s\n", cudaGetErrorString(cudaGetLastError()));
        return nullptr;
    }
    cudaGraphExec_t exec = nullptr;
    const cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) {
        fprintf(stderr, "det_b200: graph instantiation failed: %s\n", cudaGetErrorString(e));
        return nullptr;
    }
    return exec;
}

void det_graph_launch(void* graph) { DETB_CUDA_OK(cudaGraphLaunch(static_cast<cudaGraphExec_t>(graph), queue_of(nullptr))); }

void det_graph_free(void* graph) {
    if (graph) DETB_CUDA_OK(cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(graph)));
}

void det_token_feedback(const int* pick, int* pos, int* log, int log_base, int log_cap, cudaStream_t st) {
    launch_pdl(k_token_feedback, dim3(1), dim3(1), 0, queue_of(st), 1, pick, pos, log, log_base, log_cap);
}

}  // extern "C"
