// Internal interface of the runtime shared by the kernel translation units.
#pragma once
#include "../../../include/det_b200.h"
#include "prims.cuh"

namespace detb {
bool runtime_ready();
cudaStream_t queue_of(cudaStream_t st);   // maps the ABI's stream 0 onto the library's queue
int sm_count();
size_t smem_optin();
int* error_word();   // device word that bounded waits report into

// Error codes reported by det_last_error().
enum : int { DETB_ERR_NONE = 0, DETB_ERR_WAIT_EXPIRED = 1, DETB_ERR_SIZE = 2 };
}  // namespace detb
