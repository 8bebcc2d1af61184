// NcclComm: ncclAllGather of fp32 slices on the library queue.  NCCL is resolved at run time (dlopen of libnccl.so.2) so
// that a process which already carries a copy (PyTorch bundles one) uses that one and single-GPU users need none.
#include "comm.hpp"
#include "cuda_backend.hpp"
#include <dlfcn.h>
#include <nccl.h>
#include <stdexcept>
#include <string>

namespace det {

namespace {
struct Api {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    const char* (*GetErrorString)(ncclResult_t);
};
Api& api() {
    static Api a = [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) throw std::runtime_error(std::string("cannot load libnccl.so.2: ") + dlerror());
        Api r;
        r.GetUniqueId = reinterpret_cast<decltype(r.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
        r.CommInitRank = reinterpret_cast<decltype(r.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
        r.CommDestroy = reinterpret_cast<decltype(r.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
        r.AllGather = reinterpret_cast<decltype(r.AllGather)>(dlsym(h, "ncclAllGather"));
        r.GetErrorString = reinterpret_cast<decltype(r.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
        if (!r.GetUniqueId || !r.CommInitRank || !r.CommDestroy || !r.AllGather || !r.GetErrorString)
            throw std::runtime_error("libnccl.so.2 lacks a required symbol");
        return r;
    }();
    return a;
}
void check(ncclResult_t r, const char* what) {
    if (r != ncclSuccess) throw std::runtime_error(std::string(what) + ": " + api().GetErrorString(r));
}
}  // namespace

static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");

void NcclComm::unique_id(uint8_t out[128]) {
    ncclUniqueId id;
    check(api().GetUniqueId(&id), "ncclGetUniqueId");
    std::memcpy(out, &id, 128);
}

NcclComm::NcclComm(const uint8_t idb[128], int rank_, int size_) {
    rank = rank_;
    size = size_;
    ncclUniqueId id;
    std::memcpy(&id, idb, 128);
    ncclComm_t c;
    check(api().CommInitRank(&c, size_, id, rank_), "ncclCommInitRank");
    comm_ = c;
}

NcclComm::~NcclComm() {
    if (comm_) api().CommDestroy(static_cast<ncclComm_t>(comm_));
}

void NcclComm::all_gather(Backend& bk, const Buf<float>& local, const Buf<float>& tmp, const Buf<float>& full, size_t m,
                          size_t slice) {
    bk.flush();
    cudaStream_t q = static_cast<cudaStream_t>(det_cuda_stream());
    float* dst = m == 1 ? full.ptr() : tmp.ptr();
    check(api().AllGather(local.ptr(), dst, m * slice, ncclFloat, static_cast<ncclComm_t>(comm_), q), "ncclAllGather");
    if (m > 1) det_unshard(tmp.ptr(), full.ptr(), size, (int)m, (int)slice, nullptr);
}

}  // namespace det
