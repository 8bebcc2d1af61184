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

// ---- PeerComm

PeerComm::PeerComm(int rank_, int size_, size_t region_bytes, std::unique_ptr<Comm> bulk) : bulk_(std::move(bulk)) {
    rank = rank_;
    size = size_;
    x_ = det_xchg_create(region_bytes, rank_, size_);
    base_ = static_cast<uint8_t*>(det_xchg_base(x_));
    bytes_ = det_xchg_bytes(x_);
}
PeerComm::~PeerComm() {
    if (x_) det_xchg_destroy(x_);
}
void PeerComm::handle(uint8_t out[64]) const { det_xchg_ipc_handle(x_, out); }
void PeerComm::open(const uint8_t* handles) {
    det_xchg_open(x_, handles);
    opened_ = true;
}
Buf<float> PeerComm::alloc_gathered(Backend&, size_t n) {
    const size_t need = (n * sizeof(float) + 255) & ~(size_t)255;
    if (used_ + need > bytes_) throw std::runtime_error("exchange region too small for the gathered buffers");
    float* p = reinterpret_cast<float*>(base_ + used_);
    used_ += need;
    return Buf<float>::view(p, n);
}
void PeerComm::all_gather(Backend& bk, const Buf<float>& local, const Buf<float>& tmp, const Buf<float>& full, size_t m,
                          size_t slice) {
    const uint8_t* f = reinterpret_cast<const uint8_t*>(full.ptr());
    const bool inside = f >= base_ && f + m * size * slice * sizeof(float) <= base_ + bytes_;
    if (m > small_rows || !inside || slice % 4 != 0) {
        if (!bulk_) throw std::runtime_error("exchange too large for the peer path and no bulk communicator given");
        last_full_ = nullptr;
        bulk_->all_gather(bk, local, tmp, full, m, slice);
        return;
    }
    if (!opened_) throw std::runtime_error("PeerComm::open has not run");
    // a rank may still be reading the result of the previous exchange when this one starts: never the same buffer twice in a row
    if (last_full_ == full.ptr()) throw std::runtime_error("two consecutive exchanges into the same gathered buffer");
    last_full_ = full.ptr();
    bk.flush();
    det_xchg_all_gather(x_, local.ptr(), (size_t)(f - base_), (int)m, (int)slice, nullptr);
}

}  // namespace det
