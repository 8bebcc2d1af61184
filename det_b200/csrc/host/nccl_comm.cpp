// NcclComm: ncclAllGather of fp32 slices on the library queue.  NCCL is resolved at run time (dlopen of libnccl.so.2) so
// that a process which already carries a copy (PyTorch bundles one) uses that one and single-GPU users need none.
#include "comm.hpp"
#include "cuda_backend.hpp"
#include <dlfcn.h>
#include <nccl.h>
#include <algorithm>
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

PeerComm::PeerComm(int rank_, int size_, size_t staging_bytes, std::unique_ptr<Comm> bulk) : bulk_(std::move(bulk)) {
    rank = rank_;
    size = size_;
    x_ = det_xchg_create(staging_bytes, rank_, size_);
    capacity_ = det_xchg_capacity(x_);
}
PeerComm::~PeerComm() {
    if (x_) det_xchg_destroy(x_);
}
void PeerComm::handle(uint8_t out[64]) const { det_xchg_ipc_handle(x_, out); }
void PeerComm::open(const uint8_t* handles) {
    det_xchg_open(x_, handles);
    opened_ = true;
}
void PeerComm::open_loopback() {
    det_xchg_open_loopback(x_);
    opened_ = true;
    small_rows = 1 << 30;   // no bulk communicator in this mode: everything that fits goes through the staging
}
bool PeerComm::small(size_t t, size_t slice) const {
    if (t > small_rows || slice % 2 != 0 || t * size * slice > capacity_) return false;
    if (!opened_) throw std::runtime_error("PeerComm::open has not run");
    return true;
}
void PeerComm::all_gather(Backend& bk, const Buf<float>& local, const Buf<float>& tmp, const Buf<float>& full, size_t m,
                          size_t slice) {
    if (!small(m, slice)) {
        if (!bulk_) throw std::runtime_error("exchange too large for the peer path and no bulk communicator given");
        bulk_->all_gather(bk, local, tmp, full, m, slice);
        return;
    }
    bk.flush();
    det_xchg_all_gather(x_, local.ptr(), full.ptr(), (int)m, (int)slice, nullptr);
}
void PeerComm::gather_add_norm_quant(Backend& bk, const Buf<float>& y_l, const Buf<float>& tmp, const Buf<float>& y_full,
                                     size_t t, size_t slice, const Buf<float>& x, const Buf<float>& w, float eps,
                                     const Buf<int8_t>& q, const Buf<float>& s, const Buf<uint16_t>& mm) {
    if (!(fuse && det_xchg_fusable((int)t, (int)(slice * size)) && small(t, slice)))
        return Comm::gather_add_norm_quant(bk, y_l, tmp, y_full, t, slice, x, w, eps, q, s, mm);
    bk.flush();
    det_xchg_add_rmsnorm_quant(x_, y_l.ptr(), (int)slice, x.ptr(), w.ptr(), eps, (int)t, q.ptr(), s.ptr(), mm.ptr(), nullptr);
}
bool PeerComm::gather_add_norm_quant_alt(Backend& bk, const Buf<float>& y_l, const Buf<float>& tmp, const Buf<float>& y_full,
                                         size_t t, size_t slice, const Buf<float>& x, const Buf<float>& x_alt,
                                         const Buf<float>& w, float eps, const Buf<int8_t>& q, const Buf<float>& s,
                                         const Buf<uint16_t>& mm) {
    CudaBackend* cb = dynamic_cast<CudaBackend*>(&bk);
    if (fuse && fuse_gemv && cb && small(t, slice) &&
        cb->hold_exchange(DET_ACT_RMSNORM, x_, y_l.ptr(), slice, (size_t)size, x.ptr(), x_alt.ptr(), w.ptr(), eps, t, q.ptr(),
                          s.ptr(), mm.ptr()))
        return true;
    gather_add_norm_quant(bk, y_l, tmp, y_full, t, slice, x, w, eps, q, s, mm);
    return false;
}
void PeerComm::gather_quant(Backend& bk, const Buf<float>& local, const Buf<float>& tmp, const Buf<float>& full, size_t t,
                            size_t slice, const Buf<int8_t>& q, const Buf<float>& s, const Buf<uint16_t>& mm) {
    CudaBackend* cb = dynamic_cast<CudaBackend*>(&bk);
    if (fuse && fuse_gemv && cb && small(t, slice) &&
        cb->hold_exchange(DET_ACT_PLAIN, x_, local.ptr(), slice, (size_t)size, nullptr, nullptr, nullptr, 0.0f, t, q.ptr(), s.ptr(),
                          mm.ptr()))
        return;
    if (!(fuse && det_xchg_fusable((int)t, (int)(slice * size)) && small(t, slice)))
        return Comm::gather_quant(bk, local, tmp, full, t, slice, q, s, mm);
    bk.flush();
    det_xchg_quant(x_, local.ptr(), nullptr, (int)slice, (int)t, q.ptr(), s.ptr(), mm.ptr(), nullptr);
}
void PeerComm::silu_gather_quant(Backend& bk, const Buf<float>& g, const Buf<float>& u, const Buf<float>& h_l,
                                 const Buf<float>& tmp, const Buf<float>& h_full, size_t t, size_t slice,
                                 const Buf<int8_t>& q, const Buf<float>& s, const Buf<uint16_t>& mm) {
    if (!(fuse && det_xchg_fusable((int)t, (int)(slice * size)) && small(t, slice)))
        return Comm::silu_gather_quant(bk, g, u, h_l, tmp, h_full, t, slice, q, s, mm);
    bk.flush();
    det_xchg_quant(x_, g.ptr(), u.ptr(), (int)slice, (int)t, q.ptr(), s.ptr(), mm.ptr(), nullptr);
}

}  // namespace det
