// Exchange step of the tensor-parallel token loop.  The reference is single-device (no collective anywhere in it);
// sharding follows its exactness rules (docs/SPEC.md §3: output rows are independent; §5: heads are independent), so
// the only thing that ever crosses between ranks is a copy of finished fp32 values: every rank holds a slice of a row
// and needs the whole row.  One primitive covers all of it.
#pragma once
#include "backend.hpp"
#include <memory>

namespace det {

class Comm {
  public:
    virtual ~Comm() = default;
    int rank = 0, size = 1;
    // full[m][size * slice] <- for every row, the ranks' local[m][slice] blocks side by side in rank order.
    // `tmp` holds size * m * slice floats of scratch.
    virtual void all_gather(Backend& bk, const Buf<float>& local, const Buf<float>& tmp, const Buf<float>& full,
                            size_t m, size_t slice) = 0;
    // Storage for a gathered buffer (`full` above).  An exchange that writes straight into its peers' gathered buffers
    // hands out pieces of its own shared region here; the default is ordinary backend memory.
    virtual Buf<float> alloc_gathered(Backend& bk, size_t n) { return bk.alloc<float>(n); }
};

// Host-memory exchange through a caller-supplied function (tests run it over torch.distributed / gloo):
// fn(local, gathered, bytes) must fill gathered[size][bytes] with every rank's `local` block in rank order.
class CallbackComm : public Comm {
  public:
    using Fn = void (*)(const void* local, void* gathered, size_t bytes);
    CallbackComm(int rank_, int size_, Fn fn) : fn_(fn) {
        rank = rank_;
        size = size_;
    }
    void all_gather(Backend& bk, const Buf<float>& local, const Buf<float>& tmp, const Buf<float>& full, size_t m,
                    size_t slice) override {
        bk.sync();
        fn_(local.ptr(), tmp.ptr(), m * slice * sizeof(float));
        for (int r = 0; r < size; r++)
            for (size_t t = 0; t < m; t++)
                std::memcpy(full.ptr() + (t * size + r) * slice, tmp.ptr() + ((size_t)r * m + t) * slice,
                            slice * sizeof(float));
    }

  private:
    Fn fn_;
};

// NCCL over NVLink, issued on the CUDA backend's queue (capturable into the decode graph).  nccl_comm.cpp.
class NcclComm : public Comm {
  public:
    static void unique_id(uint8_t out[128]);
    NcclComm(const uint8_t id[128], int rank_, int size_);
    ~NcclComm() override;
    void all_gather(Backend& bk, const Buf<float>& local, const Buf<float>& tmp, const Buf<float>& full, size_t m,
                    size_t slice) override;

  private:
    void* comm_ = nullptr;
};

// Decode-sized exchanges as ONE kernel per rank over NVLink peer memory (det_xchg_* of the C ABI): the local slice is
// stored directly into every rank's gathered buffer, then a flag handshake.  Exchanges of more than `small_rows` rows
// (prefill chunks: megabytes, bandwidth-bound) go through the NCCL communicator given at construction.
// Set-up is collective: construct on every rank, pass every rank's handle() to open() in rank order.
class PeerComm : public Comm {
  public:
    PeerComm(int rank_, int size_, size_t region_bytes, std::unique_ptr<Comm> bulk);
    ~PeerComm() override;
    void handle(uint8_t out[64]) const;
    void open(const uint8_t* handles);
    void all_gather(Backend& bk, const Buf<float>& local, const Buf<float>& tmp, const Buf<float>& full, size_t m,
                    size_t slice) override;
    Buf<float> alloc_gathered(Backend& bk, size_t n) override;
    size_t small_rows = 8;

  private:
    void* x_ = nullptr;
    uint8_t* base_ = nullptr;
    size_t bytes_ = 0, used_ = 0;
    const float* last_full_ = nullptr;
    std::unique_ptr<Comm> bulk_;
    bool opened_ = false;
};

}  // namespace det
