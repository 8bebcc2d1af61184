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

    // The three exchange-plus-consumer steps of the sharded token loop.  The defaults spell them out op by op; an
    // exchange that can run them as one launch overrides them (same values either way).
    // x[t][size*slice] += gather(y_l); rmsnorm_quant(x, w) -> q, s, mm
    virtual void gather_add_norm_quant(Backend& bk, const Buf<float>& y_l, const Buf<float>& tmp, const Buf<float>& y_full,
                                       size_t t, size_t slice, const Buf<float>& x, const Buf<float>& w, float eps,
                                       const Buf<int8_t>& q, const Buf<float>& s, const Buf<uint16_t>& mm) {
        all_gather(bk, y_l, tmp, y_full, t, slice);
        bk.add(x, y_full, t * slice * size);
        bk.rmsnorm_quant(x, w, eps, t, slice * size, q, s, mm);
    }
    // The same step for callers that keep two copies of the residual stream: the sums may land in x_alt instead of x
    // (returns true then; the caller swaps its buffers).  An exchange that runs as the prologue of the GEMV consuming
    // q / s / mm needs this: the CTAs of that launch read x while one of them stores the sums.
    virtual bool gather_add_norm_quant_alt(Backend& bk, const Buf<float>& y_l, const Buf<float>& tmp, const Buf<float>& y_full,
                                           size_t t, size_t slice, const Buf<float>& x, const Buf<float>& x_alt,
                                           const Buf<float>& w, float eps, const Buf<int8_t>& q, const Buf<float>& s,
                                           const Buf<uint16_t>& mm) {
        (void)x_alt;
        gather_add_norm_quant(bk, y_l, tmp, y_full, t, slice, x, w, eps, q, s, mm);
        return false;
    }
    // quant(gather(local)) -> q, s, mm
    virtual void gather_quant(Backend& bk, const Buf<float>& local, const Buf<float>& tmp, const Buf<float>& full, size_t t,
                              size_t slice, const Buf<int8_t>& q, const Buf<float>& s, const Buf<uint16_t>& mm) {
        all_gather(bk, local, tmp, full, t, slice);
        bk.quant(full, t, slice * size, q, s, mm);
    }
    // h_l = silu(g) * u over the local columns; quant(gather(h_l)) -> q, s, mm
    virtual void silu_gather_quant(Backend& bk, const Buf<float>& g, const Buf<float>& u, const Buf<float>& h_l,
                                   const Buf<float>& tmp, const Buf<float>& h_full, size_t t, size_t slice,
                                   const Buf<int8_t>& q, const Buf<float>& s, const Buf<uint16_t>& mm) {
        bk.silu_mul(g, u, t, slice, h_l);
        gather_quant(bk, h_l, tmp, h_full, t, slice, q, s, mm);
    }
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
// stored into every rank's staging area as self-validating packets; where det_xchg_fusable(rows, row length) holds the
// consumer (residual add + RMSNorm + quantization, or quantization) runs in the same launch.  Exchanges of more than `small_rows` rows
// (prefill chunks: megabytes, bandwidth-bound) go through the NCCL communicator given at construction.
// Set-up is collective: construct on every rank, pass every rank's handle() to open() in rank order.
class PeerComm : public Comm {
  public:
    PeerComm(int rank_, int size_, size_t staging_bytes, std::unique_ptr<Comm> bulk);
    ~PeerComm() override;
    void handle(uint8_t out[64]) const;
    void open(const uint8_t* handles);
    void open_loopback();   // timing aid: one process runs the launch sequence of one rank (values meaningless)
    void all_gather(Backend& bk, const Buf<float>& local, const Buf<float>& tmp, const Buf<float>& full, size_t m,
                    size_t slice) override;
    void gather_add_norm_quant(Backend& bk, const Buf<float>& y_l, const Buf<float>& tmp, const Buf<float>& y_full, size_t t,
                               size_t slice, const Buf<float>& x, const Buf<float>& w, float eps, const Buf<int8_t>& q,
                               const Buf<float>& s, const Buf<uint16_t>& mm) override;
    bool gather_add_norm_quant_alt(Backend& bk, const Buf<float>& y_l, const Buf<float>& tmp, const Buf<float>& y_full, size_t t,
                                   size_t slice, const Buf<float>& x, const Buf<float>& x_alt, const Buf<float>& w, float eps,
                                   const Buf<int8_t>& q, const Buf<float>& s, const Buf<uint16_t>& mm) override;
    void gather_quant(Backend& bk, const Buf<float>& local, const Buf<float>& tmp, const Buf<float>& full, size_t t,
                      size_t slice, const Buf<int8_t>& q, const Buf<float>& s, const Buf<uint16_t>& mm) override;
    void silu_gather_quant(Backend& bk, const Buf<float>& g, const Buf<float>& u, const Buf<float>& h_l,
                           const Buf<float>& tmp, const Buf<float>& h_full, size_t t, size_t slice, const Buf<int8_t>& q,
                           const Buf<float>& s, const Buf<uint16_t>& mm) override;
    size_t small_rows = 32;   // the serving step of 32 sequences still goes through the peer kernels
    bool fuse = true;   // run exchange + consumer as one launch (measurement switch; results are the same)
    bool fuse_gemv = true;   // ... and, where the consumer's output feeds a decode GEMV, as that GEMV's prologue

  private:
    bool small(size_t t, size_t slice) const;   // the exchange fits the staging and is decode-sized
    void* x_ = nullptr;
    size_t capacity_ = 0;
    std::unique_ptr<Comm> bulk_;
    bool opened_ = false;
};

}  // namespace det
