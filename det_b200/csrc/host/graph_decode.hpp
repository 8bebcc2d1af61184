// Greedy decode with the whole step resident on the device: the token comes from the previous step's argmax in device
// memory, the position from a device counter, and the step (embed -> network -> argmax -> feedback) is captured once
// into a CUDA graph and replayed.  Same kernels and same op order as Model::forward + Model::pick (model.rs:439-496),
// so the tokens and logits equal the eager loop's bit for bit; only the host round trips per token are gone.
#pragma once
#include "cuda_backend.hpp"
#include "model.hpp"

namespace det {

class GraphDecoder {
  public:
    explicit GraphDecoder(Model& m);   // the model must live on a CudaBackend
    ~GraphDecoder();
    // Queues `n` decode steps that start from token `first_id` at the model's current position.  Returns at once;
    // `use_graph` replays the captured step, otherwise the same calls are issued eagerly.
    std::string enqueue(int32_t first_id, size_t n, bool use_graph);
    // Waits, advances the model's position by the queued steps and returns their tokens (the pick after each step).
    std::vector<int32_t> finish();

  private:
    void step();   // one decode step through the C ABI, device-resident token and position
    Model& m_;
    CudaBackend* bk_;
    Buf<uint8_t> table_;    // embedding table [vocab][hidden] of ggml type table_type_ (30 = bf16 for a synthetic model)
    int table_type_ = 30;
    Buf<int32_t> pick_, pos_, log_;
    void* graph_ = nullptr;
    size_t queued_ = 0, log_base_ = 0;
};

}  // namespace det
