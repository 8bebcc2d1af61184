// Batched serving decode: several independent sequences advance one token per step through ONE pass over the weights.
// The reference has no such loop (its Model holds one position, one KV cache and one GDN state per layer,
// model.rs:143-161); this one is composed from the unchanged op set: the sequences' current rows are stacked as M = B
// for rmsnorm_quant / gemm / quant / silu_mul_quant (rows are independent, so each row equals its batch-1 result,
// docs/SPEC.md §3), attention and Gated DeltaNet run per row against that sequence's own cache / state
// (Backend::attention_rows / gdn_rows), and every row is sampled with its own generator.  Each stream therefore
// equals the stream the same sequence produces alone.
#pragma once
#include "model.hpp"

namespace det {

struct Sequence {
    std::vector<KvCache> kv;       // one per attention layer, in layer order
    std::vector<GdnState> st;      // one per GDN layer, in layer order
    size_t pos = 0;
    Sampling sampling;
    int32_t last = 0;              // the token that the next step feeds
    std::vector<int32_t> out;      // tokens produced so far
};

class BatchDecoder {
  public:
    // `model` must have max_batch >= n_seq; every sequence gets room for `ctx` positions.
    BatchDecoder(Model& model, size_t n_seq, size_t ctx);
    // Runs the prompt of sequence i through the model (its own chunked prefill) and draws the sequence's first token.
    std::string prefill(size_t i, const int32_t* ids, size_t n, const Sampling& s);
    // One decode step: every sequence consumes its last token and draws the next one.
    std::string step();
    std::vector<Sequence> seqs;

  private:
    void bind(size_t i);     // swaps sequence i's caches / states / position into the model (and back)
    void network_rows(size_t rows);
    Model& m_;
    size_t ctx_;
    std::vector<std::unique_ptr<RowSet>> rowsets_;   // one per layer
    Buf<int32_t> pos_;
};

}  // namespace det
