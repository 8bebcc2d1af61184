#include "graph_decode.hpp"
#include <stdexcept>

namespace det {

namespace {
constexpr cudaStream_t ST = nullptr;
}  // namespace

GraphDecoder::GraphDecoder(Model& m) : m_(m), bk_(dynamic_cast<CudaBackend*>(m.backend)) {
    if (!bk_) throw std::runtime_error("GraphDecoder needs a model on the CUDA backend");
    const size_t count = m.cfg.vocab * m.cfg.hidden;
    if (m.gguf) {   // the file's own table, whatever float type it has (model.rs:389-413 reads it row by row on the host)
        GgmlType ty = GgmlType::BF16;
        m.embed.type(ty);
        table_type_ = (int)ty;
        table_ = bk_->alloc<uint8_t>(m.embed.bytes());
        bk_->write_bytes(table_.ptr(), m.gguf->data(m.embed), m.embed.bytes());
    } else {
        table_ = bk_->alloc<uint8_t>(count * 2);
        det_synth_bf16(m.seed, tensor_id(GLOBAL_LAYER, T_EMBED), (long long)count, reinterpret_cast<uint16_t*>(table_.ptr()), ST);
    }
    pick_ = bk_->alloc<int32_t>(1);
    pos_ = bk_->alloc<int32_t>(1);
    log_ = bk_->alloc<int32_t>(m.max_ctx);   // the pick made after the step at position p lands in log_[p]
}

GraphDecoder::~GraphDecoder() {
    if (graph_) {
        det_sync();
        det_graph_free(graph_);
    }
}

// embed(token in device memory) -> network at the device position -> argmax -> log the pick, advance the position
void GraphDecoder::step() {
    det_embed_table(table_.ptr(), table_type_, pick_.ptr(), 1, (int)m_.cfg.hidden, m_.w.x.ptr(), ST);
    bk_->pos_dev = pos_.ptr();
    bk_->max_pos = (int)m_.max_ctx - 1;
    m_.network(0, 1);
    bk_->flush();             // anything the backend still holds back goes out before the pick
    bk_->pos_dev = nullptr;
    det_argmax(m_.w.logits.ptr(), 1, (int)m_.cfg.vocab, pick_.ptr(), ST);
    det_token_feedback(pick_.ptr(), pos_.ptr(), log_.ptr(), 0, (int)m_.max_ctx, ST);
}

std::string GraphDecoder::enqueue(int32_t first_id, size_t n, bool use_graph) {
    if (queued_) return "a previous run has not been finished";
    if (m_.all_logits) return "graph decode needs last-position logits";
    if (n == 0) return "step count out of range";
    if (m_.pos + n > m_.max_ctx) return "decode would exceed the context";
    if (first_id < 0 || (size_t)first_id >= m_.cfg.vocab) return "token id outside the embedding table";
    const int32_t pos = (int32_t)m_.pos;
    log_base_ = m_.pos;
    bk_->write(pick_, 0, &first_id, 1);
    bk_->write(pos_, 0, &pos, 1);
    size_t left = n;
    if (use_graph && !graph_) {
        // The first step runs eagerly (it is a real step: it also sizes every scratch buffer and configures the
        // kernels); the capture that follows only records the same calls.
        step();
        left--;
        det_graph_begin();
        step();
        graph_ = det_graph_end();
        if (!graph_) return "graph capture failed";
    }
    for (size_t i = 0; i < left; i++) {
        if (use_graph) det_graph_launch(graph_);
        else step();
    }
    queued_ = n;
    return "";
}

std::vector<int32_t> GraphDecoder::finish() {
    std::vector<int32_t> out(queued_);
    if (queued_) bk_->read(log_, log_base_, out.data(), queued_);
    m_.pos += queued_;
    queued_ = 0;
    return out;
}

}  // namespace det
