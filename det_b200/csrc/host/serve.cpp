#include "serve.hpp"
#include <algorithm>
#include <cmath>
#include <stdexcept>

namespace det {

BatchDecoder::BatchDecoder(Model& model, size_t n_seq, size_t ctx) : seqs(n_seq), m_(model), ctx_(ctx) {
    if (n_seq == 0 || n_seq > model.max_batch) throw std::runtime_error("the model's max_batch is smaller than the number of sequences");
    Backend* bk = model.backend;
    const Config& c = model.cfg;
    // a tensor-parallel shard keeps this rank's kv heads and GDN heads of every sequence (model.hpp, Model::Tp)
    const size_t n_kv = model.comm ? model.tp.kv : c.n_kv;
    const size_t k_heads = model.comm ? model.tp.k_heads : c.gdn_k_heads, v_heads = model.comm ? model.tp.v_heads : c.gdn_v_heads;
    const size_t conv_dim = 2 * k_heads * c.gdn_dk + v_heads * c.gdn_dv;
    for (Sequence& s : seqs) {
        for (const Layer& l : model.layers) {
            if (l.is_attn) {
                KvCache kv;   // model.rs:278-283
                kv.kq = bk->alloc<int8_t>(ctx * n_kv * c.head_dim);
                kv.sk = bk->alloc<float>(ctx * n_kv);
                kv.vq = bk->alloc<int16_t>(ctx * n_kv * c.head_dim);
                kv.capacity = ctx;
                s.kv.push_back(std::move(kv));
            } else {
                GdnState st;   // model.rs:300-303
                st.conv_state = bk->alloc<float>((c.conv_k - 1) * conv_dim);
                st.s = bk->alloc<float>(v_heads * c.gdn_dk * c.gdn_dv);
                s.st.push_back(std::move(st));
            }
        }
    }
    size_t ia = 0, ig = 0;
    for (const Layer& l : model.layers) {
        std::vector<const KvCache*> kv;
        std::vector<const GdnState*> st;
        for (Sequence& s : seqs) {
            if (l.is_attn) kv.push_back(&s.kv[ia]);
            else st.push_back(&s.st[ig]);
        }
        (l.is_attn ? ia : ig)++;
        rowsets_.push_back(bk->make_rowset(std::move(kv), std::move(st)));
    }
    pos_ = bk->alloc<int32_t>(n_seq);
    model.set_all_logits(true);   // logits of every row of a step
}

void BatchDecoder::bind(size_t i) {
    Sequence& s = seqs[i];
    size_t ia = 0, ig = 0;
    for (Layer& l : m_.layers) {
        if (l.is_attn) std::swap(l.attn.kv, s.kv[ia++]);
        else std::swap(l.gdn.state, s.st[ig++]);
    }
    std::swap(m_.pos, s.pos);
}

std::string BatchDecoder::prefill(size_t i, const int32_t* ids, size_t n, const Sampling& sampling) {
    if (i >= seqs.size()) return "no such sequence";
    if (n == 0 || n + 1 > ctx_) return "prompt does not fit the sequence's context";
    Sequence& s = seqs[i];
    s.sampling = sampling;
    s.out.clear();
    // a slot that served an earlier conversation starts over: position 0 and zeroed recurrent state, as Model::reset
    // does (model.rs:378-387); cache rows need no clearing, positions >= pos are never read
    if (s.pos != 0) {
        m_.backend->sync();
        s.pos = 0;
        for (GdnState& st : s.st) {
            m_.backend->zero(st.conv_state);
            m_.backend->zero(st.s);
        }
    }
    const size_t max_ctx = m_.max_ctx;
    m_.max_ctx = ctx_;
    m_.all_logits = false;   // last-row logits into the first row of the (rows x vocab) buffer
    bind(i);
    std::string e = m_.prefill(ids, n);
    int32_t id = 0;
    if (e.empty()) e = m_.pick(s.sampling, id);
    bind(i);
    m_.all_logits = true;
    m_.max_ctx = max_ctx;
    if (!e.empty()) return e;
    s.last = id;
    s.out.push_back(id);
    return "";
}

// qwen35.rs:31-170 with the two sequence-dependent ops taken per row (Model::network with a RowsCtx; on a tensor-parallel
// shard the same exchanges as a batch of t tokens)
void BatchDecoder::network_rows(size_t t) {
    size_t max_pos = 0;
    for (const Sequence& s : seqs) max_pos = std::max(max_pos, s.pos);
    const RowsCtx rows{&rowsets_, &pos_, max_pos};
    m_.network(0, t, nullptr, &rows);
}

std::string BatchDecoder::step() {
    const size_t t = seqs.size();
    std::vector<int32_t> ids(t), pos(t);
    for (size_t b = 0; b < t; b++) {
        if (seqs[b].out.empty()) return "sequence " + std::to_string(b) + " has not been prefilled";
        if (seqs[b].pos + 1 > ctx_) return "sequence " + std::to_string(b) + " is out of context";
        ids[b] = seqs[b].last;
        pos[b] = (int32_t)seqs[b].pos;
    }
    std::string e = m_.embed_rows(ids.data(), t);
    if (!e.empty()) return e;
    m_.backend->write(pos_, 0, pos.data(), t);
    network_rows(t);
    const size_t v = m_.cfg.vocab;
    // all rows in one call when the sequences share their sampling parameters (each keeps its own generator)
    const Sampling& s0 = seqs[0].sampling;
    bool same = std::isfinite(s0.inv_temp) && !std::isnan(s0.top_p);
    for (const Sequence& s : seqs)
        same = same && s.sampling.greedy == s0.greedy && s.sampling.inv_temp == s0.inv_temp &&
               s.sampling.top_k == s0.top_k && s.sampling.top_p == s0.top_p;
    std::vector<int32_t> picked;
    if (same && s0.greedy) {
        picked = m_.backend->argmax_rows(m_.w.logits, t, v);
    } else if (same) {
        std::vector<uint64_t> z(t);
        for (size_t b = 0; b < t; b++) z[b] = Model::next_draw(seqs[b].sampling);
        picked = m_.backend->sample_rows(m_.w.logits, t, v, s0.inv_temp, s0.top_k, s0.top_p, z);
    } else {
        picked.resize(t);
        for (size_t b = 0; b < t; b++) {
            e = m_.pick_row(Buf<float>::view(m_.w.logits.ptr_at(b * v), v), seqs[b].sampling, picked[b]);
            if (!e.empty()) return e;
        }
    }
    for (size_t b = 0; b < t; b++) {
        seqs[b].pos += 1;
        seqs[b].last = picked[b];
        seqs[b].out.push_back(picked[b]);
    }
    return "";
}

}  // namespace det
