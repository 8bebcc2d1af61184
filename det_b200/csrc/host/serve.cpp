#include "serve.hpp"
#include <algorithm>
#include <cmath>
#include <stdexcept>

namespace det {

BatchDecoder::BatchDecoder(Model& model, size_t n_seq, size_t ctx) : seqs(n_seq), m_(model), ctx_(ctx) {
    if (model.comm) throw std::runtime_error("batched decode runs on an unsharded model");
    if (n_seq == 0 || n_seq > model.max_batch) throw std::runtime_error("the model's max_batch is smaller than the number of sequences");
    Backend* bk = model.backend;
    const Config& c = model.cfg;
    for (Sequence& s : seqs) {
        for (const Layer& l : model.layers) {
            if (l.is_attn) {
                KvCache kv;   // model.rs:278-283
                kv.kq = bk->alloc<int8_t>(ctx * c.n_kv * c.head_dim);
                kv.sk = bk->alloc<float>(ctx * c.n_kv);
                kv.vq = bk->alloc<int16_t>(ctx * c.n_kv * c.head_dim);
                kv.capacity = ctx;
                s.kv.push_back(std::move(kv));
            } else {
                GdnState st;   // model.rs:300-303
                st.conv_state = bk->alloc<float>((c.conv_k - 1) * c.conv_dim());
                st.s = bk->alloc<float>(c.gdn_v_heads * c.gdn_dk * c.gdn_dv);
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

// qwen35.rs:31-170 with the two sequence-dependent ops taken per row
void BatchDecoder::network_rows(size_t t) {
    Model& m = m_;
    const Config& c = m.cfg;
    Backend* bk = m.backend;
    Work& w = m.w;
    const size_t h = c.hidden;
    size_t max_pos = 0;
    for (const Sequence& s : seqs) max_pos = std::max(max_pos, s.pos);
    size_t li = 0;
    for (Layer& l : m.layers) {
        const RowSet& rows = *rowsets_[li++];
        bk->rmsnorm_quant(w.x, l.attn_norm, c.eps, t, h, w.xq, w.sx, w.mx);
        if (l.is_attn) {
            Attn& a = l.attn;
            m.project(a.qkv, w.xq, w.sx, w.mx, t, {&w.qg, &w.k, &w.v});
            AttnLayer layer{&a.q_norm, &a.k_norm, &a.v_scale, &a.v_inv_scale, &m.rope_cos, &m.rope_sin};
            Shape shape{t, 0, c.n_heads, c.n_kv, c.head_dim, c.rot_dim, c.eps};
            bk->attention_rows(layer, rows, pos_, max_pos, shape, w.qg, w.k, w.v, w.o);
            bk->quant(w.o, t, c.n_heads * c.head_dim, w.oq, w.so, w.mo);
            bk->gemm(*a.o.lins[0], w.oq, w.so, w.mo, t, GemmOut::accumulate(w.x));
        } else {
            Gdn& g = l.gdn;
            m.project(g.qkvz, w.xq, w.sx, w.mx, t, {&w.qkv, &w.z});
            GdnLayer layer{&g.conv, &g.a, &g.dt_bias, &g.norm};
            GdnShape shape{t, c.gdn_k_heads, c.gdn_v_heads, c.gdn_dk, c.gdn_dv, c.eps};
            m.project(g.ab, w.xq, w.sx, w.mx, t, {&w.a, &w.b});
            bk->gdn_rows(layer, rows, shape, w.qkv, w.z, w.a, w.b, w.on);
            bk->quant(w.on, t, c.gdn_v_heads * c.gdn_dv, w.onq, w.son, w.mon);
            bk->gemm(*g.out.lins[0], w.onq, w.son, w.mon, t, GemmOut::accumulate(w.x));
        }
        bk->rmsnorm_quant(w.x, l.ffn_norm, c.eps, t, h, w.xq, w.sx, w.mx);
        m.project(l.gu, w.xq, w.sx, w.mx, t, {&w.g, &w.u});
        bk->silu_mul_quant(w.g, w.u, t, c.intermediate, w.hq, w.sh, w.mh);
        bk->gemm(*l.down.lins[0], w.hq, w.sh, w.mh, t, GemmOut::accumulate(w.x));
    }
    bk->rmsnorm_quant(w.x, m.final_norm, c.eps, t, h, w.xq, w.sx, w.mx);
    bk->gemm(*m.lm_head.lins[0], w.xq, w.sx, w.mx, t, GemmOut::write(w.logits));
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
