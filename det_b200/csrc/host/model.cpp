// Model loading (synthetic), the network's op sequence and the token loop.  See model.hpp for the reference map.
#include "model.hpp"
#include "gguf.hpp"
#include <algorithm>
#include <cmath>
#include <stdexcept>

namespace det {

static SynthRowsProvider g_rows_provider = nullptr;
void set_synth_rows_provider(SynthRowsProvider p) { g_rows_provider = p; }

std::vector<uint8_t> synth_det_rows_any(uint64_t seed, uint64_t tid, size_t row0, size_t n, size_t k, int bits) {
    return g_rows_provider ? g_rows_provider(seed, tid, row0, n, k, bits) : synth_det_rows(seed, tid, n, k, bits, row0);
}

// Default of Backend::linear_synth: det rows on the host, then the ordinary weight-ingestion path.
std::unique_ptr<Linear> Backend::linear_synth(uint64_t seed, const std::vector<SynthPart>& parts, size_t k, int bits) {
    std::vector<std::vector<uint8_t>> rows;
    std::vector<LinearPart> lp;
    for (const SynthPart& p : parts) {
        rows.push_back(synth_det_rows_any(seed, p.tensor_id, p.row0, p.n, k, bits));
        lp.push_back(LinearPart{rows.back().data(), p.n});
    }
    return linear(lp, k, bits);
}

namespace {
struct SynthTensor {
    TensorKind kind;
    size_t n, k;
    int bits;
    size_t row0 = 0;
};
// model.rs:180-197 — consecutive tensors of equal type and K become one fused linear.
Proj make_proj(Backend* bk, uint64_t seed, size_t layer, const std::vector<SynthTensor>& ts) {
    Proj p;
    size_t i = 0;
    while (i < ts.size()) {
        size_t j = i + 1;
        while (j < ts.size() && ts[j].bits == ts[i].bits && ts[j].k == ts[i].k) j++;
        std::vector<SynthPart> parts;
        for (size_t q = i; q < j; q++) parts.push_back(SynthPart{tensor_id(layer, ts[q].kind), ts[q].n, ts[q].row0});
        p.lins.push_back(bk->linear_synth(seed, parts, ts[i].k, ts[i].bits));
        i = j;
    }
    return p;
}
Buf<float> ones(Backend* bk, size_t n) { return bk->upload(std::vector<float>(n, 1.0f)); }
}  // namespace

static void load_shard(Model& m, const Config& cfg, uint64_t seed, Backend* bk, size_t max_ctx, size_t max_batch);

// model.rs:316-347 — the activation buffers of a single-device model for max_batch rows.
static void alloc_work(Model& m) {
    const Config& cfg = m.cfg;
    Backend* bk = m.backend;
    const size_t h = cfg.hidden, inter = cfg.intermediate;
    const size_t n_h = cfg.n_heads, n_kv = cfg.n_kv, hd = cfg.head_dim;
    const size_t n_v = cfg.gdn_v_heads, dv = cfg.gdn_dv;
    const size_t conv_dim = cfg.conv_dim();
    const size_t mb = m.max_batch;
    Work& w = m.w;
    w.x = bk->alloc<float>(mb * h);
    w.xq = bk->alloc<int8_t>(mb * h);
    w.sx = bk->alloc<float>(mb);
    w.mx = bk->alloc<uint16_t>(mb * h / 128);
    w.qg = bk->alloc<float>(mb * n_h * 2 * hd);
    w.k = bk->alloc<float>(mb * n_kv * hd);
    w.v = bk->alloc<float>(mb * n_kv * hd);
    w.o = bk->alloc<float>(mb * n_h * hd);
    w.oq = bk->alloc<int8_t>(mb * n_h * hd);
    w.so = bk->alloc<float>(mb);
    w.mo = bk->alloc<uint16_t>(mb * n_h * hd / 128);
    w.qkv = bk->alloc<float>(mb * conv_dim);
    w.z = bk->alloc<float>(mb * n_v * dv);
    w.a = bk->alloc<float>(mb * n_v);
    w.b = bk->alloc<float>(mb * n_v);
    w.on = bk->alloc<float>(mb * n_v * dv);
    w.onq = bk->alloc<int8_t>(mb * n_v * dv);
    w.son = bk->alloc<float>(mb);
    w.mon = bk->alloc<uint16_t>(mb * n_v * dv / 128);
    w.g = bk->alloc<float>(mb * inter);
    w.u = bk->alloc<float>(mb * inter);
    w.hq = bk->alloc<int8_t>(mb * inter);
    w.sh = bk->alloc<float>(mb);
    w.mh = bk->alloc<uint16_t>(mb * inter / 128);
    w.logits = bk->alloc<float>(cfg.vocab);
}


std::unique_ptr<Model> Model::load_synthetic(const Config& cfg, uint64_t seed, Backend* bk, size_t max_ctx,
                                             size_t max_batch, Comm* comm) {
    auto mp = std::make_unique<Model>();
    Model& m = *mp;
    if (comm && comm->size > 1) {
        m.comm = comm;
        load_shard(m, cfg, seed, bk, max_ctx, max_batch);
        return mp;
    }
    m.cfg = cfg;
    m.backend = bk;
    m.seed = seed;
    m.max_ctx = max_ctx;
    m.max_batch = max_batch;
    const size_t h = cfg.hidden, inter = cfg.intermediate;
    const size_t n_h = cfg.n_heads, n_kv = cfg.n_kv, hd = cfg.head_dim;
    const size_t n_v = cfg.gdn_v_heads, dk = cfg.gdn_dk, dv = cfg.gdn_dv;
    const size_t conv_dim = cfg.conv_dim();
    const int wb = cfg.bits_default;

    m.final_norm = ones(bk, h);
    std::vector<float> rc, rs;
    rope_tables(cfg, max_ctx, rc, rs);
    m.rope_cos = bk->upload(rc);
    m.rope_sin = bk->upload(rs);
    m.lm_head = make_proj(bk, seed, GLOBAL_LAYER, {{T_EMBED, cfg.vocab, h, 8}});

    m.layers.resize(cfg.n_layers);
    for (size_t i = 0; i < cfg.n_layers; i++) {
        Layer& l = m.layers[i];
        l.is_attn = cfg.is_attention(i);
        if (l.is_attn) {
            Attn& a = l.attn;
            a.qkv = make_proj(bk, seed, i, {{T_ATTN_Q, n_h * 2 * hd, h, wb}, {T_ATTN_K, n_kv * hd, h, wb}, {T_ATTN_V, n_kv * hd, h, wb}});
            a.o = make_proj(bk, seed, i, {{T_ATTN_OUT, h, n_h * hd, wb}});
            a.q_norm = ones(bk, hd);
            a.k_norm = ones(bk, hd);
            std::vector<float> vs(n_kv, DEFAULT_V_SCALE), vis(n_kv);
            for (size_t q = 0; q < n_kv; q++) vis[q] = 1.0f / vs[q];   // model.rs:258
            a.v_scale = bk->upload(vs);
            a.v_inv_scale = bk->upload(vis);
            a.kv.kq = bk->alloc<int8_t>(max_ctx * n_kv * hd);
            a.kv.sk = bk->alloc<float>(max_ctx * n_kv);
            a.kv.vq = bk->alloc<int16_t>(max_ctx * n_kv * hd);
            a.kv.capacity = max_ctx;
        } else {
            Gdn& g = l.gdn;
            g.qkvz = make_proj(bk, seed, i, {{T_GDN_QKV, conv_dim, h, wb}, {T_GDN_GATE, n_v * dv, h, wb}});
            g.ab = make_proj(bk, seed, i, {{T_GDN_ALPHA, n_v, h, 8}, {T_GDN_BETA, n_v, h, 8}});
            g.out = make_proj(bk, seed, i, {{T_GDN_OUT, h, n_v * dv, wb}});
            std::vector<float> conv(conv_dim * cfg.conv_k), dtb(n_v), av(n_v);
            for (size_t q = 0; q < conv.size(); q++) conv[q] = draw_normal(seed, tensor_id(i, T_CONV), q, WEIGHT_STD);
            for (size_t q = 0; q < n_v; q++) {
                dtb[q] = draw_normal(seed, tensor_id(i, T_DT_BIAS), q, WEIGHT_STD);
                // the file stores ssm_a = -(1 + 15 u); the model keeps a = -ssm_a (model.rs:281-293)
                av[q] = 1.0f + 15.0f * draw_unit(seed, tensor_id(i, T_SSM_A), q);
            }
            g.conv = bk->upload(conv);
            g.a = bk->upload(av);
            g.dt_bias = bk->upload(dtb);
            g.norm = ones(bk, dv);
            g.state.conv_state = bk->alloc<float>((cfg.conv_k - 1) * conv_dim);
            g.state.s = bk->alloc<float>(n_v * dk * dv);
        }
        l.attn_norm = ones(bk, h);
        l.ffn_norm = ones(bk, h);
        l.gu = make_proj(bk, seed, i, {{T_FFN_GATE, inter, h, wb}, {T_FFN_UP, inter, h, wb}});
        l.down = make_proj(bk, seed, i, {{T_FFN_DOWN, h, inter, wb}});
    }
    alloc_work(m);
    return mp;
}

// model.rs:164-365
std::unique_ptr<Model> Model::load(const std::string& path, Backend* bk, size_t max_ctx, size_t max_batch, std::string& err) {
    std::shared_ptr<Gguf> g = Gguf::open(path, err);
    if (!g) return nullptr;
    auto mp = std::make_unique<Model>();
    Model& m = *mp;
    if (!(err = config_from_gguf(*g, m.cfg)).empty()) return nullptr;
    if (!(err = check_finite(*g)).empty()) return nullptr;
    const Config& cfg = m.cfg;
    m.backend = bk;
    m.max_ctx = max_ctx;
    m.max_batch = max_batch;
    m.gguf = g;
    try {
        auto tensor = [&](const std::string& name) -> const GgufTensor& {
            const GgufTensor* t = g->tensor(name);
            if (!t) throw std::runtime_error("missing tensor " + name);
            return *t;
        };
        auto vec = [&](const std::string& name) {
            const GgufTensor& t = tensor(name);
            GgmlType ty;
            if (!t.type(ty)) throw std::runtime_error(name + ": unsupported type");
            std::vector<float> out(t.n_elems());
            dequant_row(ty, g->data(t), out.size(), out.data());
            return bk->upload(out);
        };
        // model.rs:180-197 — consecutive tensors of equal type and row length become one fused linear
        auto proj = [&](const std::vector<std::string>& names) {
            std::vector<const GgufTensor*> infos;
            for (const std::string& n : names) infos.push_back(&tensor(n));
            Proj p;
            size_t i = 0;
            while (i < infos.size()) {
                size_t j = i + 1;
                while (j < infos.size() && infos[j]->type_id == infos[i]->type_id && infos[j]->dims[0] == infos[i]->dims[0]) j++;
                GgmlType ty;
                if (!infos[i]->type(ty) || !ggml_type_bits(ty) || infos[i]->dims.size() != 2)
                    throw std::runtime_error(infos[i]->name + ": not a det linear");
                std::vector<LinearPart> parts;
                for (size_t q = i; q < j; q++) parts.push_back(LinearPart{g->data(*infos[q]), infos[q]->dims[1]});
                p.lins.push_back(bk->linear(parts, infos[i]->dims[0], ggml_type_bits(ty)));
                i = j;
            }
            return p;
        };
        m.embed = tensor("token_embd.weight");
        GgmlType ety;
        if (!m.embed.type(ety) || ggml_type_bits(ety) || m.embed.dims != std::vector<size_t>{cfg.hidden, cfg.vocab})
            throw std::runtime_error("token_embd.weight: not a float [hidden][vocab] table");
        m.final_norm = vec("output_norm.weight");
        const GgufTensor* rope = g->tensor("rope_cos");
        if (!rope) throw std::runtime_error("no rope tables; run `det convert`");
        if (rope->dims.size() < 2 || rope->dims[1] < max_ctx)
            throw std::runtime_error("rope tables cover " + std::to_string(rope->dims.size() < 2 ? 0 : rope->dims[1]) +
                                     " positions, context " + std::to_string(max_ctx) + " requested");
        m.rope_cos = vec("rope_cos");
        m.rope_sin = vec("rope_sin");
        m.lm_head = proj({"output.weight"});

        std::vector<float> v_scales;
        bool have_scales = false;
        if (const GgufValue* a = g->get(V_SCALE_KEY); a && a->type == 9) {
            have_scales = true;
            const size_t want = cfg.n_attention_layers() * cfg.n_kv;
            bool ok = a->arr.size() == want;
            for (const GgufValue& x : a->arr) {
                float s = 0.0f;
                ok = ok && x.as_f32(s) && std::isfinite(s) && s > 0.0f;
                v_scales.push_back(s);
            }
            if (!ok) throw std::runtime_error(std::string(V_SCALE_KEY) + ": expected " + std::to_string(want) + " positive floats");
        }
        for (float s : v_scales) m.calibrated = m.calibrated || s != DEFAULT_V_SCALE;

        const size_t n_h = cfg.n_heads, n_kv = cfg.n_kv, hd = cfg.head_dim;
        const size_t n_v = cfg.gdn_v_heads, dk = cfg.gdn_dk, dv = cfg.gdn_dv, conv_dim = cfg.conv_dim();
        (void)n_h;
        size_t attn_index = 0;
        m.layers.resize(cfg.n_layers);
        for (size_t i = 0; i < cfg.n_layers; i++) {
            Layer& l = m.layers[i];
            auto n = [&](const char* s) { return "blk." + std::to_string(i) + "." + s; };
            l.is_attn = cfg.is_attention(i);
            if (l.is_attn) {
                Attn& a = l.attn;
                std::vector<float> vs(n_kv, DEFAULT_V_SCALE), vis(n_kv);
                if (have_scales) vs.assign(v_scales.begin() + attn_index * n_kv, v_scales.begin() + (attn_index + 1) * n_kv);
                attn_index++;
                for (size_t q = 0; q < n_kv; q++) vis[q] = 1.0f / vs[q];
                a.kv.kq = bk->alloc<int8_t>(max_ctx * n_kv * hd);
                a.kv.sk = bk->alloc<float>(max_ctx * n_kv);
                a.kv.vq = bk->alloc<int16_t>(max_ctx * n_kv * hd);
                a.kv.capacity = max_ctx;
                a.qkv = proj({n("attn_q.weight"), n("attn_k.weight"), n("attn_v.weight")});
                a.o = proj({n("attn_output.weight")});
                a.q_norm = vec(n("attn_q_norm.weight"));
                a.k_norm = vec(n("attn_k_norm.weight"));
                a.v_scale = bk->upload(vs);
                a.v_inv_scale = bk->upload(vis);
            } else {
                Gdn& gd = l.gdn;
                const GgufTensor& at = tensor(n("ssm_a"));
                GgmlType aty;
                if (!at.type(aty) || ggml_type_bits(aty)) throw std::runtime_error(at.name + ": not a float vector");
                std::vector<float> av(at.n_elems());
                dequant_row(aty, g->data(at), av.size(), av.data());
                for (float& v : av) v = -v;
                gd.qkvz = proj({n("attn_qkv.weight"), n("attn_gate.weight")});
                gd.ab = proj({n("ssm_alpha.weight"), n("ssm_beta.weight")});
                gd.out = proj({n("ssm_out.weight")});
                gd.conv = vec(n("ssm_conv1d.weight"));
                gd.a = bk->upload(av);
                gd.dt_bias = vec(n("ssm_dt.bias"));
                gd.norm = vec(n("ssm_norm.weight"));
                gd.state.conv_state = bk->alloc<float>((cfg.conv_k - 1) * conv_dim);
                gd.state.s = bk->alloc<float>(n_v * dk * dv);
            }
            l.attn_norm = vec(n("attn_norm.weight"));
            l.ffn_norm = vec(n("post_attention_norm.weight"));
            l.gu = proj({n("ffn_gate.weight"), n("ffn_up.weight")});
            l.down = proj({n("ffn_down.weight")});
        }
        alloc_work(m);
    } catch (const std::exception& ex) {
        err = ex.what();
        return nullptr;
    }
    return mp;
}

void Model::set_all_logits(bool all) {
    backend->sync();
    const size_t n = (all ? max_batch : 1) * cfg.vocab;
    if (w.logits.len() != n) w.logits = backend->alloc<float>(n);
    if (comm && tp.tmp.len() < n) tp.tmp = backend->alloc<float>(n);   // the logits gather of a tensor-parallel shard
    all_logits = all;
}

void Model::reset() {
    backend->sync();
    pos = 0;
    for (Layer& l : layers)
        if (!l.is_attn) {
            backend->zero(l.gdn.state.conv_state);
            backend->zero(l.gdn.state.s);
        }
}

std::string Model::embed_rows(const int32_t* ids, size_t t) {
    const size_t h = cfg.hidden;
    std::vector<float> x(t * h);
    const uint64_t tid = tensor_id(GLOBAL_LAYER, T_EMBED);
    GgmlType ety = GgmlType::BF16;
    if (gguf) embed.type(ety);
    const size_t rb = ggml_row_bytes(ety, h);
    for (size_t i = 0; i < t; i++) {
        if (ids[i] < 0 || (size_t)ids[i] >= cfg.vocab)
            return "token id " + std::to_string(ids[i]) + " is outside the embedding table (" +
                   std::to_string(cfg.vocab) + " rows)";
        if (gguf) dequant_row(ety, gguf->data(embed) + (size_t)ids[i] * rb, h, x.data() + i * h);
        else
            for (size_t j = 0; j < h; j++) x[i * h + j] = synth_weight(seed, tid, (uint64_t)ids[i] * h + j);
    }
    backend->write(w.x, 0, x.data(), x.size());
    return "";
}

void Model::project(const Proj& p, const Buf<int8_t>& xq, const Buf<float>& sx, const Buf<uint16_t>& mx, size_t t,
                    const std::vector<const Buf<float>*>& dsts) {
    size_t i = 0;
    for (const auto& lin : p.lins) {
        const size_t n = lin->widths.size();
        if (n == 1) backend->gemm(*lin, xq, sx, mx, t, GemmOut::write(*dsts[i]));
        else backend->gemm(*lin, xq, sx, mx, t, GemmOut::parts(std::vector<const Buf<float>*>(dsts.begin() + i, dsts.begin() + i + n)));
        i += n;
    }
    if (i != dsts.size()) throw std::logic_error("project: part count mismatch");
}

// qwen35.rs:31-170
void Model::network(size_t pos0, size_t t, Observer* obs, const RowsCtx* rows) {
    if (comm) {
        if (obs) throw std::logic_error("observers are not supported on a tensor-parallel shard");
        network_tp(pos0, t, rows);
        return;
    }
    if (obs && rows) throw std::logic_error("observers are not supported on a batched decode step");
    const Config& c = cfg;
    Backend* bk = backend;
    const size_t h = c.hidden;
    const Ctx ctx{pos0, t, bk};
    const bool gdn_io = obs && obs->wants_gdn_io();
    auto observe = [&](Tap::Kind kind, size_t layer, const Buf<float>* x, const KvCache* kv = nullptr,
                       const GdnState* st = nullptr) {
        if (!obs) return;
        Tap tap;
        tap.kind = kind;
        tap.layer = layer;
        tap.x = x;
        tap.kv = kv;
        tap.state = st;
        obs->observe(ctx, tap);
    };
    for (size_t li = 0; li < layers.size(); li++) {
        Layer& l = layers[li];
        observe(Tap::Residual, li, &w.x);
        bk->rmsnorm_quant(w.x, l.attn_norm, c.eps, t, h, w.xq, w.sx, w.mx);
        if (l.is_attn) {
            Attn& a = l.attn;
            project(a.qkv, w.xq, w.sx, w.mx, t, {&w.qg, &w.k, &w.v});
            observe(Tap::AttnV, li, &w.v);
            AttnLayer layer{&a.q_norm, &a.k_norm, &a.v_scale, &a.v_inv_scale, &rope_cos, &rope_sin};
            Shape shape{t, pos0, c.n_heads, c.n_kv, c.head_dim, c.rot_dim, c.eps};
            if (rows) bk->attention_rows(layer, *(*rows->sets)[li], *rows->pos, rows->max_pos, shape, w.qg, w.k, w.v, w.o);
            else bk->attention(layer, a.kv, shape, w.qg, w.k, w.v, w.o);
            observe(Tap::Kv, li, nullptr, &a.kv);
            observe(Tap::AttnOut, li, &w.o);
            observe(Tap::MixerOut, li, &w.o);
            bk->quant(w.o, t, c.n_heads * c.head_dim, w.oq, w.so, w.mo);
            bk->gemm(*a.o.lins[0], w.oq, w.so, w.mo, t, GemmOut::accumulate(w.x));
        } else {
            Gdn& g = l.gdn;
            project(g.qkvz, w.xq, w.sx, w.mx, t, {&w.qkv, &w.z});
            GdnLayer layer{&g.conv, &g.a, &g.dt_bias, &g.norm};
            GdnShape shape{t, c.gdn_k_heads, c.gdn_v_heads, c.gdn_dk, c.gdn_dv, c.eps};
            project(g.ab, w.xq, w.sx, w.mx, t, {&w.a, &w.b});
            GdnExport ex;
            if (gdn_io) {
                const size_t rep = c.gdn_v_heads / c.gdn_k_heads;
                const size_t gw = 2 * c.gdn_dk + c.gdn_dv * rep + 2 * rep;   // model.rs:315
                if (w.gin.len() < max_batch * c.gdn_k_heads * gw) w.gin = bk->alloc<float>(max_batch * c.gdn_k_heads * gw);
                if (w.gout.len() < max_batch * c.gdn_v_heads * c.gdn_dv) w.gout = bk->alloc<float>(max_batch * c.gdn_v_heads * c.gdn_dv);
                ex.gin = &w.gin;
                ex.gout = &w.gout;
            }
            if (rows) bk->gdn_rows(layer, *(*rows->sets)[li], shape, w.qkv, w.z, w.a, w.b, w.on);
            else bk->gdn(layer, g.state, shape, w.qkv, w.z, w.a, w.b, w.on, ex);
            if (gdn_io) {
                observe(Tap::GdnIn, li, &w.gin);
                observe(Tap::GdnOut, li, &w.gout);
            }
            observe(Tap::GdnStateTap, li, nullptr, nullptr, &g.state);
            observe(Tap::MixerOut, li, &w.on);
            bk->quant(w.on, t, c.gdn_v_heads * c.gdn_dv, w.onq, w.son, w.mon);
            bk->gemm(*g.out.lins[0], w.onq, w.son, w.mon, t, GemmOut::accumulate(w.x));
        }
        observe(Tap::PostMixer, li, &w.x);
        bk->rmsnorm_quant(w.x, l.ffn_norm, c.eps, t, h, w.xq, w.sx, w.mx);
        project(l.gu, w.xq, w.sx, w.mx, t, {&w.g, &w.u});
        bk->silu_mul_quant(w.g, w.u, t, c.intermediate, w.hq, w.sh, w.mh);
        bk->gemm(*l.down.lins[0], w.hq, w.sh, w.mh, t, GemmOut::accumulate(w.x));
    }
    observe(Tap::Residual, layers.size(), &w.x);
    if (all_logits) {
        bk->rmsnorm_quant(w.x, final_norm, c.eps, t, h, w.xq, w.sx, w.mx);
        bk->gemm(*lm_head.lins[0], w.xq, w.sx, w.mx, t, GemmOut::write(w.logits));
    } else {
        Buf<float> last = Buf<float>::view(w.x.ptr_at((t - 1) * h), h);
        bk->rmsnorm_quant(last, final_norm, c.eps, 1, h, w.xq, w.sx, w.mx);
        bk->gemm(*lm_head.lins[0], w.xq, w.sx, w.mx, 1, GemmOut::write(w.logits));
    }
    observe(Tap::Logits, 0, &w.logits);
}

// ---------------------------------------------------------------------------------------------------------------------
// Tensor parallel shard.  Rank r of P owns, per layer:
//   attention  q heads [r*n_h/P, ...) with the kv head(s) they read (a kv head shared by several ranks is recomputed on
//              each of them, identically); rows [r*H/P, ...) of the output projection
//   GDN        k heads [r*n_k/P, ...) with their v heads (conv channels, a/b rows, state); rows of ssm_out as above
//   FFN        columns [r*F/P, ...) of gate and up (whole 128-groups); rows [r*H/P, ...) of down
//   head       vocabulary rows [r*V/P, ...)
// Every fp32 value is produced by exactly one rank (or identically on several) with the single-device op sequence; the
// exchanges copy finished values (mixer output, SwiGLU product, projection rows, logits), so logits cannot change.
static void load_shard(Model& m, const Config& cfg, uint64_t seed, Backend* bk, size_t max_ctx, size_t max_batch) {
    const size_t P = (size_t)m.comm->size, r = (size_t)m.comm->rank;
    m.cfg = cfg;
    m.backend = bk;
    m.seed = seed;
    m.max_ctx = max_ctx;
    m.max_batch = max_batch;
    const size_t h = cfg.hidden, inter = cfg.intermediate;
    const size_t n_h = cfg.n_heads, n_kv = cfg.n_kv, hd = cfg.head_dim, rep = n_h / n_kv;
    const size_t n_k = cfg.gdn_k_heads, n_v = cfg.gdn_v_heads, dk = cfg.gdn_dk, dv = cfg.gdn_dv, grep = n_v / n_k;
    const int wb = cfg.bits_default;
    auto need = [](bool ok, const char* what) {
        if (!ok) throw std::runtime_error(std::string("tensor parallel size does not divide ") + what);
    };
    need(n_h % P == 0, "the attention heads");
    need(n_k % P == 0, "the GDN key heads");
    need(h % (P * 128) == 0 || h % P == 0, "the hidden size");
    need(inter % (P * 128) == 0, "the FFN groups");
    need(cfg.vocab % P == 0, "the vocabulary");
    need(n_h * hd == n_v * dv, "mixer widths (attention and GDN outputs share one gather buffer)");
    Model::Tp& tp = m.tp;
    tp.heads = n_h / P;
    const size_t h0 = r * tp.heads;
    tp.kv = n_kv >= P ? n_kv / P : 1;
    const size_t kv0 = h0 / rep;
    need(n_kv >= P ? n_kv % P == 0 : rep % tp.heads == 0, "the kv heads");
    tp.k_heads = n_k / P;
    tp.v_heads = tp.k_heads * grep;
    const size_t k0 = r * tp.k_heads, v0 = k0 * grep;
    tp.ffn = inter / P;
    tp.hid = h / P;
    tp.voc = cfg.vocab / P;
    const size_t f0 = r * tp.ffn, hr0 = r * tp.hid;

    m.final_norm = ones(bk, h);
    std::vector<float> rc, rs;
    rope_tables(cfg, max_ctx, rc, rs);
    m.rope_cos = bk->upload(rc);
    m.rope_sin = bk->upload(rs);
    m.lm_head = make_proj(bk, seed, GLOBAL_LAYER, {{T_EMBED, tp.voc, h, 8, r * tp.voc}});
    const size_t conv_l = 2 * tp.k_heads * dk + tp.v_heads * dv;
    m.layers.resize(cfg.n_layers);
    for (size_t i = 0; i < cfg.n_layers; i++) {
        Layer& l = m.layers[i];
        l.is_attn = cfg.is_attention(i);
        if (l.is_attn) {
            Attn& a = l.attn;
            a.qkv = make_proj(bk, seed, i, {{T_ATTN_Q, tp.heads * 2 * hd, h, wb, h0 * 2 * hd},
                                            {T_ATTN_K, tp.kv * hd, h, wb, kv0 * hd},
                                            {T_ATTN_V, tp.kv * hd, h, wb, kv0 * hd}});
            a.o = make_proj(bk, seed, i, {{T_ATTN_OUT, tp.hid, n_h * hd, wb, hr0}});
            a.q_norm = ones(bk, hd);
            a.k_norm = ones(bk, hd);
            std::vector<float> vs(tp.kv, DEFAULT_V_SCALE), vis(tp.kv);
            for (size_t q = 0; q < tp.kv; q++) vis[q] = 1.0f / vs[q];
            a.v_scale = bk->upload(vs);
            a.v_inv_scale = bk->upload(vis);
            a.kv.kq = bk->alloc<int8_t>(max_ctx * tp.kv * hd);
            a.kv.sk = bk->alloc<float>(max_ctx * tp.kv);
            a.kv.vq = bk->alloc<int16_t>(max_ctx * tp.kv * hd);
            a.kv.capacity = max_ctx;
        } else {
            Gdn& g = l.gdn;
            // attn_qkv rows are [q: n_k*dk | k: n_k*dk | v: n_v*dv]; the local linear keeps that order for its heads
            g.qkvz = make_proj(bk, seed, i, {{T_GDN_QKV, tp.k_heads * dk, h, wb, k0 * dk},
                                             {T_GDN_QKV, tp.k_heads * dk, h, wb, n_k * dk + k0 * dk},
                                             {T_GDN_QKV, tp.v_heads * dv, h, wb, 2 * n_k * dk + v0 * dv},
                                             {T_GDN_GATE, tp.v_heads * dv, h, wb, v0 * dv}});
            // the q, k and v row ranges are one output ([q | k | v] per token, what the mixer reads); z is the other
            g.qkvz.lins[0]->widths = {conv_l, tp.v_heads * dv};
            g.ab = make_proj(bk, seed, i, {{T_GDN_ALPHA, tp.v_heads, h, 8, v0}, {T_GDN_BETA, tp.v_heads, h, 8, v0}});
            g.out = make_proj(bk, seed, i, {{T_GDN_OUT, tp.hid, n_v * dv, wb, hr0}});
            std::vector<float> conv(conv_l * cfg.conv_k), dtb(tp.v_heads), av(tp.v_heads);
            auto global_channel = [&](size_t c) {   // local conv channel -> channel of the full model
                if (c < tp.k_heads * dk) return k0 * dk + c;
                c -= tp.k_heads * dk;
                if (c < tp.k_heads * dk) return n_k * dk + k0 * dk + c;
                c -= tp.k_heads * dk;
                return 2 * n_k * dk + v0 * dv + c;
            };
            for (size_t c = 0; c < conv_l; c++)
                for (size_t tap = 0; tap < cfg.conv_k; tap++)
                    conv[c * cfg.conv_k + tap] =
                        draw_normal(seed, tensor_id(i, T_CONV), global_channel(c) * cfg.conv_k + tap, WEIGHT_STD);
            for (size_t q = 0; q < tp.v_heads; q++) {
                dtb[q] = draw_normal(seed, tensor_id(i, T_DT_BIAS), v0 + q, WEIGHT_STD);
                av[q] = 1.0f + 15.0f * draw_unit(seed, tensor_id(i, T_SSM_A), v0 + q);
            }
            g.conv = bk->upload(conv);
            g.a = bk->upload(av);
            g.dt_bias = bk->upload(dtb);
            g.norm = ones(bk, dv);
            g.state.conv_state = bk->alloc<float>((cfg.conv_k - 1) * conv_l);
            g.state.s = bk->alloc<float>(tp.v_heads * dk * dv);
        }
        l.attn_norm = ones(bk, h);
        l.ffn_norm = ones(bk, h);
        l.gu = make_proj(bk, seed, i, {{T_FFN_GATE, tp.ffn, h, wb, f0}, {T_FFN_UP, tp.ffn, h, wb, f0}});
        l.down = make_proj(bk, seed, i, {{T_FFN_DOWN, tp.hid, inter, wb, hr0}});
    }
    const size_t mb = max_batch;
    Work& w = m.w;
    const size_t mix = n_h * hd;
    w.x = bk->alloc<float>(mb * h);
    w.xq = bk->alloc<int8_t>(mb * h);
    w.sx = bk->alloc<float>(mb);
    w.mx = bk->alloc<uint16_t>(mb * h / 128);
    w.qg = bk->alloc<float>(mb * tp.heads * 2 * hd);
    w.k = bk->alloc<float>(mb * tp.kv * hd);
    w.v = bk->alloc<float>(mb * tp.kv * hd);
    w.o = bk->alloc<float>(mb * std::max(tp.heads * hd, tp.v_heads * dv));   // local mixer output (either kind)
    w.oq = bk->alloc<int8_t>(mb * mix);
    w.so = bk->alloc<float>(mb);
    w.mo = bk->alloc<uint16_t>(mb * mix / 128);
    w.qkv = bk->alloc<float>(mb * conv_l);
    w.z = bk->alloc<float>(mb * tp.v_heads * dv);
    w.a = bk->alloc<float>(mb * tp.v_heads);
    w.b = bk->alloc<float>(mb * tp.v_heads);
    w.g = bk->alloc<float>(mb * tp.ffn);
    w.u = bk->alloc<float>(mb * tp.ffn);
    w.hq = bk->alloc<int8_t>(mb * inter);
    w.sh = bk->alloc<float>(mb);
    w.mh = bk->alloc<uint16_t>(mb * inter / 128);
    w.logits = bk->alloc<float>(cfg.vocab);
    tp.mix_full = bk->alloc<float>(mb * mix);
    tp.h_l = bk->alloc<float>(mb * tp.ffn);
    tp.h_full = bk->alloc<float>(mb * inter);
    tp.y_l = bk->alloc<float>(mb * tp.hid);
    tp.y_full = bk->alloc<float>(mb * h);
    tp.logits_l = bk->alloc<float>(mb * tp.voc);
    tp.tmp = bk->alloc<float>(std::max(mb * std::max(inter, mix), cfg.vocab));
    tp.x_alt = bk->alloc<float>(mb * h);
}

void Model::network_tp(size_t pos0, size_t t, const RowsCtx* rows) {
    const Config& c = cfg;
    Backend* bk = backend;
    const size_t h = c.hidden;
    // The residual stream lives in w.x or in tp.x_alt: an exchange that runs as the prologue of the GEMV it feeds stores
    // x + gathered into the other copy (every CTA of that launch still reads the old one).  `xc` is the current copy.
    const Buf<float>* xc = &w.x;
    const Buf<float>* xo = &tp.x_alt;
    // A projection back to the hidden size leaves this rank's rows in y_l; the exchange, the residual add and the
    // RMSNorm + quantization that follows are one step of the communicator (one launch on the peer-memory exchange, or
    // the prologue of the next GEMV).
    auto project_back = [&](const Linear& lin, const Buf<int8_t>& q, const Buf<float>& s, const Buf<uint16_t>& mm) {
        bk->gemm(lin, q, s, mm, t, GemmOut::write(tp.y_l));
    };
    auto add_norm_quant = [&](const Buf<float>& norm_w) {
        if (comm->gather_add_norm_quant_alt(*bk, tp.y_l, tp.tmp, tp.y_full, t, tp.hid, *xc, *xo, norm_w, c.eps, w.xq, w.sx, w.mx))
            std::swap(xc, xo);
    };
    bool pending = false;   // y_l of the previous layer's down projection has not been added to x yet
    for (size_t li = 0; li < layers.size(); li++) {
        Layer& l = layers[li];
        if (pending) add_norm_quant(l.attn_norm);
        else bk->rmsnorm_quant(*xc, l.attn_norm, c.eps, t, h, w.xq, w.sx, w.mx);
        if (l.is_attn) {
            Attn& a = l.attn;
            project(a.qkv, w.xq, w.sx, w.mx, t, {&w.qg, &w.k, &w.v});
            AttnLayer layer{&a.q_norm, &a.k_norm, &a.v_scale, &a.v_inv_scale, &rope_cos, &rope_sin};
            Shape shape{t, pos0, tp.heads, tp.kv, c.head_dim, c.rot_dim, c.eps};
            if (rows) bk->attention_rows(layer, *(*rows->sets)[li], *rows->pos, rows->max_pos, shape, w.qg, w.k, w.v, w.o);
            else bk->attention(layer, a.kv, shape, w.qg, w.k, w.v, w.o);
            comm->gather_quant(*bk, w.o, tp.tmp, tp.mix_full, t, tp.heads * c.head_dim, w.oq, w.so, w.mo);
            project_back(*a.o.lins[0], w.oq, w.so, w.mo);
        } else {
            Gdn& g = l.gdn;
            project(g.qkvz, w.xq, w.sx, w.mx, t, {&w.qkv, &w.z});
            GdnLayer layer{&g.conv, &g.a, &g.dt_bias, &g.norm};
            GdnShape shape{t, tp.k_heads, tp.v_heads, c.gdn_dk, c.gdn_dv, c.eps};
            project(g.ab, w.xq, w.sx, w.mx, t, {&w.a, &w.b});
            if (rows) bk->gdn_rows(layer, *(*rows->sets)[li], shape, w.qkv, w.z, w.a, w.b, w.o);
            else bk->gdn(layer, g.state, shape, w.qkv, w.z, w.a, w.b, w.o, GdnExport{});
            comm->gather_quant(*bk, w.o, tp.tmp, tp.mix_full, t, tp.v_heads * c.gdn_dv, w.oq, w.so, w.mo);
            project_back(*g.out.lins[0], w.oq, w.so, w.mo);
        }
        add_norm_quant(l.ffn_norm);
        project(l.gu, w.xq, w.sx, w.mx, t, {&w.g, &w.u});
        comm->silu_gather_quant(*bk, w.g, w.u, tp.h_l, tp.tmp, tp.h_full, t, tp.ffn, w.hq, w.sh, w.mh);
        project_back(*l.down.lins[0], w.hq, w.sh, w.mh);
        pending = true;
    }
    const size_t out_rows = all_logits ? t : 1;
    if (all_logits || t == 1) {
        if (pending) add_norm_quant(final_norm);
        else bk->rmsnorm_quant(*xc, final_norm, c.eps, t, h, w.xq, w.sx, w.mx);
    } else {
        if (pending) {
            comm->all_gather(*bk, tp.y_l, tp.tmp, tp.y_full, t, tp.hid);
            bk->add(*xc, tp.y_full, t * h);
        }
        Buf<float> last = Buf<float>::view(xc->ptr_at((t - 1) * h), h);
        bk->rmsnorm_quant(last, final_norm, c.eps, 1, h, w.xq, w.sx, w.mx);
    }
    bk->gemm(*lm_head.lins[0], w.xq, w.sx, w.mx, out_rows, GemmOut::write(tp.logits_l));
    comm->all_gather(*bk, tp.logits_l, tp.tmp, w.logits, out_rows, tp.voc);
}

std::string Model::forward(const int32_t* ids, size_t t, Observer* obs) {
    if (t == 0 || t > max_batch)
        return "batch of " + std::to_string(t) + " tokens (1 to " + std::to_string(max_batch) + " allowed)";
    if (pos + t > max_ctx)
        return std::to_string(t) + " tokens at position " + std::to_string(pos) + " exceed the context of " +
               std::to_string(max_ctx);
    std::string e = embed_rows(ids, t);
    if (!e.empty()) return e;
    network(pos, t, obs);
    pos += t;
    return "";
}

std::vector<float> Model::logits() { return backend->download(w.logits); }

std::string Model::pick(Sampling& s, int32_t& id) { return pick_row(w.logits, s, id); }

std::string Model::pick_row(const Buf<float>& row, Sampling& s, int32_t& id) {
    if (s.greedy) {
        id = backend->argmax(row, cfg.vocab);
        return "";
    }
    if (!std::isfinite(s.inv_temp) || std::isnan(s.top_p))
        return "sampling parameters inv_temp=" + std::to_string(s.inv_temp) + " top_p=" + std::to_string(s.top_p) +
               " are not finite";
    id = backend->sample(row, cfg.vocab, s.inv_temp, s.top_k, s.top_p, next_draw(s));
    return "";
}

uint64_t Model::next_draw(Sampling& s) {
    s.rng += 0x9E3779B97F4A7C15ull;   // splitmix64 (spec/prim.rs:207-215): the state advances once per draw
    uint64_t z = s.rng;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

std::string Model::prefill(const int32_t* ids, size_t n, Observer* obs) {
    for (size_t i = 0; i < n; i += max_batch) {
        std::string e = forward(ids + i, std::min(max_batch, n - i), obs);
        if (!e.empty()) return e;
    }
    return "";
}

std::string Model::generate(const int32_t* prompt, size_t n_prompt, size_t n_new, Sampling s,
                            const std::vector<int32_t>& stop, std::vector<int32_t>& out,
                            const std::function<void(int32_t)>& on_token, Observer* obs) {
    std::string e = prefill(prompt, n_prompt, obs);
    if (!e.empty()) return e;
    out.clear();
    for (size_t i = 0; i < n_new; i++) {
        int32_t id = 0;
        e = pick(s, id);
        if (!e.empty()) return e;
        if (obs) {   // model.rs:524-538
            Tap tap;
            tap.kind = Tap::Token;
            tap.id = id;
            tap.rng = s.rng;
            obs->observe(Ctx{pos - 1, 1, backend}, tap);
        }
        out.push_back(id);
        if (on_token) on_token(id);
        if (std::find(stop.begin(), stop.end(), id) != stop.end() || i + 1 == n_new) break;
        e = forward(&id, 1, obs);
        if (!e.empty()) return e;
    }
    return "";
}

}  // namespace det
