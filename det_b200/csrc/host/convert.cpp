// `det convert` and `det calibrate` on top of the GGUF container.  See convert.hpp for the reference map.
#include "convert.hpp"
#include <algorithm>
#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <thread>

namespace det {

// ---- source
bool Source::open(const std::string& path, Source& out, std::string& err) {
    out.parts.clear();
    std::shared_ptr<Gguf> first = Gguf::open(path, err);
    if (!first) return false;
    uint64_t count = 1;
    first->u64("split.count", count);
    out.parts.push_back(first);
    if (count > 1) {
        const size_t slash = path.find_last_of('/');
        const std::string dir = slash == std::string::npos ? "" : path.substr(0, slash + 1);
        const std::string name = slash == std::string::npos ? path : path.substr(slash + 1);
        const size_t marker = name.find("-00001-of-");
        if (marker == std::string::npos) {
            err = "split GGUF without -00001-of- in its name";
            return false;
        }
        for (uint64_t i = 2; i <= count; i++) {
            char num[16];
            std::snprintf(num, sizeof num, "%05llu", (unsigned long long)i);
            const std::string sibling = dir + name.substr(0, marker) + "-" + num + "-of-" + name.substr(marker + 10);
            std::shared_ptr<Gguf> g = Gguf::open(sibling, err);
            if (!g) return false;
            out.parts.push_back(g);
        }
    }
    return true;
}
bool Source::tensor(const std::string& name, const Gguf*& g, const GgufTensor*& t) const {
    for (const auto& p : parts)
        if (const GgufTensor* x = p->tensor(name)) {
            g = p.get();
            t = x;
            return true;
        }
    return false;
}
std::vector<float> Source::f32s(const std::string& name) const {
    const Gguf* g;
    const GgufTensor* t;
    if (!tensor(name, g, t)) throw std::runtime_error("missing tensor " + name);
    GgmlType ty;
    if (!t->type(ty)) throw std::runtime_error(name + ": unsupported source type");
    const size_t k = t->dims[0], rows = t->n_elems() / k, rb = ggml_row_bytes(ty, k);
    std::vector<float> out(rows * k);
    for (size_t r = 0; r < rows; r++) dequant_row(ty, g->data(*t) + r * rb, k, out.data() + r * k);
    return out;
}

// ---- bit widths
std::string Bits::parse(const std::string& s, Bits& out) {
    out = Bits();
    size_t pos = 0;
    while (pos <= s.size()) {
        size_t comma = s.find(',', pos);
        if (comma == std::string::npos) comma = s.size();
        std::string item = s.substr(pos, comma - pos);
        pos = comma + 1;
        const size_t a = item.find_first_not_of(" \t"), b = item.find_last_not_of(" \t");
        if (a == std::string::npos) continue;
        item = item.substr(a, b - a + 1);
        const size_t eq = item.find('=');
        const std::string num = eq == std::string::npos ? item : item.substr(eq + 1);
        int bits = 0;
        bool ok = !num.empty() && num.size() < 6;
        for (char ch : num) {
            ok = ok && ch >= '0' && ch <= '9';
            bits = bits * 10 + (ch - '0');
        }
        if (!ok) return "bad bit width \"" + num + "\"";
        if (bits != 4 && bits != 6 && bits != 8) return "bit width " + std::to_string(bits) + " is not 4, 6 or 8";
        if (eq == std::string::npos) out.def = bits;
        else out.per.emplace_back(item.substr(0, eq), bits);
    }
    return "";
}
int Bits::of(const std::string& linear) const {
    for (const auto& e : per)
        if (e.first == linear) return e.second;
    return def;
}

// ---- quantizer (host)
void host_quantize_rows(const uint8_t* src, GgmlType type, size_t, const std::vector<int>* row_perm,
                        const std::vector<int>* col_perm, size_t n, size_t k, int bits, uint8_t* out) {
    const size_t rb = det_row_bytes(bits, k), srb = ggml_row_bytes(type, k);
    unsigned nt = std::max(1u, std::min(std::thread::hardware_concurrency(), 32u));
    if (n * k < (1u << 20)) nt = 1;
    std::vector<std::thread> pool;
    for (unsigned w = 0; w < nt; w++)
        pool.emplace_back([&, w] {
            std::vector<float> row(k), tmp(k);
            for (size_t r = w; r < n; r += nt) {
                const size_t sr = row_perm ? (size_t)(*row_perm)[r] : r;
                if (col_perm) {
                    dequant_row(type, src + sr * srb, k, tmp.data());
                    for (size_t i = 0; i < k; i++) row[i] = tmp[(size_t)(*col_perm)[i]];
                } else dequant_row(type, src + sr * srb, k, row.data());
                quantize_row(row.data(), k, bits, out + r * rb);
            }
        });
    for (auto& t : pool) t.join();
}

std::vector<int> head_perm(size_t n_k, size_t n_v, size_t width, size_t offset, size_t total) {
    const size_t rep = n_v / n_k;
    std::vector<int> p(total);
    for (size_t i = 0; i < total; i++) p[i] = (int)i;
    for (size_t h2 = 0; h2 < n_v; h2++) {
        const size_t h = (h2 % rep) * n_k + h2 / rep;
        for (size_t j = 0; j < width; j++) p[offset + h2 * width + j] = (int)(offset + h * width + j);
    }
    return p;
}

// ---- convert
namespace {
struct Gen {
    enum Kind { Copy, Vec, Quant, Rope } kind = Copy;
    std::string name;
    int bits = 0;
    bool cos = false;
    std::vector<int> rows, cols, perm;
    bool has_rows = false, has_cols = false;
};
struct Out {
    std::string name;
    std::vector<size_t> dims;
    GgmlType ty;
    Gen gen;
};
size_t out_bytes(const Out& o) {
    size_t outer = 1;
    for (size_t i = 1; i < o.dims.size(); i++) outer *= o.dims[i];
    return ggml_row_bytes(o.ty, o.dims[0]) * outer;
}
}  // namespace

std::string convert(const Source& src, const std::string& out_path, const ConvertOptions& opt) {
    try {
        Config cfg;
        std::string e = config_from_gguf(*src.parts[0], cfg);
        if (!e.empty()) return e;
        const size_t n_k = cfg.gdn_k_heads, n_v = cfg.gdn_v_heads, dk = cfg.gdn_dk, dv = cfg.gdn_dv;
        const size_t kd = n_k * dk, conv_dim = cfg.conv_dim();
        size_t n_pos = opt.rope_positions;
        if (!n_pos) {
            uint64_t ctx = 32768;
            src.parts[0]->u64(cfg.name + ".context_length", ctx);
            n_pos = (size_t)ctx;
        }
        auto find = [&](const std::string& name, const Gguf*& g, const GgufTensor*& t) {
            if (!src.tensor(name, g, t)) throw std::runtime_error("missing tensor " + name);
        };
        std::vector<Out> plan;
        auto copy = [&](const std::string& name) {
            const Gguf* g;
            const GgufTensor* t;
            find(name, g, t);
            GgmlType ty;
            if (!t->type(ty)) throw std::runtime_error(name + ": unsupported source type");
            Out o{name, t->dims, ty, {}};
            o.gen.kind = Gen::Copy;
            o.gen.name = name;
            plan.push_back(std::move(o));
        };
        auto quant = [&](const std::string& name, const std::vector<int>* rows, const std::vector<int>* cols) {
            const Gguf* g;
            const GgufTensor* t;
            find(name, g, t);
            if (t->dims.size() != 2) throw std::runtime_error(name + ": not a matrix");
            // "blk.3.ffn_down.weight" -> "ffn_down" (convert.rs:196)
            const size_t last = name.rfind('.');
            const size_t prev = last == std::string::npos || last == 0 ? std::string::npos : name.rfind('.', last - 1);
            const std::string linear = last == std::string::npos ? name : name.substr(prev == std::string::npos ? 0 : prev + 1, last - (prev == std::string::npos ? 0 : prev + 1));
            const int bits = opt.bits.of(linear);
            Out o{name, {t->dims[0], t->dims[1]}, ggml_det_type(bits), {}};
            o.gen.kind = Gen::Quant;
            o.gen.name = name;
            o.gen.bits = bits;
            if (rows) { o.gen.rows = *rows; o.gen.has_rows = true; }
            if (cols) { o.gen.cols = *cols; o.gen.has_cols = true; }
            plan.push_back(std::move(o));
        };
        copy("token_embd.weight");
        copy("output_norm.weight");
        {
            const Gguf* g;
            const GgufTensor* t;
            const std::string head = src.tensor("output.weight", g, t) ? "output.weight" : "token_embd.weight";
            find(head, g, t);
            const int head_bits = opt.bits.of("output");
            Out o{"output.weight", {t->dims[0], t->dims[1]}, ggml_det_type(head_bits), {}};
            o.gen.kind = Gen::Quant;
            o.gen.name = head;
            o.gen.bits = head_bits;
            plan.push_back(std::move(o));
        }
        for (int cosv = 1; cosv >= 0; cosv--) {
            Out o{cosv ? "rope_cos" : "rope_sin", {cfg.rot_dim / 2, n_pos}, GgmlType::F32, {}};
            o.gen.kind = Gen::Rope;
            o.gen.cos = cosv != 0;
            plan.push_back(std::move(o));
        }
        for (size_t i = 0; i < cfg.n_layers; i++) {
            auto n = [&](const std::string& s) { return "blk." + std::to_string(i) + "." + s; };
            copy(n("attn_norm.weight"));
            copy(n("post_attention_norm.weight"));
            for (const char* s : {"ffn_gate", "ffn_up", "ffn_down"}) quant(n(std::string(s) + ".weight"), nullptr, nullptr);
            if (cfg.is_attention(i)) {
                for (const char* s : {"attn_q", "attn_k", "attn_v", "attn_output"}) quant(n(std::string(s) + ".weight"), nullptr, nullptr);
                copy(n("attn_q_norm.weight"));
                copy(n("attn_k_norm.weight"));
            } else {
                const std::vector<int> vrows = head_perm(n_k, n_v, dv, 2 * kd, conv_dim);
                const std::vector<int> zrows = head_perm(n_k, n_v, dv, 0, n_v * dv);
                const std::vector<int> heads = head_perm(n_k, n_v, 1, 0, n_v);
                quant(n("attn_qkv.weight"), &vrows, nullptr);
                quant(n("attn_gate.weight"), &zrows, nullptr);
                quant(n("ssm_alpha.weight"), &heads, nullptr);
                quant(n("ssm_beta.weight"), &heads, nullptr);
                quant(n("ssm_out.weight"), nullptr, &zrows);
                const std::pair<const char*, const std::vector<int>*> vecs[3] = {
                    {"ssm_conv1d.weight", &vrows}, {"ssm_a", &heads}, {"ssm_dt.bias", &heads}};
                for (const auto& v : vecs) {
                    const Gguf* g;
                    const GgufTensor* t;
                    find(n(v.first), g, t);
                    Out o{n(v.first), t->dims, GgmlType::F32, {}};
                    o.gen.kind = Gen::Vec;
                    o.gen.name = n(v.first);
                    o.gen.perm = *v.second;
                    plan.push_back(std::move(o));
                }
                copy(n("ssm_norm.weight"));
            }
        }

        const size_t align = 32;
        std::vector<GgufTensor> infos;
        size_t offset = 0;
        for (const Out& o : plan) {
            GgufTensor t;
            t.name = o.name;
            t.dims = o.dims;
            t.type_id = (uint32_t)o.ty;
            t.offset = offset;
            offset = (offset + out_bytes(o) + align - 1) / align * align;
            infos.push_back(std::move(t));
        }
        GgufKv kv;
        for (const auto& e2 : src.kv())
            if (e2.first.rfind("split.", 0) != 0 && e2.first != V_SCALE_KEY) kv.push_back(e2);
        kv.emplace_back(V_SCALE_KEY, GgufValue::f32_array(std::vector<float>(cfg.n_attention_layers() * cfg.n_kv, DEFAULT_V_SCALE)));
        const std::vector<uint8_t> header = gguf_write_header(kv, infos, align);
        FILE* f = std::fopen(out_path.c_str(), "wb");
        if (!f) return out_path + ": " + std::strerror(errno);
        bool ok = std::fwrite(header.data(), 1, header.size(), f) == header.size();
        size_t written = 0;
        const RowQuantizer quantizer = opt.quantizer ? opt.quantizer : RowQuantizer(host_quantize_rows);
        for (size_t pi = 0; ok && pi < plan.size(); pi++) {
            const Out& o = plan[pi];
            std::vector<uint8_t> data;
            switch (o.gen.kind) {
                case Gen::Copy: {
                    const Gguf* g;
                    const GgufTensor* t;
                    find(o.gen.name, g, t);
                    data.assign(g->data(*t), g->data(*t) + t->bytes());
                    break;
                }
                case Gen::Vec: {
                    const std::vector<float> v = src.f32s(o.gen.name);
                    const size_t inner = o.dims.size() > 1 ? o.dims[0] : 1, outer = v.size() / inner;
                    if (o.gen.perm.size() != outer) throw std::runtime_error(o.gen.name + ": permutation length");
                    data.resize(v.size() * 4);
                    for (size_t r = 0; r < outer; r++)
                        std::memcpy(data.data() + r * inner * 4, v.data() + (size_t)o.gen.perm[r] * inner, inner * 4);
                    break;
                }
                case Gen::Quant: {
                    const size_t k = o.dims[0], n = o.dims[1];
                    const Gguf* g;
                    const GgufTensor* t;
                    find(o.gen.name, g, t);
                    GgmlType sty;
                    if (!t->type(sty) || ggml_type_bits(sty)) throw std::runtime_error(o.gen.name + ": unsupported source type");
                    if (o.gen.has_rows && o.gen.rows.size() != n) throw std::runtime_error(o.gen.name + ": row permutation length");
                    if (o.gen.has_cols && o.gen.cols.size() != k) throw std::runtime_error(o.gen.name + ": column permutation length");
                    if (opt.verbose) std::fprintf(stderr, "  %s: %zu x %zu -> W%d\n", o.gen.name.c_str(), n, k, o.gen.bits);
                    data.resize(n * det_row_bytes(o.gen.bits, k));
                    quantizer(g->data(*t), sty, n, o.gen.has_rows ? &o.gen.rows : nullptr, o.gen.has_cols ? &o.gen.cols : nullptr, n, k,
                              o.gen.bits, data.data());
                    break;
                }
                case Gen::Rope: {   // convert.rs:370-385: binary64 angles, rounded once
                    const size_t half = cfg.rot_dim / 2;
                    std::vector<double> inv_freq(half);
                    for (size_t q = 0; q < half; q++) inv_freq[q] = std::pow(cfg.rope_theta, -((double)(2 * q)) / (double)cfg.rot_dim);
                    data.resize(n_pos * half * 4);
                    float* dst = reinterpret_cast<float*>(data.data());
                    for (size_t pos = 0; pos < n_pos; pos++)
                        for (size_t q = 0; q < half; q++) {
                            const double a = (double)pos * inv_freq[q];
                            dst[pos * half + q] = (float)(o.gen.cos ? std::cos(a) : std::sin(a));
                        }
                    break;
                }
            }
            if (written != infos[pi].offset || data.size() != out_bytes(o)) {
                std::fclose(f);
                return o.name + ": size or offset mismatch";
            }
            data.resize((data.size() + align - 1) / align * align, 0);
            ok = std::fwrite(data.data(), 1, data.size(), f) == data.size();
            written += data.size();
        }
        if (std::fclose(f) != 0 || !ok) return out_path + ": write failed";
        if (opt.verbose)
            std::fprintf(stderr, "wrote %s (%zu tensors, %.2f GB)\n", out_path.c_str(), infos.size(), (double)(header.size() + written) / 1e9);
        return "";
    } catch (const std::exception& ex) {
        return ex.what();
    }
}

std::string default_output(const std::string& src_path, const Bits& bits) {
    const size_t slash = src_path.find_last_of('/');
    const std::string dir = slash == std::string::npos ? "" : src_path.substr(0, slash + 1);
    std::string stem = slash == std::string::npos ? src_path : src_path.substr(slash + 1);
    const size_t dot = stem.rfind('.');
    if (dot != std::string::npos && dot != 0) stem = stem.substr(0, dot);
    // each suffix is trimmed repeatedly, in this order (Rust's trim_end_matches)
    for (const char* suffix : {"-00001-of-00002", "-BF16", "-bf16", "-F16", "-f16"}) {
        const size_t n = std::strlen(suffix);
        while (stem.size() >= n && stem.compare(stem.size() - n, n, suffix) == 0) stem.resize(stem.size() - n);
    }
    return dir + stem + "-det-w" + std::to_string(bits.def) + ".gguf";
}

// ---- synthetic float source
std::string write_synthetic_source_gguf(const Config& c, uint64_t seed, const std::string& path, size_t n_pos,
                                        bool f32_linears) {
    const size_t h = c.hidden, inter = c.intermediate, hd = c.head_dim;
    const size_t n_k = c.gdn_k_heads, n_v = c.gdn_v_heads, dk = c.gdn_dk, dv = c.gdn_dv, conv_dim = c.conv_dim();
    struct T {
        std::string name;
        std::vector<size_t> dims;
        GgmlType ty;
        std::function<std::vector<float>()> values;   // in converted order
        std::vector<int> rows, cols;                  // the conversion's permutations (perm[new] = old); empty: none
    };
    std::vector<T> plan;
    const GgmlType lty = f32_linears ? GgmlType::F32 : GgmlType::BF16;
    auto matrix = [&](const std::string& name, size_t layer, TensorKind kind, size_t n, size_t k, std::vector<int> rows = {},
                      std::vector<int> cols = {}) {
        plan.push_back({name, {k, n}, lty, [=] {
                            std::vector<float> v(n * k);
                            const uint64_t tid = tensor_id(layer, kind);
                            for (size_t i = 0; i < v.size(); i++) v[i] = synth_weight(seed, tid, i);
                            return v;
                        }, std::move(rows), std::move(cols)});
    };
    auto ones = [&](const std::string& name, size_t n) {
        plan.push_back({name, {n}, GgmlType::F32, [=] { return std::vector<float>(n, 1.0f); }, {}, {}});
    };
    plan.push_back({"token_embd.weight", {h, c.vocab}, GgmlType::BF16, [&] {
                        std::vector<float> v(c.vocab * h);
                        const uint64_t tid = tensor_id(GLOBAL_LAYER, T_EMBED);
                        for (size_t i = 0; i < v.size(); i++) v[i] = synth_weight(seed, tid, i);
                        return v;
                    }, {}, {}});
    ones("output_norm.weight", h);
    for (size_t i = 0; i < c.n_layers; i++) {
        const std::string b = "blk." + std::to_string(i) + ".";
        ones(b + "attn_norm.weight", h);
        ones(b + "post_attention_norm.weight", h);
        matrix(b + "ffn_gate.weight", i, T_FFN_GATE, inter, h);
        matrix(b + "ffn_up.weight", i, T_FFN_UP, inter, h);
        matrix(b + "ffn_down.weight", i, T_FFN_DOWN, h, inter);
        if (c.is_attention(i)) {
            matrix(b + "attn_q.weight", i, T_ATTN_Q, c.n_heads * 2 * hd, h);
            matrix(b + "attn_k.weight", i, T_ATTN_K, c.n_kv * hd, h);
            matrix(b + "attn_v.weight", i, T_ATTN_V, c.n_kv * hd, h);
            matrix(b + "attn_output.weight", i, T_ATTN_OUT, h, c.n_heads * hd);
            ones(b + "attn_q_norm.weight", hd);
            ones(b + "attn_k_norm.weight", hd);
        } else {
            const std::vector<int> vrows = head_perm(n_k, n_v, dv, 2 * n_k * dk, conv_dim);
            const std::vector<int> zrows = head_perm(n_k, n_v, dv, 0, n_v * dv);
            const std::vector<int> heads = head_perm(n_k, n_v, 1, 0, n_v);
            matrix(b + "attn_qkv.weight", i, T_GDN_QKV, conv_dim, h, vrows);
            matrix(b + "attn_gate.weight", i, T_GDN_GATE, n_v * dv, h, zrows);
            matrix(b + "ssm_alpha.weight", i, T_GDN_ALPHA, n_v, h, heads);
            matrix(b + "ssm_beta.weight", i, T_GDN_BETA, n_v, h, heads);
            matrix(b + "ssm_out.weight", i, T_GDN_OUT, h, n_v * dv, {}, zrows);
            plan.push_back({b + "ssm_conv1d.weight", {c.conv_k, conv_dim}, GgmlType::F32, [=] {
                                std::vector<float> v(conv_dim * c.conv_k);
                                for (size_t q = 0; q < v.size(); q++) v[q] = draw_normal(seed, tensor_id(i, T_CONV), q, WEIGHT_STD);
                                return v;
                            }, vrows, {}});
            plan.push_back({b + "ssm_a", {n_v}, GgmlType::F32, [=] {
                                std::vector<float> v(n_v);
                                for (size_t q = 0; q < n_v; q++) v[q] = -(1.0f + 15.0f * draw_unit(seed, tensor_id(i, T_SSM_A), q));
                                return v;
                            }, heads, {}});
            plan.push_back({b + "ssm_dt.bias", {n_v}, GgmlType::F32, [=] {
                                std::vector<float> v(n_v);
                                for (size_t q = 0; q < n_v; q++) v[q] = draw_normal(seed, tensor_id(i, T_DT_BIAS), q, WEIGHT_STD);
                                return v;
                            }, heads, {}});
            ones(b + "ssm_norm.weight", dv);
        }
    }
    const size_t align = 32;
    std::vector<GgufTensor> infos;
    size_t offset = 0;
    for (const T& t : plan) {
        GgufTensor g;
        g.name = t.name;
        g.dims = t.dims;
        g.type_id = (uint32_t)t.ty;
        g.offset = offset;
        offset = (offset + g.bytes() + align - 1) / align * align;
        infos.push_back(std::move(g));
    }
    const std::vector<uint8_t> header = gguf_write_header(config_metadata(c, n_pos), infos, align);
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f) return path + ": " + std::strerror(errno);
    bool ok = std::fwrite(header.data(), 1, header.size(), f) == header.size();
    for (size_t pi = 0; ok && pi < plan.size(); pi++) {
        const T& t = plan[pi];
        const std::vector<float> conv = t.values();
        const size_t inner = t.dims.size() > 1 ? t.dims[0] : 1, outer = conv.size() / inner;
        // undo the conversion: source[perm[new]] = converted[new], rows first, then columns
        std::vector<float> src(conv.size());
        for (size_t r = 0; r < outer; r++) {
            const size_t sr = t.rows.empty() ? r : (size_t)t.rows[r];
            for (size_t q = 0; q < inner; q++) src[sr * inner + (t.cols.empty() ? q : (size_t)t.cols[q])] = conv[r * inner + q];
        }
        std::vector<uint8_t> data(infos[pi].bytes());
        if (t.ty == GgmlType::F32) std::memcpy(data.data(), src.data(), data.size());
        else
            for (size_t q = 0; q < src.size(); q++) {
                const uint16_t b16 = f32_to_bf16(src[q]);
                std::memcpy(data.data() + 2 * q, &b16, 2);
            }
        data.resize((data.size() + align - 1) / align * align, 0);
        ok = std::fwrite(data.data(), 1, data.size(), f) == data.size();
    }
    if (std::fclose(f) != 0 || !ok) return path + ": write failed";
    return "";
}

// ---- calibration
std::vector<int32_t> calibration_ids(const std::vector<int32_t>& prefix, size_t vocab, size_t n_random) {
    std::vector<int32_t> ids = prefix;
    uint64_t state = 0x9E3779B97F4A7C15ull;
    for (size_t i = 0; i < n_random; i++) {
        state += 0x9E3779B97F4A7C15ull;   // splitmix64 (spec/prim.rs:203-211)
        uint64_t z = state;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        ids.push_back((int32_t)(z % vocab));
    }
    return ids;
}

namespace {
struct AbsMax : Observer {   // calibrate.rs:12-36; the fold itself is the backend's (host loop or one device kernel)
    size_t n_kv, hd;
    std::vector<size_t> layers;
    Buf<float> slots;
    void observe(const Ctx& ctx, const Tap& tap) override {
        if (tap.kind != Tap::AttnV) return;
        const size_t li = (size_t)(std::find(layers.begin(), layers.end(), tap.layer) - layers.begin());
        ctx.backend->absmax_heads(*tap.x, ctx.t, n_kv, hd, Buf<float>::view(slots.ptr_at(li * n_kv), n_kv));
    }
};
}  // namespace

std::string v_scales(Model& m, const int32_t* ids, size_t n, std::vector<float>& scales) {
    AbsMax obs;
    obs.n_kv = m.cfg.n_kv;
    obs.hd = m.cfg.head_dim;
    for (size_t l = 0; l < m.cfg.n_layers; l++)
        if (m.cfg.is_attention(l)) obs.layers.push_back(l);
    obs.slots = m.backend->alloc<float>(obs.layers.size() * m.cfg.n_kv);
    m.reset();
    std::string e = m.prefill(ids, n, &obs);
    if (!e.empty()) return e;
    const std::vector<float> absmax = m.backend->download(obs.slots);
    scales.clear();
    for (float a : absmax) scales.push_back(a == 0.0f ? DEFAULT_V_SCALE : a * HEADROOM / 32767.0f);
    return "";
}

bool write_scales_in_place(const Model& m, const std::vector<float>& scales, const std::string& path, std::string& err) {
    if (!m.gguf) {
        err = "the model was not loaded from a file";
        return false;
    }
    return m.gguf->set_metadata_in_place(path, V_SCALE_KEY, GgufValue::f32_array(scales), err);
}
bool write_scales_copy(const Model& m, const std::vector<float>& scales, const std::string& out, std::string& err) {
    if (!m.gguf) {
        err = "the model was not loaded from a file";
        return false;
    }
    return m.gguf->write_with_metadata(V_SCALE_KEY, GgufValue::f32_array(scales), out, err);
}

}  // namespace det
