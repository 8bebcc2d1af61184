// GGUF container, hyperparameters, row dequantization, the loader's finite check, and the writer of a synthetic det
// file.  See gguf.hpp for the reference map.
#include "gguf.hpp"
#include "backend.hpp"
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <cerrno>
#include <fcntl.h>
#include <functional>
#include <stdexcept>
#include <sys/mman.h>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>

namespace det {

// ---- values
GgufValue GgufValue::f32_array(const std::vector<float>& v) {
    std::vector<GgufValue> a;
    a.reserve(v.size());
    for (float x : v) a.push_back(GgufValue::f32(x));
    return GgufValue::array(std::move(a));
}
bool GgufValue::as_u64(uint64_t& out) const {
    switch (type) {
        case 0: case 2: case 4: case 10:
            out = u;
            return true;
        case 1: case 3: case 5: case 11:
            if ((int64_t)u < 0) return false;
            out = u;
            return true;
        default:
            return false;
    }
}
bool GgufValue::as_f32(float& out) const {
    if (type == 6 || type == 12) {
        out = (float)f;
        return true;
    }
    uint64_t v;
    if (!as_u64(v)) return false;
    out = (float)v;
    return true;
}
bool GgufValue::operator==(const GgufValue& o) const {
    if (type != o.type) return false;
    if (type == 8) return s == o.s;
    if (type == 9) return arr == o.arr;
    if (type == 6 || type == 12) return std::memcmp(&f, &o.f, sizeof f) == 0;
    return u == o.u;
}

// ---- tensor types
bool ggml_type_from_id(uint32_t id, GgmlType& out) {
    switch (id) {
        case 0: out = GgmlType::F32; return true;
        case 1: out = GgmlType::F16; return true;
        case 30: out = GgmlType::BF16; return true;
        case 0xDE04: out = GgmlType::Det4; return true;
        case 0xDE06: out = GgmlType::Det6; return true;
        case 0xDE08: out = GgmlType::Det8; return true;
        default: return false;
    }
}
GgmlType ggml_det_type(int bits) {
    if (bits == 4) return GgmlType::Det4;
    if (bits == 6) return GgmlType::Det6;
    if (bits == 8) return GgmlType::Det8;
    throw std::runtime_error("unsupported bit width " + std::to_string(bits));
}
int ggml_type_bits(GgmlType t) {
    return t == GgmlType::Det4 ? 4 : (t == GgmlType::Det6 ? 6 : (t == GgmlType::Det8 ? 8 : 0));
}
size_t ggml_row_bytes(GgmlType t, size_t k) {
    if (t == GgmlType::F32) return 4 * k;
    if (t == GgmlType::F16 || t == GgmlType::BF16) return 2 * k;
    if (k % 128) throw std::runtime_error("K = " + std::to_string(k) + " is not a multiple of 128");
    return det_row_bytes(ggml_type_bits(t), k);
}
std::string ggml_type_name(uint32_t id) {
    GgmlType t;
    if (ggml_type_from_id(id, t)) {
        switch (t) {
            case GgmlType::F32: return "F32";
            case GgmlType::F16: return "F16";
            case GgmlType::BF16: return "BF16";
            case GgmlType::Det4: return "DET_W4";
            case GgmlType::Det6: return "DET_W6";
            case GgmlType::Det8: return "DET_W8";
        }
    }
    static const char* names[31] = {"F32", "F16", "Q4_0", "Q4_1", "?4", "?5", "Q5_0", "Q5_1", "Q8_0", "Q8_1", "Q2_K",
                                    "Q3_K", "Q4_K", "Q5_K", "Q6_K", "Q8_K", "IQ2_XXS", "IQ2_XS", "IQ3_XXS", "IQ1_S", "IQ4_NL",
                                    "IQ3_S", "IQ2_S", "IQ4_XS", "I8", "I16", "I32", "I64", "F64", "IQ1_M", "BF16"};
    return id < 31 ? names[id] : "type" + std::to_string(id);
}
size_t GgufTensor::n_elems() const {
    size_t n = 1;
    for (size_t d : dims) n *= d;
    return n;
}
size_t GgufTensor::bytes() const {
    GgmlType t;
    if (!type(t)) throw std::runtime_error("tensor " + name + " has unsupported type " + ggml_type_name(type_id));
    size_t outer = 1;
    for (size_t i = 1; i < dims.size(); i++) outer *= dims[i];
    return ggml_row_bytes(t, dims[0]) * outer;
}

// ---- header writer
namespace {
void put(std::vector<uint8_t>& o, const void* p, size_t n) {
    const uint8_t* b = static_cast<const uint8_t*>(p);
    o.insert(o.end(), b, b + n);
}
void put_u32(std::vector<uint8_t>& o, uint32_t v) { put(o, &v, 4); }
void put_u64(std::vector<uint8_t>& o, uint64_t v) { put(o, &v, 8); }
void put_string(std::vector<uint8_t>& o, const std::string& s) {
    put_u64(o, s.size());
    put(o, s.data(), s.size());
}
void put_value(std::vector<uint8_t>& o, const GgufValue& v) {
    switch (v.type) {
        case 0: case 1: case 7: { uint8_t x = (uint8_t)v.u; put(o, &x, 1); break; }
        case 2: case 3: { uint16_t x = (uint16_t)v.u; put(o, &x, 2); break; }
        case 4: case 5: put_u32(o, (uint32_t)v.u); break;
        case 6: { float x = (float)v.f; put(o, &x, 4); break; }
        case 8: put_string(o, v.s); break;
        case 9: {
            const uint32_t et = v.arr.empty() ? 0u : v.arr[0].type;
            put_u32(o, et);
            put_u64(o, v.arr.size());
            for (const GgufValue& e : v.arr) {
                if (e.type != et) throw std::runtime_error("mixed array element types");
                put_value(o, e);
            }
            break;
        }
        case 10: case 11: put_u64(o, v.u); break;
        case 12: put(o, &v.f, 8); break;
        default: throw std::runtime_error("unknown GGUF value type " + std::to_string(v.type));
    }
}
}  // namespace

std::vector<uint8_t> gguf_write_header(const GgufKv& kv, const std::vector<GgufTensor>& tensors, size_t alignment) {
    std::vector<uint8_t> o;
    put(o, "GGUF", 4);
    put_u32(o, 3);
    put_u64(o, tensors.size());
    put_u64(o, kv.size());
    for (const auto& e : kv) {
        put_string(o, e.first);
        put_u32(o, e.second.type);
        put_value(o, e.second);
    }
    for (const GgufTensor& t : tensors) {
        put_string(o, t.name);
        put_u32(o, (uint32_t)t.dims.size());
        for (size_t d : t.dims) put_u64(o, d);
        put_u32(o, t.type_id);
        put_u64(o, t.offset);
    }
    o.resize((o.size() + alignment - 1) / alignment * alignment, 0);
    return o;
}

// ---- reader
namespace {
struct Cursor {
    const uint8_t* b;
    size_t len, pos = 0;
    const uint8_t* take(size_t n) {
        if (n > len - pos) throw std::runtime_error("truncated GGUF header");
        const uint8_t* p = b + pos;
        pos += n;
        return p;
    }
    uint32_t u32() { uint32_t v; std::memcpy(&v, take(4), 4); return v; }
    uint64_t u64() { uint64_t v; std::memcpy(&v, take(8), 8); return v; }
    std::string string() {
        const uint64_t n = u64();
        if (n > len - pos) throw std::runtime_error("truncated GGUF header");
        const uint8_t* p = take((size_t)n);
        return std::string(reinterpret_cast<const char*>(p), (size_t)n);
    }
    GgufValue value(uint32_t ty) {
        GgufValue v;
        v.type = ty;
        switch (ty) {
            case 0: v.u = take(1)[0]; break;
            case 1: v.u = (uint64_t)(int64_t)(int8_t)take(1)[0]; break;
            case 2: { uint16_t x; std::memcpy(&x, take(2), 2); v.u = x; break; }
            case 3: { int16_t x; std::memcpy(&x, take(2), 2); v.u = (uint64_t)(int64_t)x; break; }
            case 4: v.u = u32(); break;
            case 5: v.u = (uint64_t)(int64_t)(int32_t)u32(); break;
            case 6: { float x; std::memcpy(&x, take(4), 4); v.f = x; break; }
            case 7: v.u = take(1)[0] != 0; break;
            case 8: v.s = string(); break;
            case 9: {
                const uint32_t et = u32();
                const uint64_t n = u64();
                v.arr.reserve((size_t)std::min<uint64_t>(n, 1u << 20));
                for (uint64_t i = 0; i < n; i++) v.arr.push_back(value(et));
                break;
            }
            case 10: v.u = u64(); break;
            case 11: v.u = u64(); break;
            case 12: { uint64_t x = u64(); std::memcpy(&v.f, &x, 8); break; }
            default: throw std::runtime_error("unknown GGUF value type " + std::to_string(ty));
        }
        return v;
    }
};
std::string dims_text(const std::vector<size_t>& d) {
    std::string s = "[";
    for (size_t i = 0; i < d.size(); i++) s += (i ? ", " : "") + std::to_string(d[i]);
    return s + "]";
}
}  // namespace

Gguf::~Gguf() {
    if (map_) munmap(const_cast<uint8_t*>(map_), size_);
}

std::shared_ptr<Gguf> Gguf::open(const std::string& path, std::string& err) {
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) {
        err = path + ": " + std::strerror(errno);
        return nullptr;
    }
    struct stat sb;
    if (fstat(fd, &sb) != 0 || sb.st_size == 0) {
        err = path + ": " + (sb.st_size == 0 ? "truncated GGUF header" : std::strerror(errno));
        ::close(fd);
        return nullptr;
    }
    void* p = mmap(nullptr, (size_t)sb.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (p == MAP_FAILED) {
        err = path + ": " + std::strerror(errno);
        return nullptr;
    }
    std::shared_ptr<Gguf> g(new Gguf());
    g->map_ = static_cast<const uint8_t*>(p);
    g->size_ = (size_t)sb.st_size;
    try {
        Cursor c{g->map_, g->size_};
        if (std::memcmp(c.take(4), "GGUF", 4) != 0) throw std::runtime_error("not a GGUF file");
        const uint32_t version = c.u32();
        if (version != 3 && version != 2) throw std::runtime_error("unsupported GGUF version " + std::to_string(version));
        const uint64_t n_tensors = c.u64(), n_kv = c.u64();
        for (uint64_t i = 0; i < n_kv; i++) {
            std::string key = c.string();
            const uint32_t ty = c.u32();
            g->kv.emplace_back(std::move(key), c.value(ty));
        }
        for (uint64_t i = 0; i < n_tensors; i++) {
            GgufTensor t;
            t.name = c.string();
            const uint32_t nd = c.u32();
            for (uint32_t d = 0; d < nd; d++) t.dims.push_back((size_t)c.u64());
            t.type_id = c.u32();
            t.offset = (size_t)c.u64();
            g->tensors.push_back(std::move(t));
        }
        for (size_t i = 0; i < g->kv.size(); i++) g->index_[g->kv[i].first] = i;
        for (size_t i = 0; i < g->tensors.size(); i++) g->tindex_[g->tensors[i].name] = i;
        uint64_t al = 32;
        for (const auto& e : g->kv)
            if (e.first == "general.alignment") {   // the first one counts (gguf.rs:314-318)
                if (!e.second.as_u64(al)) al = 32;
                break;
            }
        if (al == 0) throw std::runtime_error("general.alignment is zero");
        g->alignment = (size_t)al;
        g->data_start = (c.pos + g->alignment - 1) / g->alignment * g->alignment;
        for (const GgufTensor& t : g->tensors) {
            GgmlType ty;
            const bool known = t.type(ty);
            const bool is_float = known && ggml_type_bits(ty) == 0;
            if (!known || t.dims.empty() || !(t.dims[0] % 32 == 0 || is_float) || (!is_float && t.dims[0] % 128 != 0))
                throw std::runtime_error("tensor " + t.name + " has unsupported type " + ggml_type_name(t.type_id) +
                                         " or shape " + dims_text(t.dims));
            const size_t bytes = t.bytes();
            if (t.dims.size() > 2 || g->data_start + t.offset + bytes > g->size_ || t.offset > g->size_)
                throw std::runtime_error("tensor " + t.name + " (" + dims_text(t.dims) + " at " + std::to_string(t.offset) +
                                         ") does not fit the file");
        }
    } catch (const std::exception& ex) {
        err = path + ": " + ex.what();
        return nullptr;
    }
    return g;
}

const GgufValue* Gguf::get(const std::string& key) const {
    auto it = index_.find(key);
    return it == index_.end() ? nullptr : &kv[it->second].second;
}
bool Gguf::u64(const std::string& key, uint64_t& out) const {
    const GgufValue* v = get(key);
    return v && v->as_u64(out);
}
bool Gguf::f32(const std::string& key, float& out) const {
    const GgufValue* v = get(key);
    return v && v->as_f32(out);
}
const std::string* Gguf::str(const std::string& key) const {
    const GgufValue* v = get(key);
    return v && v->type == 8 ? &v->s : nullptr;
}
const GgufTensor* Gguf::tensor(const std::string& name) const {
    auto it = tindex_.find(name);
    return it == tindex_.end() ? nullptr : &tensors[it->second];
}

std::vector<uint8_t> Gguf::header_with(const std::string& key, const GgufValue& v) const {
    GgufKv nkv;
    for (const auto& e : kv)
        if (e.first != key) nkv.push_back(e);
    nkv.emplace_back(key, v);
    return gguf_write_header(nkv, tensors, alignment);
}
bool Gguf::set_metadata_in_place(const std::string& path, const std::string& key, const GgufValue& v, std::string& err) const {
    const std::vector<uint8_t> header = header_with(key, v);
    if (header.size() > data_start) return false;
    FILE* f = std::fopen(path.c_str(), "r+b");
    if (!f) {
        err = path + ": " + std::strerror(errno);
        return false;
    }
    const std::vector<uint8_t> pad(data_start - header.size(), 0);
    const bool ok = std::fwrite(header.data(), 1, header.size(), f) == header.size() &&
                    std::fwrite(pad.data(), 1, pad.size(), f) == pad.size();
    if (std::fclose(f) != 0 || !ok) {
        err = path + ": write failed";
        return false;
    }
    return true;
}
bool Gguf::write_with_metadata(const std::string& key, const GgufValue& v, const std::string& out, std::string& err) const {
    const std::vector<uint8_t> header = header_with(key, v);
    FILE* f = std::fopen(out.c_str(), "wb");
    if (!f) {
        err = out + ": " + std::strerror(errno);
        return false;
    }
    bool ok = std::fwrite(header.data(), 1, header.size(), f) == header.size();
    for (size_t off = data_start; ok && off < size_; off += (size_t)1 << 26) {
        const size_t n = std::min<size_t>((size_t)1 << 26, size_ - off);
        ok = std::fwrite(map_ + off, 1, n, f) == n;
    }
    if (std::fclose(f) != 0 || !ok) {
        err = out + ": write failed";
        return false;
    }
    return true;
}

// ---- rows
float f16_to_f32(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1Fu;
    const uint32_t mant = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (mant == 0) bits = sign;
        else {
            uint32_t m = mant;
            int e = 127 - 15 + 1;
            while (!(m & 0x400u)) {
                m <<= 1;
                e--;
            }
            bits = sign | ((uint32_t)e << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (mant << 13);
    else bits = sign | ((exp + 127 - 15) << 23) | (mant << 13);
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}
void unpack_codes(const uint8_t* p, size_t k, int bits, int8_t* out) {
    for (size_t blk = 0; blk < k / 32; blk++) {
        int8_t* q = out + blk * 32;
        if (bits == 8) {
            for (int i = 0; i < 32; i++) q[i] = (int8_t)p[i];
            p += 32;
        } else if (bits == 4) {
            for (int i = 0; i < 16; i++) {
                q[i] = (int8_t)((p[i] & 0xF) - 8);
                q[i + 16] = (int8_t)((p[i] >> 4) - 8);
            }
            p += 16;
        } else {
            for (int i = 0; i < 16; i++) {
                q[i] = (int8_t)(p[i] & 0xF);
                q[i + 16] = (int8_t)(p[i] >> 4);
            }
            for (int i = 0; i < 8; i++) {
                const uint8_t hi = p[16 + i];
                q[i] = (int8_t)((q[i] | ((hi & 3) << 4)) - 32);
                q[i + 8] = (int8_t)((q[i + 8] | (((hi >> 2) & 3) << 4)) - 32);
                q[i + 16] = (int8_t)((q[i + 16] | (((hi >> 4) & 3) << 4)) - 32);
                q[i + 24] = (int8_t)((q[i + 24] | (((hi >> 6) & 3) << 4)) - 32);
            }
            p += 24;
        }
    }
}
void dequant_row(GgmlType t, const uint8_t* row, size_t k, float* out) {
    switch (t) {
        case GgmlType::F32:
            std::memcpy(out, row, 4 * k);
            break;
        case GgmlType::F16:
            for (size_t i = 0; i < k; i++) {
                uint16_t h;
                std::memcpy(&h, row + 2 * i, 2);
                out[i] = f16_to_f32(h);
            }
            break;
        case GgmlType::BF16:
            for (size_t i = 0; i < k; i++) {
                uint16_t h;
                std::memcpy(&h, row + 2 * i, 2);
                out[i] = bf16_to_f32(h);
            }
            break;
        default: {
            const int bits = ggml_type_bits(t);
            const size_t nc = k / 32 * (bits == 8 ? 32 : (bits == 6 ? 24 : 16));
            float c;
            std::memcpy(&c, row + nc, 4);
            std::vector<int8_t> q(k);
            unpack_codes(row, k, bits, q.data());
            for (size_t i = 0; i < k; i++) {
                uint16_t m;
                std::memcpy(&m, row + nc + 4 + 2 * (i / 128), 2);
                out[i] = (c * (float)m) * (float)q[i];
            }
        }
    }
}

// ---- config
std::string config_from_gguf(const Gguf& g, Config& c) {
    const std::string* arch = g.str("general.architecture");
    if (!arch) return "no general.architecture";
    if (*arch != "qwen35") return "architecture " + *arch + " is not supported (qwen35 only)";
    std::string missing;
    auto key = [&](const char* s) { return *arch + "." + s; };
    auto u = [&](const char* s) -> size_t {
        uint64_t v = 0;
        if (!g.u64(key(s), v) && missing.empty()) missing = "missing " + key(s);
        return (size_t)v;
    };
    uint64_t nextn = 0;
    g.u64(key("nextn_predict_layers"), nextn);
    const size_t blocks = u("block_count");
    const size_t interval = u("full_attention_interval");
    if (!missing.empty()) return missing;
    if (interval == 0) return key("full_attention_interval") + " is zero";
    if (nextn > blocks) return key("nextn_predict_layers") + " exceeds the block count";
    c = Config();
    c.name = *arch;
    c.n_layers = blocks - (size_t)nextn;
    c.full_attention_interval = interval;
    if (const GgufTensor* t = g.tensor("token_embd.weight")) {
        if (t->dims.size() < 2) return "token_embd.weight: not a float [hidden][vocab] table";
        c.vocab = t->dims[1];
    } else {
        const GgufValue* toks = g.get("tokenizer.ggml.tokens");
        if (!toks || toks->type != 9) return "no token_embd.weight and no tokenizer tokens";
        c.vocab = toks->arr.size();
    }
    c.gdn_dk = u("ssm.state_size");
    c.gdn_v_heads = u("ssm.time_step_rank");
    c.hidden = u("embedding_length");
    if (!missing.empty()) return missing;
    if (!g.f32(key("attention.layer_norm_rms_epsilon"), c.eps)) return "missing eps";
    c.n_heads = u("attention.head_count");
    c.n_kv = u("attention.head_count_kv");
    c.head_dim = u("attention.key_length");
    c.rot_dim = u("rope.dimension_count");
    if (!missing.empty()) return missing;
    float theta;
    if (!g.f32(key("rope.freq_base"), theta)) return "missing rope.freq_base";
    c.rope_theta = (double)theta;
    c.intermediate = u("feed_forward_length");
    c.gdn_k_heads = u("ssm.group_count");
    const size_t inner = u("ssm.inner_size");
    c.conv_k = u("ssm.conv_kernel");
    if (!missing.empty()) return missing;
    if (c.gdn_v_heads == 0) return key("ssm.time_step_rank") + " is zero";
    c.gdn_dv = inner / c.gdn_v_heads;
    return "";
}

GgufKv config_metadata(const Config& c, size_t context_length) {
    const std::string a = "qwen35";
    GgufKv kv;
    kv.emplace_back("general.architecture", GgufValue::str(a));
    kv.emplace_back("general.name", GgufValue::str("det synthetic " + c.name));
    auto u = [&](const char* k, size_t v) { kv.emplace_back(a + "." + k, GgufValue::u32((uint32_t)v)); };
    u("block_count", c.n_layers);
    u("context_length", context_length);
    u("full_attention_interval", c.full_attention_interval);
    u("embedding_length", c.hidden);
    u("feed_forward_length", c.intermediate);
    u("attention.head_count", c.n_heads);
    u("attention.head_count_kv", c.n_kv);
    u("attention.key_length", c.head_dim);
    u("attention.value_length", c.head_dim);
    kv.emplace_back(a + ".attention.layer_norm_rms_epsilon", GgufValue::f32(c.eps));
    u("rope.dimension_count", c.rot_dim);
    kv.emplace_back(a + ".rope.freq_base", GgufValue::f32((float)c.rope_theta));
    u("ssm.conv_kernel", c.conv_k);
    u("ssm.state_size", c.gdn_dk);
    u("ssm.group_count", c.gdn_k_heads);
    u("ssm.time_step_rank", c.gdn_v_heads);
    u("ssm.inner_size", c.gdn_v_heads * c.gdn_dv);
    return kv;
}

// ---- finite check
std::string check_finite(const Gguf& g) {
    for (const GgufTensor& t : g.tensors) {
        GgmlType ty;
        if (!t.type(ty)) return t.name + ": unsupported type";
        const uint8_t* data = g.data(t);
        const size_t bytes = t.bytes();
        const unsigned nt = bytes >= ((size_t)8 << 20) ? std::max(1u, std::min(std::thread::hardware_concurrency(), 16u)) : 1u;
        std::atomic<bool> bad{false};
        auto scan = [&](size_t lo, size_t hi) {   // [lo, hi) in units of elements (float types) or rows (det types)
            bool b = false;
            if (ty == GgmlType::F32) {
                for (size_t i = lo; i < hi && !b; i++) b = (data[4 * i + 3] & 0x7F) == 0x7F && (data[4 * i + 2] & 0x80);
            } else if (ty == GgmlType::F16) {
                for (size_t i = lo; i < hi && !b; i++) b = (data[2 * i + 1] & 0x7C) == 0x7C;
            } else if (ty == GgmlType::BF16) {
                for (size_t i = lo; i < hi && !b; i++) b = (data[2 * i + 1] & 0x7F) == 0x7F && (data[2 * i] & 0x80);
            } else {
                const size_t k = t.dims[0], rb = ggml_row_bytes(ty, k), nc = rb - 4 - k / 128 * 2;
                for (size_t r = lo; r < hi && !b; r++) {
                    float c;
                    std::memcpy(&c, data + r * rb + nc, 4);
                    b = !std::isfinite(c);
                }
            }
            if (b) bad = true;
        };
        const size_t units = ggml_type_bits(ty) ? bytes / ggml_row_bytes(ty, t.dims[0]) : t.n_elems();
        if (nt == 1) scan(0, units);
        else {
            std::vector<std::thread> pool;
            for (unsigned w = 0; w < nt; w++) pool.emplace_back(scan, units * w / nt, units * (w + 1) / nt);
            for (auto& th : pool) th.join();
        }
        if (bad) return t.name + ": non-finite value";
    }
    return "";
}

// ---- synthetic det file
namespace {
struct OutTensor {
    std::string name;
    std::vector<size_t> dims;
    GgmlType type;
    std::function<void(std::vector<uint8_t>&)> gen;   // appends the tensor's bytes
};
void put_f32s(std::vector<uint8_t>& o, const std::vector<float>& v) { put(o, v.data(), v.size() * 4); }
}  // namespace

std::string write_synthetic_gguf(const Config& c, uint64_t seed, const std::string& path, size_t n_pos) {
    const size_t h = c.hidden, inter = c.intermediate, hd = c.head_dim;
    const size_t n_v = c.gdn_v_heads, dv = c.gdn_dv, conv_dim = c.conv_dim();
    const int wb = c.bits_default;
    std::vector<OutTensor> plan;
    auto ones = [&](const std::string& name, size_t n) {
        plan.push_back({name, {n}, GgmlType::F32, [n](std::vector<uint8_t>& o) { put_f32s(o, std::vector<float>(n, 1.0f)); }});
    };
    auto lin = [&](const std::string& name, size_t layer, TensorKind kind, size_t n, size_t k, int bits) {
        plan.push_back({name, {k, n}, ggml_det_type(bits), [=](std::vector<uint8_t>& o) {
                            const std::vector<uint8_t> rows = synth_det_rows_any(seed, tensor_id(layer, kind), 0, n, k, bits);
                            o.insert(o.end(), rows.begin(), rows.end());
                        }});
    };
    std::vector<float> rc, rs;
    rope_tables(c, n_pos, rc, rs);
    // the order of convert.rs:223-301
    plan.push_back({"token_embd.weight", {h, c.vocab}, GgmlType::BF16, [&](std::vector<uint8_t>& o) {
                        const uint64_t tid = tensor_id(GLOBAL_LAYER, T_EMBED);
                        const size_t base = o.size(), count = c.vocab * h;
                        o.resize(base + 2 * count);
                        uint16_t* dst = reinterpret_cast<uint16_t*>(o.data() + base);
                        const unsigned nt = std::max(1u, std::min(std::thread::hardware_concurrency(), 16u));
                        std::vector<std::thread> pool;
                        for (unsigned w = 0; w < nt; w++)
                            pool.emplace_back([&, w] {
                                for (size_t i = count * w / nt; i < count * (w + 1) / nt; i++)
                                    dst[i] = f32_to_bf16(draw_normal(seed, tid, i, WEIGHT_STD));
                            });
                        for (auto& t : pool) t.join();
                    }});
    ones("output_norm.weight", h);
    lin("output.weight", GLOBAL_LAYER, T_EMBED, c.vocab, h, 8);
    plan.push_back({"rope_cos", {c.rot_dim / 2, n_pos}, GgmlType::F32, [&](std::vector<uint8_t>& o) { put_f32s(o, rc); }});
    plan.push_back({"rope_sin", {c.rot_dim / 2, n_pos}, GgmlType::F32, [&](std::vector<uint8_t>& o) { put_f32s(o, rs); }});
    for (size_t i = 0; i < c.n_layers; i++) {
        const std::string b = "blk." + std::to_string(i) + ".";
        ones(b + "attn_norm.weight", h);
        ones(b + "post_attention_norm.weight", h);
        lin(b + "ffn_gate.weight", i, T_FFN_GATE, inter, h, wb);
        lin(b + "ffn_up.weight", i, T_FFN_UP, inter, h, wb);
        lin(b + "ffn_down.weight", i, T_FFN_DOWN, h, inter, wb);
        if (c.is_attention(i)) {
            lin(b + "attn_q.weight", i, T_ATTN_Q, c.n_heads * 2 * hd, h, wb);
            lin(b + "attn_k.weight", i, T_ATTN_K, c.n_kv * hd, h, wb);
            lin(b + "attn_v.weight", i, T_ATTN_V, c.n_kv * hd, h, wb);
            lin(b + "attn_output.weight", i, T_ATTN_OUT, h, c.n_heads * hd, wb);
            ones(b + "attn_q_norm.weight", hd);
            ones(b + "attn_k_norm.weight", hd);
        } else {
            lin(b + "attn_qkv.weight", i, T_GDN_QKV, conv_dim, h, wb);
            lin(b + "attn_gate.weight", i, T_GDN_GATE, n_v * dv, h, wb);
            lin(b + "ssm_alpha.weight", i, T_GDN_ALPHA, n_v, h, 8);
            lin(b + "ssm_beta.weight", i, T_GDN_BETA, n_v, h, 8);
            lin(b + "ssm_out.weight", i, T_GDN_OUT, h, n_v * dv, wb);
            plan.push_back({b + "ssm_conv1d.weight", {c.conv_k, conv_dim}, GgmlType::F32, [=](std::vector<uint8_t>& o) {
                                std::vector<float> v(conv_dim * c.conv_k);
                                for (size_t q = 0; q < v.size(); q++) v[q] = draw_normal(seed, tensor_id(i, T_CONV), q, WEIGHT_STD);
                                put_f32s(o, v);
                            }});
            plan.push_back({b + "ssm_a", {n_v}, GgmlType::F32, [=](std::vector<uint8_t>& o) {
                                std::vector<float> v(n_v);   // the file stores the negative decay rate (model.rs:281-293)
                                for (size_t q = 0; q < n_v; q++) v[q] = -(1.0f + 15.0f * draw_unit(seed, tensor_id(i, T_SSM_A), q));
                                put_f32s(o, v);
                            }});
            plan.push_back({b + "ssm_dt.bias", {n_v}, GgmlType::F32, [=](std::vector<uint8_t>& o) {
                                std::vector<float> v(n_v);
                                for (size_t q = 0; q < n_v; q++) v[q] = draw_normal(seed, tensor_id(i, T_DT_BIAS), q, WEIGHT_STD);
                                put_f32s(o, v);
                            }});
            ones(b + "ssm_norm.weight", dv);
        }
    }
    const size_t align = 32;
    std::vector<GgufTensor> infos;
    size_t offset = 0;
    for (const OutTensor& o : plan) {
        GgufTensor t;
        t.name = o.name;
        t.dims = o.dims;
        t.type_id = (uint32_t)o.type;
        t.offset = offset;
        offset = (offset + t.bytes() + align - 1) / align * align;
        infos.push_back(std::move(t));
    }
    GgufKv kv = config_metadata(c, n_pos);
    kv.emplace_back(V_SCALE_KEY, GgufValue::f32_array(std::vector<float>(c.n_attention_layers() * c.n_kv, 1.0f / 1024.0f)));
    const std::vector<uint8_t> header = gguf_write_header(kv, infos, align);
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f) return path + ": " + std::strerror(errno);
    bool ok = std::fwrite(header.data(), 1, header.size(), f) == header.size();
    size_t written = 0;
    for (size_t i = 0; ok && i < plan.size(); i++) {
        std::vector<uint8_t> data;
        plan[i].gen(data);
        if (written != infos[i].offset || data.size() != infos[i].bytes()) {
            std::fclose(f);
            return plan[i].name + ": size or offset mismatch";
        }
        data.resize((data.size() + align - 1) / align * align, 0);
        ok = std::fwrite(data.data(), 1, data.size(), f) == data.size();
        written += data.size();
    }
    if (std::fclose(f) != 0 || !ok) return path + ": write failed";
    return "";
}

}  // namespace det
