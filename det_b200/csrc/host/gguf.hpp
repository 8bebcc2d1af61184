// The GGUF container as det reads and writes it: header, metadata key/values and the tensor table over a memory-mapped
// file (crates/det/src/gguf.rs:9-489), the hyperparameters read from its metadata (crates/det/src/config.rs:34-92), exact
// dequantization of one tensor row (crates/det/src/spec/tensor.rs:8-30, 73-104) and the finite-value check a loader
// runs first (crates/det/src/model.rs:12-44).
#pragma once
#include "synth.hpp"
#include <cstdint>
#include <memory>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace det {

// gguf.rs:9-24 — one metadata value.  `type` is the GGUF value type id (0 u8, 1 i8, 2 u16, 3 i16, 4 u32, 5 i32, 6 f32,
// 7 bool, 8 string, 9 array, 10 u64, 11 i64, 12 f64); integers and bool live in `u` (two's complement for the signed
// ones), floats in `f`, strings in `s`, array elements in `arr`.
struct GgufValue {
    uint32_t type = 4;
    uint64_t u = 0;
    double f = 0.0;
    std::string s;
    std::vector<GgufValue> arr;

    static GgufValue u32(uint32_t v) { GgufValue x; x.type = 4; x.u = v; return x; }
    static GgufValue u64(uint64_t v) { GgufValue x; x.type = 10; x.u = v; return x; }
    static GgufValue f32(float v) { GgufValue x; x.type = 6; x.f = v; return x; }
    static GgufValue str(std::string v) { GgufValue x; x.type = 8; x.s = std::move(v); return x; }
    static GgufValue array(std::vector<GgufValue> v) { GgufValue x; x.type = 9; x.arr = std::move(v); return x; }
    static GgufValue f32_array(const std::vector<float>& v);

    bool as_u64(uint64_t& out) const;   // gguf.rs:27-39: unsigned types, and signed ones when non-negative
    bool as_f32(float& out) const;      // gguf.rs:40-46: f32, f64 (rounded), or as_u64 converted
    bool operator==(const GgufValue& o) const;
};

// gguf.rs:79-146 — the tensor types det accepts.
enum class GgmlType : uint32_t { F32 = 0, F16 = 1, BF16 = 30, Det4 = 0xDE04, Det6 = 0xDE06, Det8 = 0xDE08 };
bool ggml_type_from_id(uint32_t id, GgmlType& out);
GgmlType ggml_det_type(int bits);
int ggml_type_bits(GgmlType t);                  // 4 / 6 / 8 for det linears, 0 for float types
size_t ggml_row_bytes(GgmlType t, size_t k);
std::string ggml_type_name(uint32_t id);         // gguf.rs:148-162 (names of foreign ggml types for messages)

// gguf.rs:164-190
struct GgufTensor {
    std::string name;
    std::vector<size_t> dims;   // ggml order: dims[0] is the fastest-varying (the row length of a matrix)
    uint32_t type_id = 0;
    size_t offset = 0;          // from the start of the data section
    bool type(GgmlType& t) const { return ggml_type_from_id(type_id, t); }
    size_t n_elems() const;
    size_t bytes() const;       // throws on an unsupported type
};

using GgufKv = std::vector<std::pair<std::string, GgufValue>>;

// gguf.rs:405-451
std::vector<uint8_t> gguf_write_header(const GgufKv& kv, const std::vector<GgufTensor>& tensors, size_t alignment);

class Gguf {
  public:
    // gguf.rs:261-359.  Returns null and a message on an unreadable, truncated or unsupported file.
    static std::shared_ptr<Gguf> open(const std::string& path, std::string& err);
    ~Gguf();
    Gguf(const Gguf&) = delete;
    Gguf& operator=(const Gguf&) = delete;

    const GgufValue* get(const std::string& key) const;
    bool u64(const std::string& key, uint64_t& out) const;
    bool f32(const std::string& key, float& out) const;
    const std::string* str(const std::string& key) const;
    const GgufTensor* tensor(const std::string& name) const;
    const uint8_t* data(const GgufTensor& t) const { return map_ + data_start + t.offset; }
    const uint8_t* file_bytes() const { return map_; }
    size_t file_size() const { return size_; }

    // gguf.rs:464-480: rewrites the header in the file itself when the new header fits before the tensor data (true);
    // otherwise nothing is written (false).  `det convert` reserves the room for det.v_scale.
    bool set_metadata_in_place(const std::string& path, const std::string& key, const GgufValue& v, std::string& err) const;
    // gguf.rs:482-488: a copy of the file with `key` set (replacing an existing key).
    bool write_with_metadata(const std::string& key, const GgufValue& v, const std::string& out, std::string& err) const;

    GgufKv kv;
    std::vector<GgufTensor> tensors;
    size_t data_start = 0, alignment = 32;

  private:
    Gguf() = default;
    std::vector<uint8_t> header_with(const std::string& key, const GgufValue& v) const;
    const uint8_t* map_ = nullptr;
    size_t size_ = 0;
    std::unordered_map<std::string, size_t> index_, tindex_;
};

// spec/tensor.rs:8-30
float f16_to_f32(uint16_t h);
// spec/tensor.rs:73-104: `k` elements of one row; float types exactly, det rows as (c * f32(m[g])) * f32(q).
void dequant_row(GgmlType t, const uint8_t* row, size_t k, float* out);
// Unpacks the codes of one det row (the inverse of pack_codes).
void unpack_codes(const uint8_t* packed, size_t k, int bits, int8_t* out);

// config.rs:34-92.  Returns "" and fills `c`, or the reference's message.
std::string config_from_gguf(const Gguf& g, Config& c);
// model.rs:12-44.  "" when every float tensor and every det row scale is finite.
std::string check_finite(const Gguf& g);

constexpr const char* V_SCALE_KEY = "det.v_scale";   // model.rs:48

// The metadata a converted qwen35 file carries for `c` (the keys config_from_gguf reads, general.alignment excluded).
GgufKv config_metadata(const Config& c, size_t context_length);

// Writes the seeded synthetic model of synth.hpp as the det GGUF `det convert` would produce for it (tensor order,
// types, rope tables and the reserved det.v_scale array of convert.rs:223-402): bf16 embedding table, W8 tied head,
// det rows for every linear, fp32 vectors.  `n_pos` rope positions.  Returns "" on success.
std::string write_synthetic_gguf(const Config& c, uint64_t seed, const std::string& path, size_t n_pos);

}  // namespace det
