// Hyperparameters (crates/det/src/config.rs:9-32) and the seeded synthetic models the benchmarks and end-to-end
// parity tests run on.  There is no checkpoint in reach, so every tensor is a pure function of (seed, tensor id, element
// index) that host code and a device kernel evaluate identically:
//   * an approximately normal draw: the sum of the four 16-bit fields of one splitmix64 output, centred and scaled to
//     the requested standard deviation with one fp32 multiply, then rounded to bf16 (RNE).  No libm call is involved,
//     which is what makes the host and device twins bit-identical;
//   * linears go through the reference quantizer (crates/det/src/quantize.rs:33-85, restated in synth.cpp) into det
//     rows; `output.weight` is the W8 quantization of the embedding table (tied head, convert.rs:218-235).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace det {

struct Config {
    std::string name;
    size_t hidden = 0, n_layers = 0, full_attention_interval = 4, vocab = 0;
    float eps = 1e-6f;
    size_t n_heads = 0, n_kv = 0, head_dim = 0, rot_dim = 64;
    double rope_theta = 1e7;
    size_t intermediate = 0;
    size_t gdn_k_heads = 0, gdn_v_heads = 0, gdn_dk = 128, gdn_dv = 128, conv_k = 4;
    int bits_default = 6;   // width preset: W6, with W8 for the output head and the GDN a/b projections
    bool is_attention(size_t layer) const { return (layer + 1) % full_attention_interval == 0; }   // config.rs:94-96
    size_t n_attention_layers() const { return n_layers / full_attention_interval; }
    size_t conv_dim() const { return 2 * gdn_k_heads * gdn_dk + gdn_v_heads * gdn_dv; }             // config.rs:103-105
};

// The three model shapes of the benchmark configurations (tiny, 4B, 27B).  `layers` overrides the depth when non-zero (bounded CPU-baseline samples).
Config config_tiny();
Config config_4b();
Config config_27b();
Config config_by_name(const std::string& name, size_t layers = 0);

// ---- tensor ids of the synthetic model: layer * 32 + kind (global tensors use layer = 0xFFFF)
enum TensorKind : uint64_t {
    T_ATTN_Q = 1, T_ATTN_K, T_ATTN_V, T_ATTN_OUT, T_GDN_QKV, T_GDN_GATE, T_GDN_ALPHA, T_GDN_BETA, T_GDN_OUT,
    T_FFN_GATE, T_FFN_UP, T_FFN_DOWN, T_CONV, T_DT_BIAS, T_SSM_A, T_EMBED
};
inline uint64_t tensor_id(size_t layer, TensorKind kind) { return (uint64_t)layer * 32 + (uint64_t)kind; }
constexpr size_t GLOBAL_LAYER = 0xFFFF;
constexpr float WEIGHT_STD = 0.02f;

// ---- generator (host twin; the device twin lives in csrc/cuda/synth.cu)
inline uint64_t mix64(uint64_t key) {   // the splitmix64 output function (spec/prim.rs:207-215) of state `key`
    uint64_t z = key + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
inline uint64_t elem_key(uint64_t seed, uint64_t tid, uint64_t i) { return seed ^ (tid << 40) ^ i; }
// Sum of four uniform 16-bit integers, centred: variance 4 * (2^32 - 1) / 12, i.e. std 37837.2267...
constexpr double IRWIN_HALL4_STD = 37837.22676;
inline float draw_normal(uint64_t seed, uint64_t tid, uint64_t i, float stddev) {
    const uint64_t z = mix64(elem_key(seed, tid, i));
    const int t = (int)(z & 0xFFFF) + (int)((z >> 16) & 0xFFFF) + (int)((z >> 32) & 0xFFFF) + (int)(z >> 48) - 131070;
    const float unit = (float)(1.0 / IRWIN_HALL4_STD);
    return ((float)t * unit) * stddev;
}
inline float draw_unit(uint64_t seed, uint64_t tid, uint64_t i) {   // uniform in [0, 1), 24 bits
    return (float)(mix64(elem_key(seed, tid, i)) >> 40) * (1.0f / 16777216.0f);
}
inline uint16_t f32_to_bf16(float f) {
    uint32_t b;
    __builtin_memcpy(&b, &f, 4);
    b += 0x7FFFu + ((b >> 16) & 1u);
    return (uint16_t)(b >> 16);
}
inline float bf16_to_f32(uint16_t h) {
    uint32_t b = (uint32_t)h << 16;
    float f;
    __builtin_memcpy(&f, &b, 4);
    return f;
}
// The bf16 weight element i of tensor tid, widened back to fp32 (what `det convert` reads from a bf16 file).
inline float synth_weight(uint64_t seed, uint64_t tid, uint64_t i) {
    return bf16_to_f32(f32_to_bf16(draw_normal(seed, tid, i, WEIGHT_STD)));
}

// ---- quantizer (quantize.rs:8-100)
size_t det_row_bytes(int bits, size_t k);                                     // spec/tensor.rs:49-55
void pack_codes(const int8_t* codes, size_t n, int bits, uint8_t* out);       // quantize.rs:8-31
void quantize_row(const float* w, size_t k, int bits, uint8_t* out_row);      // quantize.rs:58-85
// `n` det rows of a synthetic tensor (rows generated on the fly, threads over rows).
std::vector<uint8_t> synth_det_rows(uint64_t seed, uint64_t tid, size_t n, size_t k, int bits, size_t row0 = 0);

// The same rows through the provider set with set_synth_rows_provider when there is one (backend.hpp), else the host path.
std::vector<uint8_t> synth_det_rows_any(uint64_t seed, uint64_t tid, size_t row0, size_t n, size_t k, int bits);

// ---- rope tables [pos][rot/2], computed in binary64 and rounded once (convert.rs:370-385)
void rope_tables(const Config& c, size_t n_pos, std::vector<float>& cos, std::vector<float>& sin);

// Prompt ids uniform in [0, vocab) from the generator (tensor id 0 of seed `seed`).
std::vector<int32_t> synth_prompt(uint64_t seed, size_t n, size_t vocab);

}  // namespace det
