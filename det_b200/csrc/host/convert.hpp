// `det convert` and `det calibrate` (crates/det/src/convert.rs:13-420, crates/det/src/calibrate.rs:10-130): a float GGUF
// (BF16 / F16 / F32 tensors as llama.cpp's converter writes them) becomes a det GGUF — the same metadata and vectors,
// every linear quantized into det rows, the output head always present, the rotary tables as tensors, the Gated DeltaNet
// value heads reordered so that v head h reads k head h / (n_v / n_k) — and the value-cache scales of a det file are set
// from a calibration run.  The row quantizer is pluggable: the host one (threads over rows) or the device one of the
// CUDA backend (cuda_quantize_rows, same bytes).
#pragma once
#include "gguf.hpp"
#include "model.hpp"
#include <functional>

namespace det {

// convert.rs:13-69 — a GGUF model, possibly split over several files.
struct Source {
    std::vector<std::shared_ptr<Gguf>> parts;
    static bool open(const std::string& path, Source& out, std::string& err);
    const GgufKv& kv() const { return parts[0]->kv; }
    bool tensor(const std::string& name, const Gguf*& g, const GgufTensor*& t) const;
    std::vector<float> f32s(const std::string& name) const;   // row-major, dims[0] fastest; throws when missing
};

// convert.rs:71-117 — a default width and overrides per linear name, parsed from "6,output=8,ffn_down=8".
struct Bits {
    int def = 6;
    std::vector<std::pair<std::string, int>> per;
    static std::string parse(const std::string& s, Bits& out);   // "" on success
    int of(const std::string& linear) const;
};
constexpr const char* DEFAULT_BITS = "6,output=8,ssm_alpha=8,ssm_beta=8";   // convert.rs:119-120

// Quantizes `n` output rows of K codes from a float tensor in host memory ([src_rows][K] of `type`): output row r reads
// source row row_perm[r] (null: r), element k reads column col_perm[k] (null: k).  Writes n det file rows to `out`.
using RowQuantizer = std::function<void(const uint8_t* src, GgmlType type, size_t src_rows, const std::vector<int>* row_perm,
                                        const std::vector<int>* col_perm, size_t n, size_t k, int bits, uint8_t* out)>;
void host_quantize_rows(const uint8_t* src, GgmlType type, size_t src_rows, const std::vector<int>* row_perm,
                        const std::vector<int>* col_perm, size_t n, size_t k, int bits, uint8_t* out);

struct ConvertOptions {   // convert.rs:122-126
    Bits bits;
    size_t rope_positions = 0;   // 0 takes the model's context length (32768 when the file states none)
    RowQuantizer quantizer;      // empty: host_quantize_rows
    bool verbose = false;
};
// convert.rs:153-156 — perm[new] = old over `width`-element blocks of the v heads.
std::vector<int> head_perm(size_t n_k, size_t n_v, size_t width, size_t offset, size_t total);
std::string convert(const Source& src, const std::string& out, const ConvertOptions& opt);   // "" on success
std::string default_output(const std::string& src_path, const Bits& bits);                   // convert.rs:404-420

// The float source whose conversion (default widths, n_pos rope positions) is byte for byte write_synthetic_gguf's file:
// bf16 (or fp32, `f32_linears`) matrices in the unconverted head order, tied head (no output.weight), fp32 vectors.
std::string write_synthetic_source_gguf(const Config& c, uint64_t seed, const std::string& path, size_t n_pos,
                                        bool f32_linears);

// ---- calibration (calibrate.rs)
constexpr float HEADROOM = 8.0f;   // calibrate.rs:10
// The generator part of calibrate.rs:38-64: `prefix` (the caller's tokenized text, may be empty) followed by n_random ids.
std::vector<int32_t> calibration_ids(const std::vector<int32_t>& prefix, size_t vocab, size_t n_random);
// calibrate.rs:66-89 — runs `ids` through the model and returns the per-(attention layer, kv head) value scales.
std::string v_scales(Model& m, const int32_t* ids, size_t n, std::vector<float>& scales);
// calibrate.rs:91-109
bool write_scales_in_place(const Model& m, const std::vector<float>& scales, const std::string& path, std::string& err);
bool write_scales_copy(const Model& m, const std::vector<float>& scales, const std::string& out, std::string& err);

}  // namespace det
