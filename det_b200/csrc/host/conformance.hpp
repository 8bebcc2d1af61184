// Backend conformance: every op of a backend under test against a reference backend on random inputs and on the edge
// cases of the numerics, bit for bit — the C++ mirror of crates/det/src/conformance.rs (run, primitives, gemm, norms,
// attention, gdn, sampling).  The reference backend is passed in by the caller (tests wire the CPU oracle there), so
// this file carries no reference arithmetic of its own.
#pragma once
#include "backend.hpp"
#include <functional>
#include <string>
#include <utility>
#include <vector>

namespace det {

// conformance.rs:13-33
struct Report {
    std::vector<std::pair<std::string, std::string>> checks;   // (name, first mismatch or "")
    void add(std::string name, std::string mismatch) { checks.emplace_back(std::move(name), std::move(mismatch)); }
    bool ok() const {
        for (const auto& c : checks)
            if (!c.second.empty()) return false;
        return true;
    }
};

// The elementwise primitive hook of the backend under test (det_test_prim): (op, x, m, n) -> out
using Prim = std::function<std::vector<float>(int, const std::vector<float>&, size_t, size_t)>;
// The scalar spec primitives the `primitives` suite compares against, supplied by the caller: same op numbers, applied
// on the host.
using PrimRef = std::function<std::vector<float>(int, const std::vector<float>&, size_t, size_t)>;

void conformance_primitives(const Prim& prim, const PrimRef& ref, Report& r);
void conformance_gemm(Backend& ref, Backend& dut, Report& r);
void conformance_norms(Backend& ref, Backend& dut, Report& r);
void conformance_attention(Backend& ref, Backend& dut, Report& r);
void conformance_gdn(Backend& ref, Backend& dut, Report& r);
void conformance_sampling(Backend& ref, Backend& dut, Report& r);
// conformance.rs:164-175
Report conformance_run(Backend& ref, Backend& dut, const Prim* prim, const PrimRef* prim_ref);

}  // namespace det
