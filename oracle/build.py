"""Builds the CPU oracle (TEST INFRASTRUCTURE — not part of the product).

  oracle/_build/liboracle.so   the restated spec + reference backend (spec.hpp, ref_ops.hpp, ref_backend.hpp) with the
                               C entry points of oracle_capi.cpp; links the driver library for the shared model driver
                               and conformance suites.

The reference itself is Rust (crates/det); neither cargo nor rustc exists here, so there is no `oracle/_ref` build of
the real reference — the restatement is the only oracle.  Flags follow docs/SPEC.md §8: no contraction, no fast math.
"""
from __future__ import annotations

import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
OUT = HERE / "_build"
CUDA_INC = Path("/usr/local/cuda/include")

FLAGS = ["-O2", "-std=c++17", "-fPIC", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-Wall",
         "-I", str(ROOT / "include"), "-I", str(CUDA_INC)]


def build(force: bool = False) -> Path:
    OUT.mkdir(exist_ok=True)
    lib = OUT / "liboracle.so"
    srcs = sorted(HERE.glob("*.cpp"))
    deps = srcs + sorted(HERE.glob("*.hpp")) + sorted((ROOT / "det_b200" / "csrc" / "host").glob("*.hpp"))
    host_lib = ROOT / "det_b200" / "lib" / "libdet_host.so"
    if host_lib.exists():
        deps.append(host_lib)
    if not force and lib.exists() and all(d.stat().st_mtime <= lib.stat().st_mtime for d in deps):
        return lib
    cmd = ["g++"] + FLAGS + ["-shared", "-o", str(lib)] + [str(s) for s in srcs] + \
          ["-L", str(host_lib.parent), "-ldet_host", "-ldet_b200", f"-Wl,-rpath,{host_lib.parent}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("oracle build failed")
    if r.stderr.strip():
        sys.stderr.write(r.stderr)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
