"""In-tree build of the native libraries.

  det_b200/lib/libdet_b200.so   the C-ABI CUDA backend (include/det_b200.h), sm_100a only
  det_b200/lib/libdet_host.so   the host driver above the C ABI (model, forward pass, token loop, conformance)

The compiler flags are part of the numerics contract (crates/det-sys/build.rs:117-122, docs/SPEC.md §8): no FMA
contraction on the device (-fmad=false) or the host (-ffp-contract=off), no fast math, denormals kept.
`python -m det_b200.build` builds everything that is out of date; `--force` rebuilds.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "det_b200"
LIB = PKG / "lib"
OBJ = PKG / "build"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-fmad=false", "-ftz=false", "-prec-div=true", "-prec-sqrt=true",
    "-Xcompiler", "-fPIC,-ffp-contract=off,-O2",
    "-I", str(ROOT / "include"),
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-ffp-contract=off", "-fno-fast-math", "-pthread", "-Wall",
             "-I", str(ROOT / "include"), "-I", str(CUDA_HOME / "include")]


def _newer(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(s.stat().st_mtime > t for s in sources)


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} {cmd[-1]}")
    if r.stderr.strip():
        sys.stderr.write(r.stderr)


def cuda_sources() -> list[Path]:
    return sorted((PKG / "csrc" / "cuda").glob("*.cu"))


def host_sources() -> list[Path]:
    return sorted((PKG / "csrc" / "host").glob("*.cpp"))


def build_cuda(force: bool = False, verbose_ptxas: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    headers = list((PKG / "csrc" / "cuda").glob("*.cuh")) + list((ROOT / "include").glob("*.h"))
    objs, jobs = [], []
    for src in cuda_sources():
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        if force or _newer(obj, [src] + headers):
            cmd = [NVCC] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose_ptxas else []) + ["-c", str(src), "-o", str(obj)]
            jobs.append(cmd)
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(_run, jobs))
    out = LIB / "libdet_b200.so"
    if force or jobs or _newer(out, objs):
        _run([NVCC, "-shared", "-o", str(out)] + [str(o) for o in objs] +
             ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"])
    return out


def build_host(force: bool = False) -> Path | None:
    srcs = host_sources()
    if not srcs:
        return None
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    headers = list((PKG / "csrc" / "host").glob("*.hpp")) + list((ROOT / "include").glob("*.h"))
    objs, jobs = [], []
    for src in srcs:
        obj = OBJ / ("host_" + src.stem + ".o")
        objs.append(obj)
        if force or _newer(obj, [src] + headers):
            jobs.append(["g++"] + CXX_FLAGS + ["-c", str(src), "-o", str(obj)])
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(_run, jobs))
    out = LIB / "libdet_host.so"
    if force or jobs or _newer(out, objs):
        _run(["g++", "-shared", "-o", str(out)] + [str(o) for o in objs] +
             ["-L", str(LIB), "-ldet_b200", "-Wl,-rpath,$ORIGIN", "-pthread", "-ldl"])
    return out


def build_all(force: bool = False) -> None:
    if shutil.which(NVCC) is None:
        raise RuntimeError(f"nvcc not found at {NVCC}")
    build_cuda(force)
    build_host(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built:", *(p.name for p in sorted(LIB.glob("*.so"))))
