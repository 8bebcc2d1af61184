"""The C-ABI library loads without a GPU and exports every symbol include/det_b200.h declares (no compute calls)."""
import ctypes as C
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _declared():
    text = (ROOT / "include" / "det_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(det_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(libs):
    lib = libs.cuda()
    names = _declared()
    assert len(names) >= 40
    for name in names:
        assert hasattr(lib, name), f"libdet_b200.so does not export {name}"
    assert set(names) == set(libs.CUDA_ABI), set(names) ^ set(libs.CUDA_ABI)


def test_reference_symbols_present(libs):
    """The 30 entry points det's FFI crate binds (crates/det-sys/src/lib.rs:54-228)."""
    ref = ["det_init", "det_device_name", "det_malloc", "det_free", "det_allocated_bytes", "det_sync", "det_flush",
           "det_memset", "det_memcpy", "det_cuda_stream", "det_rmsnorm_quant", "det_quant", "det_embed", "det_add",
           "det_silu_mul_quant", "det_argmax", "det_gemm", "det_gemm_ex", "det_gemm_scratch_bytes",
           "det_gemm_set_scratch", "det_attention", "det_attn_scratch_bytes", "det_attention_dev", "det_gdn",
           "det_gdn_ex", "det_gdn_scratch_bytes", "det_sample", "det_sample_topkp", "det_sample_scratch_bytes",
           "det_test_prim"]
    lib = libs.cuda()
    for name in ref:
        assert hasattr(lib, name), name


def test_struct_layouts_match_the_reference(libs):
    """#[repr(C)] twins in crates/det-sys/src/lib.rs:12-52: pointer-sized fields then ints, natural alignment."""
    assert C.sizeof(libs.QLinear) == 3 * 8 + 3 * 4 + 4
    assert C.sizeof(libs.AttnLayer) == 4 * 8
    assert C.sizeof(libs.KvCache) == 3 * 8 + 8 + 2 * 8
    assert libs.KvCache.capacity.offset == 24 and libs.KvCache.vlo.offset == 32
    assert C.sizeof(libs.GdnLayer) == 4 * 8 and C.sizeof(libs.GdnState) == 2 * 8


def test_size_queries_need_no_device(libs):
    lib = libs.cuda()
    assert lib.det_gemm_scratch_bytes(512, 5120) == 512 * 40 * 4
    assert lib.det_attn_scratch_bytes(1, 24, 256) > 24 * 256 * 9
    assert lib.det_gdn_scratch_bytes(1, 16, 48, 128, 128) >= (10240 + 2 * 48 + 48 * 128) * 4
    assert lib.det_sample_scratch_bytes(1, 248320) == 248320 * 8
    # W6, K = 5120: a record = 4 rows x one 1024-wide K chunk = 4 * 768 code bytes + 4 * 8 * 2 (m); 5 chunks per row quad
    assert lib.det_linear_repack_bytes(17408, 5120, 6) == 17408 // 4 * 5 * (4 * 768 + 64)
    # K = 2560 (an odd multiple of 512): 512-wide chunks
    assert lib.det_linear_repack_bytes(10240, 2560, 6) == 10240 // 4 * 5 * (4 * 384 + 32)


def test_host_library_loads(libs):
    h = libs.host()
    assert h.dh_det_row_bytes(6, 5120) == 5120 // 32 * 24 + 4 + 40 * 2


def test_ctypes_mirror_has_the_layout_the_c_compiler_gives_the_header(libs, tmp_path):
    """Every struct of include/det_b200.h: size and the offset of every field as gcc lays them out, against the ctypes
    mirror in det_b200/capi.py (a field added to one side only, or out of order, shows here and not as a wrong pointer
    on the GPU)."""
    import os
    import shutil
    import subprocess
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    cuda_inc = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"
    if shutil.which("gcc") is None or not (cuda_inc / "cuda_runtime.h").exists():
        pytest.skip("needs gcc and the CUDA headers")
    pairs = {"det_qlinear": libs.QLinear, "det_attn_layer": libs.AttnLayer, "det_kv_cache": libs.KvCache,
             "det_gdn_layer": libs.GdnLayer, "det_gdn_state": libs.GdnState, "det_act_source": libs.ActSource,
             "det_gemv_op": libs.GemvOp}
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "det_b200.h"', "int main(void) {"]
    for cname, mirror in pairs.items():
        lines.append(f'  printf("{cname} %zu\\n", sizeof({cname}));')
        for field, _ in mirror._fields_:
            lines.append(f'  printf("{cname}.{field} %zu\\n", offsetof({cname}, {field}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", str(root / "include"), "-I", str(cuda_inc), str(src), "-o", str(exe)], check=True)
    got = dict(line.split() for line in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    for cname, mirror in pairs.items():
        assert int(got[cname]) == C.sizeof(mirror), cname
        for field, _ in mirror._fields_:
            assert int(got[f"{cname}.{field}"]) == getattr(mirror, field).offset, f"{cname}.{field}"
