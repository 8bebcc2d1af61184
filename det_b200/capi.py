"""ctypes bindings of the two native libraries.

  cuda()  libdet_b200.so — the C ABI of include/det_b200.h (loading it needs the CUDA runtime, not a GPU)
  host()  libdet_host.so — the driver above it (backends, synthetic model, token loop)

Nothing here falls back to a CPU implementation: a missing library raises, and the first call that needs a device
aborts inside the library when none is present.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_DIR = Path(__file__).resolve().parent / "lib"

c_void_p, c_int, c_size_t, c_float, c_char_p = C.c_void_p, C.c_int, C.c_size_t, C.c_float, C.c_char_p
c_u64, c_i32 = C.c_uint64, C.c_int32


class QLinear(C.Structure):
    """det_qlinear (include/det_b200.h; kernels/cuda/det_cuda.h:26-32)."""
    _fields_ = [("wq", c_void_p), ("c", c_void_p), ("m", c_void_p), ("N", c_int), ("K", c_int), ("bits", c_int)]


class AttnLayer(C.Structure):
    _fields_ = [("q_norm", c_void_p), ("k_norm", c_void_p), ("v_scale", c_void_p), ("v_inv_scale", c_void_p)]


class KvCache(C.Structure):
    _fields_ = [("kq", c_void_p), ("sk", c_void_p), ("vq", c_void_p), ("capacity", c_int), ("vlo", c_void_p),
                ("vhi", c_void_p)]


class GdnLayer(C.Structure):
    _fields_ = [("conv", c_void_p), ("A", c_void_p), ("dt_bias", c_void_p), ("norm", c_void_p)]


class GdnState(C.Structure):
    _fields_ = [("conv_state", c_void_p), ("S", c_void_p)]


class ActSource(C.Structure):
    """det_act_source (include/det_b200.h): fp32 inputs of a GEMM whose activation quantization is fused in."""
    _fields_ = [("kind", c_int), ("a", c_void_p), ("b", c_void_p), ("eps", c_float), ("xq", c_void_p), ("sx", c_void_p),
                ("mx", c_void_p), ("amax", c_void_p), ("xchg", c_void_p), ("local", c_void_p), ("slice", c_int),
                ("acc_out", c_void_p)]


class GemvOp(C.Structure):
    """det_gemv_op (include/det_b200.h): one decode GEMV launch with its fused neighbours."""
    _fields_ = [("lin", C.POINTER(QLinear)), ("lin2", C.POINTER(QLinear)), ("src", C.POINTER(ActSource)),
                ("xq", c_void_p), ("sx", c_void_p), ("mx", c_void_p), ("M", c_int),
                ("y", c_void_p), ("accumulate", c_int), ("nparts", c_int), ("offs", C.POINTER(c_int)),
                ("dsts", C.POINTER(c_void_p)),
                ("y2", c_void_p), ("nparts2", c_int), ("offs2", C.POINTER(c_int)), ("dsts2", C.POINTER(c_void_p)),
                ("h", c_void_p), ("h_amax", c_void_p)]


DET_LAYOUT_STREAM = 0x100
DET_LAYOUT_INT8 = 0x200
DET_LAYOUT_PAIRS = 0x400
DET_ACT_RMSNORM, DET_ACT_PLAIN = 1, 2
# tile pins of the tensor-core GEMM (det_debug_set_tc_variant) that take large batches; 0 = chosen by shape
TC_VARIANTS_LARGE = (0, 2, 3)

# every symbol include/det_b200.h declares: name -> (restype, argtypes)
CUDA_ABI = {
    "det_init": (c_int, []),
    "det_device_name": (c_char_p, []),
    "det_malloc": (c_void_p, [c_size_t]),
    "det_free": (None, [c_void_p]),
    "det_allocated_bytes": (c_size_t, []),
    "det_sync": (None, []),
    "det_flush": (None, []),
    "det_memset": (None, [c_void_p, c_int, c_size_t, c_void_p]),
    "det_memcpy": (None, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "det_cuda_stream": (c_void_p, []),
    "det_rmsnorm_quant": (None, [c_void_p, c_void_p, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "det_quant": (None, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "det_embed": (None, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "det_add": (None, [c_void_p, c_void_p, C.c_longlong, c_void_p]),
    "det_silu_mul_quant": (None, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "det_argmax": (None, [c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "det_gemm": (None, [C.POINTER(QLinear), c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "det_gemm_ex": (None, [C.POINTER(QLinear), c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                           C.POINTER(c_int), C.POINTER(c_void_p), c_void_p]),
    "det_gemm_pair": (None, [C.POINTER(QLinear), C.POINTER(QLinear), c_void_p, c_void_p, c_void_p, c_int,
                             c_int, C.POINTER(c_int), C.POINTER(c_void_p), c_int, C.POINTER(c_int), C.POINTER(c_void_p), c_void_p]),
    "det_gemv": (None, [C.POINTER(GemvOp), c_void_p]),
    "det_gemm_scratch_bytes": (c_size_t, [c_int, c_int]),
    "det_gemm_set_scratch": (None, [c_void_p, c_size_t]),
    "det_attention": (None, [C.POINTER(AttnLayer), C.POINTER(KvCache), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_int, c_float, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "det_attn_scratch_bytes": (c_size_t, [c_int, c_int, c_int]),
    "det_attention_dev": (None, [C.POINTER(AttnLayer), C.POINTER(KvCache), c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_int, c_float, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                 c_void_p, c_void_p]),
    "det_gdn": (None, [C.POINTER(GdnLayer), C.POINTER(GdnState), c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int,
                       c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "det_gdn_scratch_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "det_gdn_ex": (None, [C.POINTER(GdnLayer), C.POINTER(GdnState), c_void_p, c_void_p, c_void_p, c_void_p, c_float,
                          c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "det_sample": (None, [c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p]),
    "det_sample_topkp": (None, [c_void_p, c_int, c_int, c_float, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p]),
    "det_sample_scratch_bytes": (c_size_t, [c_int, c_int]),
    "det_sample_topkp_static": (c_int, [c_void_p, c_int, c_int, c_float, c_int, c_float, c_void_p, c_void_p, c_void_p]),
    "det_test_prim": (None, [c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "det_linear_repack_bytes": (c_size_t, [c_int, c_int, c_int]),
    "det_linear_repack": (None, [C.POINTER(QLinear), c_void_p, c_void_p]),
    "det_linear_repack_pairs": (None, [C.POINTER(QLinear), c_void_p, c_void_p]),
    "det_linear_expand_bytes": (c_size_t, [c_int, c_int]),
    "det_linear_expand": (None, [C.POINTER(QLinear), c_void_p, c_void_p]),
    "det_synth_linear": (None, [c_u64, c_u64, C.c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p]),
    "det_unshard": (None, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "det_synth_bf16": (None, [c_u64, c_u64, C.c_longlong, c_void_p, c_void_p]),
    "det_graph_begin": (None, []),
    "det_graph_end": (c_void_p, []),
    "det_graph_launch": (None, [c_void_p]),
    "det_graph_free": (None, [c_void_p]),
    "det_token_feedback": (None, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "det_attention_rows": (None, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_int, c_float, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "det_gdn_rows": (None, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int,
                            c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "det_xchg_create": (c_void_p, [c_size_t, c_int, c_int]),
    "det_xchg_ipc_handle": (None, [c_void_p, c_void_p]),
    "det_xchg_open": (None, [c_void_p, c_void_p]),
    "det_xchg_open_loopback": (None, [c_void_p]),
    "det_xchg_capacity": (c_size_t, [c_void_p]),
    "det_xchg_all_gather": (None, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "det_xchg_destroy": (None, [c_void_p]),
    "det_xchg_fusable": (c_int, [c_int, c_int]),
    "det_xchg_add_rmsnorm_quant": (None, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_int,
                                          c_void_p, c_void_p, c_void_p, c_void_p]),
    "det_xchg_quant": (None, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "det_quantize_rows": (None, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "det_absmax_heads": (None, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "det_embed_table": (None, [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "det_attn_set_workspace": (None, [c_void_p, c_size_t]),
    "det_debug_set_attn_tc": (None, [c_int, c_int]),
    "det_debug_set_pdl": (None, [c_int]),
    "det_debug_set_tc_variant": (None, [c_int]),
    "det_debug_set_gemv": (None, [c_int]),
    "det_debug_set_rows": (None, [c_int]),
    "det_debug_umma_peak": (C.c_double, [c_int]),
    "det_debug_stream_peak": (C.c_double, [c_void_p, c_size_t, c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    "det_last_error": (c_int, []),
    "det_clear_error": (None, []),
    "det_debug_set_wait_limit": (None, [C.c_longlong]),
    "det_debug_xchg_drop": (None, [c_void_p, c_int]),
}

HOST_API = {
    "dh_last_error": (c_char_p, []),
    "dh_cuda_backend_new": (c_void_p, [c_int, c_int]),
    "dh_backend_free": (None, [c_void_p]),
    "dh_backend_name": (c_int, [c_void_p, c_char_p, c_size_t]),
    "dh_cuda_debug": (None, [c_void_p, C.c_uint, c_int]),
    "dh_cuda_test_prim": (None, [c_int, c_void_p, c_size_t, c_size_t, c_size_t, c_void_p, c_size_t]),
    "dh_model_new_synth": (c_void_p, [c_void_p, c_char_p, c_size_t, c_u64, c_size_t, c_size_t]),
    "dh_model_load": (c_void_p, [c_void_p, c_char_p, c_size_t, c_size_t]),
    "dh_model_calibrated": (c_int, [c_void_p]),
    "dh_write_synthetic_gguf": (c_int, [c_char_p, c_size_t, c_u64, c_char_p, c_size_t]),
    "dh_write_synthetic_source_gguf": (c_int, [c_char_p, c_size_t, c_u64, c_char_p, c_size_t, c_int]),
    "dh_convert": (c_int, [c_char_p, c_char_p, c_char_p, c_size_t, c_int]),
    "dh_convert_default_output": (c_int, [c_char_p, c_char_p, c_char_p, c_size_t]),
    "dh_v_scales": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p, c_size_t, C.POINTER(c_size_t)]),
    "dh_calibration_ids": (None, [c_void_p, c_size_t, c_size_t, c_size_t, c_void_p]),
    "dh_write_scales_in_place": (c_int, [c_void_p, c_void_p, c_size_t, c_char_p]),
    "dh_write_scales_copy": (c_int, [c_void_p, c_void_p, c_size_t, c_char_p]),
    "dh_gguf_open": (c_void_p, [c_char_p]),
    "dh_gguf_close": (None, [c_void_p]),
    "dh_gguf_n_tensors": (c_size_t, [c_void_p]),
    "dh_gguf_data_start": (c_size_t, [c_void_p]),
    "dh_gguf_tensor": (c_int, [c_void_p, c_size_t, c_char_p, c_size_t, c_void_p, C.POINTER(c_size_t),
                               C.POINTER(C.c_uint32), C.POINTER(c_size_t), C.POINTER(c_size_t)]),
    "dh_gguf_get": (c_int, [c_void_p, c_char_p, c_char_p, c_size_t]),
    "dh_gguf_config": (c_int, [c_void_p, c_char_p, c_size_t]),
    "dh_gguf_check_finite": (c_int, [c_void_p]),
    "dh_dequant_row": (c_int, [C.c_uint32, c_void_p, c_size_t, c_void_p]),
    "dh_quantize_row": (None, [c_void_p, c_size_t, c_int, c_void_p]),
    "dh_model_forward_observed": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p, c_void_p, c_int]),
    "dh_model_generate_observed": (c_int, [c_void_p, c_void_p, c_size_t, c_size_t, c_int, c_float, c_size_t, c_float, c_u64,
                                           c_void_p, C.POINTER(c_size_t), c_void_p, c_void_p, c_int]),
    "dh_backend_read": (None, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "dh_nccl_unique_id": (None, [c_void_p]),
    "dh_nccl_comm_new": (c_void_p, [c_void_p, c_int, c_int]),
    "dh_callback_comm_new": (c_void_p, [c_int, c_int, c_void_p]),
    "dh_peer_comm_new": (c_void_p, [c_void_p, c_int, c_int, c_size_t]),
    "dh_peer_comm_handle": (None, [c_void_p, c_void_p]),
    "dh_peer_comm_open": (None, [c_void_p, c_void_p]),
    "dh_peer_comm_set_fuse": (None, [c_void_p, c_int]),
    "dh_peer_comm_open_loopback": (None, [c_void_p]),
    "dh_comm_free": (None, [c_void_p]),
    "dh_model_new_synth_tp": (c_void_p, [c_void_p, c_char_p, c_size_t, c_u64, c_size_t, c_size_t, c_void_p]),
    "dh_model_free": (None, [c_void_p]),
    "dh_model_vocab": (c_size_t, [c_void_p]),
    "dh_model_pos": (c_size_t, [c_void_p]),
    "dh_model_set_all_logits": (c_int, [c_void_p, c_int]),
    "dh_model_reset": (c_int, [c_void_p]),
    "dh_model_forward": (c_int, [c_void_p, c_void_p, c_size_t]),
    "dh_model_prefill": (c_int, [c_void_p, c_void_p, c_size_t]),
    "dh_model_logits": (c_size_t, [c_void_p, c_void_p, c_size_t]),
    "dh_model_pick": (c_int, [c_void_p, c_int, c_float, c_size_t, c_float, C.POINTER(c_u64), C.POINTER(c_i32)]),
    "dh_model_generate": (c_int, [c_void_p, c_void_p, c_size_t, c_size_t, c_int, c_float, c_size_t, c_float, c_u64,
                                  c_void_p, C.POINTER(c_size_t)]),
    "dh_cuda_set_fuse_rows": (None, [c_void_p, c_int]),
    "dh_batch_new": (c_void_p, [c_void_p, c_size_t, c_size_t]),
    "dh_batch_free": (None, [c_void_p]),
    "dh_batch_prefill": (c_int, [c_void_p, c_size_t, c_void_p, c_size_t, c_int, c_float, c_size_t, c_float, c_u64]),
    "dh_batch_step": (c_int, [c_void_p, c_size_t]),
    "dh_batch_tokens": (c_size_t, [c_void_p, c_size_t, c_void_p, c_size_t]),
    "dh_graph_decoder_new": (c_void_p, [c_void_p]),
    "dh_graph_decoder_free": (None, [c_void_p]),
    "dh_graph_decoder_enqueue": (c_int, [c_void_p, c_i32, c_size_t, c_int]),
    "dh_graph_decoder_finish": (c_size_t, [c_void_p, c_void_p, c_size_t]),
    "dh_gemv_sweep": (c_int, [c_void_p, c_int, C.POINTER(c_size_t), C.POINTER(c_size_t)]),
    "dh_use_cuda_synth_rows": (None, [c_int]),
    "dh_synth_prompt": (None, [c_u64, c_size_t, c_size_t, c_void_p]),
    "dh_synth_det_rows": (None, [c_u64, c_u64, c_size_t, c_size_t, c_int, c_void_p]),
    "dh_det_row_bytes": (c_size_t, [c_int, c_size_t]),
}

# The tap callback of dh_model_forward_observed: (user, kind, layer, pos0, t, data, len, id, rng)
TAP_FN = C.CFUNCTYPE(None, c_void_p, c_int, c_size_t, c_size_t, c_size_t, c_void_p, c_size_t, c_i32, c_u64)
TAP_KINDS = ("Residual", "MixerOut", "PostMixer", "AttnV", "Kv", "AttnOut", "GdnIn", "GdnOut", "GdnState", "Logits", "Token")

_cache: dict[str, C.CDLL] = {}


def _load(name: str, table: dict) -> C.CDLL:
    if name in _cache:
        return _cache[name]
    path = LIB_DIR / name
    if not path.exists():
        raise RuntimeError(f"{path} is missing: run `python -m det_b200.build` (there is no fallback implementation)")
    lib = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
    for sym, (res, args) in table.items():
        fn = getattr(lib, sym)   # AttributeError when the library does not export a declared symbol
        fn.restype = res
        fn.argtypes = args
    _cache[name] = lib
    return lib


def cuda() -> C.CDLL:
    return _load("libdet_b200.so", CUDA_ABI)


def host() -> C.CDLL:
    cuda()
    return _load("libdet_host.so", HOST_API)
