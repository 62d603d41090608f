"""ctypes loader for libtriebwerk_b200.so (the C ABI declared in include/triebwerk_b200.h).

There is no fallback: if the shared library is missing or a symbol cannot be resolved, importing the
product path raises.  Build it with ``python -c "import __graft_entry__ as g; g.build()"`` or
``python -m triebwerk_b200.build``.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libtriebwerk_b200.so")

# Every extern "C" symbol of include/triebwerk_b200.h; the CPU test suite checks this list against the header.
SYMBOLS = [
    "tq_status_string", "tq_version", "tq_last_compat_status",
    "launch_turbo_kv_quantize", "launch_turbo_kv_quantize_batch", "launch_turbo_gqa_attention_batch",
    "launch_turbo_gqa_attention", "launch_turbo_gqa_prefill_attention", "launch_kv_cache_write_batch",
    "launch_gqa_attention_batch", "launch_gqa_attention", "launch_gqa_prefill_attention",
    "tq_rotation_generate", "tq_workspace_bytes", "tq_append_decode", "tq_decode_attention",
    "tq_fp16_append_decode", "tq_fp16_decode_attention", "tq_workspace_status", "tq_decode_attention_static",
    "tq_engine_create", "tq_engine_destroy", "tq_engine_kv_bits", "tq_engine_set_fused", "tq_engine_arena_bytes", "tq_engine_set_arena",
    "tq_engine_alloc_batch", "tq_engine_reset", "tq_engine_sleep", "tq_engine_wake", "tq_engine_positions",
    "tq_engine_set_positions", "tq_engine_advance", "tq_engine_layer_ptrs", "tq_engine_row_base",
    "tq_engine_rotation", "tq_engine_set_rotation", "tq_engine_decode_layer", "tq_engine_prefill_append", "tq_engine_prefill_append_batch",
    "tq_engine_decode_step_host", "tq_engine_attend_layer", "tq_engine_decode_step", "tq_engine_status", "tq_engine_attend_step",
    "tq_engine_output_f32", "tq_engine_read_output_f32", "tq_engine_decode_layers", "tq_static_status", "tq_selftest_bounded_wait",
    "tq_engine_sequence_blob_bytes", "tq_engine_export_sequence", "tq_engine_import_sequence", "tq_engine_sleep_keep", "tq_engine_prefill_shared", "tq_engine_decode_step_produce", "tq_fold_rotation_into_projection",
    "tq_engine_time_attention", "tq_engine_last_attention_ms", "tq_engine_prefill_layer", "tq_engine_prefill_layer_batch", "tq_engine_step_prepare", "tq_engine_step_attend_layers",
    "tq_peer_buffer_create", "tq_peer_buffer_open", "tq_peer_buffer_close", "tq_peer_buffer_destroy", "tq_peer_copy", "tq_peer_signal", "tq_peer_wait",
]


class StepProducer(C.Structure):
    _fields_ = [("q_norm_weight", C.c_void_p), ("k_norm_weight", C.c_void_p), ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p),
                ("rope_dim", C.c_int), ("eps", C.c_float), ("biased", C.c_int), ("rotated_output", C.c_int)]


class ModelShape(C.Structure):
    _fields_ = [("num_layers", C.c_int), ("num_heads", C.c_int), ("num_kv_heads", C.c_int), ("head_dim", C.c_int)]


_lib = None


def lib() -> C.CDLL:
    """The loaded library with argument/return types set.  Raises if it was not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: the CUDA library has not been built (run __graft_entry__.build()). "
            "triebwerk_b200 has no CPU or PyTorch fallback.")
    L = C.CDLL(LIB_PATH)
    vp, i, ll, sz = C.c_void_p, C.c_int, C.c_longlong, C.c_size_t
    ip = C.c_void_p  # device int* / int64* cross as raw addresses

    def sig(name, restype, argtypes):
        f = getattr(L, name)
        f.restype = restype
        f.argtypes = argtypes

    sig("tq_status_string", C.c_char_p, [i])
    sig("tq_version", i, [])
    sig("tq_last_compat_status", i, [])
    sig("launch_turbo_kv_quantize", None, [vp, vp, vp, vp, ip, i, i, i, i, i, i, vp])
    sig("launch_turbo_kv_quantize_batch", None, [vp, vp, vp, vp, ip, i, i, i, i, i, i, vp])
    sig("launch_turbo_gqa_attention_batch", None, [vp, vp, vp, vp, vp, vp, vp, vp, ip, i, i, i, i, i, i, i, i, vp])
    sig("launch_turbo_gqa_attention", None, [vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, vp])
    sig("launch_turbo_gqa_prefill_attention", None, [vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i, i, vp])
    sig("launch_kv_cache_write_batch", None, [vp, vp, vp, vp, ip, i, i, i, vp])
    sig("launch_gqa_attention_batch", None, [vp, vp, vp, vp, vp, ip, i, i, i, i, i, i, i, vp])
    sig("launch_gqa_attention", None, [vp, vp, vp, vp, vp, i, i, i, i, i, vp])
    sig("launch_gqa_prefill_attention", None, [vp, vp, vp, vp, vp, i, i, i, i, i, i, i, vp])
    sig("tq_rotation_generate", i, [C.c_uint32, vp])
    sig("tq_workspace_bytes", sz, [i, i])
    sig("tq_append_decode", i, [vp, vp, vp, vp, vp, vp, vp, vp, ip, ip, i, i, i, i, i, i, i, i, vp, sz, vp])
    sig("tq_decode_attention", i, [vp, vp, vp, vp, vp, vp, ip, i, ip, ll, i, i, i, i, i, i, i, i, vp, sz, vp])
    sig("tq_fp16_append_decode", i, [vp, vp, vp, vp, ip, ip, i, i, i, vp])
    sig("tq_fp16_decode_attention", i, [vp, vp, vp, vp, ip, i, ip, ll, i, i, i, i, i, i, i, vp, sz, vp])
    sig("tq_workspace_status", i, [vp, vp])
    sig("tq_decode_attention_static", i, [vp, vp, vp, vp, vp, vp, vp, ip, ll, i, i, i, i, i, i, i, i, vp])
    sig("tq_engine_create", i, [C.POINTER(ModelShape), i, i, C.POINTER(vp)])
    sig("tq_engine_destroy", None, [vp])
    sig("tq_engine_kv_bits", i, [vp])
    sig("tq_engine_set_fused", i, [vp, i])
    sig("tq_engine_arena_bytes", sz, [vp, i, i, C.POINTER(i)])
    sig("tq_engine_set_arena", i, [vp, vp, sz])
    sig("tq_engine_alloc_batch", i, [vp, i, i, C.POINTER(i)])
    sig("tq_engine_reset", i, [vp, i, vp])
    sig("tq_engine_sleep", i, [vp])
    sig("tq_engine_wake", i, [vp])
    sig("tq_engine_positions", vp, [vp])
    sig("tq_engine_set_positions", i, [vp, C.POINTER(i), i, vp])
    sig("tq_engine_advance", i, [vp, vp])
    sig("tq_engine_layer_ptrs", i, [vp, i, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(ll)])
    sig("tq_engine_row_base", vp, [vp])
    sig("tq_engine_rotation", vp, [vp])
    sig("tq_engine_set_rotation", i, [vp, vp, vp])
    sig("tq_engine_decode_layer", i, [vp, i, vp, vp, vp, vp, vp])
    sig("tq_engine_prefill_append", i, [vp, i, i, vp, vp, i, i, vp])
    sig("tq_engine_prefill_append_batch", i, [vp, i, i, i, vp, vp, i, i, vp])
    sig("tq_engine_decode_step_host", i, [vp, vp, vp, vp, vp, vp])
    sig("tq_engine_attend_layer", i, [vp, i, vp, vp])
    sig("tq_engine_decode_step", i, [vp, vp, vp, vp, vp, vp])
    sig("tq_engine_status", i, [vp, vp])
    sig("tq_engine_attend_step", i, [vp, vp, vp])
    sig("tq_static_status", i, [vp])
    sig("tq_engine_decode_step_produce", i, [vp, vp, vp, vp, vp, C.POINTER(StepProducer), vp])
    sig("tq_fold_rotation_into_projection", i, [vp, vp, vp, ll, i, vp])
    sig("tq_peer_buffer_create", i, [sz, C.POINTER(vp), vp])
    sig("tq_peer_buffer_open", i, [vp, C.POINTER(vp)])
    sig("tq_peer_buffer_close", i, [vp])
    sig("tq_peer_buffer_destroy", i, [vp])
    sig("tq_peer_copy", i, [vp, vp, sz, vp])
    sig("tq_peer_signal", i, [C.POINTER(vp), i, i, C.c_ulonglong, vp])
    sig("tq_peer_wait", i, [vp, i, C.c_ulonglong, vp, C.c_uint, vp])
    sig("tq_engine_prefill_shared", i, [vp, i, i, i, vp, vp, i, vp])
    sig("tq_engine_sequence_blob_bytes", sz, [vp, i])
    sig("tq_engine_export_sequence", i, [vp, i, i, vp, sz, vp])
    sig("tq_engine_import_sequence", i, [vp, i, vp, sz, vp])
    sig("tq_engine_sleep_keep", i, [vp])
    sig("tq_selftest_bounded_wait", i, [vp, C.c_uint, vp])
    sig("tq_engine_decode_layers", i, [vp, i, i, vp, vp, vp, vp, vp])
    sig("tq_engine_output_f32", i, [vp, i])
    sig("tq_engine_prefill_layer", i, [vp, i, i, vp, vp, vp, vp, i, i, vp])
    sig("tq_engine_prefill_layer_batch", i, [vp, i, i, i, vp, vp, vp, vp, i, i, vp])
    sig("tq_engine_step_prepare", i, [vp, vp, vp, vp, vp])
    sig("tq_engine_step_attend_layers", i, [vp, i, i, vp, vp])
    sig("tq_engine_time_attention", i, [vp, i])
    sig("tq_engine_last_attention_ms", i, [vp, C.POINTER(C.c_float)])
    sig("tq_engine_read_output_f32", i, [vp, vp, i, i, vp])
    _lib = L
    return L


class TqError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().tq_status_string(status)
        super().__init__(f"{where}: {msg.decode() if msg else status} ({status})")


def check(status: int, where: str) -> None:
    if status != 0:
        raise TqError(status, where)
