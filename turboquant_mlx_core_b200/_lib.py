"""ctypes loader for libturboquant_b200.so — the C-ABI of the CUDA library.

Loading fails loudly: there is no CPU fallback behind these bindings.  Declares the
argument types of every symbol in include/turboquant_c/turboquant_c.h and
include/turboquant_c/turboquant_b200.h.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libturboquant_b200.so")

TQ_F32, TQ_F16, TQ_U8, TQ_U32 = 0, 1, 2, 3

# Every exported symbol, by header.  tests/test_abi.py checks this list against the
# headers and against the built library.
SYMBOLS_C = [
    "tq_model_load", "tq_model_forward", "tq_model_free",
    "tq_kv_cache_create", "tq_kv_cache_append", "tq_kv_cache_get_keys_fp16", "tq_kv_cache_get_values_fp16",
    "tq_kv_cache_attention", "tq_kv_cache_seq_length", "tq_kv_cache_free",
    "tq_distributed_init", "tq_distributed_init_local", "tq_distributed_rank", "tq_distributed_world_size",
    "tq_distributed_free",
    "tq_cluster_create", "tq_cluster_add_node", "tq_cluster_plan", "tq_cluster_node_count",
    "tq_cluster_get_layer_start", "tq_cluster_get_layer_end", "tq_cluster_free",
    "tq_model_dequant", "tq_array_free", "tq_version",
]

_lib = None


class LibraryMissing(RuntimeError):
    pass


def load() -> C.CDLL:
    """Return the loaded library, raising LibraryMissing if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise LibraryMissing(
            f"{LIB_PATH} not found: build it with `python -m turboquant_mlx_core_b200.build` "
            "(needs nvcc; there is no CPU fallback)")
    L = C.CDLL(LIB_PATH)
    vp, i, u32, f32p = C.c_void_p, C.c_int, C.c_uint32, C.c_void_p

    def sig(name, res, args):
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args

    sig("tq_last_error", C.c_char_p, [])
    sig("tq_device_count", i, [])
    sig("tq_set_device", i, [i])
    sig("tq_version", C.c_char_p, [])

    sig("tq_array_create", vp, [vp, i, i, C.POINTER(C.c_int)])
    sig("tq_array_wrap_device", vp, [vp, i, i, C.POINTER(C.c_int)])
    sig("tq_array_ndim", i, [vp])
    sig("tq_array_dim", i, [vp, i])
    sig("tq_array_dtype", i, [vp])
    sig("tq_array_nbytes", C.c_size_t, [vp])
    sig("tq_array_data", vp, [vp])
    sig("tq_array_to_host", i, [vp, vp, C.c_size_t])
    sig("tq_array_free", None, [vp])

    sig("tq_codebook_generate", i, [i, f32p, f32p])
    sig("tq_wht_rotate", i, [vp, vp, i, i, u32, u32, i, vp])
    sig("tq_quantize_weight", i, [vp, i, i, vp, i, vp, i, i, i, u32, i, vp, vp, vp, vp, vp])
    sig("tq_quantize_weight_seeded", i, [vp, i, i, vp, i, vp, i, i, i, u32, i, u32, u32, vp, vp, vp, vp, vp])

    sig("tq_linear_create", vp, [i, i, vp, i, vp, vp, vp, vp, i, vp, i, u32])
    sig("tq_linear_forward", i, [vp, vp, i, i, vp, vp])
    sig("tq_linear_forward_noalloc", i, [vp, vp, i, vp, vp])
    sig("tq_linear_forward_strided", i, [vp, vp, i, vp, C.c_long, vp])
    sig("tq_linear_noalloc_scratch_limit", C.c_size_t, [])
    sig("tq_linear_forward_group", i, [C.POINTER(C.c_void_p), i, vp, i, C.POINTER(C.c_void_p), vp])
    sig("tq_linear_dequantize", i, [vp, vp, i, vp])
    sig("tq_linear_status", i, [vp])
    sig("tq_linear_forward_scatter", i, [vp, vp, i, C.POINTER(C.c_void_p), i, C.c_long, C.c_long, vp])
    sig("tq_linear_forward_scatter_signal", i, [vp, vp, i, C.POINTER(C.c_void_p), i, C.c_long, C.c_long,
                                                C.POINTER(C.c_void_p), i, C.c_uint, vp])
    sig("tq_linear_wait_peers", i, [vp, vp, i, C.c_uint, vp])
    sig("tq_shared_alloc", vp, [C.c_size_t])
    sig("tq_shared_free", None, [vp])
    sig("tq_shared_export", i, [vp, vp, C.c_size_t])
    sig("tq_shared_open", vp, [vp, C.c_size_t])
    sig("tq_shared_close", i, [vp])
    sig("tq_exchange_create", vp, [i, i])
    sig("tq_exchange_broadcast", i, [vp, vp, C.POINTER(C.c_void_p), i, i, C.c_long, C.c_long, C.c_long, C.POINTER(C.c_void_p), i, vp])
    sig("tq_exchange_wait", i, [vp, vp, i, vp])
    sig("tq_exchange_sum_f16", i, [vp, i, C.c_long, C.c_long, vp, vp, vp])
    sig("tq_rmsnorm_f16", i, [vp, vp, vp, C.c_long, i, C.c_float, vp])
    sig("tq_rope_f16", i, [vp, vp, C.c_long, i, i, C.c_float, vp])
    sig("tq_rope_qk_f16", i, [vp, vp, vp, C.c_long, i, i, i, C.c_float, vp])
    sig("tq_exchange_sum_f16_rmsnorm", i, [vp, i, C.c_long, C.c_long, i, vp, vp, vp, vp, C.c_float, vp])
    sig("tq_swiglu_f16", i, [vp, vp, C.c_long, i, vp])
    sig("tq_exchange_merge_attention", i, [vp, vp, i, C.c_long, i, C.c_long, C.c_long, vp, vp])
    sig("tq_linear_forward_allgather", i, [vp, vp, vp, i, C.POINTER(C.c_void_p), i, C.c_long, C.c_long, C.POINTER(C.c_void_p), i,
                                            vp, i, vp])
    sig("tq_exchange_status", i, [vp])
    sig("tq_exchange_free", None, [vp])
    sig("tq_linear_in_features", i, [vp])
    sig("tq_linear_out_features", i, [vp])
    sig("tq_linear_free", None, [vp])

    sig("tq_model_load", vp, [C.c_char_p])
    sig("tq_model_forward", vp, [vp, vp])
    sig("tq_model_free", None, [vp])
    sig("tq_model_dequant", i, [C.c_char_p, C.c_char_p])
    sig("tq_model_layer_count", i, [vp])
    sig("tq_model_layer_name", C.c_char_p, [vp, i])
    sig("tq_model_layer", vp, [vp, C.c_char_p])

    sig("tq_kv_cache_create", vp, [i, i, i, i, i, i])
    sig("tq_kv_cache_append", None, [vp, i, vp, vp])
    sig("tq_kv_cache_get_keys_fp16", vp, [vp, i, i, i])
    sig("tq_kv_cache_get_values_fp16", vp, [vp, i, i, i])
    sig("tq_kv_cache_attention", vp, [vp, i, vp, i, i])
    sig("tq_kv_cache_seq_length", i, [vp])
    sig("tq_kv_cache_free", None, [vp])

    sig("tq_kv_append", i, [vp, i, vp, vp, i, i, vp])
    sig("tq_kv_get_fp16", i, [vp, i, i, i, i, vp, vp])
    sig("tq_kv_export", i, [vp, i, vp, vp, vp, vp, vp, vp])
    sig("tq_kv_snapshot", C.c_long, [vp, vp, C.c_size_t, u32, u32])
    sig("tq_kv_restore", i, [vp, vp, C.c_size_t])
    sig("tq_kv_delta", C.c_long, [vp, vp, C.c_size_t, C.c_uint32, C.c_uint32])
    sig("tq_kv_apply_delta", i, [vp, vp, C.c_size_t])
    sig("tq_kv_reserve", i, [vp, i, i, vp])
    sig("tq_kv_set_attention_kernel", i, [vp, i])
    sig("tq_kv_attention_status", i, [vp])
    sig("tq_kv_append_batch", i, [C.POINTER(C.c_void_p), i, i, vp, vp, i, vp])
    sig("tq_kv_attention", i, [C.POINTER(C.c_void_p), i, i, vp, i, i, vp, i, i, i, vp])
    sig("tq_kv_attention_lse", i, [C.POINTER(C.c_void_p), i, i, vp, i, i, vp, vp, i, i, i, vp])

    sig("tq_codebook_fit", i, [vp, C.c_long, i, i, vp, vp, C.POINTER(C.c_int), vp])
    sig("tq_fit_layer_codebooks", i, [vp, i, i, u32, i, i, i, vp, vp, vp, vp, vp])
    sig("tq_adaptive_block_size", u32, [i, u32])
    sig("tq_layer_index", i, [C.c_char_p])
    sig("tq_is_sensitive_layer", i, [i, i, i, i])
    sig("tq_qjl_compress", i, [vp, i, i, i, i, u32, vp, vp, vp])
    sig("tq_qjl_dot_correction", i, [vp, vp, vp, i, i, i, i, i, vp, vp])
    sig("tq_linear_forward_allgather_packets", i, [vp, vp, vp, i, vp, C.c_long, C.POINTER(C.c_void_p), i, vp])
    sig("tq_exchange_unpack_packets", i, [vp, C.c_long, vp, vp])
    sig("tq_exchange_wait_packets", i, [vp, vp, C.c_long, i, vp, C.c_long, vp])
    sig("tq_exchange_sum_packets", i, [vp, vp, vp, C.c_long, vp, vp, vp])
    sig("tq_exchange_sum_packets_rmsnorm", i, [vp, vp, vp, C.c_long, i, vp, vp, vp, vp, C.c_float, vp])
    sig("tq_decode_buffer_create", vp, [i, i, i])
    sig("tq_decode_buffer_free", None, [vp])
    sig("tq_decode_buffer_window_size", i, [vp])
    sig("tq_decode_buffer_current_length", i, [vp])
    sig("tq_decode_buffer_rebuild", i, [vp, vp, vp, i, i, vp])
    sig("tq_decode_buffer_append_token", i, [vp, vp, vp, i, vp])
    sig("tq_decode_buffer_slide_window", i, [vp, vp, vp, i, i, vp])
    sig("tq_decode_buffer_keys", i, [vp, i, i, vp, vp])
    sig("tq_decode_buffer_values", i, [vp, i, i, vp, vp])
    sig("tq_hybrid_attention", i, [vp, vp, i, vp, i, i, vp, vp])

    sig("tq_distributed_init", vp, [C.c_char_p, C.c_char_p])
    sig("tq_distributed_init_local", vp, [])
    sig("tq_distributed_rank", i, [vp])
    sig("tq_distributed_world_size", i, [vp])
    sig("tq_distributed_free", None, [vp])

    sig("tq_cluster_create", vp, [i, i, i])
    sig("tq_cluster_add_node", i, [vp, C.c_char_p, C.c_double])
    sig("tq_cluster_plan", i, [vp])
    sig("tq_cluster_node_count", i, [vp])
    sig("tq_cluster_get_layer_start", i, [vp, i])
    sig("tq_cluster_get_layer_end", i, [vp, i])
    sig("tq_cluster_free", None, [vp])
    _lib = L
    return L


def last_error() -> str:
    return load().tq_last_error().decode()


class TQError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise TQError(f"{what}: {last_error()}")
