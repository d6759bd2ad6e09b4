"""ctypes loader of ``libpaged_attention.so`` (the C-ABI in include/paged_attention.h).

There is no fallback: if the library is missing it is built with nvcc, and if
that fails the import error is raised to the caller.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

_LIB = None

# every symbol include/paged_attention.h declares (checked by the CPU tests)
SYMBOLS = [
    "pa_last_error", "pa_pool_create", "pa_pool_destroy", "pa_pool_free_blocks",
    "pa_pool_set_free_order", "pa_pool_layer_storage", "pa_seq_create", "pa_seq_free",
    "pa_seq_reserve", "pa_seq_length", "pa_seq_block_table", "pa_batch_set", "pa_batch_set_sharded", "pa_append",
    "pa_decode", "pa_decode_step", "pa_prefill", "pa_merge_partials", "pa_gather_kv", "pa_build_rope_tables",
    "pa_pool_check", "pa_pool_set_decode_chunk_blocks", "pa_pool_set_decode_cluster", "pa_pool_set_decode_shape", "pa_pool_set_step_kernel", "pa_pool_set_layer_overlap", "pa_pool_set_step_combiners", "pa_pool_step_launches", "pa_qkv_project", "pa_rmsnorm_qkv_project", "pa_rmsnorm", "pa_attention_step", "pa_ffn", "pa_ffn_rows", "pa_block_step", "pa_lm_head", "pa_argmax", "pa_embedding", "pa_decode_token", "pa_out_project", "pa_out_project_rows", "pa_qkv_project_packed", "pa_qkv_project_append", "pa_pack_projection_weights",
    "pa_decode_noalloc", "pa_decode_noalloc_check", "pa_decode_step_sharded_colocated", "pa_exchange_create", "pa_exchange_handle", "pa_exchange_connect",
    "pa_exchange_destroy", "pa_decode_step_sharded", "pa_exchange_buffer", "pa_exchange_connect_ptrs",
    "pa_decode_push", "pa_exchange_merge", "pa_gather_create", "pa_gather_handle", "pa_gather_connect",
    "pa_gather_buffer", "pa_gather_connect_ptrs", "pa_gather_destroy", "pa_decode_step_gathered",
    "pa_gather_wait",
]


LEGACY_SYMBOLS = ["lt_launch_flash_attention", "lt_launch_rope_qkv", "lt_launch_flash_output_layout"]


class FlashAttentionParams(C.Structure):
    """lt_flash_attention_params of include/legacy_kernels.h."""
    _fields_ = [("Q", C.c_void_p), ("K", C.c_void_p), ("V", C.c_void_p), ("O", C.c_void_p),
                ("L", C.c_void_p), ("batch_size", C.c_int), ("num_heads", C.c_int),
                ("num_kv_heads", C.c_int), ("q_seq_len", C.c_int), ("kv_seq_len", C.c_int),
                ("kv_stride", C.c_int), ("d_head", C.c_int), ("scale", C.c_float),
                ("causal", C.c_int), ("dtype", C.c_int), ("stream", C.c_void_p)]


class AttentionWeights(C.Structure):
    """pa_attention_weights of include/paged_attention.h."""
    _fields_ = [("input_norm", C.c_void_p), ("wq", C.c_void_p), ("wk", C.c_void_p), ("wv", C.c_void_p),
                ("wo", C.c_void_p), ("norm_layer_stride", C.c_int64), ("wq_layer_stride", C.c_int64),
                ("wkv_layer_stride", C.c_int64), ("wo_layer_stride", C.c_int64), ("rms_eps", C.c_float),
                ("hidden", C.c_int)]


class FfnWeights(C.Structure):
    """pa_ffn_weights of include/paged_attention.h."""
    _fields_ = [("ffn_norm", C.c_void_p), ("gate", C.c_void_p), ("up", C.c_void_p), ("down", C.c_void_p),
                ("norm_layer_stride", C.c_int64), ("gate_layer_stride", C.c_int64), ("up_layer_stride", C.c_int64),
                ("down_layer_stride", C.c_int64), ("rms_eps", C.c_float), ("hidden", C.c_int), ("inter", C.c_int)]


class ModelWeights(C.Structure):
    """pa_model_weights of include/paged_attention.h."""
    _fields_ = [("embed_tokens", C.c_void_p), ("attention", C.POINTER(AttentionWeights)), ("ffn", C.POINTER(FfnWeights)),
                ("final_norm", C.c_void_p), ("lm_head", C.c_void_p), ("vocab", C.c_int), ("rms_eps", C.c_float)]


class PagedAttentionError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"[{code}] {msg}")
        self.code = code


def lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    path = _build.LIB
    if not os.path.exists(path):
        _build.build()
    L = C.CDLL(path)
    vp, i, i64, f = C.c_void_p, C.c_int, C.c_int64, C.c_float
    ip = C.POINTER(C.c_int)
    L.pa_last_error.restype = C.c_char_p
    L.pa_last_error.argtypes = []
    sigs = {
        "pa_pool_create": [C.POINTER(vp), i, i, i, i, i, i],
        "pa_pool_destroy": [vp],
        "pa_pool_free_blocks": [vp, ip],
        "pa_pool_set_free_order": [vp, vp, i],
        "pa_pool_layer_storage": [vp, i, C.POINTER(vp), C.POINTER(C.c_uint64)],
        "pa_seq_create": [vp, ip],
        "pa_seq_free": [vp, i],
        "pa_seq_reserve": [vp, i, i],
        "pa_seq_length": [vp, i, ip],
        "pa_seq_block_table": [vp, i, C.POINTER(C.POINTER(C.c_int32)), ip],
        "pa_batch_set": [vp, vp, vp, i, vp],
        "pa_batch_set_sharded": [vp, vp, vp, vp, vp, vp, i, vp],
        "pa_append": [vp, i, vp, vp, vp, vp, vp, vp, vp],
        "pa_decode": [vp, i, vp, vp, i64, vp, vp, f, vp],
        "pa_decode_step": [vp, i, i, vp, vp, vp, i64, i64, vp, vp, vp, vp, i64, i64, vp, f, vp],
        "pa_prefill": [vp, i, vp, vp, vp, f, vp],
        "pa_merge_partials": [vp, vp, i, i, vp, vp, vp, vp],
        "pa_gather_kv": [vp, i, i, vp, vp, i, vp],
        "pa_build_rope_tables": [vp, vp, i],
        "pa_pool_check": [vp, vp],
        "pa_pool_set_decode_chunk_blocks": [vp, i],
        "pa_pool_set_decode_shape": [vp, i, i],
        "pa_pool_set_step_kernel": [vp, i],
        "pa_pool_set_layer_overlap": [vp, i],
        "pa_pool_set_step_combiners": [vp, i],
        "pa_pool_step_launches": [vp, C.POINTER(C.c_longlong)],
        "pa_qkv_project": [vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i64, i64, i64, i64, i64, vp],
        "pa_qkv_project_append": [vp, i, vp, vp, vp, vp, vp, vp, vp, i, vp],
        "pa_rmsnorm_qkv_project": [vp, vp, i64, f, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i64, i64, i64, i64, i64, vp],
        "pa_rmsnorm": [vp, vp, vp, i, i, f, vp],
        "pa_attention_step": [vp, vp, i, i, vp, vp, vp, i, vp, vp, f, vp],
        "pa_pool_set_decode_cluster": [vp, i],
        "pa_ffn": [vp, i, vp, vp, vp, i, i, vp],
        "pa_ffn_rows": [vp, vp, i, vp, vp, vp, i, i, vp],
        "pa_lm_head": [vp, vp, f, vp, vp, i, i, i, vp],
        "pa_argmax": [vp, vp, i, i, vp],
        "pa_embedding": [vp, vp, vp, i, i, i, vp],
        "pa_decode_token": [vp, vp, vp, vp, vp, vp, vp, f, i, vp],
        "pa_block_step": [vp, vp, i, i, vp, vp, vp, vp, vp, vp, f, vp],
        "pa_out_project": [vp, vp, vp, vp, i, i, i, i, i64, i64, i64, vp],
        "pa_out_project_rows": [vp, vp, vp, vp, vp, i, i, i, vp],
        "pa_qkv_project_packed": [vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i64, i64, i64, i64, i64, vp, vp],
        "pa_pack_projection_weights": [vp, vp, i, i, vp],
        "pa_decode_noalloc": [vp, i, i, vp, i, vp, i, vp, vp, i64, vp, f, vp],
        "pa_decode_noalloc_check": [vp],
        "pa_decode_step_sharded_colocated": [vp, vp, i, i, i, vp, vp, vp, i64, i64, vp, vp, vp, vp, i64, i64, f, vp],
        "pa_exchange_create": [C.POINTER(vp), i, i, i, i, i],
        "pa_exchange_handle": [vp, vp],
        "pa_exchange_connect": [vp, vp],
        "pa_exchange_destroy": [vp],
        "pa_exchange_buffer": [vp, C.POINTER(vp), C.POINTER(C.c_uint64)],
        "pa_exchange_connect_ptrs": [vp, C.POINTER(vp)],
        "pa_decode_push": [vp, vp, i, vp, f, vp],
        "pa_exchange_merge": [vp, vp, vp, i64, vp],
        "pa_decode_step_sharded": [vp, vp, i, i, vp, vp, vp, i64, i64, vp, vp, vp, vp, i64, i64, f, vp],
        "pa_gather_create": [C.POINTER(vp), i, i, i, i, i, i],
        "pa_gather_handle": [vp, vp],
        "pa_gather_connect": [vp, vp],
        "pa_gather_buffer": [vp, C.POINTER(vp), C.POINTER(C.c_uint64)],
        "pa_gather_connect_ptrs": [vp, C.POINTER(vp)],
        "pa_gather_destroy": [vp],
        "pa_decode_step_gathered": [vp, vp, vp, vp, vp, i64, i64, vp, vp, vp, f, i, vp, C.POINTER(vp)],
        "pa_gather_wait": [vp, vp, vp, C.POINTER(vp)],
        "lt_launch_flash_attention": [vp],
        "lt_launch_rope_qkv": [vp, vp, vp, vp, vp, vp, vp, vp, i, i, vp],
        "lt_launch_flash_output_layout": [vp, vp, i, vp],
    }
    for name, args in sigs.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = i
    _LIB = L
    return L


def check(code: int) -> None:
    if code != 0:
        raise PagedAttentionError(code, lib().pa_last_error().decode())
