"""ctypes binding of librelay_b200.so (include/relay_b200.h).

The library is the product: there is no Python or CPU fallback behind it. Loading fails
loudly when it has not been built (`python -m relay_b200.build`).
"""
from __future__ import annotations

import ctypes as C
import os

from .types import CModelConfig, CWeights

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "librelay_b200.so")

ERR_INVALID_ARGUMENT, ERR_OUT_OF_RANGE, ERR_RUNTIME, ERR_LOGIC = 1, 2, 3, 4
DECODE_SLICE = 512
PREFILL_ROWS = 64
NCCL_ID_BYTES = 128
KV_LINK_HANDLE_BYTES = 128
STATIC_DECODE_SCRATCH_BYTES = 8 << 20

LAYER_CB = C.CFUNCTYPE(None, C.c_void_p, C.c_int)


class CTokenMeta(C.Structure):
    _fields_ = [("pos", C.c_void_p), ("seq", C.c_void_p), ("table_off", C.c_void_p), ("tables", C.c_void_p)]


class CAttnShape(C.Structure):
    _fields_ = [("heads", C.c_int32), ("kv_heads", C.c_int32), ("head_dim", C.c_int32), ("block_size", C.c_int32),
                ("q_stride", C.c_int32), ("o_stride", C.c_int32)]


class CSamplingParams(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("top_k", C.c_int32), ("reserved", C.c_int32),
                ("seed", C.c_uint64), ("index", C.c_uint64)]


class CProfile(C.Structure):
    _fields_ = [("total_ms", C.c_double), ("decode_attn_ms", C.c_double), ("prefill_attn_ms", C.c_double),
                ("forwards", C.c_uint64), ("decode_attn_calls", C.c_uint64), ("prefill_attn_calls", C.c_uint64)]


# name -> (restype, argtypes); every symbol include/relay_b200.h declares
P, I, F, SZ, U32 = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_uint32
SIGNATURES = {
    "rb200_last_error": (C.c_char_p, []),
    "rb200_last_error_kind": (I, []),
    "rb200_device_count": (I, []),
    "rb200_flags_from_env": (U32, []),
    "rb200_rope_inv_freq": (I, [C.POINTER(CModelConfig), P]),
    "rb200_quantize_rows_int8": (I, [P, I, I, P, P]),
    "rb200_create": (P, [C.POINTER(CModelConfig), C.POINTER(CWeights), I, I, I, I, I, U32]),
    "rb200_destroy": (None, [P]),
    "rb200_name": (C.c_char_p, [P]),
    "rb200_get_config": (I, [P, C.POINTER(CModelConfig)]),
    "rb200_get_kv_layout": (I, [P, P]),
    "rb200_forward": (I, [P, I, P, P, P, P, P, P, I, LAYER_CB, P, P, SZ]),
    "rb200_forward_greedy": (I, [P, I, P, P, P, P, P, P, I, LAYER_CB, P, P, P, SZ]),
    "rb200_forward_sample": (I, [P, I, P, P, P, P, P, P, I, LAYER_CB, P, P, P, P, SZ]),
    "rb200_decode_open": (I, [P, I, P, P, P]),
    "rb200_decode_set_slot": (I, [P, I, I, I, P]),
    "rb200_decode_step": (I, [P, P, I, P, P, P, P, P, P, SZ]),
    "rb200_decode_close": (I, [P]),
    "rb200_kv_block_bytes": (SZ, [P]),
    "rb200_read_kv_layer": (I, [P, I, P, I, P, P]),
    "rb200_write_kv_layer": (I, [P, I, P, I, P, P]),
    "rb200_wait_kv_written": (I, [P, I]),
    "rb200_update_weight": (I, [P, C.c_char_p, P, SZ]),
    "rb200_set_profiling": (I, [P, I]),
    "rb200_get_profile": (I, [P, P]),
    "rb200_forward_replay": (I, [P, I, P]),
    "rb200_debug_fill_kv": (I, [P, C.c_uint64]),
    "rb200_kernel_launches": (C.c_uint64, []),
    "rb200_nccl_unique_id": (I, [P]),
    "rb200_nccl_init": (I, [P, P, I, I]),
    "rb200_nccl_finalize": (I, [P]),
    "rb200_send_kv_layer": (I, [P, I, I, P, I]),
    "rb200_recv_kv_layer": (I, [P, I, I, P, I]),
    "rb200_kv_hop_sync": (I, [P, I]),
    "rb200_kv_link_create": (I, [P, I, SZ, P]),
    "rb200_kv_link_connect": (I, [P, I, P]),
    "rb200_kv_link_send_layer": (I, [P, I, I, P, I]),
    "rb200_kv_link_recv_layer": (I, [P, I, I, P, I]),
    "rb200_kv_link_send_layers": (I, [P, I, I, I, P, I]),
    "rb200_kv_link_recv_layers": (I, [P, I, I, I, P, I]),
    "rb200_kv_link_skip_layers": (I, [P, I, I, I]),
    "rb200_kv_link_plan": (I, [SZ, SZ, I, I, P]),
    "rb200_kv_link_connect_local": (I, [P, I, P, I]),
    "rb200_kv_link_skip_layer": (I, [P, I, I]),
    "rb200_kv_link_wait": (I, [P, I, I]),
    "rb200_kv_link_wait_gathered": (I, [P, I, I]),
    "rb200_kv_link_close": (I, [P, I]),
    "rb200_decode_scratch_bytes": (SZ, [C.POINTER(CAttnShape), I, I]),
    "rb200_decode_plan": (SZ, [C.POINTER(CAttnShape), I, I, P, P]),
    "rb200_decode_attention": (I, [C.POINTER(CAttnShape), P, C.POINTER(CTokenMeta), P, I, I, P, P, P, SZ, P, P]),
    "rb200_decode_attention_static": (I, [C.POINTER(CAttnShape), P, C.POINTER(CTokenMeta), P, I, I, P, P, P, P]),
    "rb200_prefill_attention": (I, [C.POINTER(CAttnShape), P, C.POINTER(CTokenMeta), P, I, P, P, P, P]),
    "rb200_reference_attention": (I, [C.POINTER(CAttnShape), P, C.POINTER(CTokenMeta), I, P, P, P, P]),
    "rb200_gemv_scratch_bytes": (SZ, [I, I]),
    "rb200_gemv_int8": (I, [P, P, P, P, I, I, I, I, I, F, P, SZ, P]),
    "rb200_gemv_f16": (I, [P, P, P, I, I, I, I, I, F, P, SZ, P]),
    "rb200_gemm": (I, [P, P, P, P, P, I, I, I, I, I, F, P]),
    "rb200_gemm_status": (I, []),
    "rb200_rmsnorm": (I, [P, P, P, P, I, I, I, F, P]),
    "rb200_embed": (I, [P, P, P, I, I, I, P]),
    "rb200_qkv_post": (I, [P, P, P, C.POINTER(CTokenMeta), I, P, P, I, I, I, I, P]),
    "rb200_silu_mul": (I, [P, P, I, I, I, P]),
    "rb200_f32_to_f16": (I, [P, P, SZ, P]),
    "rb200_kv_gather": (I, [P, P, P, I, SZ, P, P]),
    "rb200_kv_scatter": (I, [P, P, P, I, SZ, P, P]),
    "rb200_argmax_rows": (I, [P, I, I, P, P, P]),
    "rb200_sample_rows": (I, [P, I, I, P, P, P, P]),
}

_lib = None


class B200Error(RuntimeError):
    pass


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200Error(f"{LIB_PATH} is missing: build it with `python -m relay_b200.build` "
                            "(there is no fallback implementation)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


_KINDS = {ERR_INVALID_ARGUMENT: ValueError, ERR_OUT_OF_RANGE: IndexError, ERR_RUNTIME: B200Error, ERR_LOGIC: TypeError}


def raise_last_error():
    """Maps the library's error kinds onto Python's closest exceptions: invalid argument ->
    ValueError, out of range -> IndexError, runtime (CUDA / NCCL) -> B200Error, logic -> TypeError."""
    L = lib()
    raise _KINDS.get(L.rb200_last_error_kind(), B200Error)(L.rb200_last_error().decode())


def check(rc: int) -> int:
    if rc < 0:
        raise_last_error()
    return rc
