"""ctypes binding of libb200mla.so (declarations: include/b200_mla.h).

There is deliberately no fallback: if the library is missing or fails to load, importing this
module raises, and so does every call into the package.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libb200mla.so")

Q_BF16, Q_E4M3, Q_BF16_CAST_E4M3 = 0, 1, 2
Q_AMAX_PARTS = 256
KV_E4M3, KV_MXFP4, KV_HYBRID = 0, 1, 2
IMPL_AUTO, IMPL_GENERIC, IMPL_TCGEN05 = 0, 1, 2

_vp, _i32, _i64, _f32 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_float


class DecodeArgs(ctypes.Structure):
    """struct b200_mla_decode_args"""
    _fields_ = [
        ("batch", _i32), ("heads", _i32), ("q_len", _i32), ("q_format", _i32), ("kv_format", _i32),
        ("causal", _i32), ("page_size", _i32), ("impl", _i32), ("sm_scale", _f32), ("max_ctas", _i32),
        ("q", _vp), ("q_row_stride", _i64), ("q_head_stride", _i64), ("q_scale", _vp),
        ("kv_codes", _vp), ("kv_codes_stride", _i64),
        ("kv_block_scales", _vp), ("kv_block_scales_stride", _i64),
        ("kv_rope", _vp), ("kv_rope_stride", _i64),
        ("kv_scale", _vp), ("num_slots", _i64),
        ("kv_indptr", _vp), ("kv_indices", _vp), ("kv_page_indptr", _vp), ("total_kv_hint", _i64),
        ("kv_pos_offset", _vp), ("kv_total_len", _vp),
        ("out", _vp), ("out_o_f32", _vp), ("out_lse", _vp),
        ("workspace", _vp), ("workspace_bytes", _i64),
    ]


class KvAppendArgs(ctypes.Structure):
    """struct b200_mla_kv_append_args"""
    _fields_ = [
        ("rows_bf16", _vp), ("n", _i64), ("row_stride", _i64), ("slots", _vp), ("base_slot", _i64), ("num_slots", _i64),
        ("kv_format", _i32), ("reserved", _i32),
        ("kv_codes", _vp), ("kv_codes_stride", _i64), ("kv_block_scales", _vp), ("kv_block_scales_stride", _i64),
        ("kv_rope", _vp), ("kv_rope_stride", _i64), ("kv_scale", _vp), ("status", _vp),
    ]


class PeerMergeArgs(ctypes.Structure):
    """struct b200_mla_peer_merge_args"""
    _fields_ = [
        ("world", _i32), ("rank", _i32), ("epoch", ctypes.c_uint32), ("wait_limit_ms", ctypes.c_uint32),
        ("bases", ctypes.POINTER(_vp)), ("rows", _i64), ("out", _vp), ("workspace", _vp),
    ]


PEER_HANDLE_BYTES = 64

EXPORTS = ("b200_mla_version", "b200_mla_last_error", "b200_mla_workspace_bytes", "b200_mla_decode",
           "b200_mla_combine", "b200_mla_quantize_fp8", "b200_mla_q_amax", "b200_mla_set_stage1_events",
           "b200_mla_decode_static", "b200_mla_read_status", "b200_mla_reset_status", "b200_mla_kv_append",
           "b200_mla_peer_exchange_bytes", "b200_mla_peer_partial_offset", "b200_mla_peer_alloc", "b200_mla_peer_open",
           "b200_mla_peer_close", "b200_mla_peer_free", "b200_mla_peer_merge")
STATUS_TIMEOUT, STATUS_BAD_PAGE = 1, 2


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m amd_optimization_challenge_b200.build` "
            "(needs nvcc; there is no CPU fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    lib.b200_mla_version.restype = _i32
    lib.b200_mla_last_error.restype = ctypes.c_char_p
    lib.b200_mla_workspace_bytes.restype = _i64
    lib.b200_mla_workspace_bytes.argtypes = [_i32, _i32, _i32]
    lib.b200_mla_decode.restype = _i32
    lib.b200_mla_decode.argtypes = [ctypes.POINTER(DecodeArgs), _vp]
    lib.b200_mla_combine.restype = _i32
    lib.b200_mla_combine.argtypes = [_vp, _vp, _i32, _i64, _i64, _i64, _vp, _vp, _vp]
    lib.b200_mla_quantize_fp8.restype = _i32
    lib.b200_mla_quantize_fp8.argtypes = [_vp, _i64, _vp, _vp, _vp, _vp]
    lib.b200_mla_q_amax.restype = _i32
    lib.b200_mla_q_amax.argtypes = [_vp, _i64, _vp, _vp]
    lib.b200_mla_decode_static.restype = _i32
    lib.b200_mla_decode_static.argtypes = [ctypes.POINTER(DecodeArgs), _vp]
    lib.b200_mla_read_status.restype = _i32
    lib.b200_mla_read_status.argtypes = [_vp, _vp, _vp]
    lib.b200_mla_reset_status.restype = _i32
    lib.b200_mla_reset_status.argtypes = [_vp, _vp]
    lib.b200_mla_kv_append.restype = _i32
    lib.b200_mla_kv_append.argtypes = [ctypes.POINTER(KvAppendArgs), _vp]
    lib.b200_mla_peer_exchange_bytes.restype = _i64
    lib.b200_mla_peer_exchange_bytes.argtypes = [_i64]
    lib.b200_mla_peer_partial_offset.restype = _i64
    lib.b200_mla_peer_partial_offset.argtypes = [_i64, ctypes.c_uint32]
    lib.b200_mla_peer_alloc.restype = _i32
    lib.b200_mla_peer_alloc.argtypes = [_i64, ctypes.POINTER(_vp), ctypes.c_char_p]
    lib.b200_mla_peer_open.restype = _i32
    lib.b200_mla_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(_vp)]
    lib.b200_mla_peer_close.restype = _i32
    lib.b200_mla_peer_close.argtypes = [_vp]
    lib.b200_mla_peer_free.restype = _i32
    lib.b200_mla_peer_free.argtypes = [_vp]
    lib.b200_mla_peer_merge.restype = _i32
    lib.b200_mla_peer_merge.argtypes = [ctypes.POINTER(PeerMergeArgs), _vp]
    lib.b200_mla_set_stage1_events.restype = _i32
    lib.b200_mla_set_stage1_events.argtypes = [_vp, _vp]
    return lib


lib = _load()


def check(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"{what} failed with status {status}: {lib.b200_mla_last_error().decode()}")
