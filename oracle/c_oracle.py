"""ctypes loader for oracle/libmla_oracle.so (test infrastructure only)."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
FMT = {"fp8": 0, "mxfp4": 1, "hybrid": 2}


def build() -> str:
    subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return os.path.join(_HERE, "libmla_oracle.so")


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libmla_oracle.so")
        if not os.path.exists(path):
            build()
        L = ctypes.CDLL(path)
        L.mo_e4m3fn_to_float.restype = ctypes.c_float
        L.mo_e4m3fn_to_float.argtypes = [ctypes.c_uint8]
        L.mo_e2m1_to_float.restype = ctypes.c_float
        L.mo_e2m1_to_float.argtypes = [ctypes.c_uint8]
        L.mo_e8m0_to_float.restype = ctypes.c_float
        L.mo_e8m0_to_float.argtypes = [ctypes.c_uint8]
        L.mo_mla_decode.restype = ctypes.c_int
        _LIB = L
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def quantize_mxfp4(x: np.ndarray):
    x = np.ascontiguousarray(x, dtype=np.float32)
    n = x.shape[-1]
    rows = x.reshape(-1, n)
    packed = np.zeros((rows.shape[0], n // 2), np.uint8)
    scales = np.zeros((rows.shape[0], n // 32), np.uint8)
    L = lib()
    for r in range(rows.shape[0]):
        for b in range(n // 32):
            L.mo_quantize_mxfp4_block(
                ctypes.c_void_p(rows.ctypes.data + 4 * (r * n + b * 32)),
                ctypes.c_void_p(packed.ctypes.data + r * (n // 2) + b * 16),
                ctypes.c_void_p(scales.ctypes.data + r * (n // 32) + b))
    return packed.reshape(*x.shape[:-1], n // 2), scales.reshape(*x.shape[:-1], n // 32)


def mla_decode(q_f32: np.ndarray, fmt: str, planes, scales, kv_indptr, kv_indices, heads, q_len,
               causal, sm_scale, pos_offset=None, total_len=None):
    """planes: list of up to three 2-D uint8 arrays; scales: (s0, s2)."""
    q_f32 = np.ascontiguousarray(q_f32, dtype=np.float32)
    planes = [np.ascontiguousarray(p, dtype=np.uint8) for p in planes] + [None] * (3 - len(planes))
    kv_indptr = np.ascontiguousarray(kv_indptr, dtype=np.int32)
    ki = None if kv_indices is None else np.ascontiguousarray(kv_indices, dtype=np.int32)
    po = None if pos_offset is None else np.ascontiguousarray(pos_offset, dtype=np.int32)
    tl_ = None if total_len is None else np.ascontiguousarray(total_len, dtype=np.int32)
    batch = len(kv_indptr) - 1
    out = np.zeros((batch * q_len, heads, 512), np.float32)
    lse = np.zeros((batch * q_len, heads), np.float32)
    st = [0 if p is None else p.strides[0] for p in planes]
    rc = lib().mo_mla_decode(
        _p(q_f32), ctypes.c_int(FMT[fmt]), _p(planes[0]), _p(planes[1]), _p(planes[2]),
        ctypes.c_int64(st[0]), ctypes.c_int64(st[1]), ctypes.c_int64(st[2]),
        ctypes.c_float(scales[0]), ctypes.c_float(scales[1]),
        _p(kv_indptr), _p(ki), ctypes.c_int(batch), ctypes.c_int(heads), ctypes.c_int(q_len),
        ctypes.c_int(1 if causal else 0), _p(po), _p(tl_), ctypes.c_float(sm_scale),
        _p(out), _p(lse))
    if rc != 0:
        raise RuntimeError(f"mo_mla_decode failed: {rc}")
    return out, lse
