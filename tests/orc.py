"""ctypes access to the CPU oracle (oracle/liboracle.so) for tests.  Builds it on demand."""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_LIB = None

F32, F16, Q8_0, Q4_K, Q5_K, Q6_K, BF16 = 0, 1, 8, 12, 13, 14, 30


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(ROOT, "oracle", "liboracle.so")
        srcs = [os.path.join(ROOT, "oracle", f) for f in ("oracle_capi.cpp", "forward.hpp", "quants.hpp")]
        if not os.path.exists(path) or any(os.path.getmtime(s) > os.path.getmtime(path) for s in srcs if os.path.exists(s)):
            subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "liboracle.so"],
                                  stdout=subprocess.DEVNULL)
        L = C.CDLL(path)
        L.orc_last_error.restype = C.c_char_p
        L.orc_storage_bytes.restype = C.c_uint64
        L.orc_storage_bytes.argtypes = [C.c_int32, C.c_uint64]
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_greedy_token.restype = C.c_int32
        for name in ("orc_model_create", "orc_state_create", "orc_state_clone", "orc_drafter_create"):
            getattr(L, name).restype = C.c_void_p
        L.orc_state_n_pos.restype = C.c_uint64
        _LIB = L
    return _LIB


def _p(a, t=C.c_void_p):
    return a.ctypes.data_as(t)


def check(rc):
    if rc != 0:
        raise RuntimeError(lib().orc_last_error().decode())


def storage_bytes(dtype, n):
    return int(lib().orc_storage_bytes(dtype, n))


def quantize(dtype, x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.zeros(storage_bytes(dtype, x.size), dtype=np.uint8)
    check(lib().orc_quantize(C.c_int32(dtype), _p(x), C.c_uint64(x.size), _p(out)))
    return out


def dequant(dtype, raw, n):
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    out = np.zeros(n, dtype=np.float32)
    check(lib().orc_dequant(C.c_int32(dtype), _p(raw), C.c_uint64(n), _p(out)))
    return out


def matmul(dtype, raw, n_in, n_out, x):
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, n_in)
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    y = np.zeros((x.shape[0], n_out), dtype=np.float32)
    check(lib().orc_matmul(C.c_int32(dtype), _p(raw), C.c_uint64(n_in), C.c_uint64(n_out), _p(x),
                           C.c_int32(x.shape[0]), _p(y)))
    return y


def greedy_token(row):
    row = np.ascontiguousarray(row, dtype=np.float32)
    return int(lib().orc_greedy_token(_p(row), C.c_uint64(row.size)))
