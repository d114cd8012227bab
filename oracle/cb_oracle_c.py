"""ctypes front end of the C oracle (oracle/cb_oracle.c).  TEST INFRASTRUCTURE ONLY.

Loads ``oracle/libcb_oracle.so`` (built by ``make -C oracle``) and exposes numpy-level wrappers
with the same names and meanings as ``oracle/cb_oracle.py``.  The shipped package never imports
this module; the test suite, the smoke entry point and the benchmark's CPU-baseline leg do.
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libcb_oracle.so")
_lib = None

_i64, _int = ctypes.c_int64, ctypes.c_int
_pf = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_pi = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")


def build(force: bool = False) -> str:
    """Compile the C oracle with the Makefile next to it."""
    src = os.path.join(_HERE, "cb_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B"])
    return _SO


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = ctypes.CDLL(_SO)
        L.cbo_num_threads.restype = _int
        L.cbo_unpack_codes.argtypes = [_pi, _i64, _i64, _int, _i64, _pi]
        L.cbo_pack_codes.argtypes = [_pi, _i64, _i64, _int, _pi]
        L.cbo_quantize_affine.argtypes = [_pf, _i64, _i64, _int, _i64, _pi, _pf, _pf]
        L.cbo_gemv_partials.argtypes = [_pf, _i64, _pi, _pf, _pf, _i64, _i64, _int, _i64, _i64, _pf]
        L.cbo_gemv.argtypes = [_pf, _i64, _pi, _pf, _pf, _i64, _i64, _int, _i64, _i64, _pf]
        L.cbo_dequantize.argtypes = [_pi, _pf, _pf, _i64, _i64, _int, _i64, _pf]
        L.cbo_matmul_nt.argtypes = [_pf, _pf, _i64, _i64, _i64, _pf]
        for f in ("cbo_unpack_codes", "cbo_pack_codes", "cbo_quantize_affine", "cbo_gemv_partials",
                  "cbo_gemv", "cbo_dequantize", "cbo_matmul_nt"):
            getattr(L, f).restype = None
        _lib = L
    return _lib


def num_threads() -> int:
    return int(lib().cbo_num_threads())


def use_all_host_threads() -> int:
    """Make the OpenMP loops use every core this process may run on, whatever OMP_NUM_THREADS says."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    L = lib()
    L.cbo_set_num_threads.argtypes = [_int]
    L.cbo_set_num_threads.restype = None
    L.cbo_set_num_threads(n)
    return num_threads()


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def unpack_codes(packed, bits, k):
    packed = _i(packed)
    out = np.empty((packed.shape[0], k), dtype=np.int32)
    lib().cbo_unpack_codes(packed, packed.shape[0], packed.shape[1], bits, k, out)
    return out


def pack_codes(q, bits):
    q = _i(q)
    n, k = q.shape
    out = np.empty((n, math.ceil(k / 32) * bits), dtype=np.int32)
    lib().cbo_pack_codes(q, n, k, bits, out)
    return out


def quantize_affine(w, bits, group_size=128):
    w = _f(w)
    n, k = w.shape
    g = math.ceil(k / group_size)
    q = np.empty((n, k), dtype=np.int32)
    s = np.empty((n, g), dtype=np.float32)
    z = np.empty((n, g), dtype=np.float32)
    lib().cbo_quantize_affine(w, n, k, bits, group_size, q, s, z)
    return q, s, z


def gemv_partials(x, packed, scales, zeros, bits, k, gs, split_k):
    x, packed, scales, zeros = _f(x), _i(packed), _f(scales), _f(zeros)
    c = math.ceil(k / 32)
    p = max(1, min(int(split_k), c))
    out = np.empty((p, x.shape[0], packed.shape[0]), dtype=np.float32)
    lib().cbo_gemv_partials(x, x.shape[0], packed, scales, zeros, packed.shape[0], k, bits, gs, p, out)
    return out


def gemv(x, packed, scales, zeros, bits, k, gs, split_k=1):
    """float32 x W^T with the decode chunk algebra; no bias / activation / output rounding."""
    x, packed, scales, zeros = _f(x), _i(packed), _f(scales), _f(zeros)
    out = np.empty((x.shape[0], packed.shape[0]), dtype=np.float32)
    lib().cbo_gemv(x, x.shape[0], packed, scales, zeros, packed.shape[0], k, bits, gs, int(split_k), out)
    return out


def dequantized_weight(packed, scales, zeros, bits, k, gs):
    packed, scales, zeros = _i(packed), _f(scales), _f(zeros)
    out = np.empty((packed.shape[0], k), dtype=np.float32)
    lib().cbo_dequantize(packed, scales, zeros, packed.shape[0], k, bits, gs, out)
    return out


def matmul_nt(x, wdq):
    """x [M,K] @ wdq[N,K]^T, float32 accumulate."""
    x, wdq = _f(x), _f(wdq)
    out = np.empty((x.shape[0], wdq.shape[0]), dtype=np.float32)
    lib().cbo_matmul_nt(x, wdq, x.shape[0], wdq.shape[0], x.shape[1], out)
    return out
