"""ctypes loader for ``oracle/_ref/libref_fp8.so`` (the reference's software FP8 cast).

Test infrastructure.  The library is built by ``oracle/ref_fp8/Makefile`` from the
reference's ``src/common/float8.h``; it exists only where the reference checkout was
available at build time, so ``available()`` must be consulted first.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libref_fp8.so")
_lib = None


def available() -> bool:
    return os.path.exists(_PATH)


def _load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_PATH)
        for name in ("ref_float_to_e4m3fn", "ref_float_to_e4m3fnuz"):
            getattr(_lib, name).argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_long]
            getattr(_lib, name).restype = None
        for name in ("ref_e4m3fn_to_float", "ref_e4m3fnuz_to_float"):
            getattr(_lib, name).argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_long]
            getattr(_lib, name).restype = None
    return _lib


def float_to_fp8(x: np.ndarray, fnuz: bool) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint8)
    fn = _load().ref_float_to_e4m3fnuz if fnuz else _load().ref_float_to_e4m3fn
    fn(x.ctypes.data, out.ctypes.data, x.size)
    return out


def fp8_to_float(c: np.ndarray, fnuz: bool) -> np.ndarray:
    c = np.ascontiguousarray(c, dtype=np.uint8)
    out = np.empty(c.shape, dtype=np.float32)
    fn = _load().ref_e4m3fnuz_to_float if fnuz else _load().ref_e4m3fn_to_float
    fn(c.ctypes.data, out.ctypes.data, c.size)
    return out


def max_values():
    lib = _load()
    return int(lib.ref_e4m3fn_max()), int(lib.ref_e4m3fnuz_max())
