"""ctypes loader for ``oracle/_ref/libref_ar_fusion.so``: the reference's own fused CUDA kernels.

Test / benchmark infrastructure.  The library is built by ``oracle/ref_kernels/Makefile`` from the
reference's ``src/impl/all_reduce_fusion_impl.h`` (compiled for sm_100a where the reference checkout is
present); ``available()`` must be consulted first.  One process drives all GPUs with peer access, as the
reference's C++ harness does (``test/cpp/test_all_reduce.cpp:337-356``).
"""
from __future__ import annotations

import ctypes
import os

import torch

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libref_ar_fusion.so")
_lib = None


def available() -> bool:
    return os.path.exists(_PATH)


def _load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_PATH)
        _lib.ref_arf_last_error.restype = ctypes.c_char_p
        _lib.ref_arf_run.restype = ctypes.c_int
        _lib.ref_arf_run.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p,
                                     ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                     ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_float)]
    return _lib


def run(parts, residual, weight, eps, warmup=5, iters=50):
    """The reference's fused call (bf16, policy 1: e4m3fn, per-token scale = amax / 240) on ``len(parts)`` GPUs.
    ``parts``: CPU bf16 tensors [tokens, hidden] (hidden 1024, 2048 or 4096).  Returns
    ``((residual_out, norm_out, scale) of rank 0 on the CPU, microseconds per call)``."""
    world = len(parts)
    tokens, hidden = parts[0].shape
    parts = [p.contiguous() for p in parts]
    residual, weight = residual.contiguous(), weight.contiguous()
    res_out = torch.empty_like(residual)
    norm_out = torch.empty(tokens, hidden, dtype=torch.uint8)
    scale = torch.empty(tokens, 1, dtype=torch.float32)
    xs = (ctypes.c_void_p * world)(*[p.data_ptr() for p in parts])
    us = ctypes.c_float(0)
    lib = _load()
    rc = lib.ref_arf_run(world, tokens, hidden, xs, residual.data_ptr(), weight.data_ptr(), eps, res_out.data_ptr(),
                         norm_out.data_ptr(), scale.data_ptr(), warmup, iters, ctypes.byref(us))
    if rc:
        raise RuntimeError("reference kernels: " + lib.ref_arf_last_error().decode())
    return (res_out, norm_out.view(torch.float8_e4m3fn), scale), float(us.value)
