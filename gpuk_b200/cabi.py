"""ctypes binding of the C ABI in ``include/gpuk_b200.h`` (``libgpuk_core.so``).

This is the same surface a binding for the reference's operator API would link against;
the tests drive the kernels through it, and ``gpuk_b200`` itself uses it for the planning
helper.  There is no fallback: a missing library is an ImportError.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int64, c_uint8, c_uint32, c_uint64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
CORE_LIB = os.path.join(HERE, "libgpuk_core.so")

(OK, ERR_INVALID_ARGUMENT, ERR_CUDA, ERR_UNSUPPORTED, ERR_NOT_READY, ERR_TOO_LARGE, ERR_PEER_TIMEOUT,
 ERR_BAD_LAUNCH) = range(8)
DTYPE_BF16, DTYPE_F16, DTYPE_F32 = 0, 1, 2
QUANT_NONE, QUANT_FP8_E4M3FN_240, QUANT_FP8_E4M3FNUZ_120, QUANT_FP8_E4M3FN_448, QUANT_FP8_E4M3FN_448_STATIC = range(5)
IPC_HANDLE_BYTES = 64
MODE_AUTO, MODE_ONE_SHOT, MODE_TWO_SHOT, MODE_SYMMETRIC = range(4)
SYM_FLAG_BYTES = 2 * 2048 * 8 * 8   # tail of a symmetric buffer that holds the flags (include/gpuk_b200.h)


class Plan(ctypes.Structure):
    _fields_ = [("one_shot", c_int), ("vpt", c_int), ("threads", c_int), ("rows_per_chunk", c_int),
                ("grid", c_int), ("rows", c_int), ("row_vecs", c_int), ("message_bytes", c_int64),
                ("cluster", c_int), ("lead_push", c_int), ("lead_reduce", c_int),
                ("ws", c_int), ("ws_grid", c_int), ("ws_vpt", c_int), ("ws_tf", c_int), ("ws_tr", c_int), ("ws_ts", c_int)]


class GpukError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"gpuk status {status}: {message}")
        self.status = status


if not os.path.exists(CORE_LIB):
    raise ImportError(
        f"{CORE_LIB} is missing: build it with `python gpuk_b200/_build.py` (needs nvcc; there is no CPU fallback)")

lib = ctypes.CDLL(CORE_LIB)

_P = c_void_p
_SIGNATURES = {
    "gpuk_last_error": (c_char_p, []),
    "gpuk_status_string": (c_char_p, [c_int]),
    "gpuk_ws_create": (c_int, [c_int, c_int, c_int, c_int64, c_int64, POINTER(_P)]),
    "gpuk_ws_destroy": (c_int, [_P]),
    "gpuk_ws_get_barrier_handle": (c_int, [_P, POINTER(c_uint8)]),
    "gpuk_ws_get_data_handle": (c_int, [_P, POINTER(c_uint8)]),
    "gpuk_ws_open_barrier_handles": (c_int, [_P, POINTER(c_uint8), c_int]),
    "gpuk_ws_open_data_handles": (c_int, [_P, POINTER(c_uint8), c_int]),
    "gpuk_ws_local_pointers": (c_int, [_P, POINTER(_P), POINTER(_P)]),
    "gpuk_ws_set_peer_pointers": (c_int, [_P, POINTER(_P), POINTER(_P), c_int]),
    "gpuk_ws_attach_symmetric": (c_int, [_P, POINTER(_P), c_int, _P, c_int64]),
    "gpuk_enable_peer_access": (c_int, [c_int]),
    "gpuk_ws_capture_clear": (c_int, [_P]),
    "gpuk_ws_captured_count": (c_int, [_P, POINTER(c_int)]),
    "gpuk_ws_open_captured_handles": (c_int, [_P, POINTER(c_uint8), POINTER(c_int64), c_int, c_int64]),
    "gpuk_tensor_ipc_handle": (c_int, [_P, POINTER(c_uint8)]),
    "gpuk_tensor_ipc_offset": (c_int, [_P, POINTER(c_int64)]),
    "gpuk_allreduce_rms": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int64, c_int, c_int, c_float, c_int, _P]),
    "gpuk_allreduce_inplace": (c_int, [_P, _P, c_int64, c_int, _P]),
    "gpuk_residual_rms_quant": (c_int, [_P, _P, _P, _P, _P, _P, c_int64, c_int, c_int, c_float, c_int, _P]),
    "gpuk_plan_allreduce_rms": (c_int, [c_int, c_int64, c_int, c_int, c_int, c_int, c_int64, POINTER(Plan)]),
    "gpuk_ws_set_oneshot_max_bytes": (c_int, [_P, c_int64]),
    "gpuk_ws_set_option": (c_int, [_P, c_char_p, c_int64]),
    "gpuk_set_tuning": (c_int, [c_char_p, c_int64]),
    "gpuk_ws_set_ready_words": (c_int, [_P, _P, c_int, c_uint32]),
    "gpuk_ws_set_timeout_ns": (c_int, [_P, c_uint64]),
    "gpuk_ws_status": (c_int, [_P, POINTER(c_uint32)]),
    "gpuk_ws_clear_status": (c_int, [_P]),
    "gpuk_ws_selftest_wait": (c_int, [_P, _P]),
    "gpuk_emulated_allreduce_rms": (c_int, [POINTER(_P), c_int, POINTER(_P), _P, _P, POINTER(_P), POINTER(_P),
                                            POINTER(_P), c_int64, c_int, c_int, c_float, c_int, c_int, _P]),
    "gpuk_selfcheck_allreduce_rms": (c_int, [c_int, POINTER(_P), _P, _P, POINTER(_P), POINTER(_P), POINTER(_P),
                                             c_int64, c_int, c_int, c_float, c_int, c_int, _P]),
    "gpuk_selfcheck_status": (c_int, [POINTER(c_uint32), _P]),
    "gpuk_fp8_linear_skinny": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P]),
    "gpuk_fp8_pack_weight": (c_int, [_P, _P, c_int, c_int, _P]),
    "gpuk_fp8_linear_status": (c_int, []),
}
for _name, (_res, _args) in _SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    return lib.gpuk_last_error().decode()


def check(status: int) -> None:
    if status != OK:
        raise GpukError(status, last_error())


def plan(world_size: int, numel: int, hidden: int, dtype: int = DTYPE_BF16, sm_count: int = 148,
         ctas_per_sm_limit: int = 0, oneshot_max_bytes: int = 0) -> Plan:
    p = Plan()
    check(lib.gpuk_plan_allreduce_rms(world_size, numel, hidden, dtype, sm_count, ctas_per_sm_limit,
                                      oneshot_max_bytes, ctypes.byref(p)))
    return p


def dtype_code(torch_dtype) -> int:
    import torch
    return {torch.bfloat16: DTYPE_BF16, torch.float16: DTYPE_F16, torch.float32: DTYPE_F32}[torch_dtype]
