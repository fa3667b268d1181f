"""gpuk_b200 -- B200-native tensor-parallel epilogue behind the gpuk operator API.

Mirrors the reference's Python surface (``gpuk/__init__.py``): the operator aliases
(``:18-31``), the FP8 policy constants (``:38-51``) and ``GPUKDistEnv`` (``:54-205``).  The
operators come from ``libgpuk_b200.so`` (``torch.ops.gpuk.*``, schema strings identical to
``src/register.cpp:5-40``), which sits on the C ABI of ``include/gpuk_b200.h``.

There is no CPU or PyTorch fallback for the fused path: a missing native library is an
ImportError, and the fused calls raise when they cannot reach the CUDA kernels.
"""
from __future__ import annotations

import os
from contextlib import contextmanager
from typing import Optional

import torch
import torch.distributed as dist

this_dir = os.path.dirname(os.path.abspath(__file__))
package_name = "gpuk"   # operator namespace, as in the reference (gpuk/__init__.py:11,15)
filename = os.path.join(this_dir, "libgpuk_b200.so")
if not os.path.exists(filename):
    raise ImportError(
        f"{filename} is missing: build it with `python gpuk_b200/_build.py` (needs nvcc and g++; "
        "there is no CPU fallback)")

from . import cabi  # noqa: E402  (loads libgpuk_core.so first; libgpuk_b200.so links against it)

torch.ops.load_library(filename)
_ops = torch.ops.gpuk

init_ar_fusion = _ops.init_ar_fusion
destroy_ar_fusion = _ops.destroy_ar_fusion
get_ar_fusion_barrier_handle = _ops.get_ar_fusion_barrier_handle
get_ar_fusion_data_handle = _ops.get_ar_fusion_data_handle
open_ar_fusion_barrier_handles = _ops.open_ar_fusion_barrier_handles
open_ar_fusion_data_handles = _ops.open_ar_fusion_data_handles
ar_fusion_capture_clear = _ops.ar_fusion_capture_clear
get_ar_fusion_tensor_handle = _ops.get_ar_fusion_tensor_handle
get_ar_fusion_tensor_offset = _ops.get_ar_fusion_tensor_offset
get_ar_fusion_captured_handles = _ops.get_ar_fusion_captured_handles
get_ar_fusion_captured_offsets = _ops.get_ar_fusion_captured_offsets
open_ar_fusion_captured_handles = _ops.open_ar_fusion_captured_handles
allreduce_inplace = _ops.allreduce_inplace
allreduce_rms = _ops.allreduce_rms

# ---------------------------------------------------------------------------------------
# FP8 policy (gpuk/__init__.py:38-51).  The reference selects the flavour by editing these
# module constants and ships with the AMD fnuz flavour; on B200 the default is OCP e4m3fn
# with its full range.  `set_fp8_policy` (or GPUK_FP8_POLICY) switches to the reference's
# own two settings.
# ---------------------------------------------------------------------------------------
QUANT_NONE = 0
_POLICIES = {
    "e4m3fn_240": (torch.float8_e4m3fn, 240, 1),      # reference policy 1 (float8.h:216-218)
    "e4m3fnuz_120": (torch.float8_e4m3fnuz, 120, 2),  # reference policy 2 (float8.h:249-251), its default
    "e4m3fn_448": (torch.float8_e4m3fn, 448, 3),      # OCP range, per-token dynamic scale
}
QUANT_STATIC_E4M3FN_448 = 4                            # one caller-supplied scale per tensor

fp8 = torch.float8_e4m3fn
fp8_max_val = 448
fp8_policy_id = 3


def set_fp8_policy(name: str) -> None:
    """Select the FP8 flavour, saturation value and operator policy id for this process."""
    global fp8, fp8_max_val, fp8_policy_id
    if name not in _POLICIES:
        raise ValueError(f"unknown FP8 policy {name!r}; choose from {sorted(_POLICIES)}")
    fp8, fp8_max_val, fp8_policy_id = _POLICIES[name]


if os.environ.get("GPUK_FP8_POLICY"):
    set_fp8_policy(os.environ["GPUK_FP8_POLICY"])


def fp8_linear_supported(tokens: int, out_features: int, in_features: int) -> bool:
    """Shapes ``fp8_linear`` is built for: decode batches (at most 32 tokens), 128-channel tiles, 64-byte k steps."""
    return 0 < tokens <= 32 and out_features % 128 == 0 and in_features % 64 == 0


def fp8_pack_weight(w_fp8: torch.Tensor) -> torch.Tensor:
    """FP8 weights [n, k] rearranged once into the blocked layout ``fp8_linear(..., packed=True)`` reads fastest
    (16 rows x 64 bytes per contiguous KiB); n a multiple of 16, k of 64.  Returns a new [n, k]-shaped tensor whose
    bytes are in blocked order."""
    import ctypes
    if w_fp8.dtype != torch.float8_e4m3fn or not (w_fp8.is_cuda and w_fp8.is_contiguous() and w_fp8.dim() == 2):
        raise RuntimeError("gpuk: fp8_pack_weight takes a contiguous 2-d float8_e4m3fn CUDA tensor")
    packed = torch.empty_like(w_fp8)
    with torch.cuda.device(w_fp8.device):
        cabi.check(cabi.lib.gpuk_fp8_pack_weight(ctypes.c_void_p(w_fp8.data_ptr()), ctypes.c_void_p(packed.data_ptr()),
                                                 w_fp8.shape[0], w_fp8.shape[1],
                                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return packed


def fp8_linear(x_fp8: torch.Tensor, x_scale: torch.Tensor, w_fp8: torch.Tensor, w_scale: torch.Tensor,
               out: Optional[torch.Tensor] = None, *, packed: bool = False, k_split: int = 0) -> torch.Tensor:
    """``(x_fp8 @ w_fp8.T) * x_scale[:, None] * w_scale[None, :]`` in bf16 for at most 32 tokens: the linear layer
    that consumes ``norm_out`` / ``scale_out`` of the fused operator (``F.linear`` in ``model/tensor_parallel.py:66``;
    the reference has no FP8 path).  ``x_fp8`` [tokens, k] and ``w_fp8`` [n, k] are ``float8_e4m3fn``, ``x_scale``
    holds one fp32 scale per token (any shape with ``tokens`` elements), ``w_scale`` one per output channel;
    ``packed=True`` says ``w_fp8`` came from ``fp8_pack_weight``.
    Hand-written weight-streaming kernel (``csrc/fp8_linear.cu``); raises for shapes it is not built for --
    ``fp8_linear_supported`` tells, and larger batches belong to a library GEMM."""
    import ctypes
    if x_fp8.dtype != torch.float8_e4m3fn or w_fp8.dtype != torch.float8_e4m3fn:
        raise RuntimeError("gpuk: fp8_linear takes float8_e4m3fn operands")
    if not (x_fp8.is_cuda and x_fp8.is_contiguous() and w_fp8.is_contiguous() and x_fp8.dim() == 2 and w_fp8.dim() == 2):
        raise RuntimeError("gpuk: fp8_linear takes contiguous 2-d CUDA tensors")
    m, k = x_fp8.shape
    n = w_fp8.shape[0]
    if w_fp8.shape[1] != k or x_scale.numel() != m or w_scale.numel() != n:
        raise RuntimeError("gpuk: fp8_linear operand shapes do not match")
    if x_scale.dtype != torch.float32 or w_scale.dtype != torch.float32 or not x_scale.is_contiguous() or not w_scale.is_contiguous():
        raise RuntimeError("gpuk: fp8_linear takes contiguous fp32 scales")
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=x_fp8.device)
    elif out.dtype != torch.bfloat16 or out.shape != (m, n) or not out.is_contiguous():
        raise RuntimeError("gpuk: fp8_linear writes a contiguous bf16 [tokens, n] tensor")
    with torch.cuda.device(x_fp8.device):
        cabi.check(cabi.lib.gpuk_fp8_linear_skinny(
            ctypes.c_void_p(x_fp8.data_ptr()), ctypes.c_void_p(x_scale.data_ptr()), ctypes.c_void_p(w_fp8.data_ptr()),
            ctypes.c_void_p(w_scale.data_ptr()), ctypes.c_void_p(out.data_ptr()), m, n, k, 1 if packed else 0, k_split,
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return out


class _TorchOps:
    """The operator set GPUKDistEnv drives; tests substitute a recording fake."""
    init_ar_fusion = staticmethod(init_ar_fusion)
    destroy_ar_fusion = staticmethod(destroy_ar_fusion)
    get_ar_fusion_barrier_handle = staticmethod(get_ar_fusion_barrier_handle)
    get_ar_fusion_data_handle = staticmethod(get_ar_fusion_data_handle)
    open_ar_fusion_barrier_handles = staticmethod(open_ar_fusion_barrier_handles)
    open_ar_fusion_data_handles = staticmethod(open_ar_fusion_data_handles)
    ar_fusion_capture_clear = staticmethod(ar_fusion_capture_clear)
    get_ar_fusion_captured_handles = staticmethod(get_ar_fusion_captured_handles)
    get_ar_fusion_captured_offsets = staticmethod(get_ar_fusion_captured_offsets)
    open_ar_fusion_captured_handles = staticmethod(open_ar_fusion_captured_handles)
    allreduce_inplace = staticmethod(allreduce_inplace)
    allreduce_rms = staticmethod(allreduce_rms)
    set_device = staticmethod(lambda d: torch.cuda.set_device(d))
    synchronize = staticmethod(lambda d: torch.cuda.synchronize(d))
    is_capturing = staticmethod(lambda: torch.cuda.is_current_stream_capturing())


class GPUKDistEnv:
    """Per-process handle on the fused tensor-parallel epilogue (``gpuk/__init__.py:54-205``).

    Same constructor, methods and return values as the reference class.  Differences a
    caller can observe:

    * a group of one works: the fused call runs the no-communication kernel (the reference
      leaves ``fptr = None``, ``:72-73``, and its fused call then fails);
    * any hidden size that is a multiple of 16 bytes is accepted (reference: 1024/2048/4096);
    * ``allreduce_add_rms_fused`` takes two keyword-only additions, ``static_scale`` (one
      per-tensor scale instead of per-token dynamic scales) and ``quant_type`` (override of
      the module-level FP8 policy);
    * inputs are never registered or copied into staging by the host, so ``capture`` /
      ``consume_capture`` exchange nothing (they still synchronise the group as before);
    * ``gather_multicast`` (keyword-only; default: on from four ranks where it can be had,
      ``GPUK_GATHER_MULTICAST=0`` switches it off): the gather areas of the two-shot exchange are placed in a buffer from
      ``torch.distributed._symmetric_memory`` and, where the NVSwitch offers a multicast mapping,
      a reduced slice is sent ONCE and copied to all ranks by the switch (``multimem.st``) instead of
      once per peer.  Pure data movement: results are bit-identical either way.  Without a
      multicast mapping (or if the allocation fails) the exchange pushes to every peer itself.
    * ``symmetric_bytes`` (keyword-only, or ``GPUK_SYMMETRIC_BYTES``, with ``gather_multicast=False``)
      adds a second exchange for large messages: a buffer of that size from
      ``torch.distributed._symmetric_memory`` is attached to the workspace, and where the NVSwitch
      offers a multicast mapping the reduction runs inside the switch (which rounds 16-bit sums its
      own way).  ``set_option("sym_min_bytes", n)`` sends fused calls of at least ``n`` bytes through it.
    """

    _SUPPORTED_WORLD_SIZES = [2, 4, 8]

    def __init__(self, group=None, device_id: int = None, max_size_in_bytes=16384 * 16384,
                 comm_ptrs_buf_len=1024 * 256, dtype: torch.dtype = torch.bfloat16, *, symmetric_bytes: Optional[int] = None,
                 gather_multicast: Optional[bool] = None, _ops=None) -> None:
        self._o = _ops or _TorchOps
        self.group = group
        self.device_id = device_id
        self.rank = dist.get_rank(group=self.group)
        self.world_size = dist.get_world_size(group=self.group)
        self.fptr = None
        self._IS_CAPTURING = False
        self._IS_CAPTURED = False
        self.disabled = False
        self.multicast = False     # True once a symmetric buffer with an NVSwitch multicast mapping is attached
        self._o.set_device(self.device_id)

        if self.world_size == 1:
            return
        if self.world_size not in GPUKDistEnv._SUPPORTED_WORLD_SIZES:
            return

        self.fptr = self._o.init_ar_fusion(self.device_id, self.rank, self.world_size, max_size_in_bytes,
                                           comm_ptrs_buf_len)
        barrier_handle = self._o.get_ar_fusion_barrier_handle(self.fptr)
        data_handle = self._o.get_ar_fusion_data_handle(self.fptr)
        self.barrier()
        barrier_handle_list = [None] * self.world_size
        data_handle_list = [None] * self.world_size
        dist.all_gather_object(barrier_handle_list, barrier_handle, group=self.group)
        dist.all_gather_object(data_handle_list, data_handle, group=self.group)
        self._o.open_ar_fusion_barrier_handles(self.fptr, barrier_handle_list)
        self._o.open_ar_fusion_data_handles(self.fptr, data_handle_list)
        self.barrier()
        if symmetric_bytes is None and os.environ.get("GPUK_SYMMETRIC_BYTES"):
            symmetric_bytes = int(os.environ["GPUK_SYMMETRIC_BYTES"])
        if gather_multicast is None:
            # measured on B200 (224 MiB message): eight ranks 663 us with the switch copying the gathered slices,
            # 741 us without; two ranks 557 us with, 403 us without (nothing to save when there is one peer)
            gather_multicast = (self.world_size >= 4 and not symmetric_bytes and _ops is None
                                and os.environ.get("GPUK_GATHER_MULTICAST", "1") != "0")
        self.gather_multicast = False
        if gather_multicast and not symmetric_bytes:
            self._try_gather_multicast(int(max_size_in_bytes))
        elif symmetric_bytes:
            self._attach_symmetric(int(symmetric_bytes))

    def _attach_symmetric(self, nbytes: int) -> None:
        """Allocates this rank's symmetric buffer, maps the peers' (and the multicast address where
        the fabric has one) and hands the addresses to the workspace."""
        import ctypes
        import torch.distributed._symmetric_memory as symm
        nbytes = (nbytes + 255) // 256 * 256
        group = self.group if self.group is not None else dist.group.WORLD
        self._sym = symm.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", self.device_id))
        self._sym.zero_()
        self._sym_handle = symm.rendezvous(self._sym, group.group_name)
        bases = (ctypes.c_void_p * self.world_size)(*[int(p) for p in self._sym_handle.buffer_ptrs])
        mc = int(getattr(self._sym_handle, "multicast_ptr", 0) or 0)
        cabi.check(cabi.lib.gpuk_ws_attach_symmetric(ctypes.c_void_p(self.fptr), bases, self.world_size,
                                                     ctypes.c_void_p(mc) if mc else None, nbytes))
        self.multicast = bool(mc)
        self.barrier()

    def _try_gather_multicast(self, max_size_in_bytes: int) -> None:
        """Gather areas in symmetric memory behind the NVSwitch multicast address, where that can be had.
        Every rank must reach the same decision, so the outcome is agreed on through the group."""
        ok = 0
        try:
            self._attach_symmetric(2 * ((max_size_in_bytes + 255) // 256 * 256) + cabi.SYM_FLAG_BYTES + 1024)
            ok = 1 if self.multicast else 0
        except Exception:   # no symmetric memory in this build / on this fabric: the exchange pushes to every peer
            ok = 0
        agreed = [None] * self.world_size
        dist.all_gather_object(agreed, ok, group=self.group)
        if all(agreed):
            self.set_option("gather_multicast", 1)
            self.gather_multicast = True
        self.barrier()

    def check(self) -> None:
        """Synchronises the device and raises if a wait of an earlier fused call gave up on a peer
        (``gpuk_ws_status``): the message names the rank, CTA, stage and peer that was waited for.
        The reference has no counterpart; its waits spin for ever (``communicator.h:98-99``)."""
        import ctypes
        if self.fptr:
            out = (ctypes.c_uint32 * 8)()
            if cabi.lib.gpuk_ws_status(ctypes.c_void_p(self.fptr), out) != cabi.OK:
                raise RuntimeError(cabi.last_error())

    def set_option(self, name: str, value: int) -> None:
        """Tuning options of the workspace (``gpuk_ws_set_option``); every rank must set the same."""
        import ctypes
        if self.fptr:
            cabi.check(cabi.lib.gpuk_ws_set_option(ctypes.c_void_p(self.fptr), name.encode(), int(value)))

    def barrier(self):
        self._o.set_device(self.device_id)
        self._o.synchronize(self.device_id)
        dist.barrier(group=self.group)

    def consume_capture(self):
        if not self.fptr:
            return
        self.barrier()
        handles = self._o.get_ar_fusion_captured_handles(self.fptr)
        offsets = self._o.get_ar_fusion_captured_offsets(self.fptr)
        for idx in range(len(handles)):
            handle_list = [None] * self.world_size
            offset_list = [None] * self.world_size
            dist.all_gather_object(handle_list, handles[idx], group=self.group)
            dist.all_gather_object(offset_list, int(offsets[idx].item()), group=self.group)
            self.barrier()
            self._o.open_ar_fusion_captured_handles(self.fptr, handle_list, offset_list, idx)
        self._o.ar_fusion_capture_clear(self.fptr)
        self.barrier()

    @contextmanager
    def capture(self):
        try:
            self._IS_CAPTURING = True
            yield
        finally:
            self._IS_CAPTURING = False
            if not self.disabled:
                self.consume_capture()

    def capture_(self, input: torch.Tensor):
        if self._o.is_capturing():
            self._IS_CAPTURED = True
        else:
            if self._IS_CAPTURED:
                self.consume_capture()
                self._IS_CAPTURED = False

    def __del__(self):
        fptr = getattr(self, "fptr", None)
        if fptr:
            try:
                self._o.destroy_ar_fusion(fptr)
            except Exception:
                pass
            self.fptr = None

    def _require_workspace(self):
        if self.world_size != 1 and not self.fptr:
            raise RuntimeError(
                f"gpuk: world size {self.world_size} is not supported by the fused path "
                f"(supported: 1 and {GPUKDistEnv._SUPPORTED_WORLD_SIZES})")

    def allreduce_native(self, allreduce_in):
        allreduce_out = allreduce_in.clone()
        dist.all_reduce(allreduce_out, group=self.group)
        return allreduce_out

    def allreduce(self, allreduce_in):
        self._require_workspace()
        allreduce_out = allreduce_in.clone()
        if self.world_size > 1:
            self._o.allreduce_inplace(self.fptr, allreduce_out)
        return allreduce_out

    def allreduce_add_rms_native(self, allreduce_in, residual_in, rms_weight, eps, fp8_out=False):
        """The PyTorch operator sequence the fused call must match (``gpuk/__init__.py:147-173``)."""
        def rms_norm_forward(x: torch.Tensor, weight: torch.Tensor, eps: float):
            input_dtype = x.dtype
            variance = x.float().pow(2).mean(-1, keepdim=True)
            x = x * torch.rsqrt(variance + eps)
            x = x.to(input_dtype)
            return weight * x
        if self.world_size > 1:
            dist.all_reduce(allreduce_in, group=self.group)
        residual_out = allreduce_in + residual_in
        norm_out = rms_norm_forward(residual_out, rms_weight, eps)
        if fp8_out:
            norm_out_scale, _ = norm_out.float().abs().max(dim=-1, keepdim=True)
            norm_out_scale = norm_out_scale / fp8_max_val
            norm_out = norm_out / norm_out_scale
            norm_out.clamp_(min=-fp8_max_val, max=fp8_max_val)
            norm_out = norm_out.to(fp8)
            return residual_out, norm_out, norm_out_scale
        scale_out = torch.empty(allreduce_in.shape[0], 1, dtype=torch.float32, device=allreduce_in.device)
        return residual_out, norm_out, scale_out

    def takes_ready_words(self, tokens: int, hidden: int, dtype: torch.dtype = torch.bfloat16) -> bool:
        """True when a fused call of this shape can start before its input is complete (``ready=`` of
        ``allreduce_add_rms_fused``): it must run the two-shot exchange with specialised warps."""
        if not self.fptr:
            return False
        p = cabi.plan(self.world_size, tokens * hidden, hidden, cabi.dtype_code(dtype))
        return bool(p.ws)

    def allreduce_add_rms_fused(self, allreduce_in, residual_in, rms_weight, eps, fp8_out=False, *,
                                static_scale: Optional[torch.Tensor] = None, quant_type: Optional[int] = None,
                                ready=None):
        """Fused all-reduce + residual add + RMSNorm (+ FP8), ``gpuk/__init__.py:175-205``.

        Returns ``(residual_out, norm_out, scale_out)`` like the reference.  With
        ``static_scale`` (a one-element fp32 CUDA tensor, or a float) the output is quantised
        with that single scale and ``scale_out`` is that tensor.

        ``ready = (words, rows_per_word, value)`` lets the call start while ``allreduce_in`` is still being
        written (by the row-parallel GEMM in front of it, ``model/tensor_parallel.py:117``): ``words`` is an int32
        CUDA tensor, word i stands for rows ``[i * rows_per_word, (i + 1) * rows_per_word)`` and the kernel reads a row
        only once its word is ``>= value``.  The producer stores the word after the rows, on any stream; the
        fused call is then NOT ordered behind the producer by the caller.  Only for shapes for which
        ``takes_ready_words`` is true; a producer that needs SMs while the exchange runs must be left room with
        ``set_option("ws_max_ctas", n)``.  The reference has no counterpart.
        """
        self._require_workspace()
        self.capture_(allreduce_in)
        if ready is not None:
            import ctypes
            words, rows_per_word, value = ready
            if not self.fptr or words.dtype not in (torch.int32, torch.uint32) or not words.is_cuda:
                raise RuntimeError("gpuk: ready words need a multi-rank environment and an int32 CUDA tensor")
            need = -(-allreduce_in.shape[0] // int(rows_per_word))
            if words.numel() < need:
                raise RuntimeError(f"gpuk: {need} ready words needed, {words.numel()} given")
            cabi.check(cabi.lib.gpuk_ws_set_ready_words(ctypes.c_void_p(self.fptr), ctypes.c_void_p(words.data_ptr()),
                                                        int(rows_per_word), int(value)))
        residual_out = torch.empty_like(residual_in)
        if static_scale is not None:
            fp8_out = True
            qt = QUANT_STATIC_E4M3FN_448
            if not isinstance(static_scale, torch.Tensor):
                static_scale = torch.tensor([float(static_scale)], dtype=torch.float32, device=allreduce_in.device)
            scale_out = static_scale.reshape(-1)
            out_dtype = torch.float8_e4m3fn
        elif fp8_out:
            qt = fp8_policy_id if quant_type is None else quant_type
            out_dtype = torch.float8_e4m3fnuz if qt == 2 else torch.float8_e4m3fn
            scale_out = torch.empty(allreduce_in.shape[0], 1, dtype=torch.float32, device=allreduce_in.device)
        else:
            qt = QUANT_NONE
            out_dtype = allreduce_in.dtype
            scale_out = torch.empty(1, dtype=torch.float32, device=allreduce_in.device)
        norm_out = torch.empty_like(allreduce_in, dtype=out_dtype)
        self._o.allreduce_rms(self.fptr or 0, allreduce_in, residual_in, rms_weight, residual_out, norm_out,
                              scale_out, eps, qt)
        return residual_out, norm_out, scale_out

    def allreduce_add_rms_fused_host(self, allreduce_in, residual_in, rms_weight, eps, out, *, chunks: int = 4,
                                     static_scale: Optional[torch.Tensor] = None, quant_type: Optional[int] = None):
        """The fused call for inputs and results that live in pinned host memory.

        ``allreduce_in`` and ``residual_in`` are pinned CPU tensors ``[tokens, hidden]``; ``out`` is a triple
        of pinned CPU tensors ``(residual_out, norm_out as FP8 or uint8, scale_out [tokens, 1] fp32)`` that
        receives the results.  The rows are cut into ``chunks`` pieces that travel as a pipeline over three
        streams -- host-to-device copy of piece i + 1, the fused kernel on piece i, device-to-host copy of piece
        i - 1 -- so the two directions of the host link are busy at the same time.  Rows are independent, so
        the results are those of one call on the whole tensor.  Returns after the last copy has completed.
        Every rank must call it with the same shapes and the same ``chunks``.  The reference has no
        counterpart: its callers keep activations on the device.
        """
        self._require_workspace()
        tokens, hidden = allreduce_in.shape
        dev = torch.device("cuda", self.device_id)
        key = (tokens, hidden, allreduce_in.dtype, out[1].dtype)
        st = getattr(self, "_host_path", None)
        if st is None or st["key"] != key:
            st = self._host_path = {
                "key": key,
                "x": torch.empty(tokens, hidden, dtype=allreduce_in.dtype, device=dev),
                "r": torch.empty(tokens, hidden, dtype=allreduce_in.dtype, device=dev),
                "res_out": torch.empty(tokens, hidden, dtype=allreduce_in.dtype, device=dev),
                "norm_out": torch.empty(tokens, hidden, dtype=out[1].dtype, device=dev),
                "scale": torch.empty(tokens, 1, dtype=torch.float32, device=dev),
                "s_in": torch.cuda.Stream(device=dev), "s_out": torch.cuda.Stream(device=dev),
            }
        if static_scale is not None:
            qt = QUANT_STATIC_E4M3FN_448
            scale_dev = static_scale.reshape(-1)
        else:
            qt = fp8_policy_id if quant_type is None else quant_type
            scale_dev = None
        cur = torch.cuda.current_stream(dev)
        s_in, s_out = st["s_in"], st["s_out"]
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        chunks = max(1, min(int(chunks), tokens))
        step = (tokens + chunks - 1) // chunks
        for lo in range(0, tokens, step):
            hi = min(lo + step, tokens)
            with torch.cuda.stream(s_in):
                st["x"][lo:hi].copy_(allreduce_in[lo:hi], non_blocking=True)
                st["r"][lo:hi].copy_(residual_in[lo:hi], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(s_in)
            cur.wait_event(ready)
            self._o.allreduce_rms(self.fptr or 0, st["x"][lo:hi], st["r"][lo:hi], rms_weight, st["res_out"][lo:hi],
                                  st["norm_out"][lo:hi], scale_dev if scale_dev is not None else st["scale"][lo:hi], eps, qt)
            done = torch.cuda.Event()
            done.record(cur)
            s_out.wait_event(done)
            with torch.cuda.stream(s_out):
                out[0][lo:hi].copy_(st["res_out"][lo:hi], non_blocking=True)
                out[1][lo:hi].copy_(st["norm_out"][lo:hi], non_blocking=True)
                if scale_dev is None:
                    out[2][lo:hi].copy_(st["scale"][lo:hi], non_blocking=True)
        s_out.synchronize()
        return out
