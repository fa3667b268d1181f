"""Shared helpers for the GPU parity tests: call the C ABI with torch tensors, build the
one-GPU emulation of an N-rank group, compare against the CPU oracle."""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from gpuk_b200 import cabi
from oracle import epilogue_oracle as eo

FP8_DTYPE = {1: torch.float8_e4m3fn, 2: torch.float8_e4m3fnuz, 3: torch.float8_e4m3fn, 4: torch.float8_e4m3fn}


def ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def stream_ptr():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def alloc_outputs(x: torch.Tensor, quant: int, static_scale: Optional[float] = None):
    m = x.shape[0]
    res_out = torch.empty_like(x)
    if quant == 0:
        norm_out = torch.empty_like(x)
        scale = torch.full((1,), -1.0, dtype=torch.float32, device=x.device)
    elif quant == 4:
        norm_out = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
        scale = torch.tensor([static_scale], dtype=torch.float32, device=x.device)
    else:
        norm_out = torch.empty(x.shape, dtype=FP8_DTYPE[quant], device=x.device)
        scale = torch.full((m, 1), -1.0, dtype=torch.float32, device=x.device)
    return res_out, norm_out, scale


def k1(x, residual, weight, eps, quant, static_scale=None):
    """gpuk_residual_rms_quant through the C ABI; returns CPU tensors."""
    res_out, norm_out, scale = alloc_outputs(x, quant, static_scale)
    hidden = x.shape[-1]
    cabi.check(cabi.lib.gpuk_residual_rms_quant(
        ptr(x), ptr(residual), ptr(weight), ptr(res_out), ptr(norm_out), ptr(scale), x.numel(), hidden,
        cabi.dtype_code(x.dtype), eps, quant, stream_ptr()))
    torch.cuda.synchronize()
    return res_out.cpu(), norm_out.cpu(), (scale.cpu() if quant else None)


class EmulatedGroup:
    """N workspaces on one GPU wired to each other; the N-rank kernels run in one cooperative launch."""

    def __init__(self, world: int, max_bytes: int = 8 << 20, device: int = 0):
        self.world = world
        self.device = device
        self.ws = []
        for r in range(world):
            h = ctypes.c_void_p()
            cabi.check(cabi.lib.gpuk_ws_create(device, r, world, max_bytes, 0, ctypes.byref(h)))
            self.ws.append(h)
        flags = (ctypes.c_void_p * world)()
        data = (ctypes.c_void_p * world)()
        for r in range(world):
            f, d = ctypes.c_void_p(), ctypes.c_void_p()
            cabi.check(cabi.lib.gpuk_ws_local_pointers(self.ws[r], ctypes.byref(f), ctypes.byref(d)))
            flags[r], data[r] = f, d
        for r in range(world):
            cabi.check(cabi.lib.gpuk_ws_set_peer_pointers(self.ws[r], flags, data, world))

    def close(self):
        for h in self.ws:
            cabi.lib.gpuk_ws_destroy(h)
        self.ws = []

    def set_option(self, name: str, value: int):
        for h in self.ws:
            cabi.check(cabi.lib.gpuk_ws_set_option(h, name.encode(), value))

    def attach_symmetric(self, message_bytes: int):
        """One zeroed buffer per emulated rank for the exchange through symmetric memory (no multicast)."""
        nbytes = (2 * ((message_bytes + 255) // 256 * 256) + cabi.SYM_FLAG_BYTES + 1023) // 256 * 256
        self.sym = [torch.zeros(nbytes, dtype=torch.uint8, device=f"cuda:{self.device}") for _ in range(self.world)]
        bases = (ctypes.c_void_p * self.world)(*[t.data_ptr() for t in self.sym])
        for h in self.ws:
            cabi.check(cabi.lib.gpuk_ws_attach_symmetric(h, bases, self.world, None, nbytes))

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _arr(self, tensors: Sequence[Optional[torch.Tensor]]):
        a = (ctypes.c_void_p * self.world)()
        for i, t in enumerate(tensors):
            a[i] = t.data_ptr() if t is not None else None
        return a

    def status(self, rank: int = 0):
        out = (ctypes.c_uint32 * 8)()
        rc = cabi.lib.gpuk_ws_status(self.ws[rank], out)
        return rc, list(out)

    def clear_status(self):
        for h in self.ws:
            cabi.check(cabi.lib.gpuk_ws_clear_status(h))

    def fused(self, parts: List[torch.Tensor], residual, weight, eps, quant, static_scale=None, force_mode=0,
              outs=None, check_status=True):
        """Returns per-rank (residual_out, norm_out, scale) on the CPU."""
        if outs is None:
            outs = [alloc_outputs(p, quant, static_scale) for p in parts]
        ws = (ctypes.c_void_p * self.world)(*[h.value for h in self.ws])
        hidden = parts[0].shape[-1]
        cabi.check(cabi.lib.gpuk_emulated_allreduce_rms(
            ws, self.world, self._arr(parts), ptr(residual), ptr(weight), self._arr([o[0] for o in outs]),
            self._arr([o[1] for o in outs]), self._arr([o[2] for o in outs]), parts[0].numel(), hidden,
            cabi.dtype_code(parts[0].dtype), eps, quant, force_mode, stream_ptr()))
        torch.cuda.synchronize()
        for r in range(self.world):
            rc, st = self.status(r)
            assert rc == 0 or not check_status, (r, st, cabi.last_error())
        return [(o[0].cpu(), o[1].cpu(), o[2].cpu() if quant else None) for o in outs]

    def plain(self, parts: List[torch.Tensor], force_mode=0):
        """In-place all-reduce of every rank's tensor; returns CPU copies."""
        ws = (ctypes.c_void_p * self.world)(*[h.value for h in self.ws])
        cabi.check(cabi.lib.gpuk_emulated_allreduce_rms(
            ws, self.world, self._arr(parts), None, None, None, None, None, parts[0].numel(), 0,
            cabi.dtype_code(parts[0].dtype), 0.0, 0, force_mode, stream_ptr()))
        torch.cuda.synchronize()
        for r in range(self.world):
            rc, st = self.status(r)
            assert rc == 0, (r, st, cabi.last_error())
        return [p.cpu() for p in parts]


def h2d_async(dst: torch.Tensor, src_pinned: torch.Tensor, stream: torch.cuda.Stream) -> None:
    """One cudaMemcpyAsync from pinned host memory on `stream`: a copy-engine transfer, whatever its size
    (torch's copy_ turns a one-element host tensor into a fill kernel, which needs an SM)."""
    from cuda.bindings import runtime as cudart
    assert src_pinned.is_pinned() and dst.is_contiguous() and src_pinned.is_contiguous()
    nbytes = dst.numel() * dst.element_size()
    assert nbytes == src_pinned.numel() * src_pinned.element_size()
    err, = cudart.cudaMemcpyAsync(dst.data_ptr(), src_pinned.data_ptr(), nbytes, cudart.cudaMemcpyKind.cudaMemcpyHostToDevice,
                                  stream.cuda_stream)
    assert err == cudart.cudaError_t.cudaSuccess, err


def random_case(world, tokens, hidden, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    parts = [torch.randn(tokens, hidden, generator=g).to(dtype) for _ in range(world)]
    residual = torch.randn(tokens, hidden, generator=g).to(dtype)
    weight = (1.0 + 0.1 * torch.randn(hidden, generator=g)).to(dtype)
    return parts, residual, weight


def check_against_oracle(got, want, quant, *, exact_residual=True, fp8_frac=0.999):
    """The parity bars: bf16 outputs atol/rtol 2e-2, FP8 within one e4m3 step on >= 99.9 % of
    elements, scales within 1e-3 relative (a row whose 16-bit maximum rounded to the neighbouring
    value counts as an outlier, see ParityReport.check).  The residual stream has no
    reduction-order freedom, so it is additionally required to be bit-exact."""
    rep = eo.compare(got, want, atol=2e-2, rtol=2e-2)
    if exact_residual:
        assert rep.residual_mismatch_frac == 0.0, rep
    if quant:
        rep.check(fp8_frac=fp8_frac, scale_rel=1e-3, scale_step=2.0 ** -7 if got[0].dtype != torch.float16 else 2.0 ** -10)
    return rep
