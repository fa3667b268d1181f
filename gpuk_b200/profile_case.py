"""Run one small, fixed case of a kernel a few times -- the command to put under `ncu`.

    python -m gpuk_b200.profile_case --kernel norm_quant --tokens 4096 --hidden 8192 --iters 6
    python -m gpuk_b200.profile_case --kernel emulated --world 8 --mode 2 --tokens 1024 --hidden 8192

`norm_quant` is the one-GPU kernel; `emulated` runs the N-rank exchange for all ranks inside
one cooperative launch on this GPU (mode 1 = one-shot, 2 = two-shot).  Inputs are seeded
random bf16; nothing is checked here (the tests do that), the point is a short, bounded run.
"""
from __future__ import annotations

import argparse
import ctypes

import torch

from . import cabi


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="norm_quant", choices=["norm_quant", "emulated"])
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--quant", type=int, default=3)
    ap.add_argument("--iters", type=int, default=6)
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--mode", type=int, default=2)
    a = ap.parse_args()
    torch.cuda.set_device(0)
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    w = (1 + 0.1 * torch.randn(a.hidden, device=dev)).bfloat16()
    res = torch.randn(a.tokens, a.hidden, device=dev).bfloat16()
    if a.kernel == "norm_quant":
        x = torch.randn(a.tokens, a.hidden, device=dev).bfloat16()
        res_out = torch.empty_like(x)
        q = torch.empty(x.shape, dtype=torch.uint8, device=dev)
        scale = torch.full((max(a.tokens, 1),), 0.05, dtype=torch.float32, device=dev)
        for _ in range(a.iters):
            cabi.check(cabi.lib.gpuk_residual_rms_quant(_p(x), _p(res), _p(w), _p(res_out), _p(q), _p(scale), x.numel(),
                                                        a.hidden, cabi.DTYPE_BF16, 1e-6, a.quant, stream))
        torch.cuda.synchronize()
        print("norm_quant", a.tokens, a.hidden, "scale0", float(scale[0]))
        return
    n = a.world
    msg = a.tokens * a.hidden * 2
    ws = []
    for r in range(n):
        h = ctypes.c_void_p()
        cabi.check(cabi.lib.gpuk_ws_create(0, r, n, max(msg, 1 << 20), 0, ctypes.byref(h)))
        ws.append(h)
    flags, data = (ctypes.c_void_p * n)(), (ctypes.c_void_p * n)()
    for r in range(n):
        f, d = ctypes.c_void_p(), ctypes.c_void_p()
        cabi.check(cabi.lib.gpuk_ws_local_pointers(ws[r], ctypes.byref(f), ctypes.byref(d)))
        flags[r], data[r] = f, d
    for r in range(n):
        cabi.check(cabi.lib.gpuk_ws_set_peer_pointers(ws[r], flags, data, n))
    xs = [torch.randn(a.tokens, a.hidden, device=dev).bfloat16() for _ in range(n)]
    outs = [(torch.empty_like(xs[0]), torch.empty(xs[0].shape, dtype=torch.uint8, device=dev),
             torch.full((max(a.tokens, 1),), 0.05, dtype=torch.float32, device=dev)) for _ in range(n)]
    arr = lambda ts: (ctypes.c_void_p * n)(*[t.data_ptr() for t in ts])
    wsa = (ctypes.c_void_p * n)(*[h.value for h in ws])
    for _ in range(a.iters):
        cabi.check(cabi.lib.gpuk_emulated_allreduce_rms(
            wsa, n, arr(xs), _p(res), _p(w), arr([o[0] for o in outs]), arr([o[1] for o in outs]),
            arr([o[2] for o in outs]), xs[0].numel(), a.hidden, cabi.DTYPE_BF16, 1e-6, a.quant, a.mode, stream))
    torch.cuda.synchronize()
    st = (ctypes.c_uint32 * 8)()
    rc = cabi.lib.gpuk_ws_status(ws[0], st)
    print("emulated", n, a.mode, a.tokens, a.hidden, "status", rc, list(st))
    for h in ws:
        cabi.lib.gpuk_ws_destroy(h)


if __name__ == "__main__":
    main()
