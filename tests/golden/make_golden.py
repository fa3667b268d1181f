"""Generate golden vectors by running the reference's own Python on CPU ranks (gloo).

Run where a checkout of the reference project is available (``--ref`` names its directory):

    python tests/golden/make_golden.py --ref <reference checkout>

The reference module ``gpuk/__init__.py`` loads a CUDA library at import time and binds
``torch.ops.gpuk.*`` names (``gpuk/__init__.py:10-35``).  Neither is needed for
``GPUKDistEnv.allreduce_add_rms_native`` (``:147-173``), which is pure PyTorch, so this
script declares empty ``gpuk::*`` operator schemas, turns ``torch.ops.load_library`` into
a no-op for the import, and then calls the *unmodified* reference method on gloo ranks.
The FP8 flavour is selected the way the reference does it, by module constants
(``gpuk/__init__.py:38-51``).

Each case is written to ``tests/golden/<name>.npz`` with the inputs, the collective's own
output and the three results (bf16/fp16 stored as uint16 bit patterns, FP8 as uint8).
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))

_OPS = [
    "init_ar_fusion", "destroy_ar_fusion", "get_ar_fusion_barrier_handle", "get_ar_fusion_data_handle",
    "open_ar_fusion_barrier_handles", "open_ar_fusion_data_handles", "ar_fusion_capture_clear",
    "get_ar_fusion_tensor_handle", "get_ar_fusion_tensor_offset", "get_ar_fusion_captured_handles",
    "get_ar_fusion_captured_offsets", "open_ar_fusion_captured_handles", "allreduce_inplace",
    "allreduce_rms", "fused_rope_rms", "fused_mrope_3d_rms", "fused_mrope_3d_rms_set_kv",
    "fused_rope_rms_2way",
]

# name, world, tokens, hidden, dtype, fp8 flavour (None = no quantisation), fp8 max, seed[, input distribution]
# input distribution: absent = N(0,1) partials; "outliers" = 0.1 % of the partials' elements times 20 (the
# prefill benchmark's inputs); "div_sqrt8" = partials N(0,1) / sqrt(8) (the decode benchmark's inputs)
CASES = [
    ("n2_bf16_16x1024_fn240", 2, 16, 1024, "bfloat16", "float8_e4m3fn", 240, 11),
    ("n2_bf16_16x1024_fnuz120", 2, 16, 1024, "bfloat16", "float8_e4m3fnuz", 120, 12),
    ("n2_bf16_16x1024_fn448", 2, 16, 1024, "bfloat16", "float8_e4m3fn", 448, 13),
    ("n2_bf16_5x2048_noquant", 2, 5, 2048, "bfloat16", None, 0, 14),
    ("n2_f16_9x1024_fn448", 2, 9, 1024, "float16", "float8_e4m3fn", 448, 15),
    ("n2_f32_7x1024_fn240", 2, 7, 1024, "float32", "float8_e4m3fn", 240, 16),
    ("n2_bf16_3x7168_fn448", 2, 3, 7168, "bfloat16", "float8_e4m3fn", 448, 17),
    ("n4_bf16_8x1024_fn448", 4, 8, 1024, "bfloat16", "float8_e4m3fn", 448, 18),
    ("n8_bf16_4x2048_fn448", 8, 4, 2048, "bfloat16", "float8_e4m3fn", 448, 19),
    ("n2_bf16_3x8192_fn448_outliers", 2, 3, 8192, "bfloat16", "float8_e4m3fn", 448, 20, "outliers"),
    ("n2_bf16_2x8192_fn448_div_sqrt8", 2, 2, 8192, "bfloat16", "float8_e4m3fn", 448, 21, "div_sqrt8"),
]


def load_reference(ref_root: str):
    lib = torch.library.Library("gpuk", "DEF")
    for name in _OPS:
        lib.define(f"{name}() -> ()")
    real_load = torch.ops.load_library
    torch.ops.load_library = lambda path: None
    try:
        spec = importlib.util.spec_from_file_location("gpuk_reference", os.path.join(ref_root, "gpuk", "__init__.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        torch.ops.load_library = real_load
    return mod, lib


def _bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e4m3fnuz):
        return t.contiguous().view(torch.uint8).numpy()
    return t.contiguous().numpy()


def make_inputs(world, tokens, hidden, dtype, seed, distribution=None):
    g = torch.Generator().manual_seed(seed)
    parts = [torch.randn(tokens, hidden, generator=g) for _ in range(world)]
    if distribution == "outliers":
        parts = [torch.where(torch.rand(tokens, hidden, generator=g) < 0.001, x * 20.0, x) for x in parts]
    elif distribution == "div_sqrt8":
        parts = [x / 8.0 ** 0.5 for x in parts]
    parts = [x.to(dtype) for x in parts]
    residual = torch.randn(tokens, hidden, generator=g).to(dtype)
    weight = (1.0 + 0.1 * torch.randn(hidden, generator=g)).to(dtype)
    return parts, residual, weight


def worker(rank, world, port, ref_root, case, out_dir):
    name, _, tokens, hidden, dtype_s, fp8_s, fp8_max, seed = case[:8]
    distribution = case[8] if len(case) > 8 else None
    torch.set_num_threads(1)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    mod, _lib = load_reference(ref_root)
    dtype = getattr(torch, dtype_s)
    parts, residual, weight = make_inputs(world, tokens, hidden, dtype, seed, distribution)
    if fp8_s is not None:
        mod.fp8 = getattr(torch, fp8_s)
        mod.fp8_max_val = fp8_max
    env = object.__new__(mod.GPUKDistEnv)   # __init__ needs a GPU; the native path needs only .group
    env.group = None
    env.fptr = None
    eps = 1e-6
    x = parts[rank].clone()
    res_out, norm_out, scale = env.allreduce_add_rms_native(x, residual, weight, eps, fp8_s is not None)
    # x now holds the collective's own result (all_reduce is in place, gpuk/__init__.py:156)
    if rank == 0:
        arrays = {f"part{r}": _bits(parts[r]) for r in range(world)}
        arrays.update(residual=_bits(residual), weight=_bits(weight), allreduce_out=_bits(x),
                      residual_out=_bits(res_out), norm_out=_bits(norm_out))
        if fp8_s is not None:
            arrays["scale"] = scale.numpy()
        arrays["meta"] = np.array([world, tokens, hidden, fp8_max, seed], dtype=np.int64)
        arrays["dtype"] = np.array(dtype_s)
        arrays["fp8"] = np.array(fp8_s or "")
        arrays["eps"] = np.array(eps, dtype=np.float64)
        np.savez(os.path.join(out_dir, name + ".npz"), **arrays)
        print("wrote", name, flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("GPUK_REFERENCE_DIR"), required=not os.environ.get("GPUK_REFERENCE_DIR"),
                    help="directory of the reference checkout (or set GPUK_REFERENCE_DIR)")
    ap.add_argument("--out", default=HERE)
    ap.add_argument("--only", default=None, help="generate only the cases whose name contains this text")
    args = ap.parse_args()
    port = 29710
    for case in CASES:
        if args.only and args.only not in case[0]:
            continue
        mp.spawn(worker, args=(case[1], port, args.ref, case, args.out), nprocs=case[1], join=True)
        port += 1


if __name__ == "__main__":
    sys.exit(main())
