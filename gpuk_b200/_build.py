"""In-tree build of the native libraries (sm_100a only).

    python gpuk_b200/_build.py [core] [torch] [oracle]

* ``libgpuk_core.so``  the CUDA kernels and the C ABI of ``include/gpuk_b200.h`` (nvcc, no torch)
* ``libgpuk_b200.so``  the PyTorch operator library ``torch.ops.gpuk.*`` on top of it (g++)

Both land next to this file so that a snapshot of the source tree carries them.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
CORE_LIB = os.path.join(HERE, "libgpuk_core.so")
TORCH_LIB = os.path.join(HERE, "libgpuk_b200.so")

NVCC = os.environ.get("NVCC", "nvcc")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]
CORE_SOURCES = ["core.cu", "launch_bf16.cu", "launch_f16.cu", "launch_f32.cu", "noalloc.cu", "fp8_linear.cu"]
HEADERS = ["common.cuh", "epilogue.cuh", "kernels.cuh", "launch.cuh", "launch_impl.cuh",
           os.path.join(ROOT, "include", "gpuk_b200.h")]


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("command failed: " + " ".join(cmd))
    return res.stdout + res.stderr


def build_core(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]
    jobs = []
    objs = []
    for src in CORE_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src[:-3] + ".o")
        objs.append(o)
        if force or not _newer(o, [s] + headers):
            jobs.append([NVCC] + NVCC_FLAGS + ["-c", s, "-o", o])
    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as ex:
        list(ex.map(lambda c: _run(c, verbose), jobs))
    if force or jobs or not _newer(CORE_LIB, objs):
        _run([NVCC, "-shared", "-cudart", "static", "-o", CORE_LIB] + objs, verbose)
    return CORE_LIB


def build_torch(verbose: bool = False, force: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension as ce

    src = os.path.join(CSRC, "torch_ops.cpp")
    deps = [src, os.path.join(ROOT, "include", "gpuk_b200.h"), CORE_LIB]
    if not force and _newer(TORCH_LIB, deps):
        return TORCH_LIB
    inc = []
    for p in ce.include_paths(device_type="cuda") if "device_type" in ce.include_paths.__code__.co_varnames else ce.include_paths(cuda=True):
        inc += ["-I", p]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
           "-DTORCH_EXTENSION_NAME=gpuk_b200", "-I", os.path.join(ROOT, "include")] + inc + [
           src, "-o", TORCH_LIB, "-L", HERE, "-lgpuk_core", "-Wl,-rpath,$ORIGIN",
           "-L", torch_lib, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
           f"-Wl,-rpath,{torch_lib}"]
    _run(cmd, verbose)
    return TORCH_LIB


def build_oracle_ref(verbose: bool = False, ref: str | None = None) -> str | None:
    """Compile the reference's software FP8 cast and its fused CUDA kernels into oracle/_ref, from the
    reference checkout named by `ref` or the environment variable GPUK_REFERENCE_DIR (skipped where none is given
    or present: the built files travel with the tree)."""
    ref = ref or os.environ.get("GPUK_REFERENCE_DIR")
    if not ref or not os.path.isdir(ref):
        return None
    for sub in ("ref_fp8", "ref_kernels"):
        mk = os.path.join(ROOT, "oracle", sub)
        if os.path.isdir(mk):
            _run(["make", "-C", mk, f"REF={ref}"], verbose)
    return os.path.join(ROOT, "oracle", "_ref")


def main(argv):
    what = [a for a in argv if not a.startswith("-")] or ["core", "torch", "oracle"]
    verbose = "-v" in argv
    force = "-f" in argv
    if "core" in what:
        print(build_core(verbose, force))
    if "torch" in what:
        print(build_torch(verbose, force))
    if "oracle" in what:
        print(build_oracle_ref(verbose))


if __name__ == "__main__":
    main(sys.argv[1:])
