"""In-tree builds: the C-ABI CUDA library (nvcc, sm_100a) and the `int4matmul` torch extension (g++).

Nothing is JIT-compiled at import time; call `build_all()` (or run `python -m int4matmul_kernels_b200._build`)
once after a checkout.  Objects are rebuilt only when a source or header is newer than them.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT_DIR = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
INCLUDE_DIR = os.path.join(ROOT_DIR, "include")

CAPI_LIB = os.path.join(LIB_DIR, "libint4matmul_b200.so")
CUDA_SOURCES = ["capi.cu", "stream_kernel.cu", "umma_kernel.cu", "pack_kernel.cu", "noalloc.cu", "rownorm_kernel.cu", "gather.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def torch_ext_path() -> str:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(LIB_DIR, "int4matmul" + suffix)


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _headers() -> list[str]:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(INCLUDE_DIR, "int4matmul_b200.h"))
    return hs


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build step failed:\n  " + " ".join(cmd) + "\n" + proc.stdout)


def build_capi(verbose: bool = False) -> str:
    """nvcc -> lib/libint4matmul_b200.so (CUDA runtime linked statically; no torch, no libcuda link)."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    sources = [s for s in CUDA_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    hdrs = _headers()
    jobs = []
    objs = []
    for s in sources:
        src = os.path.join(CSRC, s)
        obj = os.path.join(OBJ_DIR, s[:-3] + ".o")
        objs.append(obj)
        if _newer(obj, [src] + hdrs):
            jobs.append([_nvcc(), *NVCC_FLAGS, "-I", INCLUDE_DIR, "-c", src, "-o", obj])
    if jobs:
        if verbose:
            print(f"[build] compiling {len(jobs)} CUDA source(s) for sm_100a", file=sys.stderr)
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1)) as ex:
            list(ex.map(_run, jobs))
    if _newer(CAPI_LIB, objs):
        _run([_nvcc(), "-shared", "-o", CAPI_LIB, *objs, "-cudart", "static"])
    return CAPI_LIB


def build_torch_ext(verbose: bool = False) -> str:
    """g++ -> lib/int4matmul.<abi>.so, the drop-in torch extension module, linked against the C-ABI library."""
    import torch
    from torch.utils import cpp_extension

    build_capi(verbose)
    out = torch_ext_path()
    src = os.path.join(CSRC, "torch_binding.cpp")
    if not _newer(out, [src, CAPI_LIB] + _headers()):
        return out
    if verbose:
        print("[build] compiling the torch extension module int4matmul", file=sys.stderr)
    inc = []
    for p in cpp_extension.include_paths("cuda"):
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=int4matmul",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DUSE_CUDA",
           *inc, "-I", INCLUDE_DIR, src, "-o", out,
           "-L", torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
           "-L", LIB_DIR, "-lint4matmul_b200",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    _run(cmd)
    return out


def build_all(verbose: bool = False) -> None:
    build_capi(verbose)
    build_torch_ext(verbose)


if __name__ == "__main__":
    build_all(verbose=True)
    print(CAPI_LIB)
    print(torch_ext_path())
