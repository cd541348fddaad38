"""Build the UNMODIFIED reference (mstnegate/int4matmul_kernels) into oracle/_ref/ as the torch extension module
`int4matmul_ref`, from its sources where they lie (never copied into this repository).

TEST / MEASUREMENT INFRASTRUCTURE ONLY.  The module built here is a checker: GPU tests compare the product's
outputs with the reference's own kernels on the same inputs, tests/golden/make_reference_gpu_vectors.py records
such outputs as fixtures, and bench.py can time the reference's kernels beside the product's.

Two things stand between the sources and a current toolchain, both handled from the outside:
  * torch >= 2.x dropped `detail::scalar_type(const at::DeprecatedTypeProperties&)`, which the sources' dispatch
    macro calls (matmul_kernel.cu:444, matvec_kernel.cu:365): a forced-include header supplies that one overload;
  * int4matmul.cpp includes device code (int4matmul.cpp:7), so it is compiled as CUDA (`nvcc -x cu`).
The dense int3 matvec kernel does not assemble for sm_100 (ptxas C7600 at -O1..-O3), so matvec_kernel.cu is
assembled with `-Xptxas -O1` first and, if that fails, with `-Xptxas -O0`; the module records which.

A second module, `int4matmul_ref_timing`, exists only so that the reference's matvec kernels can be TIMED as the
compiler would normally build them: its matvec translation unit is compiled at default optimisation from a
build directory (oracle/_ref/shadow/) that holds symbolic links to the reference's matvec_kernel.cu and
matmul.cuh and a kernel_specs.cuh generated from the reference's list with the dense int3 row filtered out
(a quoted #include is looked up beside the including file first, so the list beside the links is the one found).
In that module the dense int3 matvec launches nothing; every other kernel is the reference's own.

Usage:  python oracle/build_reference.py [/path/to/reference]
        (default: $INT4MATMUL_REFERENCE_DIR, else a checkout named `reference` beside this repository)
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SHIM = os.path.join(OUT, "dispatch_shim.h")
SHIM_TEXT = """// forced-include shim for building the reference against a current torch (see oracle/build_reference.py)
#pragma once
#include <ATen/ATen.h>
namespace detail {
inline c10::ScalarType scalar_type(const at::DeprecatedTypeProperties& t) { return t.scalarType(); }
}
"""


def main(ref_dir: str) -> int:
    if not os.path.isdir(ref_dir):
        print(f"[ref] no reference checkout at {ref_dir}: nothing to build")
        return 0
    import torch
    from torch.utils import cpp_extension
    os.makedirs(os.path.join(OUT, "obj"), exist_ok=True)
    with open(SHIM, "w") as f:
        f.write(SHIM_TEXT)
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    target = os.path.join(OUT, "int4matmul_ref" + suffix)
    sources = ["int4matmul.cpp", "matmul_kernel.cu", "matvec_kernel.cu", "utils_kernel.cu"]
    newest_src = max(os.path.getmtime(os.path.join(ref_dir, s)) for s in sources + ["matmul.cuh", "kernel_specs.cuh"])
    timing = os.path.join(OUT, "int4matmul_ref_timing" + suffix)
    if all(os.path.exists(t) and os.path.getmtime(t) > newest_src for t in (target, timing)):
        print("[ref] up to date:", target)
        return 0
    inc = []
    for p in cpp_extension.include_paths("cuda"):
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    base = ["nvcc", "-gencode", "arch=compute_100,code=sm_100", "-O2", "--generate-line-info", "-std=c++17", "-x", "cu",
            "-Xcompiler", "-fPIC", "-include", SHIM, "-DTORCH_EXTENSION_NAME=int4matmul_ref",
            "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-w",
            # the flags torch's CUDAExtension passes to nvcc (the reference's setup.py builds through it)
            "--expt-relaxed-constexpr", "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
            "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__", *inc, "-I", ref_dir]
    objs, notes = [], []
    procs = []
    for s in sources:
        obj = os.path.join(OUT, "obj", s.replace(".", "_") + ".o")
        objs.append(obj)
        procs.append((s, obj, subprocess.Popen(base + ["-c", os.path.join(ref_dir, s), "-o", obj],
                                               stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for s, obj, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0 and s == "matvec_kernel.cu":
            for opt in ("-O1", "-O0"):
                r = subprocess.run(base + ["-Xptxas", opt, "-c", os.path.join(ref_dir, s), "-o", obj],
                                   stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
                if r.returncode == 0:
                    notes.append(f"matvec_kernel.cu assembled with ptxas {opt} (default optimisation fails: ptxas C7600)")
                    break
            else:
                print(r.stdout[-2000:])
                return 1
        elif pr.returncode != 0:
            print(out[-3000:])
            return 1
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    libs = ["-L", torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-Xlinker", f"-rpath={torch_lib}"]
    link = ["nvcc", "-shared", "-o", target, *objs, *libs]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        print(r.stdout[-3000:])
        return 1
    # ---- the timing module: matvec translation unit at default optimisation, without the dense int3 row ----
    shadow = os.path.join(OUT, "shadow")
    os.makedirs(shadow, exist_ok=True)
    for name in ("matvec_kernel.cu", "matmul.cuh"):
        link_path = os.path.join(shadow, name)
        if os.path.lexists(link_path):
            os.remove(link_path)
        os.symlink(os.path.join(ref_dir, name), link_path)
    with open(os.path.join(ref_dir, "kernel_specs.cuh")) as f:
        rows = [ln for ln in f.read().splitlines() if ln.replace(" ", "") != "MACRO_OP(false,3)"]
    with open(os.path.join(shadow, "kernel_specs.cuh"), "w") as f:
        f.write("\n".join(rows) + "\n")
    timing_target = os.path.join(OUT, "int4matmul_ref_timing" + suffix)
    tbase = [a.replace("int4matmul_ref", "int4matmul_ref_timing") if a.startswith("-DTORCH_EXTENSION_NAME") else a for a in base]
    tobjs = []
    ok = True
    for s in sources:
        src = os.path.join(shadow if s == "matvec_kernel.cu" else ref_dir, s)
        obj = os.path.join(OUT, "obj", "timing_" + s.replace(".", "_") + ".o")
        if s in ("matmul_kernel.cu", "utils_kernel.cu"):           # no module name inside: the objects above serve
            tobjs.append(os.path.join(OUT, "obj", s.replace(".", "_") + ".o"))
            continue
        r = subprocess.run(tbase + ["-c", src, "-o", obj], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            notes.append("timing module not built: " + s + " failed at default optimisation")
            print(r.stdout[-2000:])
            ok = False
            break
        tobjs.append(obj)
    if ok:
        r = subprocess.run(["nvcc", "-shared", "-o", timing_target, *tobjs, *libs],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            print(r.stdout[-3000:])
            notes.append("timing module not linked")
        else:
            notes.append("int4matmul_ref_timing: matvec_kernel.cu at default ptxas optimisation, dense int3 matvec left out")
    with open(os.path.join(OUT, "BUILD_NOTES.txt"), "w") as f:
        f.write("\n".join(notes) + ("\n" if notes else "built with default flags\n"))
    print("[ref] built", target, "|", "; ".join(notes) if notes else "default flags")
    return 0


def default_reference_dir() -> str:
    env = os.environ.get("INT4MATMUL_REFERENCE_DIR")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


if __name__ == "__main__":
    sys.exit(main(sys.argv[1] if len(sys.argv) > 1 else default_reference_dir()))
