"""CPU: the C-ABI shared library loads, exports every symbol the header declares, and rejects bad
arguments with the documented status codes before anything touches a device."""
import ctypes
import os
import re

import pytest

from int4matmul_kernels_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "int4matmul_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(i4mm_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(built_library):
    assert header_symbols() == capi.exported_symbols()


def test_library_exports_every_declared_symbol(built_library):
    for name in header_symbols():
        assert hasattr(built_library, name), name


def test_version_and_strings(built_library):
    assert built_library.i4mm_version() >= 100
    assert capi.status_string(0) == "ok"
    assert "bit width" in capi.status_string(capi.ERR_BITS)
    assert built_library.i4mm_workspace_bytes() > 0


def call(lib, bits=4, acc=0, path=0, out=16, matrix=16, mask=None, x=16, scales=16, zeros=16,
         rows=1, N=128, S=64, ng=1, g=128, ws=16, wsb=1 << 30):
    return lib.i4mm_quant_matmul(bits, acc, path, out, matrix, mask, x, scales, zeros, rows, N, S, ng, g, ws, wsb, None)


def test_argument_validation_without_a_device(built_library):
    lib = built_library
    assert call(lib, bits=5) == capi.ERR_BITS
    assert call(lib, bits=8) == capi.ERR_BITS
    assert call(lib, bits=3, mask=16) == capi.ERR_UNSUPPORTED       # sparse int3 traps in the reference
    assert call(lib, bits=2, mask=16) == capi.ERR_UNSUPPORTED
    assert call(lib, N=100) == capi.ERR_SHAPE                        # N % 64
    assert call(lib, S=96) == capi.ERR_SHAPE                         # S % 64 (matmul_kernel.cu:416)
    assert call(lib, g=96) == capi.ERR_SHAPE                         # group_size % 64 (matmul_kernel.cu:383)
    assert call(lib, g=0) == capi.ERR_SHAPE
    assert call(lib, g=64, ng=1, N=128) == capi.ERR_SHAPE            # groups do not cover N (matmul_kernel.cu:414)
    assert call(lib, rows=-1) == capi.ERR_SHAPE
    assert call(lib, rows=0) == capi.OK                              # empty input: nothing to do
    assert call(lib, out=None) == capi.ERR_NULL
    assert call(lib, x=None) == capi.ERR_NULL
    assert call(lib, matrix=8) == capi.ERR_ALIGN
    assert call(lib, path=7) == capi.ERR_SHAPE
    assert call(lib, path=1, ws=None) == capi.ERR_WORKSPACE
    assert call(lib, path=1, wsb=1024) == capi.ERR_WORKSPACE
    assert call(lib, g=-1, ng=1, rows=0) == capi.OK                  # negative group size = one group


def test_pack_validation_without_a_device(built_library):
    lib = built_library
    assert lib.i4mm_sparse_pack(16, 16, 16, 16, 64, 48, None, None) == capi.ERR_SHAPE    # N % 32 (utils_kernel.cu:101)
    assert lib.i4mm_sparse_pack(16, 16, 16, 16, 0, 64, None, None) == capi.OK
    assert lib.i4mm_sparse_pack(None, 16, 16, 16, 64, 64, None, None) == capi.ERR_NULL
    assert lib.i4mm_check_mask(None, 64, 64, 16, None) == capi.ERR_NULL


def test_torch_extension_surface():
    """The compiled module keeps the reference's eleven names and docstrings (int4matmul.cpp:65-82)."""
    import int4matmul_kernels_b200 as pkg
    from int4matmul_kernels_b200 import _build
    if not os.path.exists(_build.torch_ext_path()):
        _build.build_torch_ext()
    m = pkg.load_extension()
    names = ["weight_matrix_packing", "quant_matmul"] + [
        f"quant_int{b}_linear_mult{s}" for b in (4, 3, 2) for s in ("", "_mtx", "_vec")]
    for n in names:
        assert callable(getattr(m, n)), n
    assert "intn_fp16_mult" in m.quant_matmul.__doc__
    assert "int4_sparse_pack" in m.weight_matrix_packing.__doc__
    assert "int3_fp16_mult_vec" in m.quant_int3_linear_mult_vec.__doc__
    import torch
    cpu = torch.zeros((1, 1, 64), dtype=torch.float16)
    with pytest.raises(ValueError):
        m.quant_matmul(5, cpu, cpu, cpu, cpu, cpu, 64, None)        # std::invalid_argument -> ValueError
    with pytest.raises(RuntimeError):
        m.quant_matmul(4, cpu, cpu, cpu, cpu, cpu, 64, None)        # CPU tensors are rejected, not computed
