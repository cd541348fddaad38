"""B200 (sm_100a) implementation of the quantized matvec / matmul path of int4matmul_kernels.

  capi      ctypes binding of the C-ABI shared library (the drop-in boundary)
  ops       the reference's eleven operator entry points, on torch CUDA tensors, over that C ABI
  packing   producers of the packed weight formats (dense int4/int3/int2, 16:32 sparse int4)
  sharding  column-sharded execution over several GPUs with an all-gather of the outputs
  int4matmul (compiled, in lib/)  the torch extension module with the reference's module name

The CUDA library must be built first (`python -m int4matmul_kernels_b200._build`); nothing here computes
on the CPU and nothing falls back to PyTorch ops.
"""
__all__ = ["capi", "ops", "packing", "sharding", "load_extension"]


def load_extension():
    """Import and return the compiled torch extension module `int4matmul` from lib/."""
    import importlib.util
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    from ._build import torch_ext_path

    path = torch_ext_path()
    spec = importlib.util.spec_from_file_location("int4matmul", path)
    if spec is None or spec.loader is None:
        raise ImportError(f"cannot load the int4matmul extension from {path}; build it first")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
