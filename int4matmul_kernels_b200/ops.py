"""The reference's operator entry points (int4matmul.cpp:26-82) on torch CUDA tensors, over the C ABI.

Same names, argument order and in-place convention as the reference's torch extension; the compiled
module `int4matmul` (lib/) offers the identical surface from C++.  This Python mirror exists so that
the C ABI can be driven directly (ctypes) with a chosen kernel path and stream.

Semantics kept from the reference:
  * seq_len == 1 (or any `_vec` entry) takes the matvec route, which ADDS into `outs`
    (matvec_kernel.cu:351, 381-382); everything else overwrites `outs`;
  * `bits` outside {4, 3, 2} raises ValueError (std::invalid_argument at int4matmul.cpp:35, 45);
  * `group_size` < 0 means one group over all of in_size (matmul_kernel.cu:379-381).
Every other violated precondition raises (the reference asserts, or traps the device).
"""
from __future__ import annotations

import torch

from . import capi

_workspaces: dict[tuple[int, int], torch.Tensor] = {}
_static_weights = False


def set_static_weights(flag: bool) -> None:
    """Declare that the weight-side tensors (matrix, mask, scales, zeros) passed to the multiply entries are never
    written by the kernel that precedes the call in the stream, as is the case for the weights of a loaded model.
    Launches may then begin (set-up, first weight copies) while that kernel is still finishing; activations, outputs
    and scratch are still only touched once it is complete.  Off by default: the reference orders every launch after
    the whole preceding kernel, and a caller that rewrites weights right before a call relies on that."""
    global _static_weights
    _static_weights = bool(flag)


class Int4MatmulError(RuntimeError):
    """A non-zero status from the C ABI other than a bad bit width."""

    def __init__(self, status: int, what: str):
        self.status = status
        msg = f"{what}: {capi.status_string(status)}"
        if status == capi.ERR_LAUNCH:
            msg += f" (cudaError {capi.load().i4mm_last_cuda_error()})"
        super().__init__(msg)


def _require_cuda(t: torch.Tensor, name: str, device: torch.device) -> None:
    if not t.is_cuda or t.device != device:
        raise ValueError(f"{name} must be a CUDA tensor on {device}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def workspace(device: torch.device, stream: torch.cuda.Stream) -> torch.Tensor:
    """The zero-initialised scratch buffer for (device, stream); allocated on first use, then reused."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream.cuda_stream)
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.zeros(capi.load().i4mm_workspace_bytes(), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def check_device_status(device: torch.device | None = None) -> None:
    """Waits for every stream `workspace()` has served on `device` and raises Int4MatmulError(ERR_TIMEOUT) if a
    kernel gave up on one of its bounded device-side waits since the last check (the results of that launch are
    void).  Not called by the multiply entries themselves, because it synchronises; no reference counterpart."""
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    lib = capi.load()
    worst = capi.OK
    with torch.cuda.device(index):
        for (dev, stream), ws in list(_workspaces.items()):
            if dev != index:
                continue
            status = lib.i4mm_device_status(ws.data_ptr(), stream)
            if status == capi.ERR_TIMEOUT:
                ws.zero_()            # the scratch of a cut-short launch is not all-zero any more
                torch.cuda.synchronize(index)
            if status != capi.OK:
                worst = status
    if worst != capi.OK:
        raise Int4MatmulError(worst, "int4matmul device status")


def _mult(bits: int, route: str, outs, matrix, multiplier, scales, zeros, group_size, sparse_mask, path: int) -> None:
    if bits not in (4, 3, 2):
        raise ValueError("Unsupported bit width for " +
                         ("matvec" if multiplier.dim() == 3 and multiplier.shape[1] == 1 else "matmul"))
    if not multiplier.is_cuda:
        raise ValueError("multiplier must be a CUDA tensor")
    dev = multiplier.device
    for t, name in ((outs, "outs"), (matrix, "matrix"), (multiplier, "multiplier"), (scales, "scales"), (zeros, "zeros")):
        _require_cuda(t, name, dev)
    if multiplier.dtype != torch.float16 or outs.dtype != torch.float16:
        raise TypeError("multiplier and outs must be float16 (the reference implements fp16 only)")
    if scales.dtype != torch.float16 or zeros.dtype != torch.float16:
        raise TypeError("scales and zeros must be float16")
    if matrix.dtype != torch.int32:
        raise TypeError("matrix must be int32")
    if multiplier.dim() != 3 or outs.dim() != 3 or matrix.dim() != 2 or scales.dim() != 2 or zeros.dim() != 2:
        raise ValueError("expected multiplier/outs 3-D and matrix/scales/zeros 2-D")
    sparse = sparse_mask is not None
    if sparse and bits != 4:
        raise ValueError("16:32 sparsity is only implemented for 4-bit weights")
    batch, seq_len, in_size = multiplier.shape
    mtx_in, out_size = matrix.shape
    if route == "vec" and seq_len != 1:
        raise ValueError("the _vec entry needs seq_len == 1")
    if sparse:
        if mtx_in * 16 != in_size:
            raise ValueError("sparse matrix rows * 16 must equal in_size")
        _require_cuda(sparse_mask, "sparse_mask", dev)
        if sparse_mask.dtype != torch.int32 or tuple(sparse_mask.shape) != (mtx_in // 2, out_size) or mtx_in % 2:
            raise ValueError("sparse_mask must be int32 (matrix rows / 2, out_size)")
    elif (mtx_in * 32) % bits or mtx_in * 32 // bits != in_size:
        raise ValueError("matrix rows * 32 / bits must equal in_size")
    if tuple(outs.shape) != (batch, seq_len, out_size):
        raise ValueError("outs must be (batch, seq_len, out_size)")
    if scales.shape[1] != out_size or zeros.shape[1] != out_size or scales.shape[0] != zeros.shape[0]:
        raise ValueError("scales and zeros must be (n_groups, out_size)")
    group_size = int(group_size)
    if group_size == 0 or (group_size > 0 and group_size % 64):
        raise ValueError("group_size must be a positive multiple of 64, or negative")

    matvec = route == "vec" or (route == "auto" and seq_len == 1)
    lib = capi.load()
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev)
        ws = workspace(dev, stream)
        status = lib.i4mm_quant_matmul(
            bits, 1 if matvec else 0, path | (capi.PATH_STATIC_WEIGHTS if _static_weights else 0), outs.data_ptr(), matrix.data_ptr(),
            sparse_mask.data_ptr() if sparse else None, multiplier.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
            batch * seq_len, in_size, out_size, scales.shape[0], group_size,
            ws.data_ptr(), ws.numel(), stream.cuda_stream)
    if status != capi.OK:
        raise Int4MatmulError(status, "int4matmul")


def quant_matmul(bits, outs, matrix, multiplier, scales, zeros, group_size, sparse_mask, *, path: int = capi.PATH_AUTO):
    """intn_fp16_mult (int4matmul.cpp:26, 68)."""
    _mult(int(bits), "auto", outs, matrix, multiplier, scales, zeros, group_size, sparse_mask, path)


def _make(bits: int, route: str, doc: str):
    def fn(outs, matrix, multiplier, scales, zeros, group_size, sparse_mask, *, path: int = capi.PATH_AUTO):
        _mult(bits, route, outs, matrix, multiplier, scales, zeros, group_size, sparse_mask, path)
    fn.__doc__ = doc
    return fn


# compat names (int4matmul.cpp:71-81)
quant_int4_linear_mult = _make(4, "auto", "int4_fp16_mult")
quant_int4_linear_mult_mtx = _make(4, "mtx", "int4_fp16_mult_mtx")
quant_int4_linear_mult_vec = _make(4, "vec", "int4_fp16_mult_vec")
quant_int3_linear_mult = _make(3, "auto", "int3_fp16_mult")
quant_int3_linear_mult_mtx = _make(3, "mtx", "int3_fp16_mult_mtx")
quant_int3_linear_mult_vec = _make(3, "vec", "int3_fp16_mult_vec")
quant_int2_linear_mult = _make(2, "auto", "int2_fp16_mult")
quant_int2_linear_mult_mtx = _make(2, "mtx", "int2_fp16_mult_mtx")
quant_int2_linear_mult_vec = _make(2, "vec", "int2_fp16_mult_vec")


def weight_matrix_packing(wt_outs, msk_outs, wt_in, msk_in) -> None:
    """int4_sparse_pack (int4matmul.cpp:56-66; utils_kernel.cu:67-119).

    wt_in, msk_in uint8 (out_size, in_size); wt_outs int32 (in_size/16, out_size); msk_outs int32
    (in_size/32, out_size).  Raises ValueError if a 32-block does not keep exactly 16 weights (the
    reference device-asserts); to report that it waits for the kernel to finish.
    """
    if not wt_in.is_cuda:
        raise ValueError("wt_in must be a CUDA tensor")
    dev = wt_in.device
    for t, name in ((wt_outs, "wt_outs"), (msk_outs, "msk_outs"), (wt_in, "wt_in"), (msk_in, "msk_in")):
        _require_cuda(t, name, dev)
        if t.dim() != 2:
            raise ValueError(f"{name} must be 2-D")
    if wt_outs.dtype != torch.int32 or msk_outs.dtype != torch.int32:
        raise TypeError("wt_outs and msk_outs must be int32")
    if wt_in.dtype != torch.uint8 or msk_in.dtype != torch.uint8:
        raise TypeError("wt_in and msk_in must be uint8")
    s, n = wt_in.shape
    if tuple(msk_in.shape) != (s, n) or n % 32:
        raise ValueError("wt_in and msk_in must share a shape (out_size, in_size) with in_size % 32 == 0")
    if tuple(wt_outs.shape) != (n // 16, s) or tuple(msk_outs.shape) != (n // 32, s):
        raise ValueError("wt_outs must be (in_size/16, out_size) and msk_outs (in_size/32, out_size)")
    lib = capi.load()
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev)
        violations = torch.zeros(1, dtype=torch.int32, device=dev)
        status = lib.i4mm_sparse_pack(wt_outs.data_ptr(), msk_outs.data_ptr(), wt_in.data_ptr(), msk_in.data_ptr(),
                                      s, n, violations.data_ptr(), stream.cuda_stream)
        if status != capi.OK:
            raise Int4MatmulError(status, "weight_matrix_packing")
        bad = int(violations.item())
    if bad:
        raise ValueError(f"weight_matrix_packing: {bad} block(s) of 32 weights do not keep exactly 16 (16:32 sparsity)")


def row_norm(mode: int, a: torch.Tensor, b: torch.Tensor | None = None, c: torch.Tensor | None = None) -> torch.Tensor:
    """Row-wise glue of the layer-stack runner (`i4mm_row_norm`): v / rms(v) per row with
    v = a (mode 0), a + b + c (1), a + b / rms(b) (2), a * b (3).  Inputs fp16 (rows, width), last dim contiguous.
    Mode 4 returns (2, rows, width): mode 2's result, and mode 0 of that result, from one launch."""
    rows, width = a.shape
    for t in (a, b, c):
        if t is not None and (t.dtype != torch.float16 or t.stride(-1) != 1 or tuple(t.shape) != (rows, width)):
            raise ValueError("row_norm inputs must be fp16 (rows, width) with a contiguous last dim")
    y = torch.empty((2, rows, width) if mode == 4 else (rows, width), dtype=torch.float16, device=a.device)
    stream = torch.cuda.current_stream(a.device)
    status = capi.load().i4mm_row_norm(
        mode, y.data_ptr(), a.data_ptr(), b.data_ptr() if b is not None else None, c.data_ptr() if c is not None else None,
        rows, width, a.stride(0), b.stride(0) if b is not None else 0, c.stride(0) if c is not None else 0, stream.cuda_stream)
    if status != capi.OK:
        raise Int4MatmulError(status, "row_norm")
    return y
