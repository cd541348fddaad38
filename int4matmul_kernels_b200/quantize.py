"""The missing caller layer of the reference ("integration happens in other libs", README.md:1): a round-to-nearest
group quantiser that produces the reference's tensors, and a thin nn.Module that owns them and calls the operator.

    q[n, s]   = clamp(round(W[n, s] / scale[g, s]) + zero[g, s], 0, 2^bits - 1)          g = n // group_size
    W16[n, s] = (q[n, s] - zero[g, s]) * scale[g, s]                                      (matmul.cuh:115-125)

scale = (max - min) / (2^bits - 1) per (group, column), zero = round(-min / scale): integer zero-points stored as
fp16, as the reference's test draws them (kernel_test.py:184).  With `sparse=True` (int4 only) the 16 smallest-
magnitude weights of every 32 along N are dropped (16:32) before quantisation.
"""
from __future__ import annotations

import torch

from . import packing


def quantize_groupwise(weight: torch.Tensor, bits: int = 4, group_size: int = 128, sparse: bool = False):
    """weight (N, S) float -> dict(q uint8 (N, S), scales fp16 (G, S), zeros fp16 (G, S), keep uint8 (S, N) or None)."""
    if bits not in (4, 3, 2):
        raise ValueError("bits must be 4, 3 or 2")
    n, s = weight.shape
    g = n if group_size < 0 else group_size
    if n % 64 or s % 64 or g % 64 or n % g:
        raise ValueError("N, S and group_size must be multiples of 64 and group_size must divide N")
    if sparse and bits != 4:
        raise ValueError("16:32 sparsity is only defined for int4")
    w = weight.float()
    keep = None
    if sparse:
        mag = w.abs().t().reshape(s, n // 32, 32)                       # (S, blocks, 32)
        rank = mag.argsort(dim=2, descending=True).argsort(dim=2)
        keep = (rank < 16).reshape(s, n).to(torch.uint8)                # (S, N), 1 = keep
        w = w * keep.t().float()
    levels = (1 << bits) - 1
    wg = w.view(n // g, g, s)
    lo = wg.amin(dim=1).clamp(max=0.0)
    hi = wg.amax(dim=1).clamp(min=0.0)
    # clamped after the cast: a tiny fp32 scale would underflow to 0 in fp16, and an all-zero group (zero-padded
    # columns, a fully pruned block) would turn into 0 / 0.  2^-14 is the smallest normal fp16.
    scale = ((hi - lo) / levels).to(torch.float16).clamp(min=2.0 ** -14)
    zero = torch.round(-lo / scale.float()).clamp(0, levels).to(torch.float16)
    q = torch.round(wg / scale.float()[:, None, :]) + zero.float()[:, None, :]
    q = q.clamp(0, levels).to(torch.uint8).view(n, s)
    return dict(q=q, scales=scale.contiguous(), zeros=zero.contiguous(), keep=keep)


def dequantize(q: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, group_size: int, keep: torch.Tensor | None = None):
    """fp16 weights exactly as the kernels rebuild them (linear coding): two fp16 roundings, dropped entries exact zeros."""
    n, s = q.shape
    g = n if group_size < 0 else group_size
    w = ((q.to(torch.float16).view(n // g, g, s) - zeros[:, None, :]) * scales[:, None, :]).view(n, s)
    if keep is not None:
        w = torch.where(keep.t().bool(), w, torch.zeros((), dtype=torch.float16, device=w.device))
    return w


class QuantLinear(torch.nn.Module):
    """y = x @ W16 with W stored in the reference's packed layout; bias-free.  x (..., N) fp16 CUDA -> (..., S)."""

    def __init__(self, bits, n, s, group_size, matrix, scales, zeros, mask=None):
        super().__init__()
        self.bits, self.in_features, self.out_features, self.group_size = bits, n, s, group_size
        self.register_buffer("matrix", matrix)
        self.register_buffer("scales", scales)
        self.register_buffer("zeros", zeros)
        self.register_buffer("mask", mask)

    @classmethod
    def from_float(cls, weight: torch.Tensor, bits: int = 4, group_size: int = 128, sparse: bool = False, device="cuda"):
        """weight (N, S) = in-features x out-features (the transpose of nn.Linear.weight)."""
        qz = quantize_groupwise(weight, bits, group_size, sparse)
        n, s = weight.shape
        if sparse:
            matrix, mask = packing.pack_sparse(qz["q"].t().contiguous().to(device), qz["keep"].to(device))
        else:
            matrix, mask = packing.pack_dense(bits, qz["q"].to(device)), None
        return cls(bits, n, s, group_size, matrix, qz["scales"].to(device), qz["zeros"].to(device), mask)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from . import ops
        lead = x.shape[:-1]
        x3 = x.reshape(1, -1, self.in_features).to(torch.float16).contiguous()
        out = torch.empty((1, x3.shape[1], self.out_features), dtype=torch.float16, device=x.device)
        # the _mtx entry overwrites `out` for any row count (the auto route would add into it when there is one row)
        getattr(ops, f"quant_int{self.bits}_linear_mult_mtx")(out, self.matrix, x3, self.scales, self.zeros,
                                                              self.group_size, self.mask)
        return out.view(*lead, self.out_features)
