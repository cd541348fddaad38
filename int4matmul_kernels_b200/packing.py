"""Producers of the packed weight formats the kernels consume, vectorised in torch (CPU or CUDA tensors).

The layouts are the reference's on-device formats; its own packers are per-row Python loops
(kernel_test.py:60-123) or CUDA-only (utils_kernel.cu:19-64):
  dense int4 / int2   int32 (N*bits/32, S); word [r, s] bits [bits*j, bits*j+bits) = q[r*(32/bits)+j, s]
  dense int3          int32 (3N/32, S); every 32 n of a column form a 96-bit little-endian stream over
                      three rows, weight k at stream bits [3k, 3k+3)
  16:32 sparse int4   int32 (N/16, S) compacted kept nibbles (rows 2b, 2b+1 = low/high word of block b)
                      + int32 (N/32, S) keep mask (bit l of [b, s] = keep(n = 32b + l, s))
"""
from __future__ import annotations

import torch


def pack_dense(bits: int, q: torch.Tensor) -> torch.Tensor:
    """q: integer tensor (N, S) with values in [0, 2^bits) -> packed int32 matrix in the layout above."""
    if bits not in (4, 3, 2):
        raise ValueError("bits must be 4, 3 or 2")
    n, s = q.shape
    if n % 64:
        raise ValueError("N must be a multiple of 64")
    v = q.to(torch.int64) & ((1 << bits) - 1)
    if bits in (4, 2):
        per = 32 // bits
        shifts = (torch.arange(per, device=q.device, dtype=torch.int64) * bits).view(1, per, 1)
        words = (v.view(n // per, per, s) << shifts).sum(dim=1)
    else:
        blocks = v.view(n // 32, 32, s)

        def fields(k0, k1, base):
            sh = (3 * torch.arange(k0, k1, device=q.device, dtype=torch.int64) - base).view(1, k1 - k0, 1)
            return (blocks[:, k0:k1, :] << sh).sum(dim=1)

        # weight 10 spans stream bits 30..32 and weight 21 spans 63..65 (matmul.cuh:286-301)
        w0 = fields(0, 10, 0) | ((blocks[:, 10, :] & 3) << 30)
        w1 = (blocks[:, 10, :] >> 2) | fields(11, 21, 32) | ((blocks[:, 21, :] & 1) << 31)
        w2 = (blocks[:, 21, :] >> 1) | fields(22, 32, 64)
        words = torch.stack([w0, w1, w2], dim=1).reshape(3 * n // 32, s)
    words = words & 0xFFFFFFFF
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words)
    return words.to(torch.int32).contiguous()


def unpack_dense(bits: int, packed: torch.Tensor) -> torch.Tensor:
    """Inverse of pack_dense: int32 (R, S) -> uint8 (N, S)."""
    w = packed.to(torch.int64) & 0xFFFFFFFF
    r, s = w.shape
    if bits in (4, 2):
        per = 32 // bits
        shifts = (torch.arange(per, device=w.device, dtype=torch.int64) * bits).view(1, per, 1)
        q = (w.view(r, 1, s) >> shifts) & ((1 << bits) - 1)
        return q.reshape(r * per, s).to(torch.uint8)
    if bits != 3 or r % 3:
        raise ValueError("bits must be 4, 3 or 2 (and int3 needs rows % 3 == 0)")
    w = w.view(r // 3, 3, s)
    out = []
    for k in range(32):
        bit = 3 * k
        word, off = divmod(bit, 32)
        val = w[:, word, :] >> off
        if off + 3 > 32:
            val = val | (w[:, word + 1, :] << (32 - off))
        out.append(val & 7)
    return torch.stack(out, dim=1).reshape(r // 3 * 32, s).to(torch.uint8)


def random_keep_mask(s: int, n: int, generator: torch.Generator | None = None, device="cpu") -> torch.Tensor:
    """uint8 (S, N): in every 32 contiguous n exactly 16 ones, positions uniformly random per block."""
    if n % 32:
        raise ValueError("N must be a multiple of 32")
    r = torch.rand((s, n // 32, 32), generator=generator, device=device)
    rank = r.argsort(dim=2).argsort(dim=2)
    return (rank < 16).reshape(s, n).to(torch.uint8)


def pack_sparse(q_sn: torch.Tensor, keep_sn: torch.Tensor):
    """16:32 packing on the GPU through the library's own packer.

    q_sn, keep_sn: uint8 (S, N) CUDA tensors (low nibble = weight; keep > 0).  Returns
    (weights int32 (N/16, S), mask int32 (N/32, S)).  Raises ValueError on a 16:32 violation."""
    from . import ops
    s, n = q_sn.shape
    wt = torch.empty((n // 16, s), dtype=torch.int32, device=q_sn.device)
    msk = torch.empty((n // 32, s), dtype=torch.int32, device=q_sn.device)
    ops.weight_matrix_packing(wt, msk, q_sn.contiguous(), keep_sn.contiguous())
    return wt, msk


def shard_columns(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Contiguous copy of columns [rank*S/world, (rank+1)*S/world) of a weight-side tensor (last dim = S).
    S/world must stay a multiple of 64 (the kernels' column granularity)."""
    s = t.shape[-1]
    if s % world or (s // world) % 64:
        raise ValueError("S / world must be a multiple of 64")
    w = s // world
    return t[..., rank * w:(rank + 1) * w].contiguous()


def synthetic_weights(bits: int, n: int, s: int, group_size: int, *, sparse: bool = False, seed: int = 0,
                      device="cuda", scale_range=None):
    """Seeded synthetic layer in the benchmark's value distributions: q uniform over the bit range,
    scales ~ U[lo, hi] fp16, integer zero-points stored as fp16 (the reference draws zeros the same way,
    kernel_test.py:184).  Drawn with a CPU generator so the bits do not depend on the GPU.
    Returns dict(matrix, mask, scales, zeros) on `device`."""
    gen = torch.Generator().manual_seed(seed)
    lo, hi = scale_range if scale_range else ((0.002, 0.02) if bits == 4 else (0.005, 0.05))
    g = n if group_size < 0 else group_size
    n_groups = (n + g - 1) // g
    q = torch.randint(0, 1 << bits, (n, s), generator=gen, dtype=torch.uint8)
    scales = (torch.rand((n_groups, s), generator=gen) * (hi - lo) + lo).to(torch.float16)
    zeros = torch.randint(0, 1 << bits, (n_groups, s), generator=gen).to(torch.float16)
    if sparse:
        keep = random_keep_mask(s, n, generator=gen)
        matrix, mask = pack_sparse(q.t().contiguous().to(device), keep.to(device))
    else:
        matrix, mask = pack_dense(bits, q.to(device)), None
    return dict(matrix=matrix, mask=mask, scales=scales.to(device), zeros=zeros.to(device))
