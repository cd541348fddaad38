"""The reference's algorithm on host CPU cores, with torch: the timed CPU baseline of the benchmark.

TEST / MEASUREMENT INFRASTRUCTURE ONLY (see reference_oracle.py).  The reference has no CPU
implementation; what runs here is its test script's comparator moved to the CPU: dequantise the
whole matrix per group in fp16, W = (q - zero) * scale (kernel_test.py:138-157), then x @ W
(kernel_test.py:248-249).  Multi-threaded through torch's intra-op pool.
"""
from __future__ import annotations

import time

import numpy as np
import torch


def dequantize(bits: int, q: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, group_size: int,
               keep: torch.Tensor | None = None) -> torch.Tensor:
    """q uint8 (N, S), scales/zeros fp16 (n_groups, S) -> fp16 W (N, S), linear coding
    (kernel_test.py:146-152; two fp16 roundings, as matmul.cuh:120)."""
    n, s = q.shape
    g = n if group_size < 0 else group_size
    w = q.to(torch.float16).view(-1, min(g, n), s) if n % g == 0 else None
    if w is None:
        idx = torch.arange(n) // g
        w16 = (q.to(torch.float16) - zeros[idx]) * scales[idx]
    else:
        ng = n // min(g, n)
        w16 = ((w - zeros[:ng, None, :]) * scales[:ng, None, :]).view(n, s)
    if keep is not None:
        w16 = torch.where(keep, w16, torch.zeros((), dtype=torch.float16))   # exact +0 (matmul.cuh:398)
    return w16


def timed_pass(problem: dict, rows: int, threads: int):
    """One dequantise + matmul pass over `rows` activation rows.  Returns (t_dequant, t_matmul) seconds."""
    torch.set_num_threads(threads)
    p = problem
    q = torch.from_numpy(p["q"])
    scales, zeros = torch.from_numpy(p["scales"]), torch.from_numpy(p["zeros"])
    keep = torch.from_numpy(p["keep"]) if p["keep"] is not None else None
    x = torch.from_numpy(np.ascontiguousarray(p["x"][:, :rows, :]))
    t0 = time.perf_counter()
    w16 = dequantize(p["bits"], q, scales, zeros, p["group_size"], keep)
    t1 = time.perf_counter()
    y = x @ w16
    _ = float(y.flatten()[0])
    t2 = time.perf_counter()
    return t1 - t0, t2 - t1


def synthetic_unpacked(bits: int, n: int, s: int, m: int, group_size: int, sparse: bool = False, seed: int = 0) -> dict:
    """A seeded problem in the UNPACKED form the comparator above starts from (the reference's test script also
    dequantises from the unpacked weights it drew, kernel_test.py:126-157), with the benchmark's value
    distributions; drawn as uint8 so that a 16384 x 16384 matrix costs 268 MB, not gigabytes."""
    from . import reference_oracle as oracle
    rng = np.random.default_rng(seed)
    lo, hi = (0.002, 0.02) if bits == 4 else (0.005, 0.05)
    g = n if group_size < 0 else group_size
    n_groups = (n + g - 1) // g
    q = rng.integers(0, 1 << bits, size=(n, s), dtype=np.uint8)
    scales = rng.uniform(lo, hi, size=(n_groups, s)).astype(np.float16)
    zeros = rng.integers(0, 1 << bits, size=(n_groups, s)).astype(np.float16)
    x = rng.standard_normal(size=(1, m, n), dtype=np.float32).astype(np.float16)
    keep = None
    if sparse:
        words = oracle.random_keep_words(rng, (n // 32, s)).view(np.uint32)
        keep = ((words[:, None, :] >> np.arange(32, dtype=np.uint32)[None, :, None]) & 1).astype(bool).reshape(n, s)
    return dict(bits=bits, n=n, s=s, m=m, batch=1, group_size=group_size, sparse=sparse, q=q, keep=keep,
                scales=scales, zeros=zeros, x=x)
