"""CPU restatement (numpy) of the quantized matvec / matmul path of mstnegate/int4matmul_kernels.

TEST INFRASTRUCTURE ONLY.  This module is the checker the CUDA path is compared against; it is
imported by the tests, by the smoke check and by the benchmark's CPU-baseline leg, and by nothing
that ships.  The product path never routes through it.

Parity pin: the dense packers and the linear dequantisation are pinned against vectors produced by
the reference's own Python helpers (see tests/golden/make_golden.py, which imports the reference's
kernel_test.py).  The reference holds no stored vectors for the 16:32 sparse format, the exponent
coding or the kernels' outputs (it is CUDA-only and ships no expected results), so those parts are
pinned by formula and by closed-form known-answer cases only.

Notation: x is (B, M, N); the logical weight is (N, S); N = in-features (reduction dim, the packing
direction), S = out-features (contiguous dim of every weight-side tensor); g = group size along N.

Every function cites the reference file:line it restates.
"""
from __future__ import annotations

import numpy as np

SPARSE_BLOCK = 32          # 16 kept weights in every 32 (utils_kernel.cu:41)
SINGLE_GROUP = 0x0FFFFFFF  # group_size < 0 means one group (matmul_kernel.cu:379-381)


# --------------------------------------------------------------------------------------------
# packed formats
# --------------------------------------------------------------------------------------------

def pack_dense_pow2(bits: int, q: np.ndarray) -> np.ndarray:
    """q (N, S) ints in [0, 2^bits) -> int32 (N*bits/32, S).

    Word [r, s] holds q[r*(32/bits) + j, s] at bits [bits*j, bits*j + bits), LSB first
    (kernel_test.py:60-80; consumed at matmul.cuh:246-268 and matvec_kernel.cu:17-51).
    """
    assert bits in (4, 2)
    per = 32 // bits
    n, s = q.shape
    assert n % per == 0
    v = q.astype(np.uint64).reshape(n // per, per, s)
    shifts = (np.arange(per, dtype=np.uint64) * np.uint64(bits))[None, :, None]
    words = np.bitwise_or.reduce(v << shifts, axis=1)
    return words.astype(np.uint32).view(np.int32)


def unpack_dense_pow2(bits: int, packed: np.ndarray) -> np.ndarray:
    """Inverse of pack_dense_pow2: int32 (R, S) -> uint8 (R*32/bits, S)."""
    per = 32 // bits
    w = packed.view(np.uint32)
    r, s = w.shape
    shifts = (np.arange(per, dtype=np.uint32) * np.uint32(bits))[None, :, None]
    q = (w[:, None, :] >> shifts) & np.uint32((1 << bits) - 1)
    return q.reshape(r * per, s).astype(np.uint8)


def pack_dense_int3(q: np.ndarray) -> np.ndarray:
    """q (N, S) ints in [0, 8) -> int32 (3N/32, S).

    Every 32 consecutive n of one column form one 96-bit little-endian stream over three consecutive
    rows; weight k sits at stream bits [3k, 3k+3).  Weights 10 and 21 straddle word boundaries
    (kernel_test.py:82-123; consumed at matmul.cuh:270-309 and matvec_kernel.cu:53-127).
    """
    n, s = q.shape
    assert n % 32 == 0
    v = q.astype(np.uint64).reshape(n // 32, 32, s)
    out = np.zeros((n // 32, 3, s), dtype=np.uint64)
    for k in range(32):
        bit = 3 * k
        word, off = divmod(bit, 32)
        out[:, word, :] |= (v[:, k, :] << np.uint64(off)) & np.uint64(0xFFFFFFFF)
        if off + 3 > 32:  # straddles into the next word
            out[:, word + 1, :] |= v[:, k, :] >> np.uint64(32 - off)
    return out.reshape(3 * n // 32, s).astype(np.uint32).view(np.int32)


def unpack_dense_int3(packed: np.ndarray) -> np.ndarray:
    """Inverse of pack_dense_int3: int32 (R, S) -> uint8 (R*32/3, S)."""
    w = packed.view(np.uint32).astype(np.uint64)
    r, s = w.shape
    assert r % 3 == 0
    w = w.reshape(r // 3, 3, s)
    lo = w[:, 0, :] | (w[:, 1, :] << np.uint64(32))          # stream bits 0..63
    hi = (w[:, 1, :] >> np.uint64(0)) | (w[:, 2, :] << np.uint64(32))  # stream bits 32..95
    out = np.zeros((r // 3, 32, s), dtype=np.uint8)
    for k in range(32):
        bit = 3 * k
        if bit + 3 <= 64:
            out[:, k, :] = ((lo >> np.uint64(bit)) & np.uint64(7)).astype(np.uint8)
        else:
            out[:, k, :] = ((hi >> np.uint64(bit - 32)) & np.uint64(7)).astype(np.uint8)
    return out.reshape(r // 3 * 32, s)


def pack_sparse_int4(wt_in: np.ndarray, msk_in: np.ndarray):
    """16:32 sparse packer.  wt_in, msk_in are uint8 (S, N) as the reference's entry point takes them.

    Returns (wt_out int32 (N/16, S), msk_out int32 (N/32, S)):
      msk_out[b, s] bit l  = msk_in[s, 32b + l] > 0                       (utils_kernel.cu:34-39)
      wt_out rows 2b (low word) and 2b+1 (high word) hold the kept low nibbles of block b in
      increasing-n order, rank r at bits [4r, 4r+4) of the 64-bit word     (utils_kernel.cu:44-61)
    Exactly 16 kept entries per block are required (device assert at utils_kernel.cu:41); a block
    that violates this raises ValueError here.
    """
    s, n = wt_in.shape
    assert msk_in.shape == (s, n) and n % SPARSE_BLOCK == 0
    keep = (msk_in > 0).reshape(s, n // 32, 32)
    if not np.all(keep.sum(axis=2) == 16):
        raise ValueError("16:32 sparsity violated: some 32-block does not keep exactly 16 weights")
    bitw = (np.uint64(1) << np.arange(32, dtype=np.uint64))[None, None, :]
    msk = (keep.astype(np.uint64) * bitw).sum(axis=2).astype(np.uint32)       # (S, N/32)
    nib = (wt_in.reshape(s, n // 32, 32) & 0xF).astype(np.uint64)
    rank = np.cumsum(keep, axis=2) - keep                                       # exclusive prefix
    word = ((nib << (np.uint64(4) * rank.astype(np.uint64))) * keep).sum(axis=2)  # (S, N/32) u64
    wt = np.empty((s, n // 16), dtype=np.uint32)
    wt[:, 0::2] = (word & np.uint64(0xFFFFFFFF)).astype(np.uint32)
    wt[:, 1::2] = (word >> np.uint64(32)).astype(np.uint32)
    return np.ascontiguousarray(wt.T).view(np.int32), np.ascontiguousarray(msk.T).view(np.int32)


def unpack_sparse_int4(wt: np.ndarray, msk: np.ndarray):
    """Inverse of pack_sparse_int4.  Returns (q uint8 (N, S) with dropped entries 0, keep bool (N, S)).

    Walks the mask LSB first, taking one nibble of the 64-bit word per set bit, as the consumers do
    (matvec_kernel.cu:145-165, matmul.cuh:395-398).
    """
    w = wt.view(np.uint32).astype(np.uint64)
    m = msk.view(np.uint32)
    nb, s = m.shape
    assert w.shape == (2 * nb, s)
    word = w[0::2, :] | (w[1::2, :] << np.uint64(32))                       # (N/32, S)
    keep = ((m[:, None, :] >> np.arange(32, dtype=np.uint32)[None, :, None]) & 1).astype(bool)
    rank = (np.cumsum(keep, axis=1) - keep).astype(np.uint64)
    nib = (word[:, None, :] >> (np.uint64(4) * np.minimum(rank, np.uint64(15)))) & np.uint64(0xF)
    q = np.where(keep, nib, 0).astype(np.uint8)
    return q.reshape(nb * 32, s), keep.reshape(nb * 32, s)


# --------------------------------------------------------------------------------------------
# dequantisation
# --------------------------------------------------------------------------------------------

def _group_index(n: int, group_size: int) -> np.ndarray:
    g = SINGLE_GROUP if group_size < 0 else group_size        # matmul_kernel.cu:379-381
    return np.arange(n) // g                                   # matmul_kernel.cu:261


def dequant_w16(bits: int, q: np.ndarray, scales: np.ndarray, zeros: np.ndarray, group_size: int,
                keep: np.ndarray | None = None) -> np.ndarray:
    """The fp16 weight the reference's kernels multiply with, bit for bit.  q (N, S) -> fp16 (N, S).

    scale >= 0 (linear):  W16 = hmul(hsub(half(q), zero), scale): two fp16 roundings (matmul.cuh:115-125)
    otherwise (exponent): s' = -scale, iv = (q & SGN ? -1 : 1) * 2^(q & EXP), W16 = hfma(half(iv), s', zero),
                          one rounding (matmul.cuh:127-136); the switch is on __hge(scale, 0)
                          (matmul.cuh:420, matvec_kernel.cu:182), so NaN scales take the exponent branch.
    Dropped entries of the 16:32 format are exact zeros (matmul.cuh:398).
    """
    n, s = q.shape
    gi = _group_index(n, group_size)
    sc = scales.astype(np.float16)[gi, :]
    zp = zeros.astype(np.float16)[gi, :]
    qh = (q.astype(np.int64) & ((1 << bits) - 1)).astype(np.float16)
    with np.errstate(all="ignore"):
        lin = ((qh - zp).astype(np.float16) * sc).astype(np.float16)
        sgn = 1 << (bits - 1)
        qi = q.astype(np.int64)
        iv = np.where(qi & sgn, -1.0, 1.0) * np.exp2((qi & (sgn - 1)).astype(np.float64))
        expo = (iv * (-sc.astype(np.float64)) + zp.astype(np.float64)).astype(np.float16)
    w = np.where(sc >= np.float16(0), lin, expo).astype(np.float16)
    if keep is not None:
        w = np.where(keep, w, np.float16(0)).astype(np.float16)
    return w


def dequant_fp32(bits: int, q: np.ndarray, scales: np.ndarray, zeros: np.ndarray, group_size: int,
                 keep: np.ndarray | None = None) -> np.ndarray:
    """The reference test's high-precision weight: (q - z) * s in fp32, linear mode only
    (kernel_test.py:141, 152).  Used as the accuracy truth, not as the parity target."""
    n, s = q.shape
    gi = _group_index(n, group_size)
    w = (q.astype(np.float32) - zeros.astype(np.float32)[gi, :]) * scales.astype(np.float32)[gi, :]
    if keep is not None:
        w = w * keep.astype(np.float32)
    return w.astype(np.float32)


# --------------------------------------------------------------------------------------------
# results
# --------------------------------------------------------------------------------------------

def matmul_ref(x: np.ndarray, w16: np.ndarray, outs_in: np.ndarray | None = None) -> np.ndarray:
    """Reference semantics of both kernels: fp16 x fp16 products accumulated in fp32 over all of N,
    one rounding to fp16 at the end (matmul_kernel.cu:246-253, 326-329; matvec_kernel.cu:40, 381).

    outs_in given  -> the matvec route, which adds into the caller's `outs`:
                      half(float(outs_in) + x.W)            (matvec_kernel.cu:351, 263, 381-382)
    outs_in None   -> the matmul route, which overwrites `outs` (matmul_kernel.cu:299-332)
    The summation order inside the reference is unspecified (wmma fragments; fp32 atomics), so
    equality is up to fp32 reassociation.
    """
    b, m, n = x.shape
    acc = x.reshape(b * m, n).astype(np.float32) @ w16.astype(np.float32)
    acc = acc.reshape(b, m, -1)
    if outs_in is not None:
        acc = outs_in.astype(np.float32) + acc
    with np.errstate(over="ignore"):
        return acc.astype(np.float16)


def matmul_fp32(x: np.ndarray, w32: np.ndarray) -> np.ndarray:
    """fp32 truth of the reference's test: x.float() @ hiW (kernel_test.py:251-252)."""
    b, m, n = x.shape
    return (x.reshape(b * m, n).astype(np.float32) @ w32).reshape(b, m, -1)


def matmul_abs_bound(x: np.ndarray, w16: np.ndarray) -> np.ndarray:
    """sum_n |x . W16| per output: the magnitude fp32 reassociation error scales with."""
    b, m, n = x.shape
    a = np.abs(x.reshape(b * m, n).astype(np.float32)) @ np.abs(w16.astype(np.float32))
    return a.reshape(b, m, -1)


def mean_rel_error(truth: np.ndarray, cand: np.ndarray) -> float:
    """The reference's own error metric: nanmean(|(cand - truth) / truth|) (kernel_test.py:261-262)."""
    with np.errstate(all="ignore"):
        r = np.abs((cand.astype(np.float64) - truth.astype(np.float64)) / truth.astype(np.float64))
    return float(np.nanmean(r))


def fp16_ulp_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in fp16 units-in-the-last-place between two fp16 arrays (sign-magnitude ordered)."""
    def key(v):
        u = v.astype(np.float16).view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(a) - key(b))


# --------------------------------------------------------------------------------------------
# seeded synthetic problems (CPU generator; the same bits go to the GPU)
# --------------------------------------------------------------------------------------------

def make_problem(bits: int, n: int, s: int, m: int, group_size: int, *, sparse: bool = False,
                 batch: int = 1, seed: int = 0, scale_lo: float | None = None,
                 scale_hi: float | None = None, x_dist: str = "normal", exponent_frac: float = 0.0):
    """Seeded problem with the value distributions of the benchmark configs: x ~ N(0,1) fp16,
    q uniform over the bit range, scales ~ U[lo, hi] fp16, integer zero-points stored as fp16.
    Returns a dict with raw q (N,S), keep (N,S) or None, packed matrix, mask or None, scales, zeros, x.
    exponent_frac > 0 flips that fraction of 32-column-aligned (group, column-run) scale blocks
    negative, which selects the exponent coding for them."""
    rng = np.random.default_rng(seed)
    if scale_lo is None:
        scale_lo, scale_hi = (0.002, 0.02) if bits == 4 else (0.005, 0.05)
    q = rng.integers(0, 1 << bits, size=(n, s), dtype=np.int64).astype(np.uint8)
    g = n if group_size < 0 else group_size
    n_groups = (n + g - 1) // g
    scales = rng.uniform(scale_lo, scale_hi, size=(n_groups, s)).astype(np.float16)
    zeros = rng.integers(0, 1 << bits, size=(n_groups, s)).astype(np.float16)
    if exponent_frac > 0:
        flip = rng.random(size=(n_groups, (s + 31) // 32)) < exponent_frac
        flip = np.repeat(flip, 32, axis=1)[:, :s]
        scales = np.where(flip, -scales, scales).astype(np.float16)
    if x_dist == "normal":
        x = rng.standard_normal(size=(batch, m, n)).astype(np.float16)
    else:
        x = rng.uniform(-1.0, 1.0, size=(batch, m, n)).astype(np.float16)
    keep = None
    mask = None
    if sparse:
        assert bits == 4 and n % 32 == 0
        order = np.argsort(rng.random(size=(s, n // 32, 32)), axis=2)
        keep_sn = (order < 16).reshape(s, n)
        matrix, mask = pack_sparse_int4(np.ascontiguousarray(q.T), keep_sn.astype(np.uint8))
        keep = np.ascontiguousarray(keep_sn.T)
    elif bits == 3:
        matrix = pack_dense_int3(q)
    else:
        matrix = pack_dense_pow2(bits, q)
    return dict(bits=bits, n=n, s=s, m=m, batch=batch, group_size=group_size, sparse=sparse,
                q=q, keep=keep, matrix=matrix, mask=mask, scales=scales, zeros=zeros, x=x)


def expected(problem: dict, outs_in: np.ndarray | None = None):
    """(reference-semantics fp16 result, W16, abs bound) for a problem from make_problem."""
    p = problem
    w16 = dequant_w16(p["bits"], p["q"], p["scales"], p["zeros"], p["group_size"], p["keep"])
    return matmul_ref(p["x"], w16, outs_in), w16, matmul_abs_bound(p["x"], w16)


# --------------------------------------------------------------------------------------------
# checks on sampled output columns (full-size shapes, where a whole-matrix oracle would take minutes)
# --------------------------------------------------------------------------------------------

def unpack_columns(bits: int, matrix: np.ndarray, mask: np.ndarray | None, cols: np.ndarray):
    """(q uint8 (N, len(cols)), keep bool or None) of the chosen output columns of a packed matrix: every
    output column depends only on its own column of the weight-side tensors (matmul_kernel.cu:258-267)."""
    sub = np.ascontiguousarray(matrix[:, cols])
    if mask is not None:
        return unpack_sparse_int4(sub, np.ascontiguousarray(mask[:, cols]))
    if bits == 3:
        return unpack_dense_int3(sub), None
    return unpack_dense_pow2(bits, sub), None


def expected_columns(bits: int, matrix: np.ndarray, mask: np.ndarray | None, scales: np.ndarray, zeros: np.ndarray,
                     group_size: int, x: np.ndarray, cols: np.ndarray, outs_in: np.ndarray | None = None):
    """Reference-semantics result for the output columns `cols` only, computed from the PACKED tensors.

    x (B, M, N) fp16; returns (want fp16 (B, M, len(cols)), abs bound (B, M, len(cols))).  outs_in, if given, is
    the (B, M, len(cols)) slice of the caller's `outs` that the matvec route adds to (matvec_kernel.cu:351)."""
    cols = np.asarray(cols)
    q, keep = unpack_columns(bits, matrix, mask, cols)
    w16 = dequant_w16(bits, q, scales[:, cols], zeros[:, cols], group_size, keep)
    return matmul_ref(x, w16, outs_in), matmul_abs_bound(x, w16)


def random_keep_words(rng: np.random.Generator, shape, pool: int = 1 << 16) -> np.ndarray:
    """int32 keep-mask words with exactly 16 of 32 bits set, drawn from a pool of `pool` masks whose kept
    positions are uniformly random 16-subsets (argsort of uniforms), so that large masks cost no large sort."""
    order = np.argsort(rng.random(size=(pool, 32)), axis=1)
    bits = (order < 16).astype(np.uint64) << np.arange(32, dtype=np.uint64)[None, :]
    words = bits.sum(axis=1).astype(np.uint32)
    return words[rng.integers(0, pool, size=shape)].view(np.int32)


def make_packed_problem(bits: int, n: int, s: int, m: int, group_size: int, *, sparse: bool = False,
                        batch: int = 1, seed: int = 0):
    """Seeded problem for full-size shapes, drawn directly in the packed formats (uniform packed words are
    uniform weights in every format: nibbles, crumbs, 3-bit fields of the 96-bit streams, compacted nibbles),
    with the value distributions of make_problem.  No (N, S) array of unpacked weights is ever built; check
    results with expected_columns."""
    rng = np.random.default_rng(seed)
    lo, hi = (0.002, 0.02) if bits == 4 else (0.005, 0.05)
    rows = n // 16 if sparse else n * bits // 32
    matrix = rng.integers(0, 1 << 32, size=(rows, s), dtype=np.uint64).astype(np.uint32).view(np.int32)
    mask = random_keep_words(rng, (n // 32, s)) if sparse else None
    g = n if group_size < 0 else group_size
    n_groups = (n + g - 1) // g
    scales = rng.uniform(lo, hi, size=(n_groups, s)).astype(np.float16)
    zeros = rng.integers(0, 1 << bits, size=(n_groups, s)).astype(np.float16)
    x = rng.standard_normal(size=(batch, m, n), dtype=np.float32).astype(np.float16)
    return dict(bits=bits, n=n, s=s, m=m, batch=batch, group_size=group_size, sparse=sparse,
                matrix=matrix, mask=mask, scales=scales, zeros=zeros, x=x)
