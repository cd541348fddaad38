"""CPU: the numpy oracle against the vectors recorded from the reference's own Python helpers, plus
format round trips and closed-form known answers (the reference's RANDOMIZE_* = False toggles)."""
import os

import numpy as np
import pytest

from oracle import reference_oracle as o

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_python_vectors.npz"))
TAGS = sorted({"_".join(k.split("_")[:4]) for k in GOLD.files})


@pytest.mark.parametrize("tag", TAGS)
def test_packers_and_dequant_match_reference_python(tag):
    bits = int(tag[1])
    g = int(tag.split("_g")[1])
    q = np.ascontiguousarray(GOLD[tag + "_q_sn"].T)
    packed = o.pack_dense_int3(q) if bits == 3 else o.pack_dense_pow2(bits, q)
    assert np.array_equal(packed, GOLD[tag + "_packed"])
    unpacked = o.unpack_dense_int3(packed) if bits == 3 else o.unpack_dense_pow2(bits, packed)
    assert np.array_equal(unpacked, q)
    w16 = o.dequant_w16(bits, q, GOLD[tag + "_scales"], GOLD[tag + "_zeros"], g)
    assert np.array_equal(w16.view(np.uint16), GOLD[tag + "_w16"].view(np.uint16))
    w32 = o.dequant_fp32(bits, q, GOLD[tag + "_scales"], GOLD[tag + "_zeros"], g)
    assert np.array_equal(w32, GOLD[tag + "_w32"])
    # the script's fp32 comparator; torch's and numpy's sgemm may order the sum differently
    y32 = o.matmul_fp32(GOLD[tag + "_x"], w32)
    np.testing.assert_allclose(y32, GOLD[tag + "_y32"], rtol=1e-5, atol=1e-4)
    # reference semantics vs the script's fp16 matmul: same weights, fp32 vs fp16 accumulation
    y = o.matmul_ref(GOLD[tag + "_x"], w16)
    assert o.mean_rel_error(GOLD[tag + "_y32"], y) < 0.01


def test_int3_straddling_fields_by_hand():
    # weight 10 spans bits 30..32, weight 21 spans bits 63..65 of the 96-bit stream (matmul.cuh:286-301)
    q = np.zeros((32, 64), dtype=np.uint8)
    q[10, :] = 0b101
    q[21, :] = 0b110
    w = o.pack_dense_int3(q).view(np.uint32)
    assert w.shape == (3, 64)
    assert int(w[0, 0]) == (0b01 << 30)          # low two bits of weight 10
    assert int(w[1, 0]) == 0b1 | (0b0 << 31)     # its top bit; weight 21's low bit (0) at bit 31
    assert int(w[2, 0]) == 0b11                  # weight 21's top two bits


def test_sparse_pack_by_hand():
    # one column, one block: keep the odd positions; weights = position mod 16
    n, s = 32, 64
    wt = np.tile((np.arange(n) % 16).astype(np.uint8), (s, 1))
    msk = np.tile((np.arange(n) % 2).astype(np.uint8) * 7, (s, 1))   # any value > 0 keeps (utils_kernel.cu:34)
    w, m = o.pack_sparse_int4(wt, msk)
    assert w.shape == (2, s) and m.shape == (1, s)
    assert int(m.view(np.uint32)[0, 0]) == 0xAAAAAAAA
    # kept weights in order: 1,3,5,...,15,1,3,...,15 -> nibbles LSB first
    assert int(w.view(np.uint32)[0, 0]) == 0xFDB97531
    assert int(w.view(np.uint32)[1, 0]) == 0xFDB97531
    q, keep = o.unpack_sparse_int4(w, m)
    assert np.array_equal(keep[:, 0], np.arange(n) % 2 == 1)
    assert np.array_equal(q[:, 0], np.where(np.arange(n) % 2 == 1, np.arange(n) % 16, 0))


def test_sparse_pack_rejects_bad_block():
    wt = np.zeros((64, 32), dtype=np.uint8)
    msk = np.ones((64, 32), dtype=np.uint8)
    with pytest.raises(ValueError):
        o.pack_sparse_int4(wt, msk)


@pytest.mark.parametrize("bits,sparse", [(4, False), (3, False), (2, False), (4, True)])
def test_round_trip_random(bits, sparse):
    p = o.make_problem(bits, 256, 128, 1, 64, sparse=sparse, seed=5)
    if sparse:
        q, keep = o.unpack_sparse_int4(p["matrix"], p["mask"])
        assert np.array_equal(keep, p["keep"])
        assert np.array_equal(q, np.where(p["keep"], p["q"], 0))
    elif bits == 3:
        assert np.array_equal(o.unpack_dense_int3(p["matrix"]), p["q"])
    else:
        assert np.array_equal(o.unpack_dense_pow2(bits, p["matrix"]), p["q"])


@pytest.mark.parametrize("n", [5120, 13824, 16384, 20480])
def test_all_ones_known_answer(n):
    # q = 1, z = 0, s = 1, x = 1  ->  every output equals N (dense) or N/2 (16:32), exactly in fp16
    s = 64
    q = np.ones((n, s), dtype=np.uint8)
    scales = np.ones((1, s), dtype=np.float16)
    zeros = np.zeros((1, s), dtype=np.float16)
    x = np.ones((1, 1, n), dtype=np.float16)
    w16 = o.dequant_w16(4, q, scales, zeros, -1)
    assert np.all(o.matmul_ref(x, w16) == np.float16(n))
    keep = np.tile((np.arange(n) % 32 < 16)[:, None], (1, s))
    w16s = o.dequant_w16(4, q, scales, zeros, -1, keep)
    assert np.all(o.matmul_ref(x, w16s) == np.float16(n // 2))


def test_exponent_coding_values():
    # scale < 0 selects +-2^(q & 7) * (-scale) + zero with a single rounding (matmul.cuh:127-136)
    q = np.arange(16, dtype=np.uint8).reshape(16, 1).repeat(64, axis=1)
    q = np.concatenate([q] * 4, axis=0)
    scales = np.full((1, 64), -0.5, dtype=np.float16)
    zeros = np.full((1, 64), 3.0, dtype=np.float16)
    w = o.dequant_w16(4, q, scales, zeros, -1)[:16, 0].astype(np.float32)
    want = np.array([(1 << (v & 7)) * (-1 if v & 8 else 1) * 0.5 + 3.0 for v in range(16)], dtype=np.float32)
    assert np.array_equal(w, want)


def test_matvec_accumulates_into_outs():
    p = o.make_problem(4, 128, 64, 1, 64, seed=3)
    base = np.full((1, 1, 64), 2.5, dtype=np.float16)
    y0, w16, _ = o.expected(p)
    y1, _, _ = o.expected(p, outs_in=base)
    acc = p["x"].reshape(1, -1).astype(np.float32) @ w16.astype(np.float32)
    assert np.array_equal(y1.reshape(-1), (acc.reshape(-1) + np.float32(2.5)).astype(np.float16))
    assert not np.array_equal(y0, y1)


@pytest.mark.parametrize("bits,sparse", [(4, False), (3, False), (2, False), (4, True)])
def test_sampled_columns_agree_with_the_whole_matrix(bits, sparse):
    """expected_columns works from the packed tensors and must give, column for column, what expected() gives
    from the unpacked weights, for both routes."""
    p = o.make_problem(bits, 512, 256, 5, 64, sparse=sparse, seed=3, exponent_frac=0.2)
    cols = np.array([0, 5, 77, 128, 255])
    want, _, bound = o.expected(p)
    w2, b2 = o.expected_columns(bits, p["matrix"], p["mask"], p["scales"], p["zeros"], 64, p["x"], cols)
    assert np.array_equal(w2.view(np.uint16), want[..., cols].view(np.uint16))
    assert np.allclose(b2, bound[..., cols])
    base = np.random.default_rng(1).standard_normal(want.shape).astype(np.float16)
    want_acc, _, _ = o.expected(p, outs_in=base)
    w3, _ = o.expected_columns(bits, p["matrix"], p["mask"], p["scales"], p["zeros"], 64, p["x"], cols, base[..., cols])
    assert np.array_equal(w3.view(np.uint16), want_acc[..., cols].view(np.uint16))


def test_packed_problem_generator():
    p = o.make_packed_problem(4, 256, 128, 3, 64, sparse=True, seed=9)
    assert p["matrix"].shape == (16, 128) and p["mask"].shape == (8, 128) and p["x"].shape == (1, 3, 256)
    bits = np.unpackbits(p["mask"].view(np.uint8).reshape(-1, 4), axis=1)
    assert (bits.sum(axis=1) == 16).all()                      # exactly 16 of every 32 kept (utils_kernel.cu:41)
    q, keep = o.unpack_sparse_int4(p["matrix"], p["mask"])
    assert keep.reshape(8, 32, 128).sum(axis=1).min() == 16 and q.max() <= 15
    for b, rows in ((4, 32), (3, 24), (2, 16)):
        d = o.make_packed_problem(b, 256, 64, 1, -1, seed=b)
        assert d["matrix"].shape == (rows, 64) and d["scales"].shape == (1, 64) and d["zeros"].max() < (1 << b)
