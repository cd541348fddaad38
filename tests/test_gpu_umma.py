"""GPU parity tests of the tcgen05 path (tensor-memory A operand), through the C ABI, for every format and
for row counts from 1 to several tiles."""
import numpy as np
import pytest
import torch

from int4matmul_kernels_b200 import capi, ops
from oracle import reference_oracle as oracle

from helpers import assert_parity, run_problem, to_dev
from test_gpu_stream import FORMATS, fmt_id, one_hot_problem

pytestmark = pytest.mark.gpu
P = capi.PATH_TCGEN05


@pytest.mark.parametrize("fmt", FORMATS, ids=fmt_id)
@pytest.mark.parametrize("zero_kind", ["integer", "fraction", "large"])
def test_dequantised_weights_are_bit_exact(fmt, zero_kind):
    bits, sparse = fmt
    p = one_hot_problem(bits, sparse, 256, 128, 64, 11, zero_kind)
    got = run_problem(p, path=P)[0]
    w16 = oracle.dequant_w16(bits, p["q"], p["scales"], p["zeros"], p["group_size"], p["keep"])
    assert np.array_equal(got.view(np.uint16), w16.view(np.uint16))


@pytest.mark.parametrize("fmt", FORMATS, ids=fmt_id)
def test_exponent_coding_is_bit_exact(fmt):
    bits, sparse = fmt
    p = one_hot_problem(bits, sparse, 128, 128, 64, 13, "integer", exponent_frac=0.5)
    got = run_problem(p, path=P)[0]
    w16 = oracle.dequant_w16(bits, p["q"], p["scales"], p["zeros"], p["group_size"], p["keep"])
    assert np.array_equal(got.view(np.uint16), w16.view(np.uint16))


@pytest.mark.parametrize("fmt", FORMATS, ids=fmt_id)
@pytest.mark.parametrize("n,s,g", [(64, 64, 64), (128, 192, 64), (320, 128, 64), (1024, 320, 128),
                                   (768, 256, 192), (2048, 1024, -1), (4096, 4096, 128)])
def test_matvec_parity(fmt, n, s, g):
    bits, sparse = fmt
    p = oracle.make_problem(bits, n, s, 1, g, sparse=sparse, seed=n + s)
    got = run_problem(p, path=P)
    want, _, bound = oracle.expected(p, outs_in=np.zeros((1, 1, s), np.float16))
    assert_parity(got, want, bound, f"matvec {fmt} {n}x{s} g{g}")


@pytest.mark.parametrize("fmt", FORMATS, ids=fmt_id)
@pytest.mark.parametrize("m", [2, 15, 16, 17, 33, 64, 65, 128, 129, 256, 300, 700])
def test_rows_parity(fmt, m):
    bits, sparse = fmt
    p = oracle.make_problem(bits, 640, 384, m, 128, sparse=sparse, seed=100 + m)
    got = run_problem(p, path=P)
    want, _, bound = oracle.expected(p)
    assert_parity(got, want, bound, f"rows={m} {fmt}")


@pytest.mark.parametrize("fmt", FORMATS, ids=fmt_id)
def test_batched(fmt):
    bits, sparse = fmt
    for m in (1, 5, 90):
        p = oracle.make_problem(bits, 256, 192, m, 64, sparse=sparse, batch=3, seed=7 + m)
        got = run_problem(p, path=P)
        want, _, bound = oracle.expected(p, outs_in=np.zeros((3, 1, 192), np.float16) if m == 1 else None)
        assert_parity(got, want, bound, f"batch=3 m={m} {fmt}")


def test_matvec_adds_into_outs_and_matmul_overwrites():
    p = oracle.make_problem(4, 512, 256, 1, 128, seed=21)
    base = np.random.default_rng(0).standard_normal((1, 1, 256)).astype(np.float16)
    got = run_problem(p, path=P, outs_in=base)
    want, _, bound = oracle.expected(p, outs_in=base)
    assert_parity(got, want, bound, "matvec accumulate")
    p2 = oracle.make_problem(4, 512, 256, 200, 128, seed=22)
    junk = np.full((1, 200, 256), 1000.0, dtype=np.float16)
    got2 = run_problem(p2, path=P, outs_in=junk)
    want2, _, bound2 = oracle.expected(p2)
    assert_parity(got2, want2, bound2, "matmul overwrite")


def test_results_are_bit_reproducible_and_match_streaming_path_closely():
    p = oracle.make_problem(4, 8192, 2048, 1, 128, seed=5)
    a = run_problem(p, path=P)
    b = run_problem(p, path=P)
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))
    c = run_problem(p, path=capi.PATH_STREAM)
    assert oracle.fp16_ulp_distance(a, c).max() <= 2


@pytest.mark.parametrize("shape", [(5120, 2048, 256, 128), (2048, 5120, 2048, 128)])
def test_matmul_shapes_like_the_benchmark(shape):
    n, s, m, g = shape
    p = oracle.make_problem(4, n, s, m, g, seed=1)
    got = run_problem(p, path=P)
    want, _, bound = oracle.expected(p)
    st = assert_parity(got, want, bound, f"matmul {shape}")
    assert st["frac_exact"] > 0.8


@pytest.mark.parametrize("fmt", FORMATS, ids=fmt_id)
@pytest.mark.parametrize("m", [128, 129, 300, 700])
def test_single_cta_path_matches_cta_pairs_bit_for_bit(fmt, m):
    """128 rows or more run as CTA pairs (two SMs per MMA) by default; path 3 keeps single CTAs.  Same k order per
    output element, so the two must agree exactly, and both with the oracle."""
    bits, sparse = fmt
    p = oracle.make_problem(bits, 640, 384, m, 128, sparse=sparse, seed=300 + m)
    pair = run_problem(p, path=P)
    single = run_problem(p, path=capi.PATH_TCGEN05_SINGLE_CTA)
    want, _, bound = oracle.expected(p)
    assert_parity(single, want, bound, f"single-CTA rows={m} {fmt}")
    assert np.array_equal(pair.view(np.uint16), single.view(np.uint16))


@pytest.mark.parametrize("s", [128, 256, 640, 1152])
def test_cta_pairs_with_odd_and_even_column_tile_counts(s):
    p = oracle.make_problem(4, 1024, s, 520, 128, seed=s)
    got = run_problem(p, path=P)
    want, _, bound = oracle.expected(p)
    assert_parity(got, want, bound, f"pairs S={s}")


@pytest.mark.parametrize("fmt", FORMATS, ids=fmt_id)
@pytest.mark.parametrize("m", [40, 64, 100, 128, 300, 520])
@pytest.mark.parametrize("path", [P, capi.PATH_TCGEN05_SINGLE_CTA])
def test_k_parts_for_shapes_with_few_column_tiles(fmt, m, path):
    """More than 32 rows and few tiles: K is cut into parts (one CTA or CTA pair each) whose fp32 partial outputs a
    second kernel sums in part order; afterwards the few-row split-K path must still find its scratch all-zero."""
    bits, sparse = fmt
    p = oracle.make_problem(bits, 2048, 320, m, 128, sparse=sparse, seed=700 + m)
    got = run_problem(p, path=path)
    want, _, bound = oracle.expected(p)
    assert_parity(got, want, bound, f"k-parts rows={m} {fmt}")
    again = run_problem(p, path=path)
    assert np.array_equal(got.view(np.uint16), again.view(np.uint16))
    p1 = oracle.make_problem(bits, 2048, 320, 1, 128, sparse=sparse, seed=800 + m)
    got1 = run_problem(p1, path=P)
    want1, _, bound1 = oracle.expected(p1, outs_in=np.zeros((1, 1, 320), np.float16))
    assert_parity(got1, want1, bound1, f"matvec after k-parts {fmt}")


def test_no_device_timeouts_recorded():
    ws = ops.workspace(torch.device("cuda", torch.cuda.current_device()), torch.cuda.current_stream())
    assert capi.load().i4mm_device_status(ws.data_ptr(), torch.cuda.current_stream().cuda_stream) == capi.OK
