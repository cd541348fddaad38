"""Golden vectors recorded from the reference's own CUDA kernels on a B200 (tests/golden/reference_gpu_vectors.npz,
made by tests/golden/make_reference_gpu_vectors.py): the CPU oracle is checked against them without a GPU, and the
product's two kernel paths are checked against them on the GPU."""
import os
import re

import numpy as np
import pytest

from oracle import reference_oracle as oracle

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_gpu_vectors.npz"))
CASES = sorted(k[:-4] for k in GOLD.files if k.endswith("_out"))


def problem_of(tag):
    m = re.match(r"b(\d)_(sp|dn)_n(\d+)_s(\d+)_m(\d+)_g(\d+)_seed(\d+)(_exp)?$", tag)
    bits, sparse = int(m[1]), m[2] == "sp"
    n, s, rows, g, seed = (int(m[i]) for i in range(3, 8))
    return oracle.make_problem(bits, n, s, rows, g, sparse=sparse, seed=seed, exponent_frac=0.5 if m[8] else 0.0)


def within_tolerance(got, want, bound):
    ulp = oracle.fp16_ulp_distance(got, want)
    diff = np.abs(got.astype(np.float32) - want.astype(np.float32))
    return (ulp <= 1) | (diff <= 2.0 ** -13 * bound)


@pytest.mark.parametrize("tag", CASES)
def test_oracle_reproduces_the_reference_kernels(tag):
    p = problem_of(tag)
    ref_out = GOLD[tag + "_out"]
    want, _, bound = oracle.expected(p, outs_in=np.zeros((1, 1, p["s"]), np.float16) if p["m"] == 1 else None)
    # the reference sums in its own order (wmma fragments; fp32 atomics in the matvec): equality up to fp32 reassociation
    assert within_tolerance(ref_out, want, bound).all()
    assert (oracle.fp16_ulp_distance(ref_out, want) == 0).mean() > 0.98
    if p["sparse"]:      # the 16:32 packer is integer work: bit-exact
        assert np.array_equal(GOLD[tag + "_packed"], p["matrix"])
        assert np.array_equal(GOLD[tag + "_mask"], p["mask"])


@pytest.mark.gpu
@pytest.mark.parametrize("tag", CASES)
@pytest.mark.parametrize("path", [1, 2], ids=["stream", "tcgen05"])
def test_kernels_reproduce_the_reference_kernels(tag, path):
    from helpers import run_problem
    p = problem_of(tag)
    got = run_problem(p, path=path)
    _, _, bound = oracle.expected(p)
    assert within_tolerance(got, GOLD[tag + "_out"], bound).all()
