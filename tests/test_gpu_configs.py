"""GPU: the benchmark configurations at their full shapes, through the C ABI, checked against the oracle on sampled
output columns (every output column depends only on its own column of the weight-side tensors, so a sample of
columns is checked exactly as the whole matrix would be, at a cost the CPU finishes in seconds)."""
import numpy as np
import pytest
import torch

from int4matmul_kernels_b200 import capi, ops
from oracle import reference_oracle as oracle

from helpers import assert_parity, to_dev

pytestmark = pytest.mark.gpu


def sample_columns(s, count, seed):
    """Tile edges of both tile widths (128 columns, 256 for CTA pairs), the matrix edges, and random columns."""
    rng = np.random.default_rng(seed)
    edges = [0, 1, 63, 64, 127, 128, 129, 255, 256, 257, s // 2 - 1, s // 2, s - 257, s - 129, s - 128, s - 65, s - 64, s - 1]
    cols = set(c for c in edges if 0 <= c < s)
    cols.update(int(c) for c in rng.integers(0, s, size=count))
    return np.array(sorted(cols))


def run_packed(p, path=capi.PATH_AUTO, outs_in=None):
    """ops.quant_matmul on a packed problem; returns the whole fp16 output (B, M, S) as numpy."""
    outs = to_dev(outs_in) if outs_in is not None else torch.zeros((p["batch"], p["m"], p["s"]), dtype=torch.float16, device="cuda")
    mask = to_dev(p["mask"]) if p["mask"] is not None else None
    ops.quant_matmul(p["bits"], outs, to_dev(p["matrix"]), to_dev(p["x"]), to_dev(p["scales"]), to_dev(p["zeros"]),
                     p["group_size"], mask, path=path)
    torch.cuda.synchronize()
    return outs.cpu().numpy()


def check_packed(p, what, path=capi.PATH_AUTO, n_cols=160, with_outs=False):
    outs_in = None
    if p["m"] == 1:                                           # the matvec route adds into outs (matvec_kernel.cu:351)
        rng = np.random.default_rng(11)
        outs_in = (rng.standard_normal((p["batch"], 1, p["s"])) if with_outs else np.zeros((p["batch"], 1, p["s"]))).astype(np.float16)
    got = run_packed(p, path, outs_in)
    cols = sample_columns(p["s"], n_cols, p["n"] + p["m"])
    want, bound = oracle.expected_columns(p["bits"], p["matrix"], p["mask"], p["scales"], p["zeros"], p["group_size"],
                                          p["x"], cols, outs_in[..., cols] if outs_in is not None else None)
    st = assert_parity(got[..., cols], want, bound, what)
    assert st["frac_exact"] > 0.8, (what, st)
    return got


def test_metric_shape_int4_matvec_16384():
    p = oracle.make_packed_problem(4, 16384, 16384, 1, 128, seed=0)
    a = check_packed(p, "int4 matvec 16384^2", with_outs=True)
    assert capi.load().i4mm_last_launch_shape() == 16
    b = check_packed(p, "int4 matvec 16384^2 (again)", with_outs=True)
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))            # fixed summation order: bit-reproducible
    check_packed(p, "int4 matvec 16384^2, streaming path", path=capi.PATH_STREAM)


@pytest.mark.parametrize("n,s", [(5120, 20480), (20480, 5120)])
def test_config_int4_matmul_m2048(n, s):
    p = oracle.make_packed_problem(4, n, s, 2048, 128, seed=2)
    a = check_packed(p, f"int4 matmul M=2048 {n}x{s}")
    assert capi.load().i4mm_last_launch_shape() >= 1128               # a CTA-pair instance of 128 rows or more
    b = check_packed(p, f"int4 matmul M=2048 {n}x{s}, single CTAs", path=capi.PATH_TCGEN05_SINGLE_CTA)
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))            # same k order per output element


def test_config_sparse_matvec_16384():
    p = oracle.make_packed_problem(4, 16384, 16384, 1, 64, sparse=True, seed=3)
    check_packed(p, "16:32 matvec 16384^2", with_outs=True)
    check_packed(p, "16:32 matvec 16384^2, streaming path", path=capi.PATH_STREAM)


def test_config_sparse_matmul_m2048():
    p = oracle.make_packed_problem(4, 5120, 20480, 2048, 64, sparse=True, seed=4)
    check_packed(p, "16:32 matmul M=2048 5120x20480")


@pytest.mark.parametrize("bits", [3, 2])
@pytest.mark.parametrize("m", [1, 16, 128, 2048])
def test_config_int3_int2(bits, m):
    p = oracle.make_packed_problem(bits, 20480, 5120, m, 64, seed=10 * bits + m)
    check_packed(p, f"int{bits} 20480x5120 M={m}")


@pytest.mark.parametrize("n,s", [(5120, 15360), (5120, 5120), (5120, 27648), (13824, 5120)],
                         ids=["qkv", "o", "gate_up", "down"])
@pytest.mark.parametrize("m", [1, 16, 128, 2048])
def test_config_stack_matrices(n, s, m):
    """The four launches of one layer of the 13B-class stack (q|k|v and gate|up run as one concatenated-S launch)."""
    p = oracle.make_packed_problem(4, n, s, m, 128, seed=n + s + m)
    check_packed(p, f"stack matrix {n}->{s} M={m}", n_cols=96)
    if m == 2048 and s == 5120:
        assert capi.load().i4mm_last_launch_shape() >= 1128


def test_reference_script_distributions():
    """The value distributions of the reference's own test script: x ~ U[-1, 1), scales ~ U[0.01, 1.01), seed 123
    (kernel_test.py:29, 185, 241), on the shapes of its README rows that matter here."""
    rng = np.random.default_rng(123)
    for n, s, m in [(16384, 16384, 1), (5120, 20480, 2048)]:
        p = oracle.make_packed_problem(4, n, s, m, 128, seed=123)
        p["x"] = rng.uniform(-1.0, 1.0, size=p["x"].shape).astype(np.float16)
        p["scales"] = rng.uniform(0.01, 1.01, size=p["scales"].shape).astype(np.float16)
        check_packed(p, f"reference distributions {n}x{s} M={m}")


def test_no_device_timeouts_recorded_by_the_full_size_runs():
    ops.check_device_status()
