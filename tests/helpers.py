"""Shared helpers of the GPU parity tests: run a seeded problem through the C ABI and compare with the oracle."""
import numpy as np
import torch

from int4matmul_kernels_b200 import capi, ops
from oracle import reference_oracle as oracle

# Tolerance of the parity tests against the reference-semantics oracle (fp16 weights bit-exact, fp32
# accumulation, one fp16 rounding).  The reference's own summation order is unspecified (wmma fragments,
# fp32 atomics), so results may differ by fp32 reassociation before the final rounding:
#   every element: at most 1 fp16 ulp from the oracle, OR |diff| <= 2^-13 * sum_n |x * W16|
ULP_TOL = 1
ABS_FRAC = 2.0 ** -13


def to_dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def device_problem(p):
    d = dict(matrix=to_dev(p["matrix"]), x=to_dev(p["x"]), scales=to_dev(p["scales"]), zeros=to_dev(p["zeros"]),
             mask=to_dev(p["mask"]) if p["mask"] is not None else None)
    return d


def run_problem(p, *, path=capi.PATH_AUTO, outs_in=None, route="auto"):
    """Run through the ctypes C-ABI mirror; returns the fp16 output as numpy (B, M, S)."""
    d = device_problem(p)
    if outs_in is None:
        outs = torch.zeros((p["batch"], p["m"], p["s"]), dtype=torch.float16, device="cuda")
    else:
        outs = to_dev(outs_in)
    fn = {"auto": ops.quant_matmul}.get(route)
    if route == "auto":
        ops.quant_matmul(p["bits"], outs, d["matrix"], d["x"], d["scales"], d["zeros"], p["group_size"], d["mask"], path=path)
    else:
        getattr(ops, f"quant_int{p['bits']}_linear_mult_{route}")(
            outs, d["matrix"], d["x"], d["scales"], d["zeros"], p["group_size"], d["mask"], path=path)
    torch.cuda.synchronize()
    return outs.cpu().numpy()


def assert_parity(got, want, bound, what=""):
    assert got.shape == want.shape, (got.shape, want.shape)
    ulp = oracle.fp16_ulp_distance(got, want)
    diff = np.abs(got.astype(np.float32) - want.astype(np.float32))
    ok = (ulp <= ULP_TOL) | (diff <= ABS_FRAC * bound)
    finite = np.isfinite(want.astype(np.float32))
    ok = ok | (~finite & (got.view(np.uint16) == want.view(np.uint16)))
    if not ok.all():
        bad = np.argwhere(~ok)
        i = tuple(bad[0])
        raise AssertionError(f"{what}: {len(bad)} of {ok.size} elements out of tolerance; first at {i}: "
                             f"got {got[i]} want {want[i]} ulp {ulp[i]} bound {bound[i]}")
    return dict(max_ulp=int(ulp.max()), frac_exact=float((ulp == 0).mean()))
