"""GPU: the allocation-free entry point, i4mm_quant_matvec_static.

It exists for callers that cannot call cudaMalloc (they run inside another owner's memory pool, or in a
loop where an allocation's implicit device synchronisation is not allowed), so this test drives it the way
such a caller would: straight through the C ABI with device pointers and no workspace argument, two calls in
a row on the same stream (the second call reuses the library's fixed scratch as the first one left it), and
checks each result against the ordinary entry point on its streaming path, which runs the same kernel with
caller-provided scratch.  The file name sorts last so that a run that stops at the first failure has already
run every other test.
"""
import numpy as np
import pytest
import torch

from int4matmul_kernels_b200 import capi, ops
from oracle import reference_oracle as oracle

from helpers import assert_parity, to_dev

pytestmark = pytest.mark.gpu


def call_static(lib, p, d, outs, accumulate):
    stream = torch.cuda.current_stream()
    return lib.i4mm_quant_matvec_static(
        p["bits"], accumulate, outs.data_ptr(), d["matrix"].data_ptr(),
        d["mask"].data_ptr() if d["mask"] is not None else None, d["x"].data_ptr(), d["scales"].data_ptr(),
        d["zeros"].data_ptr(), p["batch"] * p["m"], p["n"], p["s"], d["scales"].shape[0], p["group_size"],
        stream.cuda_stream)


@pytest.mark.parametrize("bits,sparse,n,s,m", [(4, False, 4096, 4096, 1), (4, True, 2048, 1024, 1),
                                                 (3, False, 1024, 640, 5), (2, False, 8192, 256, 8)])
def test_static_scratch_entry_matches_the_ordinary_entry_twice_in_a_row(bits, sparse, n, s, m):
    lib = capi.load()
    p = oracle.make_problem(bits, n, s, m, 128 if bits == 4 and not sparse else 64, sparse=sparse, seed=77)
    d = dict(matrix=to_dev(p["matrix"]), x=to_dev(p["x"]), scales=to_dev(p["scales"]), zeros=to_dev(p["zeros"]),
             mask=to_dev(p["mask"]) if sparse else None)
    base = np.random.default_rng(1).standard_normal((1, m, s)).astype(np.float16)
    # the ordinary entry, streaming path, matvec semantics (adds into outs)
    want = to_dev(base)
    ws = ops.workspace(want.device, torch.cuda.current_stream())
    st = lib.i4mm_quant_matmul(bits, 1, capi.PATH_STREAM, want.data_ptr(), d["matrix"].data_ptr(),
                               d["mask"].data_ptr() if sparse else None, d["x"].data_ptr(), d["scales"].data_ptr(),
                               d["zeros"].data_ptr(), m, n, s, d["scales"].shape[0], p["group_size"],
                               ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
    assert st == capi.OK
    torch.cuda.synchronize()
    want = want.cpu().numpy()
    ref, _, bound = oracle.expected(p, outs_in=base)
    for attempt in range(2):                      # the second call finds the scratch as the first left it
        got = to_dev(base)
        assert call_static(lib, p, d, got, 1) == capi.OK
        torch.cuda.synchronize()
        got = got.cpu().numpy()
        # same kernel, same grid, same summation order: the tolerance of the parity tests is met with zero distance
        assert_parity(got, want, bound, f"static entry, call {attempt + 1}")
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
        assert_parity(got, ref, bound, f"static entry vs oracle, call {attempt + 1}")


def test_static_scratch_entry_rejects_what_does_not_fit():
    lib = capi.load()
    p = oracle.make_problem(4, 256, 128, 9, 64, seed=3)
    d = dict(matrix=to_dev(p["matrix"]), x=to_dev(p["x"]), scales=to_dev(p["scales"]), zeros=to_dev(p["zeros"]), mask=None)
    outs = torch.zeros((1, 9, 128), dtype=torch.float16, device="cuda")
    assert call_static(lib, p, d, outs, 0) == capi.ERR_TOO_LARGE            # 9 rows > 8
    assert "fixed scratch" in capi.status_string(capi.ERR_TOO_LARGE)
    assert torch.all(outs == 0)                                             # nothing was launched
    assert lib.i4mm_quant_matvec_static(4, 0, 16, 16, None, 16, 16, 16, 1, 128, 128 * 8193, 1, 128, None) == capi.ERR_TOO_LARGE
    assert lib.i4mm_quant_matvec_static(5, 0, 16, 16, None, 16, 16, 16, 1, 128, 128, 1, 128, None) == capi.ERR_BITS
