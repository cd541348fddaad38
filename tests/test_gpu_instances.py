"""GPU: every compiled instance of the tcgen05 kernel (rows per tile x CTA pair / single CTA) against the oracle,
the matvec route's add-into-outs for any row count, repeat runs of the ring configurations whose stages are not a
multiple of the dequant warpgroups, and the host side of the device status word."""
import numpy as np
import pytest
import torch

from int4matmul_kernels_b200 import capi, ops
from oracle import reference_oracle as oracle

from helpers import assert_parity, device_problem, run_problem, to_dev
from test_gpu_stream import FORMATS, fmt_id

pytestmark = pytest.mark.gpu

PAIR, SINGLE = capi.PATH_TCGEN05, capi.PATH_TCGEN05_SINGLE_CTA


def forced(path, nt):
    return path | (nt << 8)


def last_shape():
    return capi.load().i4mm_last_launch_shape()


@pytest.mark.parametrize("fmt", FORMATS, ids=fmt_id)
@pytest.mark.parametrize("nt", [128, 160, 192, 224, 256])
@pytest.mark.parametrize("path", [PAIR, SINGLE], ids=["pair", "single"])
def test_every_many_row_instance(fmt, nt, path):
    """Rows per tile forced, so that each compiled instance is exercised whatever the shape heuristic prefers:
    several row tiles with a ragged last one, several column tiles per CTA, an odd number of column tiles."""
    bits, sparse = fmt
    g = 64 if nt in (160, 224) else 128
    p = oracle.make_problem(bits, 1152, 128 * 5, 2 * nt + 37, g, sparse=sparse, seed=nt + bits)
    got = run_problem(p, path=forced(path, nt))
    assert last_shape() % 10000 == nt + (1000 if path == PAIR else 0)
    want, _, bound = oracle.expected(p)
    assert_parity(got, want, bound, f"NT={nt} path={path} {fmt}")


@pytest.mark.parametrize("fmt", FORMATS, ids=fmt_id)
@pytest.mark.parametrize("nt,m", [(16, 9), (32, 32), (64, 50)])
def test_every_few_row_instance(fmt, nt, m):
    bits, sparse = fmt
    p = oracle.make_problem(bits, 1152, 128 * 5, m, 64, sparse=sparse, seed=nt + bits)
    got = run_problem(p, path=forced(PAIR, nt))
    assert last_shape() % 10000 == nt
    want, _, bound = oracle.expected(p)
    assert_parity(got, want, bound, f"NT={nt} {fmt}")


@pytest.mark.parametrize("path", [PAIR, SINGLE], ids=["pair", "single"])
@pytest.mark.parametrize("m,nt", [(224, 224), (448, 224), (256, 256), (512, 256)])
def test_one_wave_shapes_pick_the_tall_tiles(path, m, nt):
    """As many column tiles as the GPU has SMs (pairs: SM pairs): one wave of 224- or 256-row tiles beats two waves
    of shorter ones, so the shape heuristic itself lands on the instances the full-size matmuls run."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    p = oracle.make_problem(4, 384, 128 * sms, m, 128, seed=m)
    got = run_problem(p, path=path)
    assert last_shape() % 10000 == nt + (1000 if path == PAIR else 0)
    want, _, bound = oracle.expected(p)
    assert_parity(got, want, bound, f"one wave m={m} path={path}")


@pytest.mark.parametrize("fmt", FORMATS, ids=fmt_id)
@pytest.mark.parametrize("batch", [65, 130, 300])
@pytest.mark.parametrize("path", [capi.PATH_AUTO, PAIR, SINGLE], ids=["auto", "pair", "single"])
def test_batched_matvec_adds_into_outs_for_any_batch(fmt, batch, path):
    """seq_len == 1 is the matvec route for any batch (grid z = batch, matvec_kernel.cu:343-347) and it adds into the
    caller's outs (matvec_kernel.cu:351, 381-382); more than 64 rows take the many-row tiles here."""
    bits, sparse = fmt
    p = oracle.make_problem(bits, 512, 384, 1, 64, sparse=sparse, batch=batch, seed=batch + bits)
    base = np.random.default_rng(batch).standard_normal((batch, 1, 384)).astype(np.float16)
    got = run_problem(p, path=path, outs_in=base)
    want, _, bound = oracle.expected(p, outs_in=base)
    assert_parity(got, want, bound, f"batched matvec accumulate B={batch} {fmt} path={path}")
    if path == capi.PATH_AUTO:
        got_vec = run_problem(p, path=path, outs_in=base, route="vec")
        assert np.array_equal(got_vec.view(np.uint16), got.view(np.uint16))
        # the _mtx entry overwrites, whatever seq_len is (matmul_kernel.cu:299-332)
        got_mtx = run_problem(p, path=path, outs_in=base, route="mtx")
        want_mtx, _, _ = oracle.expected(p)
        assert_parity(got_mtx, want_mtx, bound, f"mtx overwrite B={batch} {fmt}")


def test_accumulate_through_the_c_abi_with_forced_tiles():
    lib = capi.load()
    p = oracle.make_problem(4, 640, 256, 1, 128, batch=200, seed=17)
    d = device_problem(p)
    base = np.random.default_rng(5).standard_normal((200, 1, 256)).astype(np.float16)
    want, _, bound = oracle.expected(p, outs_in=base)
    ws = ops.workspace(torch.device("cuda", torch.cuda.current_device()), torch.cuda.current_stream())
    for path in (forced(PAIR, 128), forced(PAIR, 256), forced(SINGLE, 160), forced(SINGLE, 256)):
        outs = to_dev(base)
        st = lib.i4mm_quant_matmul(4, 1, path, outs.data_ptr(), d["matrix"].data_ptr(), None, d["x"].data_ptr(),
                                   d["scales"].data_ptr(), d["zeros"].data_ptr(), 200, 640, 256, d["scales"].shape[0], 128,
                                   ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
        assert st == capi.OK
        torch.cuda.synchronize()
        assert_parity(outs.cpu().numpy(), want, bound, f"C ABI accumulate path={path:#x}")


@pytest.mark.parametrize("nt,path", [(256, PAIR), (256, SINGLE), (224, PAIR), (192, PAIR), (128, PAIR), (160, SINGLE)],
                         ids=["256-pair", "256-single", "224-pair", "192-pair", "128-pair", "160-single"])
def test_repeat_runs_of_the_guarded_ring_configurations(nt, path):
    """Ring configurations whose weight stages are not a multiple of the dequant warpgroups (3 stages / 2 groups,
    6 / 4) hand consecutive uses of a stage to different groups.  30 runs with fresh activations each, every one
    against the oracle, and a repeat of the first input that must reproduce its bits."""
    rng = np.random.default_rng(nt)
    p = oracle.make_problem(4, 2048, 128 * 12, 2 * nt, 128, seed=nt)          # 16 stages per tile, 24 / 12 tiles
    d = device_problem(p)
    _, w16, _ = oracle.expected(dict(p, x=p["x"][:, :1]))
    first = None
    for rep in range(31):
        x = p["x"] if rep in (0, 30) else rng.standard_normal(p["x"].shape).astype(np.float16)
        outs = torch.full((1, p["m"], p["s"]), 7.0, dtype=torch.float16, device="cuda")
        ops.quant_matmul(4, outs, d["matrix"], to_dev(x), d["scales"], d["zeros"], 128, None, path=forced(path, nt))
        torch.cuda.synchronize()
        got = outs.cpu().numpy()
        assert_parity(got, oracle.matmul_ref(x, w16), oracle.matmul_abs_bound(x, w16), f"NT={nt} rep {rep}")
        if rep == 0:
            first = got
    assert np.array_equal(first.view(np.uint16), got.view(np.uint16))
    ops.check_device_status()


def test_status_word_is_reported_and_cleared_on_the_host():
    """Host-side handling only: the word a kernel would set after a bounded wait ran out is written with a tensor
    store; no kernel is made to wait."""
    lib = capi.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream()
    ws = ops.workspace(dev, stream)
    assert lib.i4mm_device_status(ws.data_ptr(), stream.cuda_stream) == capi.OK
    word = ws[256 * 1024 - 64:256 * 1024 - 60].view(torch.int32)
    word.fill_(22)
    assert lib.i4mm_device_status(ws.data_ptr(), stream.cuda_stream) == capi.ERR_TIMEOUT
    assert "timed out" in capi.status_string(capi.ERR_TIMEOUT)
    assert lib.i4mm_device_status(ws.data_ptr(), stream.cuda_stream) == capi.OK
    word.fill_(31)
    with pytest.raises(ops.Int4MatmulError) as e:
        ops.check_device_status()
    assert e.value.status == capi.ERR_TIMEOUT
    ops.check_device_status()                                   # cleared, and the scratch is all-zero again
    assert int(ws.count_nonzero()) == 0
    assert lib.i4mm_static_device_status(stream.cuda_stream) == capi.OK
    # the compiled module offers the same check
    import int4matmul_kernels_b200 as pkg
    pkg.load_extension().check_device_status()


@pytest.mark.parametrize("m", [1, 16, 200])
def test_overlapped_launches_keep_stream_order_for_activations_and_outputs(m):
    """With the static-weights promise a launch may begin while the kernel before it is still running; what it reads
    (activations, old outputs) and writes (outputs, scratch) must still see that kernel's results.  A chain in which
    every call consumes the previous call's output, and a run of accumulating calls into one buffer, must give the
    same bits as the ordinary launches."""
    n = s = 1024
    probs = [oracle.make_problem(4, n, s, m, 128, seed=500 + i, scale_lo=0.01, scale_hi=0.03) for i in range(4)]
    devs = [device_problem(p) for p in probs]
    x0 = to_dev(probs[0]["x"])

    def chain():
        h = x0
        for d in devs * 3:
            out = torch.zeros((1, m, s), dtype=torch.float16, device="cuda")
            ops.quant_int4_linear_mult_mtx(out, d["matrix"], h, d["scales"], d["zeros"], 128, None)
            h = ops.row_norm(0, out.view(m, s)).view(1, m, s)
        acc = torch.zeros((1, m, s), dtype=torch.float16, device="cuda")
        for d in devs * 3:                      # the matvec route (seq_len == 1) adds into acc; others overwrite
            ops.quant_matmul(4, acc, d["matrix"], x0, d["scales"], d["zeros"], 128, None)
        torch.cuda.synchronize()
        return h.cpu().numpy(), acc.cpu().numpy()

    plain = chain()
    ops.set_static_weights(True)
    try:
        for _ in range(3):
            over = chain()
            assert np.array_equal(plain[0].view(np.uint16), over[0].view(np.uint16))
            assert np.array_equal(plain[1].view(np.uint16), over[1].view(np.uint16))
    finally:
        ops.set_static_weights(False)
    # and the first link of the chain against the oracle
    out = torch.zeros((1, m, s), dtype=torch.float16, device="cuda")
    ops.quant_int4_linear_mult_mtx(out, devs[0]["matrix"], x0, devs[0]["scales"], devs[0]["zeros"], 128, None)
    want, _, bound = oracle.expected(probs[0])
    assert_parity(out.cpu().numpy(), want, bound, f"first link m={m}")
    ops.check_device_status()
