"""GPU: the fused row-norm glue kernel and the layer-stack runner (single GPU; 2-GPU NCCL run where two devices exist)."""
import os
import socket

import numpy as np
import pytest
import torch

from int4matmul_kernels_b200 import ops, packing, sharding
from oracle import reference_oracle as oracle

from helpers import assert_parity

pytestmark = pytest.mark.gpu


def rn(f):
    return f * torch.rsqrt(f.pow(2).mean(dim=-1, keepdim=True) + 1e-6)


@pytest.mark.parametrize("rows,width", [(1, 5120), (3, 13824), (70, 256), (2, 14336), (2, 14338), (1, 27648)])
def test_row_norm_modes_match_the_fp32_expression(rows, width):
    g = torch.Generator().manual_seed(rows * 7 + width)
    buf = (torch.randn((rows, 3 * width), generator=g) * 3).to(torch.float16).cuda()
    a, b, c = buf[:, :width], buf[:, width:2 * width], buf[:, 2 * width:]         # strided column slices
    fa, fb, fc = a.float(), b.float(), c.float()
    want = [rn(fa), rn(fa + fb + fc), rn(fa + rn(fb)), rn(fa * fb)]
    got = [ops.row_norm(0, a), ops.row_norm(1, a, b, c), ops.row_norm(2, a, b), ops.row_norm(3, a, b)]
    torch.cuda.synchronize()
    for mode, (w, y) in enumerate(zip(want, got)):
        assert y.shape == (rows, width) and y.dtype == torch.float16
        # fp32 math on both sides, different summation order inside the row reduction: within 1 fp16 ulp
        ulp = oracle.fp16_ulp_distance(y.cpu().numpy(), w.to(torch.float16).cpu().numpy())
        assert ulp.max() <= 1, f"mode {mode}: {ulp.max()} ulp"
    # mode 4 = mode 2 and mode 0 of its result from one launch: the same bits as the two launches
    both = ops.row_norm(4, a, b)
    assert both.shape == (2, rows, width)
    assert torch.equal(both[0], got[2]) and torch.equal(both[1], ops.row_norm(0, got[2]))


@pytest.mark.parametrize("rows", [5, 40, 200])
def test_row_norm_launched_behind_a_multiply_reads_its_finished_output(rows):
    """The glue kernels are launched so that they may start while the kernel before them is still running (and so is
    the reduce kernel of a multiply whose K range was cut into parts); what they read must be that kernel's finished
    output.  Chains launched back to back without a synchronisation against the same chains with one, at the sizes of
    the 13B-class stack (a 13824 -> 5120 multiply: K parts at 40 rows, CTA pairs at 200), ordinary launches and
    launches that may overlap."""
    cfg = sharding.StackConfig(hidden=5120, mlp=13824, layers=1, bits=4, group_size=64)
    w = sharding.synthetic_stack_matrix(cfg, 0, "down", 13824, 5120, torch.device("cuda"))
    g = torch.Generator().manual_seed(rows)
    xs = [torch.randn((rows, w.n), generator=g).to(torch.float16).cuda() for _ in range(3)]
    h = torch.randn((rows, w.s), generator=g).to(torch.float16).cuda()

    def glue(mode, d):
        return ops.row_norm(mode, d) if mode == 0 else ops.row_norm(mode, d, h, d) if mode == 1 else ops.row_norm(mode, h, d)

    for static in (False, True):
        for mode in range(5):
            refs = []
            for x in xs:
                d = sharding.cuda_multiply(w, x)
                torch.cuda.synchronize()
                refs.append(glue(mode, d))
                torch.cuda.synchronize()
            ops.set_static_weights(static)
            try:
                outs = [glue(mode, sharding.cuda_multiply(w, xs[i % 3])) for i in range(24)]
                torch.cuda.synchronize()
            finally:
                ops.set_static_weights(False)
            bad = [i for i, o in enumerate(outs) if not torch.equal(o, refs[i % 3])]
            assert not bad, f"rows {rows} mode {mode} static {static}: launches {bad} differ from the synchronised ones"
    ops.check_device_status()


class _SynchronisedStack(sharding.DecoderStack):
    """The stack with a device synchronisation after every launch: the reference for what a pass must compute."""

    @staticmethod
    def combine(mode, a, b=None, c=None):
        y = sharding.DecoderStack.combine(mode, a, b, c)
        torch.cuda.synchronize()
        return y

    @classmethod
    def combine_and_normalise(cls, a, b):
        y = sharding.DecoderStack.combine_and_normalise(a, b)
        torch.cuda.synchronize()
        return y


@pytest.mark.parametrize("rows", [1, 5, 40, 200])
def test_stack_pass_at_full_width_is_the_same_with_and_without_synchronisation(rows):
    """Two layers at the 13B-class widths: passes launched back to back (ordinary launches, then launches that may
    overlap) must give the bits of a pass that synchronises after every launch."""
    cfg = sharding.StackConfig(hidden=5120, mlp=13824, layers=2, bits=4, group_size=64)

    def synced_multiply(w, x):
        y = sharding.cuda_multiply(w, x)
        torch.cuda.synchronize()
        return y

    plain = sharding.DecoderStack(cfg, 0, 1, torch.device("cuda"))
    synced = _SynchronisedStack(cfg, 0, 1, torch.device("cuda"), multiply=synced_multiply)
    synced.layers = plain.layers                                   # the same weights
    h = torch.randn((rows, cfg.hidden), generator=torch.Generator().manual_seed(rows)).to(torch.float16).cuda()
    want = synced.forward(h)
    torch.cuda.synchronize()
    for static in (False, True):
        ops.set_static_weights(static)
        try:
            outs = [plain.forward(h) for _ in range(6)]
            torch.cuda.synchronize()
        finally:
            ops.set_static_weights(False)
        bad = [i for i, o in enumerate(outs) if not torch.equal(o, want)]
        assert not bad, f"rows {rows} static {static}: passes {bad} differ from the synchronised pass"
    ops.check_device_status()


def test_stack_linears_match_the_oracle_on_the_inputs_they_received():
    cfg = sharding.StackConfig(hidden=256, mlp=512, layers=2, bits=4, group_size=64)
    calls = []

    def recording_multiply(w, x):
        y = sharding.cuda_multiply(w, x)
        calls.append((w, x.clone(), y.clone()))
        return y

    stack = sharding.DecoderStack(cfg, 0, 1, torch.device("cuda"), multiply=recording_multiply)
    for rows in (1, 40):
        calls.clear()
        h = torch.randn((rows, cfg.hidden), generator=torch.Generator().manual_seed(rows)).to(torch.float16).cuda()
        out = stack.forward(h)
        torch.cuda.synchronize()
        assert out.shape == (rows, cfg.hidden) and torch.isfinite(out.float()).all()
        assert len(calls) == cfg.layers * 4
        for w, x, y in calls:
            q = packing.unpack_dense(4, w.matrix).cpu().numpy()
            w16 = oracle.dequant_w16(4, q, w.scales.cpu().numpy(), w.zeros.cpu().numpy(), w.group_size)
            xs = x.cpu().numpy()[None]
            want = oracle.matmul_ref(xs, w16)
            assert_parity(y.cpu().numpy()[None], want, oracle.matmul_abs_bound(xs, w16), f"stack linear {w.n}x{w.s}")


def _nccl_worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dev = torch.device("cuda", rank)
        p = oracle.make_problem(4, 512, 1024, 1, 128, seed=17)
        full = sharding.QuantWeights(4, 512, 1024, 128, torch.from_numpy(p["matrix"]).to(dev),
                                     torch.from_numpy(p["scales"]).to(dev), torch.from_numpy(p["zeros"]).to(dev))
        for rows in (1, 33):
            x = torch.randn((rows, 512), generator=torch.Generator().manual_seed(rows)).to(torch.float16).to(dev)
            want = sharding.cuda_multiply(full, x)
            got = sharding.ShardedLinear(full, rank, world).forward(x)
            torch.cuda.synchronize()
            assert torch.equal(got, want), f"rank {rank} rows {rows}"
        cfg = sharding.StackConfig(hidden=256, mlp=512, layers=2, bits=4, group_size=64)
        full_stack = sharding.DecoderStack(cfg, 0, 1, dev)
        mine = sharding.DecoderStack.from_full(full_stack, rank, world)
        h = torch.randn((5, 256), generator=torch.Generator().manual_seed(3)).to(torch.float16).to(dev)
        a, b = full_stack.forward(h), mine.forward(h)
        torch.cuda.synchronize()
        assert torch.equal(a, b)
        # the same stack with the outputs gathered by the multiply kernels' own peer stores: bit-equal, step after step,
        # and replayed from one CUDA graph per rank (no collective library call inside the pass)
        mine.enable_peer_gather(rows=5)
        ops.set_static_weights(True)
        for _ in range(3):
            c = mine.forward(h)
            torch.cuda.synchronize()
            assert torch.equal(a, c), f"rank {rank}: peer gather differs"
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            mine.forward(h)
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            d = mine.forward(h)
        for _ in range(3):
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(a, d), f"rank {rank}: graph replay of the peer-gather pass differs"
        ops.set_static_weights(False)
        ops.check_device_status()
        dist.barrier()
        mine.peer.close()
        dist.barrier()
        mine.peer.destroy()
        torch.save(b.cpu(), os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_sharded_linear_and_stack_over_nccl(tmp_path):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_nccl_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert torch.equal(torch.load(tmp_path / "rank0.pt"), torch.load(tmp_path / "rank1.pt"))


@pytest.mark.parametrize("rows", [1, 16, 100, 300])
@pytest.mark.parametrize("parts,world", [(1, 4), (3, 2), (2, 8)])
def test_gathering_multiply_places_every_ranks_columns(rows, parts, world):
    """One GPU standing in for `world` ranks ONE AFTER THE OTHER (no kernel waits for another here): each rank's shard,
    multiplied by the gathering entry into the same (rows, S) buffer, must rebuild the unsharded product bit for bit,
    with the matrices of a concatenation (q | k | v, gate | up) sharded one by one."""
    import ctypes
    from int4matmul_kernels_b200 import capi
    lib = capi.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    n, s_part = 512, 64 * 3 * world                   # 192 columns per rank and part: tiles straddle part boundaries
    s = parts * s_part
    p = oracle.make_problem(4, n, s, rows, 128, seed=rows + parts)
    full = sharding.QuantWeights(4, n, s, 128, torch.from_numpy(p["matrix"]).to(dev), torch.from_numpy(p["scales"]).to(dev),
                                 torch.from_numpy(p["zeros"]).to(dev))
    x = torch.from_numpy(p["x"][0]).to(dev)
    want = sharding.cuda_multiply(full, x)
    gathered = torch.full((rows, s), 7.0, dtype=torch.float16, device=dev)
    ws = ops.workspace(dev, torch.cuda.current_stream())
    for rank in range(world):
        def cut(t):
            return torch.cat([packing.shard_columns(t[..., j * s_part:(j + 1) * s_part], rank, world) for j in range(parts)], dim=-1).contiguous()
        m, sc, z = cut(full.matrix), cut(full.scales), cut(full.zeros)
        ptrs = (ctypes.c_void_p * 1)(gathered.data_ptr())
        st = lib.i4mm_quant_matmul_gather(4, capi.PATH_AUTO, ptrs, 1, s, parts, rank, world, m.data_ptr(), None, x.data_ptr(),
                                          sc.data_ptr(), z.data_ptr(), rows, n, s // world, sc.shape[0], 128,
                                          ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
        assert st == capi.OK
    torch.cuda.synchronize()
    assert torch.equal(gathered, want)
    # the hand-shake of a single rank passes at once, and again (its values advance on the device)
    peer = sharding.PeerGather({"g": (rows, s)}, 0, 1, dev)
    for _ in range(2):
        (y,) = peer.multiply("g", full, x, 1)
        torch.cuda.synchronize()
        assert torch.equal(y, want)
    ops.check_device_status()
    peer.destroy()


def test_gathering_entry_rejects_bad_arguments():
    import ctypes
    from int4matmul_kernels_b200 import capi
    lib = capi.load()
    ptrs = (ctypes.c_void_p * 1)(16)
    call = lambda **k: lib.i4mm_quant_matmul_gather(4, k.get("path", 0), ptrs, k.get("n", 1), k.get("ld", 512), k.get("parts", 1),
                                                    k.get("rank", 0), k.get("world", 2), 16, None, 16, 16, 16, 1, 128, k.get("s", 256), 1, 128, 16, 1 << 30, None)
    assert call(n=9) == capi.ERR_SHAPE
    assert call(rank=2) == capi.ERR_SHAPE
    assert call(ld=256) == capi.ERR_SHAPE                       # narrower than S * world
    assert call(parts=3) == capi.ERR_SHAPE                      # S not divisible
    assert call(parts=8, s=256) == capi.ERR_SHAPE               # 32 columns per piece: not a multiple of 64
    assert call(path=1) == capi.ERR_UNSUPPORTED                 # the streaming kernel has no gathering epilogue
