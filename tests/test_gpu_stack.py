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


@pytest.mark.parametrize("rows,width", [(1, 5120), (3, 13824), (70, 256)])
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
