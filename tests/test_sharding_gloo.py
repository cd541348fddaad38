"""CPU, world_size 2 over gloo: column sharding, output gathering and the layer-stack data flow.

The local multiply is injected (the numpy oracle working on CPU tensors), so these tests exercise exactly the
host-side logic that surrounds the CUDA operator in a multi-GPU run: shard index math, the layout of the
all-gathered outputs, and the re-assembly of concatenated q|k|v and gate|up matrices."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from int4matmul_kernels_b200 import packing, sharding
from oracle import reference_oracle as oracle


def oracle_multiply(w: sharding.QuantWeights, x: torch.Tensor) -> torch.Tensor:
    q = oracle.unpack_dense_pow2(w.bits, w.matrix.numpy())
    w16 = oracle.dequant_w16(w.bits, q, w.scales.numpy(), w.zeros.numpy(), w.group_size)
    y = oracle.matmul_ref(x.numpy()[None], w16)[0]
    return torch.from_numpy(y)


def small_weights(n, s, g, seed):
    p = oracle.make_problem(4, n, s, 1, g, seed=seed)
    return sharding.QuantWeights(4, n, s, g, torch.from_numpy(p["matrix"]), torch.from_numpy(p["scales"]),
                                 torch.from_numpy(p["zeros"]))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # --- one sharded linear: gathered result == unsharded result, bit for bit, for 1 and several rows ---
        full = small_weights(256, 384, 64, seed=5)
        for rows in (1, 5):
            x = torch.from_numpy(np.random.default_rng(rows).standard_normal((rows, 256)).astype(np.float16))
            lin = sharding.ShardedLinear(full, rank, world, multiply=oracle_multiply)
            got = lin.forward(x)
            want = oracle_multiply(full, x)
            assert got.shape == want.shape
            assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"rank {rank} rows {rows}"
            lo, hi = sharding.column_range(384, rank, world)
            assert torch.equal(lin.forward_local(x), want[:, lo:hi])
        # --- the decoder stack: world-2 shards of a full stack reproduce the world-1 result exactly ---
        cfg = sharding.StackConfig(hidden=128, mlp=256, layers=2, bits=4, group_size=64)
        full_stack = sharding.DecoderStack(cfg, 0, 1, "cpu", multiply=oracle_multiply)
        mine = sharding.DecoderStack.from_full(full_stack, rank, world)
        h = torch.from_numpy(np.random.default_rng(9).standard_normal((3, 128)).astype(np.float16))
        want = full_stack.forward(h.clone())
        got = mine.forward(h.clone())
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        torch.save(got, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_world_size_2_sharding_and_gather(tmp_path):
    world = 2
    mp.spawn(worker, args=(world, free_port(), str(tmp_path)), nprocs=world, join=True)
    a, b = torch.load(tmp_path / "rank0.pt"), torch.load(tmp_path / "rank1.pt")
    assert torch.equal(a, b)                      # every rank ends with the same gathered activations


def test_column_range_rules():
    assert sharding.column_range(5120, 3, 8) == (1920, 2560)
    assert sharding.column_range(13824, 7, 8) == (12096, 13824)       # 13824 / 8 = 27 * 64
    with pytest.raises(ValueError):
        sharding.column_range(5120 + 64, 0, 8)
    t = torch.arange(2 * 256).view(2, 256)
    assert torch.equal(packing.shard_columns(t, 1, 4), t[:, 64:128])
    assert packing.shard_columns(t, 1, 4).is_contiguous()


def test_stack_config_matches_the_benchmark_shapes():
    cfg = sharding.STACK_13B
    assert cfg.weights_per_layer() == 317_194_240                      # 4 x 5120^2 + 3 x 5120 x 13824
    names = [m[0] for m in cfg.matrices()]
    assert names == ["qkv", "o", "gate_up", "down"]


def test_gathered_column_map_is_a_part_major_permutation():
    """The column map of the gathering multiply (OutMap in the kernels, `gathered_column` here): over all ranks the
    shards' columns fill the gathered buffer exactly once, piece by piece, ranks in order inside a piece."""
    from int4matmul_kernels_b200 import sharding
    for parts, world, part_cols in [(1, 8, 640), (3, 8, 640), (2, 8, 1728), (2, 2, 64)]:
        s_local = parts * part_cols
        seen = {}
        for rank in range(world):
            for c in range(s_local):
                g = sharding.gathered_column(c, part_cols, rank, world)
                assert g not in seen
                seen[g] = (rank, c)
        assert sorted(seen) == list(range(s_local * world))
        for g, (rank, c) in seen.items():
            piece, inside = divmod(g, part_cols * world)
            assert piece == c // part_cols and inside // part_cols == rank and inside % part_cols == c % part_cols
