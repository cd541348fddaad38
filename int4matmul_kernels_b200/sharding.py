"""Column-sharded execution of quantized linear layers over the GPUs of one node.

Every output column s depends only on column s of the weight-side tensors and on all of x, so the path shards
along S (out-features) without any reduction: rank r of P owns columns [r*S/P, (r+1)*S/P) as contiguous copies
(`packing.shard_columns`), x is replicated, each rank runs the unchanged single-GPU operator on its shard.
Only where the next layer needs all of S are the (rows, S/P) outputs all-gathered (NCCL over NVLink on GPUs;
the same code runs over gloo on CPU for the host-logic tests, with the local multiply injected).

The 13B-class decoder stack of the benchmark configs (hidden 5120, MLP 13824, 40 layers, int4, group 128) is
described by `STACK_13B`; `DecoderStack` runs its seven matrices per layer with a fixed, documented data flow.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import packing


def column_range(s: int, rank: int, world: int) -> tuple[int, int]:
    """Columns owned by `rank`; S / world must stay a multiple of 64 (the kernels' column granularity)."""
    if s % world or (s // world) % 64:
        raise ValueError(f"S={s} cannot be split over {world} ranks in multiples of 64 columns")
    w = s // world
    return rank * w, (rank + 1) * w


def gather_columns(local: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """All-gather (rows, S/P) shards into (rows, S) on every rank, rank r's block at columns [r*S/P, (r+1)*S/P).

    all_gather_into_tensor concatenates along dim 0, so the shards are gathered as (P, rows, S/P) and then laid
    out along the last dim; for rows == 1 that permutation is a no-op view."""
    if world == 1:
        return local
    rows, sl = local.shape
    buf = torch.empty((world, rows, sl), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf.view(world * rows, sl), local.contiguous(), group=group)
    if rows == 1:
        return buf.view(1, world * sl)
    return buf.permute(1, 0, 2).reshape(rows, world * sl)


@dataclass
class QuantWeights:
    """One quantized matrix in the reference's device layout (possibly a column shard of it)."""
    bits: int
    n: int                      # in-features
    s: int                      # out-features held here
    group_size: int
    matrix: torch.Tensor        # int32 (N*bits/32, s)   or (N/16, s) for the 16:32 format
    scales: torch.Tensor        # fp16 (n_groups, s)
    zeros: torch.Tensor         # fp16 (n_groups, s)
    mask: Optional[torch.Tensor] = None

    def shard(self, rank: int, world: int) -> "QuantWeights":
        lo, hi = column_range(self.s, rank, world)
        return QuantWeights(self.bits, self.n, hi - lo, self.group_size,
                            packing.shard_columns(self.matrix, rank, world),
                            packing.shard_columns(self.scales, rank, world),
                            packing.shard_columns(self.zeros, rank, world),
                            packing.shard_columns(self.mask, rank, world) if self.mask is not None else None)


def cuda_multiply(w: QuantWeights, x: torch.Tensor) -> torch.Tensor:
    """x (rows, N) fp16 CUDA -> (rows, w.s) fp16 through the library (overwrite semantics)."""
    from . import ops
    out = torch.empty((1, x.shape[0], w.s), dtype=torch.float16, device=x.device)
    fn = getattr(ops, f"quant_int{w.bits}_linear_mult_mtx")
    fn(out, w.matrix, x.view(1, x.shape[0], x.shape[1]), w.scales, w.zeros, w.group_size, w.mask)
    return out.view(x.shape[0], w.s)


class _DevicePointerView:
    """Lets torch wrap device memory that the library allocated (`torch.as_tensor` reads __cuda_array_interface__)."""

    def __init__(self, ptr: int, shape: tuple, typestr: str):
        self.__cuda_array_interface__ = dict(shape=shape, typestr=typestr, data=(ptr, False), version=3, strides=None)


class PeerGather:
    """Gathered output buffers that the multiply kernels of all ranks write into directly (`i4mm_quant_matmul_gather`).

    Every rank allocates one (rows, S) fp16 buffer per name plus a flags buffer through the library
    (`i4mm_peer_buffer_create`), the CUDA IPC handles go round the process group once, and every rank maps the others'
    buffers.  After that a step runs no collective library call: the multiply's epilogue stores this rank's columns
    into every rank's buffer through the peer mappings and `i4mm_gather_sync` is the hand-shake, so a pass can be
    captured in one CUDA graph per rank.  With world == 1 the same calls run on local memory only."""

    def __init__(self, shapes: dict, rank: int, world: int, device, group=None):
        import ctypes
        from . import capi
        self.lib = capi.load()
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.names = list(shapes)
        self.shapes = dict(shapes)
        hb = self.lib.i4mm_ipc_handle_bytes()
        self._owned, self._opened = [], []
        local, handles = {}, {}
        with torch.cuda.device(self.device):
            for name, nbytes in [(n, r * ld * 2) for n, (r, ld) in shapes.items()] + [("__flags", self.lib.i4mm_gather_flags_bytes(len(shapes)))]:
                ptr, h = ctypes.c_void_p(), ctypes.create_string_buffer(hb)
                self._check(self.lib.i4mm_peer_buffer_create(nbytes, ctypes.byref(ptr), h), "peer buffer")
                self._owned.append(ptr.value)
                local[name], handles[name] = ptr.value, h.raw
            everyone = [handles]
            if world > 1:
                everyone = [None] * world
                dist.all_gather_object(everyone, handles, group=group)
            self.ptrs = {}
            for name in local:
                row = []
                for r in range(world):
                    if r == rank:
                        row.append(local[name])
                    else:
                        ptr = ctypes.c_void_p()
                        self._check(self.lib.i4mm_peer_buffer_open(everyone[r][name], ctypes.byref(ptr)), "peer mapping")
                        self._opened.append(ptr.value)
                        row.append(ptr.value)
                self.ptrs[name] = (ctypes.c_void_p * world)(*row)
            self.buffers = {n: torch.as_tensor(_DevicePointerView(local[n], shapes[n], "<f2"), device=self.device) for n in shapes}
        if world > 1:
            dist.barrier(group=group)           # nobody writes before everybody has mapped

    def _check(self, status: int, what: str) -> None:
        from . import capi, ops
        if status != capi.OK:
            raise ops.Int4MatmulError(status, what)

    def multiply(self, name: str, w: QuantWeights, x: torch.Tensor, parts: int = 1) -> list:
        """x (rows, N) times this rank's shard `w`, written into every rank's gathered buffer `name`, then the hand-shake.
        Returns the `parts` gathered matrices as column slices (rows, S_part) of the local buffer."""
        from . import capi, ops
        rows_max, ld = self.shapes[name]
        rows = x.shape[0]
        if rows > rows_max or w.s * self.world != ld:
            raise ValueError("gathered buffer does not fit this multiply")
        stream = torch.cuda.current_stream(self.device)
        ws = ops.workspace(self.device, stream)
        path = capi.PATH_AUTO | (capi.PATH_STATIC_WEIGHTS if ops._static_weights else 0)
        self._check(self.lib.i4mm_quant_matmul_gather(
            w.bits, path, self.ptrs[name], self.world, ld, parts, self.rank, self.world, w.matrix.data_ptr(),
            w.mask.data_ptr() if w.mask is not None else None, x.data_ptr(), w.scales.data_ptr(), w.zeros.data_ptr(),
            rows, w.n, w.s, w.scales.shape[0], w.group_size, ws.data_ptr(), ws.numel(), stream.cuda_stream), "gathering multiply")
        self._check(self.lib.i4mm_gather_sync(self.ptrs["__flags"], self.world, self.rank, self.names.index(name), len(self.names),
                                              ws.data_ptr(), stream.cuda_stream), "gather hand-shake")
        buf = self.buffers[name][:rows]
        sp = ld // parts
        return [buf[:, i * sp:(i + 1) * sp] for i in range(parts)]

    def close(self) -> None:
        for ptr in self._opened:
            self.lib.i4mm_peer_buffer_close(ptr)
        self._opened = []

    def destroy(self) -> None:
        self.close()
        for ptr in self._owned:
            self.lib.i4mm_peer_buffer_destroy(ptr)
        self._owned = []


def gathered_column(c: int, part_cols: int, rank: int, world: int) -> int:
    """Column of a gathered buffer that local column c of rank `rank`'s shard lands in (the kernels' OutMap): piece
    c // part_cols of a concatenation whose matrices were sharded one by one."""
    part = c // part_cols
    return part * part_cols * world + rank * part_cols + c % part_cols


class ShardedLinear:
    """A column shard of one quantized linear layer plus the gather of its outputs."""

    def __init__(self, full: QuantWeights, rank: int, world: int, group=None,
                 multiply: Callable[[QuantWeights, torch.Tensor], torch.Tensor] = cuda_multiply):
        self.rank, self.world, self.group = rank, world, group
        self.full_s = full.s
        self.local = full.shard(rank, world) if world > 1 else full
        self.multiply = multiply

    def forward_local(self, x: torch.Tensor) -> torch.Tensor:
        return self.multiply(self.local, x)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return gather_columns(self.forward_local(x), self.world, self.group)


# ---- the 13B-class layer stack of the benchmark configs --------------------------------------------------------
@dataclass(frozen=True)
class StackConfig:
    hidden: int = 5120
    mlp: int = 13824            # = 64 * 216
    layers: int = 40
    bits: int = 4
    group_size: int = 128

    def matrices(self):
        """(name, in-features, out-features) of the matrices of one layer, in execution order.  q/k/v and gate/up
        read the same input, so they run as one launch over their concatenated columns."""
        h, m = self.hidden, self.mlp
        return (("qkv", h, 3 * h), ("o", h, h), ("gate_up", h, 2 * m), ("down", m, h))

    def weights_per_layer(self) -> int:
        return sum(n * s for _, n, s in self.matrices())


STACK_13B = StackConfig()


def synthetic_stack_matrix(cfg: StackConfig, layer: int, name: str, n: int, s: int, device, rank: int = 0, world: int = 1,
                           parts: int = 1) -> QuantWeights:
    """Seeded random int4 matrix of the stack, generated directly as this rank's column shard.

    Nibbles uniform over 0..15 are the same distribution as packed words uniform over int32, so the packed matrix
    is drawn directly; scales ~ U[0.002, 0.02], integer zero-points 0..15 (the benchmark's value distributions).
    `parts` > 1 marks a concatenation of `parts` equal matrices (q|k|v, gate|up): each part is sharded on its own, so
    that rank r holds [part_0 columns of r | part_1 columns of r | ...]."""
    part_s = s // parts
    lo, hi = column_range(part_s, rank, world)
    sl = (hi - lo) * parts
    seed = (layer * 131 + sum(ord(c) for c in name)) * 8 + rank
    gen = torch.Generator(device=device).manual_seed(seed)
    rows = n * cfg.bits // 32
    n_groups = n // cfg.group_size
    matrix = torch.randint(-2 ** 31, 2 ** 31 - 1, (rows, sl), dtype=torch.int32, device=device, generator=gen)
    scales = (torch.rand((n_groups, sl), device=device, generator=gen) * 0.018 + 0.002).to(torch.float16)
    zeros = torch.randint(0, 16, (n_groups, sl), device=device, generator=gen).to(torch.float16)
    return QuantWeights(cfg.bits, n, sl, cfg.group_size, matrix, scales, zeros)


class DecoderStack:
    """The linear layers of a decoder stack, column-sharded, with a fixed stand-in data flow between them:

        q, k, v = qkv(norm(h))         gathered (rows, H) each;   t = norm(q + k + v)      (stand-in for attention)
        h       = norm(h + norm(o(t)))                            gathered (rows, H)
        g, u    = gate_up(h)           gathered (rows, F) each;   a = norm(g * u)          (stand-in for the gated MLP)
        h       = norm(h + norm(down(a)))                         gathered (rows, H)

    norm = division by the row's RMS (in fp32), which keeps every activation near unit scale for any depth.  There
    is no softmax or learned parameter: the stack exists to time and check the quantized linears and their
    gathers; parity is checked per matrix on the inputs it actually received."""

    def __init__(self, cfg: StackConfig, rank: int, world: int, device, group=None, layers: Optional[int] = None,
                 multiply: Callable[[QuantWeights, torch.Tensor], torch.Tensor] = cuda_multiply):
        self.cfg, self.rank, self.world, self.group, self.multiply = cfg, rank, world, group, multiply
        self.layers = []
        for layer in range(cfg.layers if layers is None else layers):
            mats = {}
            for name, n, s in cfg.matrices():
                parts = 3 if name == "qkv" else 2 if name == "gate_up" else 1
                mats[name] = synthetic_stack_matrix(cfg, layer, name, n, s, device, rank, world, parts)
            self.layers.append(mats)

    @classmethod
    def from_full(cls, full: "DecoderStack", rank: int, world: int, group=None, multiply=None) -> "DecoderStack":
        """The shard of an unsharded (world == 1) stack that `rank` of `world` owns: every part of a concatenated
        matrix (q|k|v, gate|up) is column-sharded on its own and the rank's pieces are concatenated again."""
        self = cls.__new__(cls)
        self.cfg, self.rank, self.world, self.group = full.cfg, rank, world, group
        self.multiply = multiply if multiply is not None else full.multiply
        self.layers = []
        for mats in full.layers:
            out = {}
            for name, w in mats.items():
                parts = 3 if name == "qkv" else 2 if name == "gate_up" else 1
                part_s = w.s // parts

                def cut(t):
                    if t is None:
                        return None
                    pieces = [packing.shard_columns(t[..., i * part_s:(i + 1) * part_s], rank, world) for i in range(parts)]
                    return torch.cat(pieces, dim=-1).contiguous()

                out[name] = QuantWeights(w.bits, w.n, w.s // world, w.group_size, cut(w.matrix), cut(w.scales), cut(w.zeros), cut(w.mask))
            self.layers.append(out)
        return self

    def enable_peer_gather(self, rows: int) -> None:
        """From now on every matrix's outputs are gathered by the multiply kernels' own peer stores (PeerGather)
        instead of an NCCL all-gather; `rows` = the largest number of activation rows that will be passed."""
        shapes = {name: (rows, s) for name, _, s in self.cfg.matrices()}
        self.peer = PeerGather(shapes, self.rank, self.world, self.layers[0]["qkv"].matrix.device, self.group)

    def _linear(self, w: QuantWeights, x: torch.Tensor, parts: int, name: str = "") -> list[torch.Tensor]:
        """Local multiply + gather; returns the `parts` gathered tensors (rows, S_part)."""
        if getattr(self, "peer", None) is not None:
            return self.peer.multiply(name, w, x, parts)
        local = self.multiply(w, x)                                   # (rows, parts * S_part / P)
        rows = local.shape[0]
        if self.world == 1:
            return list(local.view(rows, parts, -1).unbind(1))
        gathered = gather_columns(local, self.world, self.group)      # (rows, P * parts * S_part / P), rank-major
        g = gathered.view(rows, self.world, parts, -1)                 # [row, rank, part, cols of that rank]
        return [g[:, :, i, :].reshape(rows, -1) for i in range(parts)]

    @staticmethod
    def combine(mode: int, a: torch.Tensor, b: Optional[torch.Tensor] = None, c: Optional[torch.Tensor] = None) -> torch.Tensor:
        """v / rms(v) per row with v = a (mode 0), a + b + c (1), a + b / rms(b) (2), a * b (3), in fp32.
        One fused kernel on CUDA tensors; the same expression in torch ops on CPU tensors (host-logic tests)."""
        if a.is_cuda:
            from . import ops
            return ops.row_norm(mode, a, b, c)

        def rn(f):
            return f * torch.rsqrt(f.pow(2).mean(dim=-1, keepdim=True) + 1e-6)
        fa = a.float()
        v = fa if mode == 0 else fa + b.float() + c.float() if mode == 1 else fa + rn(b.float()) if mode == 2 else fa * b.float()
        return rn(v).to(torch.float16)

    @classmethod
    def combine_and_normalise(cls, a: torch.Tensor, b: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """(combine(2, a, b), combine(0, of that)): a layer's output and the next layer's normalised input; one launch
        on CUDA tensors."""
        if a.is_cuda:
            from . import ops
            both = ops.row_norm(4, a, b)
            return both[0], both[1]
        h = cls.combine(2, a, b)
        return h, cls.combine(0, h)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        comb = self.combine
        x = comb(0, h)
        for i, mats in enumerate(self.layers):
            q, k, v = self._linear(mats["qkv"], x, 3, "qkv")
            t = comb(1, q, k, v)
            (o,) = self._linear(mats["o"], t, 1, "o")
            h = comb(2, h, o)
            gate, up = self._linear(mats["gate_up"], h, 2, "gate_up")
            a = comb(3, gate, up)
            (d,) = self._linear(mats["down"], a, 1, "down")
            if i + 1 < len(self.layers):
                h, x = self.combine_and_normalise(h, d)
            else:
                h = comb(2, h, d)
        return h
