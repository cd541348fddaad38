#!/usr/bin/env python
"""Benchmark of the quantized matmul / matvec path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One step = one operator call (`quant_matmul`) over one batch of synthetic activations.  The default
workload is the int4 dense matmul at M = 2048 on the 5120 x 20480 matrix (group 128), the configuration
the headline TFLOP/s figure is quoted on; the default run also times the matvec half of the metric (int4,
16384 x 16384, one activation row) with the same protocol and prints it under the key `matvec` of the same line.
With --gpus N (launched under torch.distributed.run, one rank per GPU) the weight matrix is column-
sharded along S over the ranks (every rank computes its own S/N columns of the same product: total work
fixed, "strong" scaling); there is no collective inside the timed region.

Prints ONE JSON line on rank 0.  Keys beyond the basic contract:
  roofline      dominant kernel: algorithmic flops (or bytes) per launch / CUDA-event time per launch,
                against the measured peak in MEASURED_PEAKS.json (fallback figures if that file is absent)
  cpu_baseline  the CPU restatement of the reference's algorithm (torch CPU dequantise + matmul, the
                reference test's own comparator) timed on this host's cores on a bounded sample
  e2e           the same metric through the drop-in torch extension module with HOST buffers: per step
                one pinned host->device copy of the activations and one device->host copy of the result
  clocks        SM clock samples taken with nvidia-smi during the timed region
  parity        the outputs the timed steps left behind, checked on sampled output columns against the CPU oracle
                after the timed region (every rank checks its own shard; rank 0 prints the worst)
  torch_fp16    torch's fp16 `x @ W16` (cuBLAS) on the dequantised matrix, the reference script's own comparator
                (kernel_test.py:248-249, 296), timed on the same GPU with the same events
`--impl reference` times the reference's algorithm on the host CPU (the reference itself is CUDA-only and
has no CPU implementation; its test script's torch dequantise-and-matmul comparator is what runs).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: bits, N (in), S (out), M, group, sparse
    "int4_matmul_m2048_5120x20480": dict(bits=4, n=5120, s=20480, m=2048, g=128, sparse=False),
    "int4_matmul_m2048_20480x5120": dict(bits=4, n=20480, s=5120, m=2048, g=128, sparse=False),
    "int4_matvec_16384": dict(bits=4, n=16384, s=16384, m=1, g=128, sparse=False),
    "int4_matvec_5120": dict(bits=4, n=5120, s=5120, m=1, g=128, sparse=False),
    "int4_sparse_matvec_16384": dict(bits=4, n=16384, s=16384, m=1, g=64, sparse=True),
    "int4_sparse_matmul_m2048_5120x20480": dict(bits=4, n=5120, s=20480, m=2048, g=64, sparse=True),
    "int3_matvec_20480x5120": dict(bits=3, n=20480, s=5120, m=1, g=64, sparse=False),
    "int2_matvec_20480x5120": dict(bits=2, n=20480, s=5120, m=1, g=64, sparse=False),
    "int4_matmul_m16_20480x5120": dict(bits=4, n=20480, s=5120, m=16, g=128, sparse=False),
    "int3_matmul_m2048_20480x5120": dict(bits=3, n=20480, s=5120, m=2048, g=64, sparse=False),
    "int2_matmul_m2048_20480x5120": dict(bits=2, n=20480, s=5120, m=2048, g=64, sparse=False),
}
# 13B-class decoder linear-layer stack (hidden 5120, MLP 13824, 40 layers, int4, group 128), column-sharded over
# the ranks with an all-gather of every matrix's outputs; "m" = activation rows
STACK_WORKLOADS = {f"stack13b_m{m}": m for m in (1, 16, 128, 2048)}
DEFAULT_WORKLOAD = "int4_matmul_m2048_5120x20480"
MATVEC_WORKLOAD = "int4_matvec_16384"            # the other half of the metric: timed by the default run as well

# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of
# the unsharded workload), with the first 12 hex digits of the SHA-256 of csrc/umma_kernel.cu as it was when the
# capture was made: the figure is printed only while the kernel source still is that file, else `traffic` is null.
NCU_TRAFFIC_BYTES = {
    "int4_matmul_m2048_5120x20480": (224119296 + 67726080, "3e9726a8cb99"),
    "int4_matvec_16384": (143103744 + 4355072, "3e9726a8cb99"),
}

L2_BYTES = 126 * 1024 * 1024


def algorithmic_bytes(w, s_cols=None):
    s = w["s"] if s_cols is None else s_cols
    n, m, bits = w["n"], w["m"], w["bits"]
    weights = (n // 16 if w["sparse"] else n * bits // 32) * s * 4
    mask = (n // 32) * s * 4 if w["sparse"] else 0
    groups = (n + w["g"] - 1) // w["g"]
    return weights + mask + 2 * groups * s * 2 + m * n * 2 + m * s * 2


def algorithmic_flops(w, s_cols=None):
    s = w["s"] if s_cols is None else s_cols
    return 2.0 * w["m"] * w["n"] * s


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm=float(d["hbm_gbs"]), tf_burst=float(d["bf16_tflops"]),
                    tf_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None

    def _loop(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip().splitlines()
                if out:
                    f = [x.strip() for x in out[0].split(",")]
                    self.samples.append(float(f[0]))
                    self.max_mhz = float(f[1])
                    for nm, v in zip(names, f[2:]):
                        if v.lower().startswith("active"):
                            self.reasons.add(nm)
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self):
        return dict(sm_mhz=statistics.median(self.samples) if self.samples else None, sm_max_mhz=self.max_mhz,
                    reasons=sorted(self.reasons), samples=len(self.samples))


def cpu_problem(w, seed=0):
    from oracle import cpu_baseline                  # the CPU legs and the parity check are where the benchmark runs oracle/
    return cpu_baseline.synthetic_unpacked(w["bits"], w["n"], w["s"], w["m"], w["g"], w["sparse"], seed)


def kernel_source_tag():
    import hashlib
    path = os.path.join(ROOT, "int4matmul_kernels_b200", "csrc", "umma_kernel.cu")
    with open(path, "rb") as f:
        return hashlib.sha256(f.read()).hexdigest()[:12]


def ncu_traffic(name, world):
    rec = NCU_TRAFFIC_BYTES.get(name)
    if rec is None or world != 1:
        return None
    return rec[0] if rec[1] == kernel_source_tag() else None


L2_RULE = "weights rotate over enough copies that consecutive steps miss L2 (copies x bytes per step > 2 x L2)"


def config_of(name, w):
    """Identical in both arms."""
    return dict(workload=name, **{k: w[k] for k in ("bits", "n", "s", "m", "g", "sparse")}, l2=L2_RULE)


def cpu_reference_seconds(w, problem, rows, cores):
    """Seconds the reference's algorithm takes for ONE full step on the CPU, from a bounded sample:
    the whole matrix is dequantised (timed in full), the matmul is timed on `rows` activation rows and
    scaled to all M rows."""
    from oracle import cpu_baseline
    t_deq, t_mm = cpu_baseline.timed_pass(problem, rows, cores)
    return t_deq + t_mm * (w["m"] / rows)


def reference_cuda_seconds(w, layer, x, torch):
    """Times the UNMODIFIED reference's CUDA kernels (built into oracle/_ref by oracle/build_reference.py) on the same
    tensors, beside the product: a baseline leg like the CPU one, never part of the product path.  None if absent."""
    import glob
    import importlib.util
    # the matvec kernels are timed from the module whose matvec translation unit was compiled at default optimisation
    # (oracle/build_reference.py); it has no dense int3 matvec
    modname = "int4matmul_ref_timing" if w["m"] == 1 else "int4matmul_ref"
    cand = glob.glob(os.path.join(ROOT, "oracle", "_ref", modname + ".*.so"))
    if not cand or (w["bits"] == 3 and w["m"] == 1):
        return None
    try:
        spec = importlib.util.spec_from_file_location(modname, cand[0])
        ref = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ref)
        out = torch.zeros((1, w["m"], layer["matrix"].shape[1]), dtype=torch.float16, device=x.device)

        def call():
            ref.quant_matmul(w["bits"], out, layer["matrix"], x, layer["scales"], layer["zeros"], w["g"], layer["mask"])

        for _ in range(3):
            call()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        iters = 10
        e0.record()
        for _ in range(iters):
            call()
        e1.record()
        torch.cuda.synchronize()
        sec = e0.elapsed_time(e1) / iters / 1e3
        kind = metric_of(w)[2]
        notes = ""
        np_ = os.path.join(ROOT, "oracle", "_ref", "BUILD_NOTES.txt")
        if os.path.exists(np_):
            notes = open(np_).read().strip()
        return dict(value=units_per_step(w, kind) / sec, unit=metric_of(w)[1], us_per_call=sec * 1e6, module=modname,
                    what="reference quant_matmul (its WMMA / CUDA-core kernels compiled for sm_100), same tensors, "
                         "its own stream and temporaries (the matvec route: 3 torch kernels and 2 allocations per call), 10 calls",
                    build_notes=notes)
    except Exception as e:
        return dict(unavailable=f"{type(e).__name__}: {e}")


def metric_of(w):
    if w["m"] == 1:
        return "int4 matvec HBM GB/s".replace("int4", f"int{w['bits']}"), "GB/s", "hbm"
    if w["m"] <= 64:
        return f"int{w['bits']} skinny matmul HBM GB/s", "GB/s", "hbm"
    return f"int{w['bits']} matmul TFLOP/s (M={w['m']})", "TFLOP/s", "tensor"


def units_per_step(w, kind, s_cols=None):
    return algorithmic_bytes(w, s_cols) / 1e9 if kind == "hbm" else algorithmic_flops(w, s_cols) / 1e12


def reference_line(args, w, name):
    """The reference's algorithm on this host's CPU cores for one workload: a dict in the bench line's format."""
    import torch
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    metric, unit, kind = metric_of(w)
    p = cpu_problem(w)
    rows = min(w["m"], 256)                     # bounded sample of the activation rows
    times = []
    for i in range(args.warmup + args.steps):
        dt = cpu_reference_seconds(w, p, rows, cores)
        if i >= args.warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    value = units_per_step(w, kind) / sec
    sample = (f"per step: full {w['n']}x{w['s']} dequantise timed whole, matmul timed on {rows} of {w['m']} rows "
              "and scaled to all rows")
    return dict(metric=metric, value=value, unit=unit, n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                ms_per_step=sec * 1e3, higher_is_better=True, scaling="strong", vs_baseline=None,
                dtype="f16", data="synthetic", impl="reference", config=config_of(name, w),
                cpu_baseline=dict(value=value, unit=unit, cores=cores, kind="port", sample=sample,
                                  spread=[units_per_step(w, kind) / max(times), units_per_step(w, kind) / min(times)]),
                e2e=dict(value=value, unit=unit, h2d_bytes_per_step=0, d2h_bytes_per_step=0))


def run_reference(args, w, name):
    """--impl reference: the reference's algorithm on this host's CPU cores (see module docstring)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    line = reference_line(args, w, name)
    if name == DEFAULT_WORKLOAD and not args.no_matvec:
        line["matvec"] = reference_line(args, WORKLOADS[MATVEC_WORKLOAD], MATVEC_WORKLOAD)
    print(json.dumps(line))


def run_stack(args):
    """The layer-stack workloads: every rank holds its column shard of every matrix; each matrix's outputs are
    all-gathered (NCCL) before the next one reads them.  One step = one pass of the activations through all layers."""
    import torch
    import torch.distributed as dist
    from int4matmul_kernels_b200 import capi, sharding

    m = STACK_WORKLOADS[args.workload]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = sharding.StackConfig(layers=args.layers)
    kind = "hbm" if m <= 64 else "tensor"
    unit = "GB/s" if kind == "hbm" else "TFLOP/s"
    wpl = cfg.weights_per_layer()
    groups_per_layer = sum((n // cfg.group_size) * s for _, n, s in cfg.matrices())
    act_per_layer = sum(m * (n + s) * 2 for _, n, s in cfg.matrices())
    bytes_pass = cfg.layers * (wpl // 2 + groups_per_layer * 4 + act_per_layer)          # int4 weights + scales + zeros + x + out
    flops_pass = cfg.layers * 2.0 * m * wpl
    metric = f"13B-class int4 linear stack, M={m}: " + ("effective HBM GB/s" if kind == "hbm" else "TFLOP/s")
    units = bytes_pass / 1e9 if kind == "hbm" else flops_pass / 1e12

    if args.impl == "reference":
        if rank != 0:
            return
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        # bounded sample: one layer's four (concatenated) matrices at reduced row count, scaled to 40 layers
        sec = 0.0
        rows = min(m, 64)
        for name, n, s_full in cfg.matrices():
            wl = dict(bits=4, n=n, s=s_full, m=rows, g=cfg.group_size, sparse=False)
            p = cpu_problem(wl)
            t_deq, t_mm = __import__("oracle.cpu_baseline", fromlist=["timed_pass"]).timed_pass(p, rows, cores)
            sec += t_deq + t_mm * (m / rows)
        sec *= cfg.layers
        value = units / sec
        sample = f"one layer (4 launches' matrices), dequantise timed whole, matmul on {rows} of {m} rows scaled; x{cfg.layers} layers"
        print(json.dumps(dict(metric=metric, value=value, unit=unit, n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                              ms_per_step=sec * 1e3, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="f16",
                              data="synthetic", impl="reference", config=dict(workload=args.workload, layers=cfg.layers, m=m),
                              cpu_baseline=dict(value=value, unit=unit, cores=cores, kind="port", sample=sample),
                              e2e=dict(value=value, unit=unit, h2d_bytes_per_step=0, d2h_bytes_per_step=0))))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import datetime
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # a short collective timeout: a rank that never arrives ends the run with an error instead of a long hang
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))
    capi.load()
    from int4matmul_kernels_b200 import ops
    ops.set_static_weights(True)
    stack = sharding.DecoderStack(cfg, rank, world, dev)
    if world > 1 and not args.nccl_gather:
        # the multiply kernels store their columns into every rank's gathered buffers themselves (peer mappings); the
        # pass then holds no collective library call and is captured as one CUDA graph per rank
        stack.enable_peer_gather(m)
    gen = torch.Generator().manual_seed(4321)
    h_host = torch.randn((m, cfg.hidden), generator=gen).to(torch.float16).pin_memory()
    h0 = h_host.to(dev)

    def step():
        return stack.forward(h0)

    for _ in range(max(args.warmup, 3)):
        out = step()
    torch.cuda.synchronize()
    graph = None
    # with NCCL all-gathers inside the step (--nccl-gather), the steps are launched directly (no graph capture of NCCL calls)
    if not args.no_graph and (world == 1 or not args.nccl_gather):
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            n0 = capi.load().i4mm_launch_count()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(args.steps):
                    out = step()
            k_launches = capi.load().i4mm_launch_count() - n0      # kernels of ours in the K captured steps
            graph.replay()
            torch.cuda.synchronize()
        except Exception as e:
            print(f"[bench] CUDA graph capture unavailable ({type(e).__name__}: {e}); timing direct launches", file=sys.stderr)
            graph = None

    if graph is None:
        n0 = capi.load().i4mm_launch_count()
        for _ in range(args.steps):
            step()
        k_launches = capi.load().i4mm_launch_count() - n0

    def run_steps():
        if graph is not None:
            graph.replay()
        else:
            for _ in range(args.steps):
                step()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local_rank) as clocks:
        run_steps()
        barrier()
        e0.record()
        run_steps()
        e1.record()
        barrier()
        run_steps()
        barrier()
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = units / (ms_step / 1e3)

    # end to end: activations from pinned host memory in, final activations back, every step
    out_host = torch.empty((m, cfg.hidden), dtype=torch.float16).pin_memory()
    h_dev = torch.empty_like(h0)

    def e2e_step():
        h_dev.copy_(h_host, non_blocking=True)
        out_host.copy_(stack.forward(h_dev), non_blocking=True)

    e2e_step()
    barrier()
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = float(t.item())

    # ---- parity, outside the timed region: layer 0's q|k|v multiply of this rank's shard against the CPU oracle on
    # sampled columns, and (several GPUs) the gathered buffer: this rank's block bit-equal to its own product, the
    # whole buffer identical on every rank ----
    x0 = stack.combine(0, h0)
    w0 = stack.layers[0]["qkv"]
    y_local = sharding.cuda_multiply(w0, x0)
    torch.cuda.synchronize()
    wl = dict(bits=4, n=w0.n, s=w0.s, m=m, g=cfg.group_size, sparse=False)
    cols = sample_columns(w0.s, 48, rank)
    n_el, n_bad, worst_ulp, exact = check_outputs(wl, [dict(matrix=w0.matrix, mask=None, scales=w0.scales, zeros=w0.zeros)],
                                                  x0.cpu().numpy()[None], y_local, cols, False)
    gather_ok = True
    if world > 1:
        parts = stack._linear(w0, x0, 3, "qkv")
        torch.cuda.synchronize()
        sp = w0.s // 3
        for j in range(3):
            gather_ok = gather_ok and bool(torch.equal(parts[j][:, rank * sp:(rank + 1) * sp], y_local[:, j * sp:(j + 1) * sp]))
        digest = torch.cat([t.contiguous().view(torch.int16).to(torch.float64).sum().view(1) for t in parts])
        lo, hi = digest.clone(), digest.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        gather_ok = gather_ok and bool(torch.equal(lo, hi))
        t = torch.tensor([float(n_bad), 0.0 if gather_ok else 1.0, float(worst_ulp)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        n_bad, gather_ok, worst_ulp = int(t[0].item()), t[1].item() == 0.0, int(t[2].item())
    # the whole pass: the output of the timed steps (launched back to back, launches overlapping) must be, bit for bit,
    # what a pass that synchronises the device after every launch computes
    def synchronised(fn):
        def call(*a, **k):
            y = fn(*a, **k)
            torch.cuda.synchronize()
            return y
        return call
    timed_out = out.clone()
    eager_out = stack.forward(h0).clone()                       # launched back to back once more, outside any graph
    torch.cuda.synchronize()
    patched = ("combine", "combine_and_normalise", "_linear")
    for attr in patched:
        setattr(stack, attr, synchronised(getattr(stack, attr)))
    try:
        synced_out = stack.forward(h0).clone()
        synced_again = stack.forward(h0)
        differing = [int((synced_out != timed_out).sum().item()), int((synced_out != eager_out).sum().item()),
                     int((synced_out != synced_again).sum().item())]
    finally:
        for attr in patched:
            delattr(stack, attr)
    if world > 1:
        t = torch.tensor([float(v) for v in differing], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        differing = [int(v) for v in t.tolist()]
    pass_ok = differing == [0, 0, 0]
    pass_differing = dict(timed_graph_vs_synchronised=differing[0], back_to_back_vs_synchronised=differing[1],
                          synchronised_twice=differing[2])
    from int4matmul_kernels_b200 import ops as _ops
    status_ok = True
    try:
        _ops.check_device_status()
    except Exception:
        status_ok = False
    parity = dict(checked=True, ok=(n_bad == 0 and gather_ok and status_ok and pass_ok), out_of_tolerance=n_bad, max_ulp=worst_ulp,
                  elements_per_rank=n_el, frac_bit_identical=exact, gathered_identical_on_all_ranks=gather_ok, ranks=world,
                  device_status_ok=status_ok, timed_pass_equals_synchronised_pass=pass_ok, timed_pass_differing_elements=pass_differing,
                  against="CPU oracle on sampled columns of layer 0's q|k|v product of every rank's shard; gathered buffers compared "
                          "across ranks; the timed pass's output bit-equal to a pass with a device synchronisation after every launch")

    peaks = measured_peaks()
    peak = peaks["hbm"] if kind == "hbm" else peaks["tf_sustained"]
    achieved = value / world                                    # per GPU: every rank moves / computes 1/world of the pass
    if rank == 0:
        print(json.dumps(dict(
            metric=metric, value=value, unit=unit, n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3),
            ms_per_step=ms_step, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="f16", data="synthetic",
            config=dict(workload=args.workload, layers=cfg.layers, hidden=cfg.hidden, mlp=cfg.mlp, m=m, bits=4, g=cfg.group_size,
                        sharding=(f"S columns of every matrix over {world} GPU(s); outputs gathered " +
                                  ("by NCCL all-gathers" if args.nccl_gather else "by the multiply kernels' own peer stores + a flag hand-shake per matrix")),
                        l2=f"{cfg.layers * wpl // 2 / 1e9:.1f} GB of weights per pass (>> L2)",
                        timed_as="one CUDA graph of the K steps" if graph is not None else "K direct launches"),
            roofline=dict(bound=kind, achieved=achieved, peak=peak, unit=unit, frac=achieved / peak, traffic=None,
                          peak_source=peaks["source"], kernel="umma_kernel (tcgen05)",
                          note="whole pass incl. normalisation kernels and all-gathers, per GPU; sustained peak for tensor"),
            parity=parity, cpu_baseline=None,
            e2e=dict(value=units / (ms_e2e / args.steps / 1e3), unit=unit, h2d_bytes_per_step=h_host.numel() * 2,
                     d2h_bytes_per_step=out_host.numel() * 2, ms_per_step=ms_e2e / args.steps),
            clocks=clocks.summary(), gpu_launches=int(k_launches))))
    if world > 1:
        dist.destroy_process_group()


def sample_columns(s, count, seed):
    """Output columns to check: tile edges of both tile widths, the shard's edges, and random columns."""
    import numpy as np
    rng = np.random.default_rng(seed)
    edges = [0, 1, 127, 128, 255, 256, s // 2 - 1, s // 2, s - 257, s - 129, s - 128, s - 1]
    cols = set(c for c in edges if 0 <= c < s)
    cols.update(int(c) for c in rng.integers(0, s, size=count))
    return np.array(sorted(cols))


def check_outputs(w, chain, x_cpu, out, cols, accumulate_from_zero):
    """One output buffer against the CPU oracle on the columns `cols` (reference semantics: fp16 weights as the
    reference rebuilds them, fp32 accumulation, one rounding).  `chain` = the weight copies multiplied into the
    buffer, in order: one for the overwriting matmul route; for the matvec route, which adds into the buffer,
    every launch since the buffer was zeroed (each adds to the rounded result of the one before).  Returns
    (elements checked, out of tolerance, worst ulp distance, fraction bit-identical).  Tolerance as in the tests:
    1 fp16 ulp, or 2^-13 of sum |x . W16|."""
    import numpy as np
    import torch
    from oracle import reference_oracle as oracle            # checker only, after the timed region
    ci = torch.as_tensor(cols, device=chain[0]["matrix"].device)
    sub = lambda t: t.index_select(1, ci).cpu().numpy() if t is not None else None
    want = np.zeros((1, w["m"], len(cols)), np.float16) if accumulate_from_zero else None
    bound = 0.0
    for layer in chain:
        want, b = oracle.expected_columns(w["bits"], sub(layer["matrix"]), sub(layer["mask"]), sub(layer["scales"]),
                                          sub(layer["zeros"]), w["g"], x_cpu, np.arange(len(cols)), want)
        bound = bound + b
        if not accumulate_from_zero:
            break
    got = out.index_select(out.dim() - 1, ci.to(out.device)).cpu().numpy().reshape(want.shape)
    ulp = oracle.fp16_ulp_distance(got, want)
    diff = np.abs(got.astype(np.float32) - want.astype(np.float32))
    ok = (ulp <= 1) | (diff <= 2.0 ** -13 * bound)
    return int(ok.size), int((~ok).sum()), int(ulp.max()), float((ulp == 0).mean())


def torch_fp16_leg(w, layer, x, torch, steps):
    """torch's own fp16 matmul on the dequantised weights, as the reference script times it (kernel_test.py:248-249,
    296): a library comparator beside the product, never part of its path.  Dense formats only."""
    if w["sparse"]:
        return None
    from int4matmul_kernels_b200 import packing, quantize
    try:
        q = packing.unpack_dense(w["bits"], layer["matrix"])
        w16 = quantize.dequantize(q, layer["scales"], layer["zeros"], w["g"])
        del q
        x2 = x.view(w["m"], w["n"])
        for _ in range(3):
            y = x2 @ w16
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        iters = max(steps, 10)
        e0.record()
        for _ in range(iters):
            y = x2 @ w16
        e1.record()
        torch.cuda.synchronize()
        sec = e0.elapsed_time(e1) / iters / 1e3
        del w16, y
        kind = metric_of(w)[2]
        return dict(us_per_call=sec * 1e6, value=units_per_step(w, kind, layer["matrix"].shape[1]) / sec, unit=metric_of(w)[1],
                    what=f"torch fp16 x @ W16 (cuBLAS) on the already dequantised {w['n']}x{layer['matrix'].shape[1]} matrix, {iters} back-to-back calls; "
                         "for few rows it reads 2 bytes per weight where the packed formats read bits/8")
    except Exception as e:                                # a comparator: its failure is reported, not fatal
        return dict(unavailable=f"{type(e).__name__}: {e}")


def run_workload(args, name, w, ctx):
    """Times one workload on this rank's column shard; returns the line's dict on rank 0 (None elsewhere)."""
    torch, dist, dev = ctx["torch"], ctx["dist"], ctx["dev"]
    world, rank, local_rank, ext = ctx["world"], ctx["rank"], ctx["local_rank"], ctx["ext"]
    from int4matmul_kernels_b200 import capi, ops, packing
    lib = capi.load()

    metric, unit, kind = metric_of(w)
    s_local = w["s"] // world
    if w["s"] % world or s_local % 64:
        raise SystemExit("S / gpus must be a multiple of 64")

    # ---- synthetic data: full matrix drawn from the seed, this rank keeps its column shard ----
    bytes_per_step = algorithmic_bytes(w, s_local)
    copies = max(1, -(-2 * L2_BYTES // bytes_per_step))     # rotate so that consecutive steps miss L2
    copies = min(copies, 24)
    layers = []
    for c in range(copies):
        full = packing.synthetic_weights(w["bits"], w["n"], w["s"], w["g"], sparse=w["sparse"], seed=c, device=dev)
        layers.append({k: (packing.shard_columns(v, rank, world) if v is not None else None) for k, v in full.items()})
        del full
    gen = torch.Generator().manual_seed(1234)
    x_host = torch.randn((1, w["m"], w["n"]), generator=gen).to(torch.float16).pin_memory()
    x = x_host.to(dev)
    matvec = w["m"] == 1                                     # the matvec route adds into outs
    # matvec: one output buffer per step, all zeroed by ONE fill at the start of every run of K steps, so that what a
    # buffer holds afterwards is a known chain of accumulations without a fill kernel between the timed launches
    n_out = min(args.steps, 64) if matvec else min(copies, 4)
    out_all = torch.zeros((n_out, 1, w["m"], s_local), dtype=torch.float16, device=dev)
    outs = [out_all[j] for j in range(n_out)]

    def step(i):
        L = layers[i % copies]
        if matvec and i == 0:
            out_all.zero_()
        ops.quant_matmul(w["bits"], outs[i % n_out], L["matrix"], x, L["scales"], L["zeros"], w["g"], L["mask"], path=args.path)

    use_umma = args.path != 1                       # automatic = the tcgen05 kernel for every row count
    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    shape = lib.i4mm_last_launch_shape()

    graph = None
    if not args.no_graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step(0)                                   # allocates this stream's scratch outside the capture
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            n0 = lib.i4mm_launch_count()
            with torch.cuda.graph(graph, stream=side):
                for i in range(args.steps):
                    step(i)
            k_launches = lib.i4mm_launch_count() - n0      # kernels of ours in the K captured steps
            graph.replay()
            torch.cuda.synchronize()
        except Exception as e:                            # capture is an optimisation of the harness only
            print(f"[bench] CUDA graph capture unavailable ({type(e).__name__}: {e}); timing direct launches", file=sys.stderr)
            graph = None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if graph is None:
        n0 = lib.i4mm_launch_count()
        for i in range(args.steps):
            step(i)
        k_launches = lib.i4mm_launch_count() - n0

    def run_steps():
        if graph is not None:
            graph.replay()
        else:
            for i in range(args.steps):
                step(i)

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local_rank) as clocks:
        # keep the GPU under the same load for ~0.3 s around the timed K steps so that nvidia-smi sees the clocks
        # the timed region runs at (the timed region alone lasts only milliseconds)
        t_end = time.perf_counter() + 0.15
        while time.perf_counter() < t_end:
            run_steps()
        barrier()
        e0.record()
        run_steps()
        e1.record()
        barrier()
        t_end = time.perf_counter() + 0.15
        while time.perf_counter() < t_end:
            run_steps()
        barrier()
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = units_per_step(w, kind) / (ms_step / 1e3)          # whole job: all shards together per step

    # ---- parity of what the timed steps left in the output buffers (outside the timed region) ----
    x_cpu = x_host.numpy()
    writers = {}                                             # output buffer -> the weight copies written into it, in order
    for i in range(args.steps):
        writers.setdefault(i % n_out, []).append(i % copies)
    checked = bad = 0
    worst_ulp, exact = 0, 1.0
    n_cols = 0
    for j, chain in sorted(writers.items())[:8]:
        cols = sample_columns(s_local, 64, 17 * j + rank)
        n, b, u, fe = check_outputs(w, [layers[li] for li in (chain if matvec else chain[-1:])], x_cpu, outs[j], cols, matvec)
        checked, bad, worst_ulp, exact, n_cols = checked + n, bad + b, max(worst_ulp, u), min(exact, fe), n_cols + len(cols)
    status_ok = lib.i4mm_device_status(ops.workspace(dev, torch.cuda.current_stream()).data_ptr(), torch.cuda.current_stream().cuda_stream) == capi.OK

    # ---- roofline of the dominant kernel (this rank's launch) ----
    peaks = measured_peaks()
    us_launch = ms_step * 1e3
    gbs = algorithmic_bytes(w, s_local) / 1e9 / (ms_step / 1e3)
    tfs = algorithmic_flops(w, s_local) / 1e12 / (ms_step / 1e3)
    if kind == "hbm":
        achieved, peak, runit = gbs, peaks["hbm"], "GB/s"
    else:
        achieved, peak, runit = tfs, peaks["tf_burst"], "TFLOP/s"
    roofline = dict(bound=kind, achieved=achieved, peak=peak, unit=runit, frac=achieved / peak,
                    traffic=ncu_traffic(name, world), peak_source=peaks["source"],
                    us_per_launch=us_launch, kernel="umma_kernel (tcgen05)" if use_umma else "stream_kernel (mma.sync)",
                    launch_shape=shape, frac_of_nominal=achieved / (8000.0 if kind == "hbm" else 2250.0),
                    frac_of_sustained_bf16=(tfs / peaks["tf_sustained"]) if kind == "tensor" else None)
    if 16 <= w["m"] <= 256:
        # near the ridge (arithmetic intensity ~ the machine balance): report against both roofs
        roofline["both_roofs"] = dict(hbm=dict(achieved=gbs, peak=peaks["hbm"], frac=gbs / peaks["hbm"], unit="GB/s"),
                                      tensor=dict(achieved=tfs, peak=peaks["tf_burst"], frac=tfs / peaks["tf_burst"], unit="TFLOP/s"))

    # ---- end to end through the drop-in module, host buffers: H2D(i+1) | kernel(i) | D2H(i-1) on three streams ----
    e2e = None
    if not args.no_e2e:
        s_in, s_k, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        x_dev = [torch.empty_like(x) for _ in range(2)]
        # several GPUs: every rank needs all of x, but only 1 / N of it crosses this rank's PCIe link; the ranks then
        # exchange their pieces over NVLink (one NCCL all-gather per step, inside the timed region)
        # (only worth a collective's latency when x is large: a matvec's 32 KB go straight to every GPU)
        split_x = world > 1 and x_host.numel() % (8 * world) == 0 and x_host.numel() * 2 >= (1 << 20)
        if split_x:
            chunk = x_host.numel() // world
            x_piece_host = x_host.view(-1)[rank * chunk:(rank + 1) * chunk]
            x_piece_dev = [torch.empty(chunk, dtype=torch.float16, device=dev) for _ in range(2)]
        o_dev = [torch.zeros((1, w["m"], s_local), dtype=torch.float16, device=dev) for _ in range(2)]
        out_host = [torch.empty((1, w["m"], s_local), dtype=torch.float16).pin_memory() for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_k = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]

        def e2e_step(i):
            b = i % 2
            L = layers[i % copies]
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_k[b])                   # the kernel that last read this input buffer
                if split_x:
                    x_piece_dev[b].copy_(x_piece_host, non_blocking=True)
                    dist.all_gather_into_tensor(x_dev[b].view(-1), x_piece_dev[b])
                else:
                    x_dev[b].copy_(x_host, non_blocking=True)
                ev_in[b].record(s_in)
            with torch.cuda.stream(s_k):
                s_k.wait_event(ev_in[b])
                s_k.wait_event(ev_out[b])                  # the copy that last read this output buffer
                if matvec:
                    o_dev[b].zero_()
                ext.quant_matmul(w["bits"], o_dev[b], L["matrix"], x_dev[b], L["scales"], L["zeros"], w["g"], L["mask"])
                ev_k[b].record(s_k)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_k[b])
                out_host[b].copy_(o_dev[b], non_blocking=True)
                ev_out[b].record(s_out)

        cur = torch.cuda.current_stream()

        def e2e_run(n):
            for st in (s_in, s_k, s_out):
                st.wait_stream(cur)
            for i in range(n):
                e2e_step(i)
            for st in (s_in, s_k, s_out):
                cur.wait_stream(st)

        e2e_run(3)
        barrier()
        e0.record()
        e2e_run(args.steps)
        e1.record()
        barrier()
        ms_e2e = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms_e2e], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_e2e = float(t.item())
        # the host copy of the last step's result is checked as well
        last = args.steps - 1
        cols = sample_columns(s_local, 48, 99 + rank)
        n, b, u, fe = check_outputs(w, [layers[last % copies]], x_cpu, out_host[last % 2].to(dev), cols, matvec)
        checked, bad, worst_ulp, exact, n_cols = checked + n, bad + b, max(worst_ulp, u), min(exact, fe), n_cols + len(cols)
        e2e = dict(value=units_per_step(w, kind) / (ms_e2e / args.steps / 1e3), unit=unit,
                   h2d_bytes_per_step=(x_host.numel() // world if split_x else x_host.numel()) * 2,
                   d2h_bytes_per_step=out_host[0].numel() * 2, bytes_are="per rank (every rank copies its piece of x in and its columns of the result out)",
                   ms_per_step=ms_e2e / args.steps,
                   how="int4matmul.quant_matmul on pinned host buffers; input copy, kernel and result copy of consecutive steps "
                       "overlap on three streams (double-buffered)" +
                       ("; every rank copies 1 / N of x from the host and the ranks all-gather it over NVLink (NCCL)" if split_x else ""))

    if world > 1:
        t = torch.tensor([float(checked), float(bad), float(n_cols)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        t2 = torch.tensor([float(worst_ulp), -exact, 0.0 if status_ok else 1.0], device=dev)
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        checked, bad, n_cols = int(t[0].item()), int(t[1].item()), int(t[2].item())
        worst_ulp, exact, status_ok = int(t2[0].item()), -float(t2[1].item()), t2[2].item() == 0.0
    parity = dict(checked=True, ok=(bad == 0 and status_ok), elements=checked, out_of_tolerance=bad, max_ulp=worst_ulp,
                  frac_bit_identical=exact, cols=n_cols, ranks=world, device_status_ok=status_ok,
                  against="CPU oracle (reference semantics) on sampled output columns of the buffers the timed steps wrote",
                  tolerance="1 fp16 ulp or 2^-13 * sum|x.W16|")

    # ---- CPU baseline on a bounded sample; the reference's CUDA kernels and torch fp16 beside it (rank 0, one GPU) ----
    cpu = ref_gpu = torch16 = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        p = cpu_problem(w)
        rows = min(w["m"], 256)
        cpu_reference_seconds(w, p, rows, cores)
        reps = 3
        sec = min(cpu_reference_seconds(w, p, rows, cores) for _ in range(reps))
        del p
        cpu = dict(value=units_per_step(w, kind) / sec, unit=unit, cores=cores, kind="port",
                   sample=(f"full {w['n']}x{w['s']} dequantise timed whole, matmul timed on {rows} of {w['m']} rows and "
                           f"scaled to all rows, best of {reps}"))
        ref_gpu = reference_cuda_seconds(w, layers[0], x, torch)
        torch16 = torch_fp16_leg(w, layers[0], x, torch, args.steps)

    if rank != 0:
        return None
    return dict(metric=metric, value=value, unit=unit, n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3),
                ms_per_step=ms_step, higher_is_better=True, scaling="strong", vs_baseline=None,
                dtype="f16", data="synthetic", config=config_of(name, w),
                protocol=dict(sharding=f"S columns over {world} GPU(s)", weight_copies=copies,
                              timed_as="one CUDA graph of the K steps" if graph is not None else "K direct launches",
                              outputs=(f"{n_out} output buffers zeroed by one fill per K steps (the matvec route adds into them)"
                                       if matvec else f"{n_out} output buffers, overwritten")),
                roofline=roofline, parity=parity, cpu_baseline=cpu, reference_cuda=ref_gpu, torch_fp16=torch16, e2e=e2e,
                clocks=clocks.summary(), gpu_launches=int(k_launches))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + sorted(STACK_WORKLOADS))
    ap.add_argument("--layers", type=int, default=40, help="layers of the stack workloads")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--path", type=int, default=0, help="0 auto, 1 streaming kernel, 2 tcgen05 kernel, 3 tcgen05 with single CTAs")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline and the comparator legs")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-matvec", action="store_true", help="default workload only: do not time the matvec half of the metric as well")
    ap.add_argument("--no-graph", action="store_true", help="launch the timed steps directly instead of as one CUDA graph")
    ap.add_argument("--nccl-gather", action="store_true", help="stack workloads on several GPUs: gather outputs with NCCL all-gathers (the checker path) instead of peer stores")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
    if args.workload in STACK_WORKLOADS:
        run_stack(args)
        return
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, w, args.workload)
        return

    import torch
    import torch.distributed as dist
    from int4matmul_kernels_b200 import capi, ops
    import int4matmul_kernels_b200 as pkg

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    capi.load()                                   # fails loudly if the CUDA library is missing
    # the benchmark's weights are never rewritten: launches may overlap the tail of the kernel before them
    ops.set_static_weights(True)
    ctx = dict(torch=torch, dist=dist, dev=dev, world=world, rank=rank, local_rank=local_rank, ext=pkg.load_extension())
    ctx["ext"].set_static_weights(True)

    mv = None
    if args.workload == DEFAULT_WORKLOAD and not args.no_matvec:
        # the other half of the metric, same protocol, under one extra key of the same line; it runs first because it
        # is the clock-sensitive one and the matmul leaves the GPU sitting on its power cap
        mv = run_workload(args, MATVEC_WORKLOAD, WORKLOADS[MATVEC_WORKLOAD], ctx)
        torch.cuda.empty_cache()
    line = run_workload(args, args.workload, w, ctx)
    if mv is not None and line is not None:
        line["matvec"] = mv
        line["gpu_launches_matvec"] = mv["gpu_launches"]
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
