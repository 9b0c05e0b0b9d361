#!/usr/bin/env python
"""Benchmark of the quantized decode hot path on B200.

Metric: decode tokens/s of a random-init Llama-7B-shape model (32 layers, d 4096, 32 heads of 128,
SwiGLU 11008, vocab 32000), every linear int4 (group 128, scale + zero point, the reference's
packing), paged KV cache (block 16), batch 16, 2048 positions of context per sequence, greedy next
token.  One step = one pass of the whole decode step over the batch.  At N > 1 the same step is
tensor-parallel over N ranks (strong scaling: the batch is fixed).

  python bench.py --gpus 1 --steps 20 --warmup 3
  python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
  python bench.py --impl reference ...      the CPU restatement of accel's CPU kernels, host cores

Prints ONE JSON line on rank 0."""
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
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode tok/s (7B-shape int4, paged KV)"
WORKLOAD = ("7B-shape decode step: 32 layers, d_model 4096, 32 heads x 128, SwiGLU 11008, vocab "
            "32000, int4 group-128 linears, paged KV block 16, batch 16, context 2048, greedy")


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json, STREAM-style copy)"
    return 6650.0, "fallback (6.65 TB/s, an earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for t, r in self.rows if t0 <= t <= t1 + 0.2 and len(r) >= 9] or \
               [r for _, r in self.rows if len(r) >= 9]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = [float(r[1]) for r in rows]
        reasons = set()
        for r in rows:
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6),
                              ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": float(rows[0][2]),
                "power_w_max": max(float(r[3]) for r in rows), "samples": len(rows),
                "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------------------------
# reference arm: the oracle's layer sample on the host cores
# ----------------------------------------------------------------------------------------------
def cpu_sample(steps: int, warmup: int, layers: int = 32, budget_s: float = 20.0, sample=None):
    """The CPU baseline beside the GPU number: times ONE of the step's layers per sample (plus the
    lm_head and argmax once) on every host core and scales to the `layers` a token needs.
    Returns (tok/s, seconds per layer, seconds for the head, threads used)."""
    import oracle
    from oracle.step import LayerSample
    cores = oracle.set_threads()             # not the launcher's OMP_NUM_THREADS
    s = sample if sample is not None else LayerSample()
    x = None
    for _ in range(max(warmup, 0)):
        _, x = s.time_layer()
    times, t_begin = [], time.perf_counter()
    for _ in range(max(steps, 1)):
        t, x = s.time_layer()
        times.append(t)
        if time.perf_counter() - t_begin > budget_s:
            break
    t_head = s.time_head(x)
    t_layer = statistics.median(times)
    step_s = layers * t_layer + t_head
    return s.B / step_s, t_layer, t_head, cores


def run_reference(args):
    """The reference arm: accel's CPU kernels (their C restatement; the Go module cannot be built
    without a Go toolchain) on every host core, the same decode step as the GPU arm.  A step runs
    the layer `layers` times and the lm_head + argmax once, as a token does; when that would not
    finish in a few minutes the step runs fewer layer passes and is scaled, and says so."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    from oracle.step import LayerSample
    cores = oracle.set_threads()             # torch.distributed.run exports OMP_NUM_THREADS=1
    s = LayerSample(batch=args.batch, context=args.context)
    layers, steps, warmup = args.layers, args.steps, args.warmup
    t_probe, x = s.time_layer()              # untimed probe: sizes the sample
    budget_s = float(os.environ.get("AB_REFERENCE_BUDGET_S", "240"))
    passes = max(1, min(layers, int(budget_s / max(t_probe * (steps + warmup), 1e-9))))

    def one_step():
        nonlocal x
        t0 = time.perf_counter()
        for _ in range(passes):
            x = s.layer()
        t_layers = time.perf_counter() - t0
        t0 = time.perf_counter()
        s.head_and_argmax(x)
        return t_layers, time.perf_counter() - t0

    for _ in range(warmup):
        one_step()
    w0 = time.perf_counter()
    runs = [one_step() for _ in range(steps)]
    wall = time.perf_counter() - w0
    t_layers = sum(r[0] for r in runs) / steps
    t_head = sum(r[1] for r in runs) / steps
    step_s = t_layers * layers / passes + t_head
    toks = s.B / step_s
    sample = (f"every step runs the layer {passes} time(s) of the {layers} a token needs"
              + ("" if passes == layers else f" (scaled x{layers}/{passes} to the full step)")
              + f" and the lm_head + argmax once, batch {s.B}, context {s.context}; wall time of the "
              f"{steps} timed steps {wall:.1f} s; C restatement of accel's CPU kernels, OpenMP over "
              "workgroups; the Go backend itself cannot be built here (no Go toolchain)")
    line = {
        "impl": "reference", "metric": METRIC, "value": toks, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": 1e3 * step_s,
        "ms_per_step_as_run": 1e3 * wall / steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch": s.B, "context": s.context, "layers": layers,
                   "kv_cache": "f32", "parallelism": "host cores", "layer_passes_per_step": passes},
        "cpu_baseline": {"value": toks, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": toks, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# the B200 arm
# ----------------------------------------------------------------------------------------------
def time_kernel(fn, reps, stream):
    import torch
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        fn()
    e1.record(stream)
    e1.synchronize()
    return e0.elapsed_time(e1) / reps


def run_linear(args):
    """One int4 product M x K x N on its own (the metric's second figure and the sweep over the
    batch size): a CUDA graph of the product over 8 different weight matrices (larger than L2
    together), timed with CUDA events over 10 replays.  Prints one JSON line."""
    import torch

    from accel_b200 import quant
    from accel_b200 import runtime as rt
    M, K, N = (int(v) for v in args.linear.split(","))
    dev = "cuda:0"
    torch.cuda.set_device(0)
    torch.manual_seed(7)
    nm = max(2, min(8, (1 << 30) // (K * N // 2)))
    if args.int8:
        return run_linear_int8(args, M, K, N, nm)
    mats = [quant.int4_quantize_device(torch.randn(K, N, device=dev) * 0.02) for _ in range(nm)]
    a = torch.randn(M, K, device=dev)
    out = torch.empty(M, N, device=dev)
    u = rt.gemm_dims(M if M > 1 else 0, N, K)
    name = "QuantMatMulInt4" if M > 1 else "QuantMatVecInt4"
    x = a if M > 1 else a[0]
    if not args.planes:
        # the load-time prepack (a permutation of the three planes) and the kernels that read it
        mats = [(quant.int4_prepack(c, sc, z, K, N),) for c, sc, z in mats]
        name += "Packed"

    def body():
        for m in mats:
            rt.launch(name, [x, *m, out], u)

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        body()
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            body()
    torch.cuda.current_stream().wait_stream(s)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        g.replay()
    e1.record()
    e1.synchronize()
    us = e0.elapsed_time(e1) / (10 * nm) * 1e3
    nbytes = K * N // 2 + 2 * (K * N // 128) * 2 + M * K * 4 + M * N * 4
    peak, src = measured_peaks()
    print(json.dumps({"metric": "int4 linear", "shape": {"M": M, "K": K, "N": N}, "us": us,
                      "bytes": nbytes, "gbs": nbytes / us / 1e3, "frac_of_hbm_peak": nbytes / us / 1e3 / peak,
                      "tflops": 2.0 * M * K * N / us / 1e6, "peak_source": src, "matrices_rotated": nm,
                      "kernel": rt.last_selection()}))


def run_linear_int8(args, M, K, N, nm):
    """The int8 path's product (quant.Int8Quantize weights, f32 activations) timed like run_linear."""
    import numpy as np
    import torch

    from accel_b200 import runtime as rt
    dev = "cuda:0"
    rng = np.random.default_rng(7)
    mats = []
    for _ in range(nm):
        # quants and scales of the right shape and range; the time does not depend on the values
        q = torch.from_numpy(rng.integers(-127, 128, (K, N), dtype=np.int8)).to(dev)
        sc = (torch.rand(K * N // 32, device=dev) * 0.01 + 0.001).half()
        mats.append((q, sc))
    a = torch.randn(M, K, device=dev)
    out = torch.empty(M, N, device=dev)
    name = "QuantMatMulTiledF32" if M > 1 else "QuantMatVecF32"
    u = rt.gemm_dims(M, N, K)

    def body():
        for m in mats:
            rt.launch(name, [a, *m, out], u)

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        body()
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            body()
    torch.cuda.current_stream().wait_stream(s)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        g.replay()
    e1.record()
    e1.synchronize()
    us = e0.elapsed_time(e1) / (10 * nm) * 1e3
    nbytes = K * N + (K * N // 32) * 2 + M * K * 4 + M * N * 4
    peak, src = measured_peaks()
    print(json.dumps({"metric": "int8 linear", "shape": {"M": M, "K": K, "N": N}, "us": us, "bytes": nbytes,
                      "gbs": nbytes / us / 1e3, "frac_of_hbm_peak": nbytes / us / 1e3 / peak, "peak_source": src,
                      "matrices_rotated": nm, "kernel": rt.last_selection()}))


def run_attention(args):
    """Config 3: paged-KV decode attention on its own: 32 sequences, one query token each, 32 query
    heads over 8 KV heads (GQA), head dim 128, block 16, context lengths uniform in [512, 4096],
    block table = disjoint runs of a seeded permutation of a shared pool.  Several caches (larger
    than L2 together) are rotated inside one CUDA graph; f32 (the reference's batched kernel) and
    f16 (this library's extension) caches.  Prints one JSON line."""
    import numpy as np
    import torch

    from accel_b200 import runtime as rt
    dev = "cuda:0"
    torch.cuda.set_device(0)
    B, qH, kvH, D, block, max_pages = 32, 32, 8, 128, 16, 256
    rng = np.random.default_rng(3)
    lengths = rng.integers(512, 4097, B).astype(np.int64)
    need = (lengths + block - 1) // block
    pool = int(need.sum()) + 8
    perm = rng.permutation(pool).astype(np.int32)
    pages = np.zeros((B, max_pages), np.int32)
    at = 0
    for i, n in enumerate(need):
        pages[i, :n] = perm[at:at + n]
        at += n
    peak, src = measured_peaks()
    scale = float(np.float32(1.0) / np.float32(np.sqrt(D)))
    u = rt.batched_dims(B, qH, kvH, D, block, max_pages, scale)
    q = torch.randn(B, qH, D, device=dev)
    out = torch.empty(B, qH, D, device=dev)
    pg = torch.from_numpy(pages).to(dev)
    ln = torch.from_numpy(lengths.astype(np.int32)).to(dev)
    result = {}
    for dt, name in ((torch.float32, "AttentionDecodeBatched"), (torch.float16, "AttentionDecodeBatchedF16")):
        caches = [(torch.randn(pool * block, kvH, D, device=dev).to(dt), torch.randn(pool * block, kvH, D, device=dev).to(dt))
                  for _ in range(4)]

        def body():
            for k, v in caches:
                rt.launch(name, [q, k, v, pg, ln, out], u)

        st = torch.cuda.Stream()
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st):
            body()
            st.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                body()
        torch.cuda.current_stream().wait_stream(st)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            g.replay()
        e1.record()
        e1.synchronize()
        us = e0.elapsed_time(e1) / (10 * len(caches)) * 1e3
        esz = 2 if dt == torch.float16 else 4
        nbytes = int(2 * kvH * D * esz * lengths.sum() + 2 * B * qH * D * 4 + pages.size * 4 + B * 4)
        result["f16" if esz == 2 else "f32"] = {"us": us, "bytes": nbytes, "gbs": nbytes / us / 1e3,
                                                "frac_of_hbm_peak": nbytes / us / 1e3 / peak}
        del caches
    print(json.dumps({"metric": "paged decode attention", "config": {
        "workload": "32 sequences x 1 query, 32 q heads / 8 KV heads, head dim 128, block 16, "
                    "context lengths uniform in [512, 4096] (seed 3)", "positions": int(lengths.sum())},
        "peak_source": src, **result}))


def run_moe(args):
    """Config 5: the expert half of a MoE layer, 8 experts, 4096 tokens x top-2 = 8192 routed rows,
    d 4096, expert FFN 14336 (gate, up, SwiGLU, down), int4 experts; per-expert counts from a
    seeded multinomial (top-2 distinctness per token is not modelled by the config).  At N > 1 the
    experts are split over the ranks and the rows travel by all-to-all; the 8192 rows are split
    evenly over the ranks (strong scaling).  Prints one JSON line."""
    import torch
    import torch.distributed as dist

    from accel_b200 import moe
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    E, d, ffn, rows_total = 8, 4096, 14336, 8192
    layer = moe.ExpertParallelFFN(E, d, ffn, dev, seed=5, init_on_device=True)
    g = torch.Generator().manual_seed(5)
    expert_all = torch.multinomial(torch.ones(E), rows_total, replacement=True, generator=g).to(torch.int32)
    lo, hi = rank * rows_total // world, (rank + 1) * rows_total // world
    x = torch.randn(hi - lo, d, device=dev)
    expert = expert_all[lo:hi].to(dev)
    for _ in range(max(args.warmup, 1)):
        layer.forward(x, expert)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out = layer.forward(x, expert)
    e1.record()
    e1.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    flops = 3 * 2.0 * rows_total * d * ffn
    if rank == 0:
        print(json.dumps({"metric": "grouped int4 MoE FFN", "value": flops / ms / 1e9, "unit": "TFLOP/s",
                          "ms_per_layer": ms, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                          "rows_per_s": rows_total / ms * 1e3, "scaling": "strong",
                          "config": {"workload": "8 experts, 8192 routed rows, d 4096, ffn 14336, int4 group 128",
                                     "parallelism": f"ep{world}", "counts": "seeded multinomial over 8 experts"},
                          "checksum": float(out.double().abs().sum().item())}))
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(0)


def run_allreduce(args):
    """Latency of one 256 KiB all-reduce (16 rows x 4096 floats, a row-parallel product of the decode
    step) inside a CUDA graph: this library's one-shot kernel over NVLink peer memory, copying and in
    place with the residual add and RMSNorm folded in, beside the process group's NCCL all-reduce and
    NCCL followed by the AddRMSNorm kernel.  Run under torchrun, one rank per GPU."""
    import torch
    import torch.distributed as dist

    from accel_b200 import runtime as rt
    from accel_b200.peer import PeerAllReduce
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    dist.init_process_group("nccl", device_id=dev)
    ar = PeerAllReduce(16 * 4096, dev, regions=(16 * 4096, 16 * 4096))

    def per_call_us(fn):
        y = torch.randn(16, 4096, device=dev)
        st = torch.cuda.Stream()
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st):
            for _ in range(64):
                fn(y)
            st.synchronize()
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2, stream=st):
                for _ in range(64):
                    fn(y)
            g2.replay()
            st.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            for _ in range(5):
                g2.replay()
            e1.record(st)
            e1.synchronize()
        return e0.elapsed_time(e1) / (5 * 64) * 1e3

    gain = torch.ones(4096, device=dev)
    s_out, n_out = torch.empty(16, 4096, device=dev), torch.empty(16, 4096, device=dev)
    flip = [0]

    def fused_inplace(y):
        flip[0] ^= 1
        ar.all_reduce_region_add_rms_norm(flip[0], y, gain, s_out, n_out, 1e-5)

    def nccl_then_norm(y):
        dist.all_reduce(y)
        rt.launch("AddRMSNorm", [y, y, gain, s_out, n_out], rt.row_dims(16, 4096, 1e-5))

    line = {"metric": "all_reduce_latency_256KiB", "unit": "us", "n_gpus": world, "higher_is_better": False,
            "peer_copying": per_call_us(lambda y: ar.all_reduce_(y)),
            "nccl": per_call_us(lambda y: dist.all_reduce(y)),
            "peer_inplace_add_rmsnorm": per_call_us(fused_inplace),
            "nccl_then_add_rmsnorm": per_call_us(nccl_then_norm)}
    ar.check()
    if rank == 0:
        print(json.dumps(line), flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0)


def run_b200(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    from accel_b200 import decode as dec
    from accel_b200 import runtime as rt

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: accel_b200 has no CPU path "
                         "(use --impl reference for the CPU baseline)")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch N ranks with torchrun")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        import datetime
        import faulthandler
        # a rank that never arrives must end the run with an error and a stack, not hang it
        faulthandler.dump_traceback_later(int(os.environ.get("AB_BENCH_WATCHDOG_S", "900")), exit=True)
        # no NVLink multicast objects: a rank that dies while bound to one faults its peers' GPUs
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=600))
        group = dist.group.WORLD

    cache_dtype = torch.float16 if args.kv == "f16" else torch.float32
    cfg = dec.ModelConfig(layers=args.layers, cache_dtype=cache_dtype)
    shard = dec.Shard.plan(cfg, world, rank)
    if args.shard_of > 1:
        # one rank's share of an N-way tensor-parallel step on ONE GPU, the sums over ranks left out:
        # the launch list and the per-kernel times of a rank, which a profiler cannot take from a
        # multi-rank run.  Not a benchmark figure.
        if world != 1:
            raise SystemExit("--shard-of runs in one process")
        shard = dec.Shard.plan(cfg, args.shard_of, 0)
    t_setup = time.perf_counter()
    model = dec.DecodeModel(cfg, shard, dev, seed=1234)
    B, ctx = args.batch, args.context
    total_steps = 3 * (args.steps + args.warmup) + 8
    collective, why = (args.collective if world > 1 else "none"), ""
    engine = None
    if collective == "peer":
        # mapping the peers' buffers is a collective of its own; if any rank cannot, all use NCCL
        try:
            engine = dec.DecodeEngine(model, B, max_context=ctx + total_steps + 16, group=group,
                                      collective="peer")
            ok = 1
        except Exception as e:                     # noqa: BLE001 - reported in the JSON line
            ok, why = 0, f"{type(e).__name__}: {e}"[:160]
        flag = torch.tensor([ok], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) == 0:
            collective, engine = f"nccl (peer memory unavailable{': ' + why if why else ' on another rank'})", None
    if engine is None:
        engine = dec.DecodeEngine(model, B, max_context=ctx + total_steps + 16, group=group,
                                  collective="skip" if args.shard_of > 1 else "nccl")
        if args.shard_of > 1:
            collective = f"skipped: rank 0's kernels of a tp{args.shard_of} step, results not the model's"
    engine.overlap = not args.no_overlap
    log = (lambda m: print(f"[rank {rank}] {m}", file=sys.stderr, flush=True)) if args.verbose else (lambda m: None)
    log("engine built")
    rng = np.random.default_rng(99)
    prompts = rng.integers(0, cfg.vocab, (B, ctx))       # seeded random token ids, as config 4 says
    first = rng.integers(0, cfg.vocab, B)

    def fill(eng):
        """The 2048-token context: a real prefill through the batch kernels and the paged causal
        prefill attention (--kv-fill prefill), or seeded N(0,1) K/V rows (--kv-fill random)."""
        info = {"kv_fill": "seeded N(0,1) rows stand in for the prefill (--kv-fill random)"}
        if args.kv_fill == "prefill":
            try:
                secs = eng.prefill(prompts, chunk=args.prefill_chunk)
                info = {"kv_fill": "prefill of the seeded random prompts through the batch int4 kernels and "
                                   "AttentionPrefillPaged, %d positions per sequence at a time" % args.prefill_chunk,
                        "prefill_s": round(secs, 3), "prefill_tok_s": round(B * ctx / secs, 1)}
            except Exception as e:                 # noqa: BLE001 - said in the JSON line; the run goes on
                eng.lengths_host[:] = 0
                eng.fill_context(ctx, seed=7)
                info = {"kv_fill": f"seeded N(0,1) rows; the prefill failed: {type(e).__name__}: {e}"[:300]}
        else:
            eng.fill_context(ctx, seed=7)
        for s_ in range(B):
            eng.reserve(s_, ctx + total_steps + 8)
        eng.upload_pages()
        return info

    fill_info = fill(engine)
    engine.set_inputs(first)
    log("context filled")
    if args.no_graph:
        engine.prepare()
        engine.record_step()
    else:
        engine.capture(warmup=1)
    torch.cuda.synchronize()
    log("step captured")
    t_setup = time.perf_counter() - t_setup

    # ---- parity of the sharded step, outside every timed region: the first step's logits and
    # greedy ids on N ranks against the same step of the unsharded model, built once on rank 0
    # from the same seeds (the ranks' shards are cut from bit-identical matrices)
    tp_parity = None
    if world > 1 and not args.no_tp_parity:
        engine.set_inputs(first)
        engine.run_step()
        torch.cuda.synchronize()
        tp_logits = engine.full_logits().clone()
        tp_ids = engine.next_tokens.clone()
        if rank == 0:
            m1 = dec.DecodeModel(cfg, dec.Shard.plan(cfg, 1, 0), dev, seed=1234)
            e1 = dec.DecodeEngine(m1, B, max_context=ctx + total_steps + 16)
            fill(e1)
            e1.set_inputs(first)
            e1.prepare()
            e1.record_step()
            torch.cuda.synchronize()
            ref = e1.full_logits()
            top2 = torch.topk(ref, 2, dim=1).values
            clear = (top2[:, 0] - top2[:, 1]) > 2e-3 * ref.abs().max()
            tp_parity = {
                "tp_vs_tp1_rel_err": float((tp_logits - ref).abs().max() / ref.abs().max()),
                "rows_with_clear_argmax": int(clear.sum()), "rows": B,
                "ids_equal_on_clear_rows": bool(torch.equal(tp_ids[clear], e1.next_tokens[clear])),
                "what": "first decode step, logits [batch, vocab] and greedy ids, N ranks against "
                        "the unsharded model on rank 0 (same seeds, same cache contents)"}
            del e1, m1, ref
            torch.cuda.empty_cache()
        # the other ranks wait here for rank 0: their next peer all-reduce would give up after its
        # bounded wait if rank 0 were still building the unsharded model
        torch.cuda.synchronize()
        dist.barrier()
        log("tp parity checked")

    stream = torch.cuda.current_stream(dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- value: K steps, inputs resident, the step feeding itself on the device
    engine.set_inputs(first)
    lengths0 = engine.lengths_host.copy()
    for _ in range(args.warmup):
        engine.run_step()
        engine.advance_on_device()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()              # after the sampler's start-up sleep, so every rank enters the region together
    kv_bytes_first = engine.kv_bytes_read_per_step()
    launches0 = rt.launch_count()
    t0 = time.perf_counter()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        engine.run_step()
        engine.advance_on_device()
    e1.record(stream)
    e1.synchronize()
    barrier()
    t1 = time.perf_counter()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    ms_per_step = ms_total / args.steps
    value = B * args.steps / (ms_total / 1e3)
    # kernels per step: the captured step's launches (counted when it was recorded) + the advance
    gpu_launches = args.steps * (engine.kernel_launches_per_step + 1)
    del launches0

    log(f"value timed: {ms_per_step:.3f} ms/step")
    # ---- e2e: the caller's loop; host token ids in, host token ids out, every step
    tok = engine.next_tokens.cpu().numpy()
    for _ in range(min(args.warmup, 3)):
        tok = engine.step(tok)
    barrier()
    w0 = time.perf_counter()
    for _ in range(args.steps):
        tok = engine.step(tok)
    torch.cuda.synchronize()
    w1 = time.perf_counter()
    e2e_s = max_over_ranks(w1 - w0)
    e2e_value = B * args.steps / e2e_s

    # ---- the same loop through the driver seam (N = 1): the step recorded as a plan (host-write node
    # for the inputs, a dispatch node per kernel, the ids copied into a host-visible block), compiled
    # once and driven with set_payload / ab_exec_submit / ab_fence_wait, replayed as a CUDA graph
    e2e_seam = None
    if world == 1 and not args.no_seam and args.shard_of == 1:
        try:
            seam = dec.SeamStep(engine, use_graphs=True)
            for _ in range(min(args.warmup, 3)):
                tok = seam.step(tok)
            torch.cuda.synchronize()
            s0 = time.perf_counter()
            for _ in range(args.steps):
                tok = seam.step(tok)
            s1 = time.perf_counter()
            e2e_seam = {"value": B * args.steps / (s1 - s0), "unit": "tok/s", "plan_nodes": seam.nodes,
                        "h2d_bytes_per_step": engine.h2d_bytes_per_step,
                        "d2h_bytes_per_step": engine.d2h_bytes_per_step,
                        "what": "ab_compile once; per step ab_exec_set_payload + ab_exec_submit + ab_fence_wait + "
                                "a read of the host-visible ids block (use_graphs = 1)"}
            seam.close()
        except Exception as e:                     # noqa: BLE001 - reported in the JSON line, the run goes on
            e2e_seam = {"error": f"{type(e).__name__}: {e}"[:300]}
    log("e2e timed")
    # ---- roofline of the dominant kernel: the paged decode attention (K/V of every cached
    # position, once per KV head), timed alone with events on its launching stream, one launch per
    # layer so consecutive launches read different caches (1 GB each, far larger than L2)
    peak, peak_src = measured_peaks()
    reps = 3

    def attn_all_layers():
        scale = float(np.float32(1.0) / np.float32(np.sqrt(cfg.head_dim)))
        name = "AttentionDecodeBatchedF16" if cache_dtype == torch.float16 else "AttentionDecodeBatched"
        u = dec._u("<IIIIIIfI", B, engine.hq, engine.hk, cfg.head_dim, cfg.block, engine.max_pages, scale, 0)
        for li in range(cfg.layers):
            rt.launch(name, [engine.q, engine.k_cache[li], engine.v_cache[li], engine.pages,
                             engine.lengths, engine.attn], u)

    attn_all_layers()
    torch.cuda.synchronize()
    attn_ms = time_kernel(attn_all_layers, reps, stream) / cfg.layers
    esz = 2 if cache_dtype == torch.float16 else 4
    lens = engine.lengths.cpu().numpy().astype(np.int64)
    attn_bytes = int(2 * engine.hk * cfg.head_dim * esz * lens.sum()
                     + 2 * B * engine.hq * cfg.head_dim * 4 + engine.pages.numel() * 4 + B * 4)
    attn_gbs = attn_bytes / (attn_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": ("attn_partition_gqa_mma_kernel<__half, 1>" if cache_dtype == torch.float16
                                            else "attn_partition_kernel") + " (+ attn_combine_kernel)",
                "achieved": attn_gbs, "peak": peak, "unit": "GB/s", "frac": attn_gbs / peak,
                "peak_source": peak_src, "bytes_per_launch": attn_bytes, "ms_per_launch": attn_ms,
                # dram__bytes_read + dram__bytes_write of one launch: NOT measured in this run (it needs
                # a profiler); the figure of the committed ncu capture of this kernel at this per-launch
                # size (a launch reads one layer's cache whatever the layer count), scaled by this
                # run's bytes when the cache dtype or the shard differs
                "traffic": int(1.0790e9 * attn_bytes / 1087906112),
                "traffic_source": "ncu capture of the same kernel and per-launch size, summarised under "
                                  "profiles/, scaled by bytes; not re-measured by this run"}

    # ---- int4 GEMV bandwidth (the metric's second figure): K=4096, N=11008, M=1, rotating over
    # the layers' gate and up matrices (64 x 24 MB, larger than L2).  The headline figure is the
    # kernel the step uses (the load-time prepack of the same matrices); the reference-layout
    # kernel on quant.Int4Quantize's planes is reported beside it.
    gemv = None
    if world == 1 and cfg.layers >= 4 and args.shard_of == 1:
        a1 = torch.randn(cfg.d_model, device=dev)
        out1 = torch.empty(cfg.ffn, device=dev)
        mats = [m for L in model.layers for m in (L.wg, L.wu)]
        u = dec._u("<IIII", 0, cfg.ffn, cfg.d_model, 0)
        gbytes = mats[0].nbytes + cfg.d_model * 4 + cfg.ffn * 4

        def graph_time(body):
            body()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            s2 = torch.cuda.Stream(device=dev)
            s2.wait_stream(stream)
            with torch.cuda.stream(s2):
                with torch.cuda.graph(g, stream=s2):
                    body()
            stream.wait_stream(s2)
            g.replay()
            torch.cuda.synchronize()
            return time_kernel(g.replay, 5, stream) / len(mats)

        def planes_all():
            for m in mats:
                rt.launch("QuantMatVecInt4", [a1, m.codes, m.scales, m.zeros, out1], u)

        ms_planes = graph_time(planes_all)
        packed = [dec.pack(m) for m in mats]

        def packed_all():
            for m in packed:
                rt.launch("QuantMatVecInt4Packed", [a1, m.packed, out1], u)

        ms = graph_time(packed_all)
        del packed
        gemv = {"shape": "M=1 K=4096 N=11008", "bytes": gbytes, "us": ms * 1e3,
                "gbs": gbytes / (ms * 1e-3) / 1e9, "frac": gbytes / (ms * 1e-3) / 1e9 / peak,
                "kernel": "int4_stream_kernel on the load-time prepack (what the step runs)",
                "reference_layout": {"us": ms_planes * 1e3, "gbs": gbytes / (ms_planes * 1e-3) / 1e9,
                                     "frac": gbytes / (ms_planes * 1e-3) / 1e9 / peak,
                                     "kernel": "int4_row_kernel on quant.Int4Quantize's planes"},
                "matrices_rotated": len(mats)}

    # ---- CPU baseline beside it (rank 0, N = 1 only): the oracle's layer sample
    cpu, layer_par = None, None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and args.shard_of == 1:
        # parity at the benchmarked shape first (the GPU leg wants the sample's pristine cache):
        # one full-size layer + lm_head + argmax, this library on the GPU against the oracle
        from oracle.step import LayerSample, layer_parity
        sample = LayerSample(batch=B, context=ctx)
        layer_par = layer_parity(sample, dev)
        layer_par["what"] = ("one full-size layer of the benchmarked step (batch %d, context %d, d 4096, "
                             "32 heads x 128, ffn 11008, f32 cache) + lm_head + argmax, GPU against the "
                             "CPU oracle on identical seeded inputs" % (B, ctx))
        toks, t_layer, t_head, cores = cpu_sample(3, 1, sample=sample)
        cpu = {"value": toks, "unit": "tok/s", "cores": cores, "kind": "port",
               "sample": f"1 of 32 layers of the same step timed 3 times (median {t_layer:.3f} s) + "
                         f"lm_head and argmax once ({t_head:.3f} s), scaled to 32 layers; C "
                         "restatement of accel's CPU kernels, OpenMP over workgroups"}

    # a peer all-reduce that gave up waiting (bounded) left wrong sums behind: say so
    peer_timeouts = 0
    if getattr(engine, "_peer", None) is not None:
        try:
            engine._peer.check()
        except Exception:                          # noqa: BLE001
            peer_timeouts = 1
        t = torch.tensor([peer_timeouts], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
        peer_timeouts = int(t.item())
    if rank == 0:
        weight_bytes = model.int4_bytes()
        line = {
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "batch": B, "context": ctx, "layers": cfg.layers,
                       "kv_cache": args.kv, "parallelism": f"tp{world}", "collective": collective,
                       "l2": "inputs larger than L2: each step streams "
                             f"{weight_bytes / 1e9:.2f} GB of int4 weights and "
                             f"{kv_bytes_first / 1e9:.1f} GB of K/V per rank",
                       **fill_info, "setup_s": round(t_setup, 1)},
            "e2e": {"value": e2e_value, "unit": "tok/s",
                    "h2d_bytes_per_step": engine.h2d_bytes_per_step,
                    "d2h_bytes_per_step": engine.d2h_bytes_per_step},
            "e2e_seam": e2e_seam,
            "gpu_launches": gpu_launches,
            "roofline": roofline,
            "step_hbm": {"bytes_per_step_per_rank": weight_bytes + kv_bytes_first,
                         "gbs": (weight_bytes + kv_bytes_first) / (ms_per_step * 1e-3) / 1e9,
                         "frac_of_peak": (weight_bytes + kv_bytes_first) / (ms_per_step * 1e-3) / 1e9 / peak},
            "int4_gemv": gemv,
            "peer_allreduce_ranks_timed_out": peer_timeouts,
            "cpu_baseline": cpu,
            "parity": {"layer_vs_oracle": layer_par, "tensor_parallel": tp_parity},
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # the captured step holds NCCL work; tearing the process group down under it can block, so
        # the ranks meet once more and leave without the teardown
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--kv", default="f32", choices=["f32", "f16"],
                    help="KV cache dtype; f32 is what the reference's batched decode kernel reads")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kv-fill", default="prefill", choices=["prefill", "random"],
                    help="how the context's K/V get into the cache before the timed steps")
    ap.add_argument("--prefill-chunk", type=int, default=256, help="positions per sequence and prefill pass")
    ap.add_argument("--no-tp-parity", action="store_true",
                    help="skip the N-rank against one-rank comparison of the first step (N > 1)")
    ap.add_argument("--shard-of", type=int, default=1, metavar="N",
                    help="diagnostic: run rank 0's shard of an N-way tensor-parallel step alone on one GPU, "
                         "collectives skipped (for launch lists; not a benchmark figure)")
    ap.add_argument("--no-seam", action="store_true", help="skip the end-to-end loop through ab_compile / ab_exec_submit")
    ap.add_argument("--no-graph", action="store_true", help="launch the step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-overlap", action="store_true", help="keep every operator on one stream")
    ap.add_argument("--force-overlap", action="store_true", help="side-stream overlap at N > 1 too")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="all-reduce of the row-parallel products at N > 1: this library's one-shot "
                         "kernel over NVLink peer memory, or NCCL")
    ap.add_argument("--attention", action="store_true",
                    help="time the paged decode attention of config 3 on its own, f32 and f16 caches")
    ap.add_argument("--allreduce", action="store_true",
                    help="under torchrun: latency of one 256 KiB all-reduce, peer kernel beside NCCL")
    ap.add_argument("--moe", action="store_true",
                    help="time the expert-parallel grouped int4 FFN (config 5) instead of the decode step")
    ap.add_argument("--planes", action="store_true",
                    help="with --linear: read quant.Int4Quantize's three planes as they are (the reference's "
                         "layout) instead of the load-time prepack")
    ap.add_argument("--int8", action="store_true", help="with --linear: the int8 path (QuantMatVecF32 / QuantMatMulTiledF32)")
    ap.add_argument("--linear", default=None, metavar="M,K,N",
                    help="time one int4 product on its own instead of the decode step")
    args = ap.parse_args()
    if args.linear:
        run_linear(args)
    elif args.allreduce:
        run_allreduce(args)
    elif args.attention:
        run_attention(args)
    elif args.moe:
        run_moe(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
