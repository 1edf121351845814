#!/usr/bin/env python
"""Benchmark of the NVFP4 projection path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl engine|reference]

Headline workload (N=1): one full 0.8B-class decode step, M=1: 24 layers x
{[4096,1024], [1024,2048], [7168,1024], [1024,3584]} NVFP4 projections, BF16
activations N(0,1), weights seeded N(0,0.02) quantised on the GPU.  A step is one
pass over all 96 projections; `value` is algorithmic GB/s summed over the step.
The same JSON line carries the prefill W4A4 GEMM (M=4096, gate+up [18432,2560])
as `gemm`, with its own roofline, when that kernel is available.

For N > 1 (one process per GPU under torchrun) the decode step runs as N
independent replicas (it does not shard: a cross-GPU hop costs more than the
kernel) and the GEMM runs N-sharded over output rows with an NCCL all-gather.

`--impl reference` times the reference's CPU path for the same workload (the
oracle's restatement of its scalar loop, all host threads) on rank 0.
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
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

LAYERS_0P8B = 24
SHAPES_0P8B = [(4096, 1024), (1024, 2048), (7168, 1024), (1024, 3584)]  # (N, K) per layer
GEMM_SHAPE = (18432, 2560)  # (N, K): 4B-class gate+up
GEMM_M = 4096
GEMM_SETS = 5
L2_BYTES = 126 * 1024 * 1024
# DRAM bytes of one launch from the ncu captures summarised under profiles/ (same workloads as below)
DECODE_DRAM_TRAFFIC_BYTES = 234_243_072 + 6_459_904
GEMM_DRAM_TRAFFIC_BYTES = 32_540_672 + 100_419_584


def algorithmic_bytes(n: int, k: int, m: int) -> int:
    """W4A16 projection: codes + block scales + activations + outputs + weight_scale_2."""
    return n * k // 2 + n * k // 16 + m * k * 2 + m * n * 2 + 4


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks/throttle reasons sampled every 20 ms while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- workloads
def build_decode_model(q, torch, device, seed: int, sets: int):
    """`sets` independent copies of the 96 NVFP4 projections (alternated between steps so that no weight byte can
    survive in L2 from one step to the next) with one BF16 activation vector per projection."""
    gen = torch.Generator(device=device).manual_seed(seed)
    models = []
    for _ in range(sets):
        weights = []
        for _layer in range(LAYERS_0P8B):
            for (n, k) in SHAPES_0P8B:
                w = torch.randn((n, k), generator=gen, device=device, dtype=torch.float32) * 0.02
                codes, scales, s2 = q.quantize_weight(w)
                weights.append(q.Nvfp4Weight.from_device(codes, scales, s2))
                del w, codes, scales
        models.append(weights)
    return models


def decode_buffers(torch, device, seed: int, m: int = 1):
    """Host (pinned) and device activations / outputs for one step of `m` tokens, packed back to back."""
    shapes = [s for _ in range(LAYERS_0P8B) for s in SHAPES_0P8B]
    x_elems = m * sum(k for _, k in shapes)
    y_elems = m * sum(n for n, _ in shapes)
    gen = torch.Generator().manual_seed(seed)
    x_host = torch.randn(x_elems, generator=gen, dtype=torch.float32).to(torch.bfloat16).pin_memory()
    y_host = torch.empty(y_elems, dtype=torch.bfloat16).pin_memory()
    x_dev = x_host.to(device)
    y_dev = torch.zeros(y_elems, dtype=torch.bfloat16, device=device)
    xs, ys, xo, yo = [], [], 0, 0
    for n, k in shapes:
        xs.append(x_dev[xo:xo + m * k].view(m, k))
        ys.append(y_dev[yo:yo + m * n].view(m, n))
        xo += m * k
        yo += m * n
    return shapes, x_host, y_host, x_dev, y_dev, xs, ys


def run_engine(args, rank: int, world: int, local_rank: int) -> dict | None:
    import torch
    import torch.distributed as dist

    import qwen35x_b200 as q

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    pk = peaks()
    sets = 2
    models = build_decode_model(q, torch, device, seed=42 + rank, sets=sets)
    shapes, x_host, y_host, x_dev, y_dev, xs, ys = decode_buffers(torch, device, seed=7 + rank, m=args.m)
    step_bytes = sum(algorithmic_bytes(n, k, args.m) for n, k in shapes)
    launches_per_step = len(shapes)
    stream = torch.cuda.Stream(device=device)

    # The step's work list: all 96 projections in one persistent launch (they are independent in this workload).
    batches = [q.GemvBatch(list(zip(models[s], xs, ys)), args.m) for s in range(sets)]

    def step(set_index: int):
        batches[set_index].run()

    def step_per_projection(set_index: int):
        for w, x, y in zip(models[set_index], xs, ys):
            q.gemv_w4a16(w, x, out=y, kernel=q.GEMV_STREAM)

    # One CUDA graph per weight set: device-resident step, the end-to-end step with its copies, and (secondary
    # figure) the same step as 96 separate launches.
    graphs, graphs_e2e, graphs_pp = [], [], []
    full = args.only == "all"
    with torch.cuda.stream(stream):
        for s in range(sets):
            step(s)
            if full:
                step_per_projection(s)
        stream.synchronize()
        for s in range(sets):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                step(s)
            graphs.append(g)
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2, stream=stream):
                x_dev.copy_(x_host, non_blocking=True)
                step(s)
                y_host.copy_(y_dev, non_blocking=True)
            graphs_e2e.append(g2)
            if full:
                g3 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g3, stream=stream):
                    step_per_projection(s)
                graphs_pp.append(g3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(run_one, steps: int, warmup: int) -> float:
        with torch.cuda.stream(stream):
            for i in range(warmup):
                run_one(i)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(steps):
                run_one(warmup + i)
            e1.record(stream)
            barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    launches_before = q.launch_count()
    # Device-resident steps: back-to-back stream launches.  The kernel is launched with programmatic stream
    # serialisation, so a step's weight stream starts under the tail of the previous step (its activations and
    # outputs still wait for the previous kernel to complete); one-kernel graph replays cannot overlap that way and
    # are reported beside it.
    # The K launches are issued from CUDA graphs of up to 64 consecutive steps each (programmatic edges between the
    # kernel nodes), so that the host's launch cost plays no part; every step is still one launch of the work list.
    chunk = min(args.steps, 64)
    if chunk > 1:
        chunk -= chunk % 2  # whole A/B pairs: consecutive replays keep alternating the weight sets
    n_chunks, rest = divmod(args.steps, chunk)

    def capture_steps(count: int, first_set: int):
        with torch.cuda.stream(stream):
            for i in range(count):
                step((first_set + i) % sets)
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i in range(count):
                    step((first_set + i) % sets)
        return g

    g_chunk = capture_steps(chunk, 0)
    g_rest = capture_steps(rest, (n_chunks * chunk) % sets) if rest else None

    def timed_chunks() -> float:
        with torch.cuda.stream(stream):
            for i in range(args.warmup):
                step(i % sets)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(n_chunks):
                g_chunk.replay()
            if g_rest is not None:
                g_rest.replay()
            e1.record(stream)
            barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    ms_dev = timed_chunks()
    ms_graph = timed(lambda i: graphs[i % sets].replay(), args.steps, args.warmup)

    def e2e_one(i):
        graphs_e2e[i % sets].replay()
        stream.synchronize()  # the caller reads the step's result on the host

    ms_e2e = timed(e2e_one, args.steps, args.warmup)
    clocks = sampler.stop() if sampler else None
    ms_pp = timed(lambda i: graphs_pp[i % sets].replay(), args.steps, args.warmup) if full else float("nan")
    del launches_before
    torch.cuda.synchronize()
    for b in batches:
        if b.status() != 0:
            raise RuntimeError(f"device-side wait expired in the decode step, code {b.status()}")

    gemm = None
    if args.only != "decode":
        gemm = bench_gemm(args, q, torch, dist, device, rank, world, pk, timed_barrier=barrier)

    if rank != 0:
        return None
    ms_per_step = ms_dev / args.steps
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9
    e2e_value = world * step_bytes / (ms_e2e / args.steps * 1e-3) / 1e9
    launches_per_step = 1
    per_launch_s = ms_per_step * 1e-3 / launches_per_step
    achieved = (step_bytes / launches_per_step) / per_launch_s / 1e9
    out = {
        "metric": "nvfp4_decode_step_bandwidth", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 weights x bf16 activations, fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"0.8B-class decode step, M={args.m}, " "24 layers x {[4096,1024],[1024,2048],[7168,1024],"
                               "[1024,3584]} NVFP4 projections (BASELINE configs[1])",
                   "bytes_per_step": step_bytes, "launch": "one persistent work-list launch over the step's 96 projections per step, back to back on one "
                                                          "stream with programmatic dependent launch (issued from CUDA "
                                                          "graphs of up to 64 consecutive steps)",
                   "graph_replay": {"ms_per_step": round(ms_graph / args.steps, 5),
                                    "value": round(world * step_bytes / (ms_graph / args.steps * 1e-3) / 1e9, 2),
                                    "note": "same step as one-kernel CUDA graph replays (no overlap between replays)"},
                   "per_projection_launches": {"ms_per_step": round(ms_pp / args.steps, 5),
                                               "value": round(world * step_bytes / (ms_pp / args.steps * 1e-3) / 1e9, 2),
                                               "note": "same step as 96 separate kernel launches in one CUDA graph"},
                   "l2": f"two weight sets alternated between steps ({2 * step_bytes} B total > {L2_BYTES} B L2)",
                   "parallelism": "replicas only" if world > 1 else "1 GPU"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "traffic": DECODE_DRAM_TRAFFIC_BYTES,
                     "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch, "
                                       "profiles/gemv_w4a16_stream_decode_step_0p8b.md",
                     "peak_source": pk["source"],
                     "kernel": f"gemv_w4a16_stream_kernel (M={args.m})", "bytes_per_launch": step_bytes // launches_per_step},
        "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": x_host.numel() * 2,
                "d2h_bytes_per_step": y_host.numel() * 2, "ms_per_step": round(ms_e2e / args.steps, 5)},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }
    if gemm is not None:
        out["gemm"] = gemm
    if not full:
        out["config"].pop("per_projection_launches", None)
        out["config"]["only"] = args.only
    if world == 1 and full:
        out["cpu_baseline"] = cpu_baseline(sample_layers=24)
    return out


def bench_gemm(args, q, torch, dist, device, rank, world, pk, timed_barrier) -> dict | None:
    """Prefill W4A4 projection (activation quantisation + tcgen05 GEMM), N-sharded over ranks, all-gathered."""
    n, k = GEMM_SHAPE
    m = GEMM_M
    from qwen35x_b200 import sharding

    # Inputs larger than L2: GEMM_SETS independent (weight, activation, scratch, output) sets are used round-robin,
    # so an iteration never finds its operands (32 MB per set) in the 126 MB L2 from its previous use.
    try:
        gen = torch.Generator(device=device).manual_seed(1234)
        sets = []
        for _ in range(GEMM_SETS):
            w = torch.randn((n, k), generator=gen, device=device, dtype=torch.float32) * 0.02
            codes, scales, s2 = q.quantize_weight(w)
            weight = q.Nvfp4Weight.from_device(codes, scales, s2, shard_index=rank, shard_count=world)
            del w, codes, scales
            x = torch.randn((m, k), generator=gen, device=device, dtype=torch.float32)
            ch = torch.randperm(k, generator=gen, device=device)[: max(1, -(-k // 1000))]
            x[:, ch] *= 20.0
            x = x.to(torch.bfloat16)
            scratch = q.act_scratch(m, k, device)
            out = torch.empty((m, weight.rows), dtype=torch.bfloat16, device=device)
            q.project_prefill(weight, x, out=out, scratch=scratch)
            sets.append((weight, x, scratch, out))
        torch.cuda.synchronize()
    except q.Q35bError as e:
        if "not built" in str(e):
            return None
        raise
    widest = max(c for _, c in sharding.shard_layout(n, world))
    gathered = torch.empty((world * m, widest), dtype=torch.bfloat16, device=device) if world > 1 else None
    # the gather fused into the GEMM's stores: every rank owns a full [m, n] matrix the other ranks store into
    peer, peer_error = None, None
    if world > 1:
        # every rank must reach the same decision, so the outcome of the set-up is agreed on before it is used
        try:
            peer = sharding.PeerGather(m, n)
            ok = 1
        except Exception as e:  # noqa: BLE001 - reported in the JSON line, the NCCL exchange is timed instead
            peer_error = f"{type(e).__name__}: {e}"
            ok = 0
        flag = torch.tensor([ok], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            peer = None
            peer_error = peer_error or "set-up failed on another rank"
    counter = [0]

    def one(with_quant: bool, with_gather: bool, index=None, fused: bool = True):
        weight, x, scratch, out = sets[(counter[0] if index is None else index) % GEMM_SETS]
        counter[0] += 1
        if with_quant:
            a_codes, a_scales, g = q.quantize_activations(x, scratch=scratch)
        else:
            a_codes, a_scales, g = scratch[0].view(m, k // 2), scratch[1], scratch[2]
        if peer is not None and with_gather and fused:
            peer.project(weight, a_codes, a_scales, g)  # GEMM storing into every rank's [m, n] + bounded wait
            return
        q.gemm_w4a4(weight, a_codes, a_scales, g, m, out=out)
        if world > 1 and with_gather:
            sharding.all_gather_slabs(out, n, out=gathered)  # result layout [rank][M][rows of rank]

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        times = []
        for _ in range(steps):
            timed_barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], device=device)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            times.append(float(t.item()))
        return statistics.median(times)

    steps = max(5, min(args.steps, 20))
    if world == 1:
        # one graph holding a GEMM on each of the rotating sets, timed per replay: an event pair around a single launch
        # on an idle GPU would add that launch's start-up latency to a 100 us kernel
        stg = torch.cuda.Stream(device=device)
        with torch.cuda.stream(stg):
            for i in range(GEMM_SETS):
                one(False, False, index=i)
            stg.synchronize()
            g_all = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_all, stream=stg):
                for i in range(GEMM_SETS):
                    one(False, False, index=i)
        torch.cuda.synchronize()
        ms_gemm = timed(g_all.replay, steps, max(3, args.warmup)) / GEMM_SETS
    else:
        ms_gemm = timed(lambda: one(False, False), steps, max(3, args.warmup))
    full_step = lambda: one(True, True)
    if world == 1:
        # quantise + GEMM as one CUDA graph per set, so that host launch latency between the three kernels is not timed
        st = torch.cuda.Stream(device=device)
        graphs = []
        with torch.cuda.stream(st):
            for i in range(GEMM_SETS):
                one(True, True, index=i)
            st.synchronize()
            for i in range(GEMM_SETS):
                g_ = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g_, stream=st):
                    one(True, True, index=i)
                graphs.append(g_)
        torch.cuda.synchronize()
        gi = [0]

        def full_step():
            graphs[gi[0] % GEMM_SETS].replay()
            gi[0] += 1
    ms_full = timed(full_step, steps, max(3, args.warmup))
    ms_nccl = timed(lambda: one(True, True, fused=False), steps, max(3, args.warmup)) if world > 1 else None
    if peer is not None:
        try:
            peer.check()
        except RuntimeError as e:  # a bounded device-side wait expired: keep the NCCL figure, say why
            peer_error = str(e)
            peer = None
            ms_full = ms_nccl
    flops = 2.0 * m * n * k
    fp4_peak_nominal = 9000.0
    fp4_peak_4x = 4.0 * pk["bf16_tflops"]
    tf = flops / (ms_gemm * 1e-3) / 1e12
    return {
        "workload": f"prefill W4A4 GEMM M={m}, gate+up [N={n}, K={k}] (BASELINE configs[3]), N-sharded over {world} GPU(s)",
        "gemm_only": {"ms": round(ms_gemm, 4), "tflops": round(tf, 1)},
        "quant_gemm_gather": {"ms": round(ms_full, 4), "tflops": round(flops / (ms_full * 1e-3) / 1e12, 1),
                              "exchange": "none (1 GPU)" if world == 1 else
                              ("GEMM epilogue stores into every rank's [M, N] over NVLink (peer memory) + flag wait"
                               if peer is not None else f"NCCL all-gather (peer buffers unavailable: {peer_error})")},
        **({"quant_gemm_nccl_gather": {"ms": round(ms_nccl, 4), "tflops": round(flops / (ms_nccl * 1e-3) / 1e12, 1),
                                       "exchange": "NCCL all-gather of the BF16 slabs after the GEMM"}} if world > 1 else {}),
        "roofline": {"bound": "tensor", "achieved": round(tf / world, 1), "peak": fp4_peak_nominal, "unit": "TFLOP/s",
                     "frac": round(tf / world / fp4_peak_nominal, 4),
                     "traffic": GEMM_DRAM_TRAFFIC_BYTES if world == 1 else None,
                     "peak_source": "nominal dense FP4 (no measured FP4 peak); 4x measured bf16 burst = "
                                    f"{fp4_peak_4x:.0f} TFLOP/s -> frac {tf / world / fp4_peak_4x:.4f}",
                     "kernel": "gemm_w4a4_2cta_kernel", "per_gpu": True},
        "l2": f"{GEMM_SETS} operand/output sets used round-robin ({GEMM_SETS} x 32 MB operands + {GEMM_SETS} x 151 MB outputs > 126 MB L2)",
    }


# --------------------------------------------------------------------------- CPU arms
def cpu_decode_sample(o, np, layers: int, threads: int, repeats: int = 1):
    """Time the oracle's scalar W4A16 loop on `layers` layers of the decode step; returns (seconds, bytes)."""
    rng = np.random.default_rng(1)
    tensors = []
    for (n, k) in SHAPES_0P8B:
        codes = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
        scales = rng.integers(0x20, 0x50, size=(n, k // 16), dtype=np.uint8)
        xb = o.bf16_round(rng.standard_normal((1, k)).astype(np.float32))
        tensors.append((codes, scales, xb, n, k))
    t0 = time.perf_counter()
    for _ in range(repeats):
        for _layer in range(layers):
            for codes, scales, xb, n, k in tensors:
                o.gemv_bf16(codes, scales, 3e-4, xb, threads=threads)
    dt = time.perf_counter() - t0
    nbytes = repeats * layers * sum(algorithmic_bytes(n, k, 1) for n, k in SHAPES_0P8B)
    return dt, nbytes


def cpu_baseline(sample_layers: int) -> dict:
    import numpy as np

    from oracle import q35oracle as o

    threads = o.max_threads()
    cpu_decode_sample(o, np, 1, threads)  # warm the pages
    dt, nbytes = cpu_decode_sample(o, np, sample_layers, threads, repeats=max(1, 24 // sample_layers) * 40)
    dt1, nbytes1 = cpu_decode_sample(o, np, 1, 1)
    return {"value": round(nbytes / dt / 1e9, 4), "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{sample_layers} of 24 layers x {max(1, 24 // sample_layers) * 40} repeats of the decode step (oracle restatement of "
                      f"cuda_bench.cu:2091-2100, rows split over OpenMP threads), {dt:.2f} s",
            "single_thread": {"value": round(nbytes1 / dt1 / 1e9, 4), "unit": "GB/s", "cores": 1,
                              "sample": f"1 layer, {dt1:.2f} s"}}


def cpu_reference_entries(shapes_m):
    """CPU leg of the shape report: the oracle's scalar loop (reference CPU path) on a bounded sample of each shape
    (64 output rows per thread x min(M, 2) tokens), one thread and all threads; the full-shape time is an explicit
    extrapolation."""
    import time

    import numpy as np

    from oracle import q35oracle as o

    out = []
    rng = np.random.default_rng(5)
    threads = o.max_threads()
    for n, k, m in shapes_m:
        rows, toks = min(n, 64 * threads), min(m, 2)
        codes = rng.integers(0, 256, size=(rows, k // 2), dtype=np.uint8)
        scales = rng.integers(0x20, 0x50, size=(rows, k // 16), dtype=np.uint8)
        xb = o.bf16_round(rng.standard_normal((toks, k)).astype(np.float32))
        res = {}
        for t in (1, threads):
            r = min(rows, 64) if t == 1 else rows
            t0 = time.perf_counter()
            o.gemv_bf16(codes[:r], scales[:r], 3e-4, xb, threads=t)
            dt = time.perf_counter() - t0
            res[t] = dt * (n / r) * (m / toks)
        out.append({"N": n, "K": k, "M": m, "cpu_us_1_thread_extrapolated": round(res[1] * 1e6, 1),
                    f"cpu_us_{threads}_threads_extrapolated": round(res[threads] * 1e6, 1), "cores": threads,
                    "sample": f"{rows} rows x {toks} tokens measured, scaled by rows and tokens"})
    return out



def run_reference(args, rank: int) -> dict | None:
    if rank != 0:
        return None
    import numpy as np

    from oracle import q35oracle as o

    threads = o.max_threads()
    # bounded sample: as many of the 24 layers per step as keep the whole run near 100 s of CPU time
    t_layer, _ = cpu_decode_sample(o, np, 1, threads)
    t_layer, _ = cpu_decode_sample(o, np, 1, threads)
    layers = int(max(1, min(24, 100.0 / max(t_layer * (args.steps + args.warmup), 1e-9))))
    for _ in range(args.warmup):
        cpu_decode_sample(o, np, layers, threads)
    dt = 0.0
    nbytes = 0
    for _ in range(args.steps):
        t, b = cpu_decode_sample(o, np, layers, threads)  # times the projection loops only, not the input generation
        dt += t
        nbytes += b
    value = nbytes / dt / 1e9
    sample = (f"each step = {layers} of 24 layers of the decode step on {threads} host threads (oracle port of the "
              f"reference's scalar CPU loop, cuda_bench.cu:2091-2100; the reference itself cannot run its CPU path "
              f"without a GPU)")
    return {"impl": "reference", "metric": "nvfp4_decode_step_bandwidth", "value": round(value, 4), "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dt / args.steps * 1e3, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "nvfp4 weights x bf16 activations, fp32 accumulate", "data": "synthetic",
            "config": {"workload": "0.8B-class decode step, M=1 (BASELINE configs[1]); bounded sample per step",
                       "parallelism": "host CPU"},
            "cpu_baseline": {"value": round(value, 4), "unit": "GB/s", "cores": threads, "kind": "port",
                             "sample": sample},
            "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["engine", "reference"], default="engine")
    ap.add_argument("--m", type=int, default=1, choices=range(1, 9), metavar="TOKENS",
                    help="tokens per decode step (1..8); the headline and the driver's runs use 1")
    ap.add_argument("--report", default="", help="write the per-shape throughput report (JSON) to this path and exit")
    ap.add_argument("--only", choices=["all", "decode", "gemm"], default="all",
                    help="profiling aid: 'decode' skips the GEMM, the per-projection-launch figure and the CPU "
                         "baseline; 'gemm' shrinks the decode part to its minimum")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "engine" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.report:
        import torch

        import qwen35x_b200 as q
        from qwen35x_b200 import shape_report

        torch.cuda.set_device(0)
        rep = shape_report.run("", q, torch, torch.device("cuda", 0), peaks())
        rep["cpu_reference"] = cpu_reference_entries([(3584, 1024, 1), (18432, 2560, 1), (2560, 9216, 1), (18432, 2560, 4096)])
        Path(args.report).parent.mkdir(parents=True, exist_ok=True)
        Path(args.report).write_text(json.dumps(rep, indent=1))
        Path(args.report).with_suffix(".md").write_text(shape_report.to_markdown(rep))
        print(json.dumps({"report": args.report, "entries": sum(len(v) for v in rep.values() if isinstance(v, list))}))
        return 0
    if args.impl == "reference":
        out = run_reference(args, rank)
        if out is not None:
            print(json.dumps(out), flush=True)
        return 0
    if args.gpus > 1 and world == 1:
        # launched without torchrun: start one rank per GPU ourselves
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29517"), __file__,
               "--gpus", str(args.gpus), "--steps", str(args.steps), "--warmup", str(args.warmup)]
        return subprocess.call(cmd)
    out = run_engine(args, rank, world, local_rank)
    if out is not None:
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
