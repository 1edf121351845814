#!/usr/bin/env python
"""Benchmark of the NVFP4 projection path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl engine|reference]

Headline workload (N=1): one full 0.8B-class decode step, M=1: 24 layers x
{[4096,1024], [1024,2048], [7168,1024], [1024,3584]} NVFP4 projections, BF16
activations N(0,1), weights seeded N(0,0.02) quantised on the GPU.  A step is one
pass over all 96 projections; `value` is algorithmic GB/s summed over the step.
The same JSON line carries
  `decode_4b`  the 4B-class decode step (32 layers x {[18432,2560], [2560,9216], [10240,2560], [2560,4096]}) at
               M = 1 and 8 (1 GPU only),
  `gemm`       the prefill W4A4 GEMM (M=4096, gate+up [18432,2560]) with its own roofline, end-to-end figure,
               CPU baseline and check, and the prefill MLP block (hidden 2560, intermediate 9216).

For N > 1 (one process per GPU under torchrun) the decode step runs as N independent replicas (it does not shard:
a cross-GPU hop costs more than the kernel); the GEMM and the MLP block run N-sharded over output rows, the shards
exchanged over NVLink, and every rank checks the gathered result against its own unsharded computation.

`--impl reference` times the reference's CPU path for the same decode step (the oracle's restatement of its scalar
loop, all host threads) on rank 0 and, where a GPU and the compiled reference are present, the reference's own
CUDA kernels on the same shapes beside it.
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
LAYERS_4B = 32
SHAPES_4B = [(18432, 2560), (2560, 9216), (10240, 2560), (2560, 4096)]
GEMM_SHAPE = (18432, 2560)  # (N, K): 4B-class gate+up
GEMM_M = 4096
GEMM_SETS = 5
MLP_HIDDEN, MLP_INTER = 2560, 9216
MLP_SETS = 3
MLP_CHUNKS = 1  # token groups of the sharded MLP block (PeerMlp.run chunks): 2 and 4 measured slower on 2 GPUs (203, 275 us against 186)
L2_BYTES = 126 * 1024 * 1024
PEER_COPY_GBS = 770.0  # measured peer-copy rate per direction on this pool's NVLink (nominal 900)
FP4_NOMINAL_TFLOPS = 9000.0


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


def ncu_traffic(key: str):
    """DRAM bytes of one launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures summarised under
    profiles/: profiles/traffic.json maps a workload key to {"bytes": ..., "source": "<summary file>"}."""
    p = ROOT / "profiles" / "traffic.json"
    if not p.is_file():
        return None, "profiles/traffic.json missing"
    entry = json.loads(p.read_text()).get(key)
    if not entry:
        return None, f"no entry {key} in profiles/traffic.json"
    return int(entry["bytes"]), entry.get("source", "profiles/traffic.json")


def host_threads() -> int:
    """Host threads this process may run on.  Not OMP_NUM_THREADS: torch.distributed.run forces that to 1."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


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
def build_decode_model(q, torch, device, seed: int, sets: int, shapes, layers: int):
    """`sets` independent copies of the step's NVFP4 projections (alternated between steps so that no weight byte can
    survive in L2 from one step to the next)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    models = []
    for _ in range(sets):
        weights = []
        for _layer in range(layers):
            for (n, k) in shapes:
                w = torch.randn((n, k), generator=gen, device=device, dtype=torch.float32) * 0.02
                codes, scales, s2 = q.quantize_weight(w)
                weights.append(q.Nvfp4Weight.from_device(codes, scales, s2))
                del w, codes, scales
        models.append(weights)
    return models


def decode_buffers(torch, device, seed: int, shapes, m: int = 1):
    """Host (pinned) and device activations / outputs for one step of `m` tokens, packed back to back."""
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
    return x_host, y_host, x_dev, y_dev, xs, ys


class Timer:
    """CUDA-event timing on one stream, max over ranks, with a barrier + synchronize on both sides."""

    def __init__(self, torch, dist, device, world: int):
        self.torch, self.dist, self.device, self.world = torch, dist, device, world

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, ms: float) -> float:
        if self.world > 1:
            t = self.torch.tensor([ms], device=self.device)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def region(self, stream, run_one, steps: int, warmup: int) -> float:
        """Milliseconds for `steps` calls of run_one(i) issued back to back on `stream`."""
        torch = self.torch
        with torch.cuda.stream(stream):
            for i in range(warmup):
                run_one(i)
            self.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(steps):
                run_one(warmup + i)
            e1.record(stream)
            self.barrier()
        return self.max_over_ranks(e0.elapsed_time(e1))

    def per_call(self, stream, fn, steps: int, warmup: int) -> float:
        """Median milliseconds of single calls, each between a barrier and a synchronize (max over ranks per call)."""
        torch = self.torch
        times = []
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                fn()
            for _ in range(steps):
                self.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                fn()
                e1.record(stream)
                stream.synchronize()
                times.append(self.max_over_ranks(e0.elapsed_time(e1)))
        return statistics.median(times)


def capture(torch, stream, fn):
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
    return g


def time_decode_step(torch, timer, stream, batches, steps: int, warmup: int):
    """Per-step milliseconds of a work-list step: (back-to-back launches issued from CUDA graphs of up to 64
    consecutive steps, programmatic edges between the kernel nodes), (one-kernel graph replays, no overlap)."""
    sets = len(batches)
    chunk = min(steps, 64)
    if chunk > 1 and sets > 1:
        chunk -= chunk % sets  # whole rounds: consecutive replays keep rotating the weight sets
    n_chunks, rest = divmod(steps, chunk)

    def steps_graph(count: int, first: int):
        return capture(torch, stream, lambda: [batches[(first + i) % sets].run() for i in range(count)])

    g_chunk = steps_graph(chunk, 0)
    g_rest = steps_graph(rest, (n_chunks * chunk) % sets) if rest else None
    singles = [capture(torch, stream, b.run) for b in batches]

    def replay_chunks(_i):
        for _ in range(n_chunks):
            g_chunk.replay()
        if g_rest is not None:
            g_rest.replay()

    with torch.cuda.stream(stream):
        for i in range(warmup):
            batches[i % sets].run()
    ms_b2b = timer.region(stream, replay_chunks, 1, 0) / steps
    ms_graph = timer.region(stream, lambda i: singles[i % sets].replay(), steps, warmup) / steps
    return ms_b2b, ms_graph


def run_engine(args, rank: int, world: int, local_rank: int) -> dict | None:
    import torch
    import torch.distributed as dist

    import qwen35x_b200 as q

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    pk = peaks()
    timer = Timer(torch, dist, device, world)
    full = args.only == "all"
    sets = 2
    shapes = [s for _ in range(LAYERS_0P8B) for s in SHAPES_0P8B]
    models = build_decode_model(q, torch, device, seed=42 + rank, sets=sets, shapes=SHAPES_0P8B, layers=LAYERS_0P8B)
    x_host, y_host, x_dev, y_dev, xs, ys = decode_buffers(torch, device, seed=7 + rank, shapes=shapes, m=args.m)
    step_bytes = sum(algorithmic_bytes(n, k, args.m) for n, k in shapes)
    stream = torch.cuda.Stream(device=device)

    # The step's work list: all 96 projections in one persistent launch (they are independent in this workload).
    batches = [q.GemvBatch(list(zip(models[s], xs, ys)), args.m, digits=args.digits) for s in range(sets)]

    def step_per_projection(set_index: int):
        for w, x, y in zip(models[set_index], xs, ys):
            q.gemv_w4a16(w, x, out=y, kernel=q.GEMV_STREAM)

    def e2e_step(s: int):
        x_dev.copy_(x_host, non_blocking=True)
        batches[s].run()
        y_host.copy_(y_dev, non_blocking=True)

    graphs_e2e = [capture(torch, stream, lambda s=s: e2e_step(s)) for s in range(sets)]
    graphs_pp = [capture(torch, stream, lambda s=s: step_per_projection(s)) for s in range(sets)] if full else []

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    # Device-resident steps: back-to-back stream launches.  The kernel is launched with programmatic stream
    # serialisation, so a step's weight stream starts under the tail of the previous step (its activations and
    # outputs still wait for the previous kernel to complete); one-kernel graph replays cannot overlap that way and
    # are reported beside it.
    ms_per_step, ms_graph_step = time_decode_step(torch, timer, stream, batches, args.steps, args.warmup)

    def e2e_one(i):
        graphs_e2e[i % sets].replay()
        stream.synchronize()  # the caller reads the step's result on the host

    ms_e2e = timer.region(stream, e2e_one, args.steps, args.warmup) / args.steps
    clocks = sampler.stop() if sampler else None
    ms_pp = timer.region(stream, lambda i: graphs_pp[i % sets].replay(), args.steps, args.warmup) / args.steps if full else float("nan")
    torch.cuda.synchronize()
    for b in batches:
        if b.status() != 0:
            raise RuntimeError(f"device-side wait expired in the decode step, code {b.status()}")
    del batches, graphs_e2e, graphs_pp, models
    torch.cuda.empty_cache()

    decode_4b = None
    if full and world == 1:
        decode_4b = bench_decode_4b(args, q, torch, timer, device, pk)
    gemm = None
    if args.only != "decode":
        gemm = bench_gemm(args, q, torch, dist, timer, device, rank, world, pk)

    if rank != 0:
        return None
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    achieved_graph = step_bytes / (ms_graph_step * 1e-3) / 1e9
    traffic, traffic_source = (ncu_traffic(f"decode_step_0p8b_m{args.m}") if args.m in (1, 8)
                               else (None, "no capture for this token count"))
    out = {
        "metric": "nvfp4_decode_step_bandwidth", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 weights x bf16 activations, fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"0.8B-class decode step, M={args.m}, " "24 layers x {[4096,1024],[1024,2048],[7168,1024],"
                               "[1024,3584]} NVFP4 projections (BASELINE configs[1])",
                   "bytes_per_step": step_bytes,
                   "launch": "one persistent work-list launch over the step's 96 projections per step, back to back on "
                             "one stream with programmatic dependent launch (issued from CUDA graphs of up to 64 "
                             "consecutive steps)",
                   "graph_replay": {"ms_per_step": round(ms_graph_step, 5), "value": round(world * achieved_graph, 2),
                                    "frac_of_hbm_peak": round(achieved_graph / pk["hbm_gbs"], 4),
                                    "note": "same step as one-kernel CUDA graph replays (no overlap between replays): "
                                            "what a step with other work between its projections sees"},
                   "per_projection_launches": {"ms_per_step": round(ms_pp, 5),
                                               "value": round(world * step_bytes / (ms_pp * 1e-3) / 1e9, 2),
                                               "note": "same step as 96 separate kernel launches in one CUDA graph"},
                   "l2": f"two weight sets alternated between steps ({2 * step_bytes} B total > {L2_BYTES} B L2)",
                   "parallelism": "replicas only" if world > 1 else "1 GPU"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "frac_graph_replay": round(achieved_graph / pk["hbm_gbs"], 4),
                     "traffic": traffic, "traffic_source": traffic_source, "peak_source": pk["source"],
                     "kernel": f"gemv_w4a16_stream_kernel (M={args.m})", "bytes_per_launch": step_bytes},
        "e2e": {"value": round(world * step_bytes / (ms_e2e * 1e-3) / 1e9, 2), "unit": "GB/s",
                "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2,
                "ms_per_step": round(ms_e2e, 5)},
        "gpu_launches": args.steps,
        "clocks": clocks,
    }
    if decode_4b is not None:
        out["decode_4b"] = decode_4b
    if gemm is not None:
        out["gemm"] = gemm
    if not full:
        out["config"].pop("per_projection_launches", None)
        out["config"]["only"] = args.only
    if world == 1 and full:
        out["cpu_baseline"] = cpu_baseline(sample_layers=24)
    return out


def bench_decode_4b(args, q, torch, timer, device, pk) -> list:
    """The 4B-class decode step (BASELINE configs[2]): 128 projections, 1.94 GB of weights (one set: larger than L2
    by itself), M = 1 and 8, one work-list launch per step."""
    shapes = [s for _ in range(LAYERS_4B) for s in SHAPES_4B]
    models = build_decode_model(q, torch, device, seed=4242, sets=1, shapes=SHAPES_4B, layers=LAYERS_4B)
    stream = torch.cuda.Stream(device=device)
    out = []
    steps = max(4, min(args.steps, 40))
    for m in (1, 8):
        _, _, _, _, xs, ys = decode_buffers(torch, device, seed=11 + m, shapes=shapes, m=m)
        batches = [q.GemvBatch(list(zip(models[0], xs, ys)), m)]
        ms_b2b, ms_graph = time_decode_step(torch, timer, stream, batches, steps, 3)
        torch.cuda.synchronize()
        if batches[0].status() != 0:
            raise RuntimeError(f"device-side wait expired in the 4B-class decode step, code {batches[0].status()}")
        nbytes = sum(algorithmic_bytes(n, k, m) for n, k in shapes)
        out.append({"workload": "4B-class decode step, 32 layers x {[18432,2560],[2560,9216],[10240,2560],[2560,4096]} "
                                "(BASELINE configs[2])", "M": m, "bytes_per_step": nbytes,
                    "ms_per_step": round(ms_b2b, 5), "GB/s": round(nbytes / ms_b2b / 1e6, 1),
                    "frac_of_hbm_peak": round(nbytes / ms_b2b / 1e6 / pk["hbm_gbs"], 4),
                    "graph_replay_ms_per_step": round(ms_graph, 5),
                    "graph_replay_frac_of_hbm_peak": round(nbytes / ms_graph / 1e6 / pk["hbm_gbs"], 4), "steps": steps})
        del batches
    return out


def bench_gemm(args, q, torch, dist, timer, device, rank, world, pk) -> dict | None:
    """Prefill W4A4 projection (activation quantisation + tcgen05 GEMM), N-sharded over ranks, and the prefill MLP
    block; every exchange path is checked against the rank's own unsharded result."""
    n, k = GEMM_SHAPE
    m = GEMM_M
    from qwen35x_b200 import sharding

    # Inputs larger than L2: GEMM_SETS independent (weight, activation, scratch, output) sets are used round-robin,
    # so an iteration never finds its operands (32 MB per set) in the 126 MB L2 from its previous use.
    gen = torch.Generator(device=device).manual_seed(1234)
    sets, raw0 = [], None
    for i in range(GEMM_SETS):
        w = torch.randn((n, k), generator=gen, device=device, dtype=torch.float32) * 0.02
        codes, scales, s2 = q.quantize_weight(w)
        weight = q.Nvfp4Weight.from_device(codes, scales, s2, shard_index=rank, shard_count=world)
        if i == 0:
            raw0 = (codes, scales, s2)  # set 0 keeps its checkpoint-layout bytes for the checks below
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

    steps = max(5, min(args.steps, 20))
    warm = max(3, args.warmup)
    st = torch.cuda.Stream(device=device)
    # GEMM alone, the same way at every N: one graph holding a GEMM on each of the rotating sets, timed per replay
    # (an event pair around a single eager launch would add that launch's start-up latency to a 100 us kernel)
    g_all = capture(torch, st, lambda: [one(False, False, index=i) for i in range(GEMM_SETS)])
    ms_gemm = timer.per_call(st, g_all.replay, steps, warm) / GEMM_SETS
    if world == 1:
        # quantise + GEMM as one CUDA graph per set, so that host launch latency between the kernels is not timed
        graphs = [capture(torch, st, lambda i=i: one(True, True, index=i)) for i in range(GEMM_SETS)]
        gi = [0]

        def full_step():
            graphs[gi[0] % GEMM_SETS].replay()
            gi[0] += 1
        ms_full = timer.per_call(st, full_step, steps, warm)
        ms_nccl = None
    else:
        if peer is not None:
            # quantise + gathering GEMM + wait as one CUDA graph per set (epochs are counted on the device)
            graphs = []
            for i in range(GEMM_SETS):
                timer.barrier()
                graphs.append(capture(torch, st, lambda i=i: one(True, True, index=i)))
                timer.barrier()
            gi = [0]

            def fused_step():
                graphs[gi[0] % GEMM_SETS].replay()
                gi[0] += 1
            ms_full = timer.per_call(st, fused_step, steps, warm)
        else:
            ms_full = None
        ms_nccl = timer.per_call(st, lambda: one(True, True, fused=False), steps, warm)  # eager: NCCL launches
        if ms_full is None:
            ms_full = ms_nccl
    if peer is not None:
        try:
            peer.check()
        except RuntimeError as e:  # a bounded device-side wait expired: keep the NCCL figure, say why
            peer_error = str(e)
            peer = None
            ms_full = ms_nccl

    # ---- checks, outside every timed region
    checks = {}
    weight0, x0, scratch0, out0 = sets[0]
    codes0, scales0, s20 = raw0
    with torch.cuda.stream(st):
        a_codes, a_scales, g = q.quantize_activations(x0, scratch=scratch0)
        if world > 1:
            full_w = q.Nvfp4Weight.from_device(codes0, scales0, s20)
            c_full = q.gemm_w4a4(full_w, a_codes, a_scales, g, m)
            ok_fused = None
            if peer is not None:
                timer.barrier()
                c_gathered = peer.project(weight0, a_codes, a_scales, g)
                st.synchronize()
                peer.check()
                ok_fused = bool(torch.equal(c_gathered, c_full))
                timer.barrier()
            q.gemm_w4a4(weight0, a_codes, a_scales, g, m, out=out0)
            slabs = sharding.all_gather_slabs(out0, n, out=gathered)
            ok_nccl = bool(torch.equal(sharding.assemble(slabs, n), c_full))
            verdict = torch.tensor([int(ok_nccl and ok_fused is not False)], device=device)
            dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
            checks["gather_checked"] = bool(int(verdict.item()))
            checks["gather_check"] = ("gathered [M, N] of the fused path and of the NCCL path torch.equal to this rank's "
                                      "own unsharded GEMM, on every rank" if peer is not None else
                                      "gathered [M, N] of the NCCL path torch.equal to this rank's own unsharded GEMM, on every rank")
            del full_w, c_full
        else:
            q.gemm_w4a4(weight0, a_codes, a_scales, g, m, out=out0)
        st.synchronize()
    cpu = None
    if rank == 0:
        cpu = gemm_cpu_baseline_and_check(q, torch, m, n, k, weight0, codes0, scales0, s20, a_codes, a_scales, g, out0)
        checks["checked"] = cpu.pop("checked")
        checks["check"] = cpu.pop("check")
    e2e = gemm_e2e(q, torch, timer, st, sets, m, n, k, steps, warm) if world == 1 else None
    del raw0, codes0, scales0
    if peer is not None:
        del peer
    mlp = bench_mlp(args, q, torch, dist, timer, device, rank, world)

    failed = [key for key in ("checked", "gather_checked") if checks.get(key) is False] + \
             (["mlp.checked"] if mlp.get("checked") is False else [])
    flops = 2.0 * m * n * k
    fp4_peak_4x = 4.0 * pk["bf16_tflops"]
    tf = flops / (ms_gemm * 1e-3) / 1e12
    traffic, traffic_source = ncu_traffic("gemm_m4096_n18432_k2560") if world == 1 else (None, "1-GPU capture only")
    gather_bytes_in = m * n * 2 * (world - 1) // world
    result = {
        "workload": f"prefill W4A4 GEMM M={m}, gate+up [N={n}, K={k}] (BASELINE configs[3]), N-sharded over {world} GPU(s)",
        "gemm_only": {"ms": round(ms_gemm, 4), "tflops": round(tf, 1),
                      "timing": f"one CUDA graph with a GEMM on each of {GEMM_SETS} rotating sets, per replay / {GEMM_SETS}, every N"},
        "quant_gemm_gather": {"ms": round(ms_full, 4), "tflops": round(flops / (ms_full * 1e-3) / 1e12, 1),
                              "exchange": "none (1 GPU)" if world == 1 else
                              ("GEMM epilogue stores into every rank's [M, N] over NVLink (peer memory) + flag wait"
                               if peer_error is None else f"NCCL all-gather (peer buffers unavailable: {peer_error})")},
        **({"quant_gemm_nccl_gather": {"ms": round(ms_nccl, 4), "tflops": round(flops / (ms_nccl * 1e-3) / 1e12, 1),
                                       "exchange": "NCCL all-gather of the BF16 slabs after the GEMM"},
            "best_exchange": "fused" if (peer_error is None and ms_full <= ms_nccl) else "nccl",
            "gather_roofline": {"bytes_in_per_gpu": gather_bytes_in, "peer_copy_gbs": PEER_COPY_GBS,
                                "us_at_peer_copy_rate": round(gather_bytes_in / PEER_COPY_GBS / 1e3, 1),
                                "note": "every GPU must take in (N-1)/N of the BF16 [M, N]: a lower bound for any "
                                        "exchange that leaves the whole matrix on every rank"}} if world > 1 else {}),
        **checks,
        "roofline": {"bound": "tensor", "achieved": round(tf / world, 1), "peak": FP4_NOMINAL_TFLOPS, "unit": "TFLOP/s",
                     "frac": round(tf / world / FP4_NOMINAL_TFLOPS, 4),
                     "traffic": traffic, "traffic_source": traffic_source,
                     "peak_source": "nominal dense FP4 (no measured FP4 peak); 4x measured bf16 burst = "
                                    f"{fp4_peak_4x:.0f} TFLOP/s -> frac {tf / world / fp4_peak_4x:.4f}",
                     "kernel": "gemm_w4a4_2cta_kernel", "per_gpu": True},
        "l2": f"{GEMM_SETS} operand/output sets used round-robin ({GEMM_SETS} x 32 MB operands + {GEMM_SETS} x 151 MB outputs > 126 MB L2)",
        "mlp_block": mlp,
    }
    if e2e is not None:
        result["e2e"] = e2e
    if cpu is not None:
        result["cpu_baseline"] = cpu
    if failed:
        if rank == 0:
            print(json.dumps({"error": "result check failed", "failed": failed, "gemm": result}), flush=True)
        raise SystemExit(3)
    return result


def gemm_cpu_baseline_and_check(q, torch, m, n, k, weight, codes, scales, s2, a_codes, a_scales, g, out) -> dict:
    """The reference's CPU computation of the W4A4 projection (oracle port of cuda_bench.cu:872-884) on a bounded
    sample of output rows, all host threads: its time is the CPU baseline, its values are what the GPU output of
    the same rows is checked against (relative L2 <= 1e-3)."""
    import numpy as np

    from oracle import q35oracle as o

    threads = host_threads()
    rng = np.random.default_rng(3)
    lo, hi = weight.row_begin, weight.row_begin + weight.rows
    rows = np.sort(rng.choice(np.arange(lo, hi), size=min(32, hi - lo), replace=False))
    idx = torch.from_numpy(rows).to(codes.device)
    h_codes, h_scales = codes[idx].cpu().numpy(), scales[idx].cpu().numpy()
    a_c = a_codes.cpu().numpy()
    tiled = a_scales.cpu().numpy()
    r = np.arange(m)[:, None]
    c = np.arange(k // 16)[None, :]
    slots = (k // 16 + 3) // 4 * 4
    a_s = tiled[(((r // 128) * (slots // 4) + c // 4) * 32 + (r % 32)) * 16 + ((r % 128) // 32) * 4 + (c % 4)]
    t0 = time.perf_counter()
    eb, _ = o.gemm_w4a4(h_codes, h_scales, s2, a_c, a_s, float(g.item()), threads=threads)
    dt = time.perf_counter() - t0
    got = out[:, idx - lo].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    err = o.rel_l2(o.bf16_to_f32(got), o.bf16_to_f32(eb))
    flops = 2.0 * m * len(rows) * k
    return {"value": round(flops / dt / 1e12, 6), "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"{len(rows)} of {n} output rows x all {m} tokens ({dt:.2f} s); full shape extrapolates to "
                      f"{dt * n / len(rows):.0f} s",
            "checked": bool(err <= 1e-3), "check": f"GPU output of the sampled rows vs the CPU port: relative L2 {err:.2e} (<= 1e-3)"}


def gemm_e2e(q, torch, timer, stream, sets, m, n, k, steps, warm) -> dict:
    """The projection through the public call with host buffers: x from pinned host memory, quantise, GEMM, the
    BF16 output back to pinned host memory, host synchronised every step."""
    x_host = sets[0][1].cpu().pin_memory()
    c_host = torch.empty((m, n), dtype=torch.bfloat16).pin_memory()
    graphs = []
    for weight, x, scratch, out in sets:
        def step(weight=weight, x=x, scratch=scratch, out=out):
            x.copy_(x_host, non_blocking=True)
            q.project_prefill(weight, x, out=out, scratch=scratch)
            c_host.copy_(out, non_blocking=True)
        graphs.append(capture(torch, stream, step))
    gi = [0]

    def one():
        graphs[gi[0] % len(graphs)].replay()
        gi[0] += 1
    ms = timer.per_call(stream, one, max(3, steps // 2), min(warm, 3))
    flops = 2.0 * m * n * k
    return {"value": round(flops / (ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s", "ms_per_step": round(ms, 4),
            "h2d_bytes_per_step": m * k * 2, "d2h_bytes_per_step": m * n * 2}


def bench_mlp(args, q, torch, dist, timer, device, rank, world) -> dict:
    """Prefill MLP block out = down(silu(gate x) * up x) + residual, M = 4096, hidden 2560, intermediate 9216,
    N-sharded over the ranks: gate/up shards write their columns of the NVFP4 intermediate (0.5625 B per element),
    a peer push carries them to every rank, the down shards write BF16 columns of the output, a second push gathers
    those (sharding.PeerMlp)."""
    from qwen35x_b200 import sharding

    m, hidden, inter = GEMM_M, MLP_HIDDEN, MLP_INTER
    gen = torch.Generator(device=device).manual_seed(77)
    layout = sharding.MlpLayout(m, hidden, inter)
    data = []
    h_scale = None
    for i in range(MLP_SETS):
        gw = [q.quantize_weight(torch.randn((inter, hidden), generator=gen, device=device) * 0.02) for _ in range(2)]
        dw = q.quantize_weight(torch.randn((hidden, inter), generator=gen, device=device) * 0.02)
        host = [(c.cpu().numpy(), s.cpu().numpy(), s2) for (c, s, s2) in gw]
        gu = q.Nvfp4Weight.gate_up_from_host(*host[0], *host[1], shard_index=rank, shard_count=world)
        down = q.Nvfp4Weight.from_device(dw[0], dw[1], dw[2], shard_index=rank, shard_count=world)
        x = torch.randn((m, hidden), generator=gen, device=device).to(torch.bfloat16)
        res = torch.randn((m, hidden), generator=gen, device=device).to(torch.bfloat16)
        sx = q.act_scratch(m, hidden, device)
        entry = {"gu": gu, "down": down, "x": x, "res": res, "sx": sx}
        if i == 0:
            # unsharded block of set 0: calibrates the intermediate's scale and gives the expected output
            gu_full = q.Nvfp4Weight.gate_up_from_host(*host[0], *host[1]) if world > 1 else gu
            down_full = q.Nvfp4Weight.from_device(dw[0], dw[1], dw[2]) if world > 1 else down
            codes, scales, g = q.quantize_activations(x, scratch=sx)
            h = q.gemm_w4a4(gu_full, codes, scales, g, m)
            h_scale = (h.float().abs().max() / (6.0 * 448.0)).reshape(1).to(torch.float32)
            hc, hs, hg = q.gemm_w4a4_gate_up_quant(gu_full, codes, scales, g, m, h_scale)
            entry["expected"] = q.gemm_w4a4(down_full, hc, hs, hg, m, residual=res)
            del h, hc, hs, gu_full, down_full
        data.append(entry)
        del gw, dw, host
    torch.cuda.synchronize()
    status = torch.zeros(1, dtype=torch.int32, device=device)
    st = torch.cuda.Stream(device=device)
    flops = 2.0 * m * hidden * inter * 3
    steps = max(5, min(args.steps, 20))
    if world == 1:
        bufs = [(torch.empty(m * layout.codes_ld, dtype=torch.uint8, device=device),
                 torch.empty(layout.scales_bytes, dtype=torch.uint8, device=device),
                 torch.empty((m, hidden), dtype=torch.bfloat16, device=device)) for _ in range(MLP_SETS)]

        def block(i):
            d, (hc, hs, y) = data[i], bufs[i]
            codes, scales, g = q.quantize_activations(d["x"], scratch=d["sx"])
            c2, s2_, g2 = q.gemm_w4a4_gate_up_quant(d["gu"], codes, scales, g, m, h_scale, scratch=(hc, hs, None), status=status)
            q.gemm_w4a4(d["down"], c2, s2_, g2, m, out=y, status=status, residual=d["res"])
            return y
        graphs = [capture(torch, st, lambda i=i: block(i)) for i in range(MLP_SETS)]
        gi = [0]

        def one():
            graphs[gi[0] % MLP_SETS].replay()
            gi[0] += 1
        ms = timer.per_call(st, one, steps, 3)
        with torch.cuda.stream(st):
            ok = bool(torch.equal(block(0), data[0]["expected"]))
            st.synchronize()
        ok = ok and int(status.item()) == 0
        exchange = "none (1 GPU)"
    else:
        local = q.PeerBuffer.create_bytes(layout.total)
        nb = int(q.lib().q35b_peer_buffer_handle_bytes())
        mine = torch.frombuffer(bytearray(local.export()), dtype=torch.uint8).to(device)
        handles = torch.empty((world, nb), dtype=torch.uint8, device=device)
        dist.all_gather_into_tensor(handles, mine)
        handles = handles.cpu().numpy()
        buffers = [local if r == rank else q.PeerBuffer.open_bytes(handles[r].tobytes(), layout.total) for r in range(world)]
        dist.barrier()
        runners = [sharding.PeerMlp(layout, buffers, rank, d["gu"], d["down"], h_scale, status) for d in data]
        gi = [0]

        def block(i):
            d = data[i]
            codes, scales, g = q.quantize_activations(d["x"], scratch=d["sx"])
            return runners[i].run(codes, scales, g, residual=d["res"], chunks=MLP_CHUNKS)

        # one CUDA graph per set (the epochs of pushes and waits are counted on the device, so replays line up across
        # ranks); captured between barriers, since the capture's warm-up run already exchanges data
        graphs = []
        for i in range(MLP_SETS):
            timer.barrier()
            graphs.append(capture(torch, st, lambda i=i: block(i)))
            timer.barrier()

        def one():
            graphs[gi[0] % MLP_SETS].replay()
            gi[0] += 1
        ms = timer.per_call(st, one, steps, 3)
        with torch.cuda.stream(st):
            timer.barrier()
            y = block(0)
            st.synchronize()
            okt = torch.tensor([int(torch.equal(y, data[0]["expected"]) and int(status.item()) == 0)], device=device)
            dist.all_reduce(okt, op=dist.ReduceOp.MIN)
            ok = bool(int(okt.item()))
            timer.barrier()
        exchange = ("NVFP4 intermediate columns and BF16 output columns pushed to every rank with peer-memory stores "
                    f"(q35b_peer_push) + flag waits; one CUDA graph per block")
    token_sharded = None
    if world > 1 and m % (128 * world) == 0:
        # The same block with the TOKENS dealt out instead of the weight rows: every rank keeps whole weights (as
        # the decode replicas do) and runs its M / world rows; nothing is exchanged but the activation's
        # per-tensor scale (one float, here taken from set 0's full activation outside the timed region).
        mr = m // world
        rows = slice(rank * mr, (rank + 1) * mr)
        gen2 = torch.Generator(device=device).manual_seed(77)
        gw = [q.quantize_weight(torch.randn((inter, hidden), generator=gen2, device=device) * 0.02) for _ in range(2)]
        dw = q.quantize_weight(torch.randn((hidden, inter), generator=gen2, device=device) * 0.02)
        host = [(c.cpu().numpy(), s.cpu().numpy(), s2) for (c, s, s2) in gw]
        gu_full = q.Nvfp4Weight.gate_up_from_host(*host[0], *host[1])
        down_full = q.Nvfp4Weight.from_device(dw[0], dw[1], dw[2])
        x_full, res_full = data[0]["x"], data[0]["res"]
        codes, scales, g = q.quantize_activations(x_full, scratch=data[0]["sx"])
        x_scale = float(g.item())
        h = q.gemm_w4a4(gu_full, codes, scales, g, m)
        hs_full = (h.float().abs().max() / (6.0 * 448.0)).reshape(1).to(torch.float32)
        hc, hs, hg = q.gemm_w4a4_gate_up_quant(gu_full, codes, scales, g, m, hs_full)
        expected = q.gemm_w4a4(down_full, hc, hs, hg, m, residual=res_full)[rows].clone()
        del h, hc, hs
        xs_ = [x_full[rows].contiguous()] + [torch.randn((mr, hidden), generator=gen2, device=device).to(torch.bfloat16)
                                              for _ in range(MLP_SETS - 1)]
        rs_ = [res_full[rows].contiguous()] + [torch.randn((mr, hidden), generator=gen2, device=device).to(torch.bfloat16)
                                                for _ in range(MLP_SETS - 1)]
        sxs = [q.act_scratch(mr, hidden, device) for _ in range(MLP_SETS)]
        lay = sharding.MlpLayout(mr, hidden, inter)
        tb = [(torch.empty(mr * lay.codes_ld, dtype=torch.uint8, device=device),
               torch.empty(lay.scales_bytes, dtype=torch.uint8, device=device),
               torch.empty((mr, hidden), dtype=torch.bfloat16, device=device)) for _ in range(MLP_SETS)]

        def tblock(i):
            hc_, hs_, y_ = tb[i]
            c_, s_, g_ = q.quantize_activations(xs_[i], global_scale=x_scale, scratch=sxs[i])
            c2, s2_, g2 = q.gemm_w4a4_gate_up_quant(gu_full, c_, s_, g_, mr, hs_full, scratch=(hc_, hs_, None), status=status)
            q.gemm_w4a4(down_full, c2, s2_, g2, mr, out=y_, status=status, residual=rs_[i])
            return y_
        tgraphs = [capture(torch, st, lambda i=i: tblock(i)) for i in range(MLP_SETS)]
        ti = [0]

        def tone():
            tgraphs[ti[0] % MLP_SETS].replay()
            ti[0] += 1
        tms = timer.per_call(st, tone, steps, 3)
        with torch.cuda.stream(st):
            okt = torch.tensor([int(torch.equal(tblock(0), expected) and int(status.item()) == 0)], device=device)
            st.synchronize()
        dist.all_reduce(okt, op=dist.ReduceOp.MIN)
        token_sharded = {"ms": round(tms, 4), "tflops": round(flops / (tms * 1e-3) / 1e12, 1), "tokens_per_gpu": mr,
                         "exchange": "none: whole weights on every GPU, M / N tokens each, the per-tensor activation "
                                     "scale (one float) agreed beforehand",
                         "checked": bool(int(okt.item())),
                         "check": "rows of this rank torch.equal to the same rows of the unsharded block, on every rank"}
    h_bytes = m * inter * 9 // 16
    out_bytes = m * hidden * 2
    return {"token_sharded": token_sharded,
            "workload": f"prefill MLP block M={m}, hidden {hidden}, intermediate {inter}, N-sharded over {world} GPU(s): "
                        "quantise x, gate/up GEMM writing NVFP4, down GEMM + residual",
            "ms": round(ms, 4), "tflops": round(flops / (ms * 1e-3) / 1e12, 1), "exchange": exchange,
            "gathered_bytes_in_per_gpu": (h_bytes + out_bytes) * (world - 1) // world,
            "gather_us_at_peer_copy_rate": round((h_bytes + out_bytes) * (world - 1) / world / PEER_COPY_GBS / 1e3, 1),
            "checked": ok, "check": "output of set 0 torch.equal to the unsharded block of the same library"
                                    + (", on every rank" if world > 1 else "")}


# --------------------------------------------------------------------------- CPU arms
def cpu_decode_tensors(o, np):
    """One layer of the 0.8B-class step as the CPU arms see it: weights seeded N(0, 0.02) quantised to NVFP4 by the
    oracle's quantiser (the recipe the GPU arm applies to its own seeded weights), BF16 activations N(0, 1)."""
    rng = np.random.default_rng(42)
    tensors = []
    for (n, k) in SHAPES_0P8B:
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        codes, scales, s2 = o.quantize_nvfp4(w)
        xb = o.bf16_round(rng.standard_normal((1, k)).astype(np.float32))
        tensors.append((codes, scales, s2, xb, n, k))
    return tensors


def cpu_decode_sample(o, tensors, layers: int, threads: int, repeats: int = 1):
    """Time the oracle's scalar W4A16 loop on `layers` layers of the decode step; returns (seconds, bytes)."""
    t0 = time.perf_counter()
    for _ in range(repeats):
        for _layer in range(layers):
            for codes, scales, s2, xb, n, k in tensors:
                o.gemv_bf16(codes, scales, s2, xb, threads=threads)
    dt = time.perf_counter() - t0
    nbytes = repeats * layers * sum(algorithmic_bytes(n, k, 1) for n, k in SHAPES_0P8B)
    return dt, nbytes


def cpu_baseline(sample_layers: int) -> dict:
    import numpy as np

    from oracle import q35oracle as o

    threads = host_threads()
    tensors = cpu_decode_tensors(o, np)
    cpu_decode_sample(o, tensors, 1, threads)  # warm the pages
    t_step, _ = cpu_decode_sample(o, tensors, sample_layers, threads)
    repeats = int(max(1, min(40, 10.0 / max(t_step, 1e-9))))  # about ten seconds of CPU work
    dt, nbytes = cpu_decode_sample(o, tensors, sample_layers, threads, repeats=repeats)
    dt1, nbytes1 = cpu_decode_sample(o, tensors, 1, 1)
    return {"value": round(nbytes / dt / 1e9, 4), "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{sample_layers} of 24 layers x {repeats} repeats of the decode step (oracle restatement of "
                      f"cuda_bench.cu:2091-2100, rows split over {threads} threads), {dt:.2f} s",
            "single_thread": {"value": round(nbytes1 / dt1 / 1e9, 4), "unit": "GB/s", "cores": 1,
                              "sample": f"1 layer, {dt1:.2f} s"}}


def cpu_reference_entries(shapes_m):
    """CPU leg of the shape report: the oracle's scalar loop (reference CPU path) on a bounded sample of each shape
    (64 output rows per thread x min(M, 2) tokens), one thread and all threads; the full-shape time is an explicit
    extrapolation."""
    import numpy as np

    from oracle import q35oracle as o

    out = []
    rng = np.random.default_rng(5)
    threads = host_threads()
    for n, k, m in shapes_m:
        rows, toks = min(n, 64 * threads), min(m, 2)
        w = (rng.standard_normal((rows, k)) * 0.02).astype(np.float32)
        codes, scales, s2 = o.quantize_nvfp4(w)
        xb = o.bf16_round(rng.standard_normal((toks, k)).astype(np.float32))
        res = {}
        for t in (1, threads):
            r = min(rows, 64) if t == 1 else rows
            t0 = time.perf_counter()
            o.gemv_bf16(codes[:r], scales[:r], s2, xb, threads=t)
            dt = time.perf_counter() - t0
            res[t] = dt * (n / r) * (m / toks)
        out.append({"N": n, "K": k, "M": m, "cpu_us_1_thread_extrapolated": round(res[1] * 1e6, 1),
                    f"cpu_us_{threads}_threads_extrapolated": round(res[threads] * 1e6, 1), "cores": threads,
                    "sample": f"{rows} rows x {toks} tokens measured, scaled by rows and tokens"})
    return out


def reference_gpu_kernels() -> dict:
    """The reference's own CUDA code on this GPU, through the compiled reference (oracle/_ref): its `scale-group`
    W4A16 kernel (src/runtime/cuda_bench.cu:374-429) on the 96 projections of the 0.8B-class step, launched as its
    benchmark launches it, and its cuBLASLt FP4 prefill bridge (cuda_bench.cu:1056-1167) on the gate+up GEMM.
    Timed with CUDA events on the legacy default stream, which is where the reference launches."""
    try:
        import ctypes as C

        import numpy as np
        import torch

        from oracle import q35oracle as o

        if not torch.cuda.is_available():
            return {"unavailable": "no CUDA device in this process"}
        R = o.ref_lib()
        if R is None:
            return {"unavailable": "the compiled reference (oracle/_ref/libq35ref.so) is not present"}
        torch.cuda.set_device(0)
        rng = np.random.default_rng(42)
        out = {}
        # ---- decode step with the reference's scale-group kernel
        tens = []
        for (n, k) in SHAPES_0P8B:
            w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
            codes, scales, s2 = o.quantize_nvfp4(w)
            tens.append((n, k, s2, codes, scales))
        sets = []
        for _ in range(2):  # two sets of the 96 matrices so that no weight byte is found in L2
            layer = []
            for _l in range(LAYERS_0P8B):
                for (n, k, s2, codes, scales) in tens:
                    layer.append((n, k, s2, torch.from_numpy(codes).cuda(), torch.from_numpy(scales).cuda(),
                                  torch.randn(k, device="cuda"), torch.empty(n, device="cuda")))
            sets.append(layer)

        def step(s):
            for (n, k, s2, dc, ds, dx, dy) in sets[s]:
                if R.ref_w4a16_projection(dc.data_ptr(), ds.data_ptr(), dx.data_ptr(), C.c_float(1.0), C.c_float(s2),
                                          dy.data_ptr(), n, k, 2) != 0:
                    raise RuntimeError(R.ref_last_error().decode())
        for s in (0, 1, 0, 1):
            step(s)
        torch.cuda.synchronize()
        reps = 6
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            step(i % 2)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        step_bytes = LAYERS_0P8B * sum(algorithmic_bytes(n, k, 1) for n, k in SHAPES_0P8B)
        out["decode_step_scale_group"] = {"ms_per_step": round(ms, 4), "GB/s": round(step_bytes / ms / 1e6, 1),
                                          "launches_per_step": 96,
                                          "note": "nvfp4_projection_scale_group_kernel, one launch per projection, fp32 "
                                                  "activations (the reference benchmark's contract)"}
        del sets
        torch.cuda.empty_cache()
        # ---- prefill GEMM through the reference's cuBLASLt bridge
        try:
            n, k = GEMM_SHAPE
            m = GEMM_M
            w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
            codes, scales, s2 = o.quantize_nvfp4(w)
            swapped = ((codes & 0x0F) << 4) | (codes >> 4)
            d_w = torch.from_numpy(swapped).cuda()
            d_ws = torch.from_numpy(o.swizzle_scales(scales)).cuda()
            d_s2 = torch.tensor([s2], dtype=torch.float32, device="cuda")
            x = torch.randn((m, k), device="cuda").to(torch.bfloat16)
            d_ac = torch.zeros(m * k // 2, dtype=torch.uint8, device="cuda")
            d_as = torch.zeros(o.tiled_scale_bytes(m, k // 16), dtype=torch.uint8, device="cuda")
            d_c = torch.empty((m, n), dtype=torch.float32, device="cuda")
            el = C.c_double(0)
            times = []
            for i in range(6):
                torch.cuda.synchronize()
                if R.ref_cublaslt_prefill_bf16(x.data_ptr(), d_w.data_ptr(), d_ws.data_ptr(), d_s2.data_ptr(), m, n, k,
                                               d_ac.data_ptr(), d_as.data_ptr(), d_c.data_ptr(), C.byref(el)) != 0:
                    raise RuntimeError(R.ref_last_error().decode())
                if i >= 2:
                    times.append(el.value)
            ms = statistics.median(times)
            out["prefill_cublaslt"] = {"ms": round(ms, 4), "tflops": round(2.0 * m * n * k / ms / 1e9, 1),
                                       "note": "run_nvfp4_cublaslt_prefill_projection_device_bf16: two memsets, the "
                                               "reference's activation quantiser and cublasLtMatmul (FP4, fp32 output), "
                                               "timed by the reference's own events"}
        except Exception as e:  # noqa: BLE001 - reported, the decode figure stands
            out["prefill_cublaslt"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        return out
    except Exception as e:  # noqa: BLE001 - this leg is an extra; the CPU figure is the arm's value
        return {"unavailable": f"{type(e).__name__}: {e}"[:300]}


def run_reference(args, rank: int) -> dict | None:
    if rank != 0:
        return None
    import numpy as np

    from oracle import q35oracle as o

    threads = host_threads()
    tensors = cpu_decode_tensors(o, np)
    cpu_decode_sample(o, tensors, 1, threads)
    t_layer, _ = cpu_decode_sample(o, tensors, 1, threads)
    # all 24 layers per step unless that would take the whole run beyond about 150 s of CPU time
    layers = int(max(1, min(24, 150.0 / max(t_layer * (args.steps + args.warmup), 1e-9))))
    for _ in range(args.warmup):
        cpu_decode_sample(o, tensors, layers, threads)
    dt = 0.0
    nbytes = 0
    for _ in range(args.steps):
        t, b = cpu_decode_sample(o, tensors, layers, threads)  # times the projection loops only
        dt += t
        nbytes += b
    value = nbytes / dt / 1e9
    sample = (f"each step = {layers} of 24 layers of the decode step on {threads} host threads (oracle port of the "
              f"reference's scalar CPU loop, cuda_bench.cu:2091-2100; the reference itself cannot run its CPU path "
              f"without a GPU); seeded N(0,0.02) weights quantised with the oracle's NVFP4 quantiser")
    return {"impl": "reference", "metric": "nvfp4_decode_step_bandwidth", "value": round(value, 4), "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dt / args.steps * 1e3 * (24 / layers), 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "nvfp4 weights x bf16 activations, fp32 accumulate", "data": "synthetic",
            "config": {"workload": "0.8B-class decode step, M=1 (BASELINE configs[1])"
                                   + ("" if layers == 24 else f"; bounded sample: {layers} of 24 layers per step, ms_per_step scaled to 24"),
                       "parallelism": "host CPU"},
            "cpu_baseline": {"value": round(value, 4), "unit": "GB/s", "cores": threads, "kind": "port",
                             "sample": sample},
            "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "reference_gpu": reference_gpu_kernels() if not args.no_reference_gpu else {"unavailable": "switched off (--no-reference-gpu)"}}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["engine", "reference"], default="engine")
    ap.add_argument("--m", type=int, default=1, choices=range(1, 9), metavar="TOKENS",
                    help="tokens per decode step (1..8); the headline and the driver's runs use 1")
    ap.add_argument("--digits", type=int, default=0,
                    help="decode step on the tensor cores with this many NVFP4 digit rows per token (0: the exact "
                         "BF16-activation kernel)")
    ap.add_argument("--report", default="", help="write the per-shape throughput report (JSON) to this path and exit")
    ap.add_argument("--only", choices=["all", "decode", "gemm"], default="all",
                    help="profiling aid: 'decode' skips the GEMM, the per-projection-launch figure and the CPU "
                         "baseline; 'gemm' shrinks the decode part to its minimum")
    ap.add_argument("--no-reference-gpu", action="store_true",
                    help="reference arm: skip the timing of the reference's own CUDA kernels")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "engine" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.report and world > 1:
        # the prefill cells with M >= 128, N-sharded over the ranks of this torchrun job
        import torch
        import torch.distributed as dist

        import qwen35x_b200 as q
        import shape_report

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        rep = shape_report.run_sharded(q, torch, dist, rank, world, torch.device("cuda", local_rank), peaks())
        bad = [r for r in rep["sharded_prefill"] if not r["checked"]]
        if rank == 0:
            Path(args.report).parent.mkdir(parents=True, exist_ok=True)
            Path(args.report).write_text(json.dumps(rep, indent=1))
            Path(args.report).with_suffix(".md").write_text(shape_report.sharded_to_markdown(rep))
            print(json.dumps({"report": args.report, "gpus": world, "entries": len(rep["sharded_prefill"]), "failed_checks": len(bad)}))
        dist.barrier()
        dist.destroy_process_group()
        return 3 if bad else 0
    if args.report:
        import torch

        import qwen35x_b200 as q
        import shape_report

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
