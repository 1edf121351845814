"""Per-shape throughput report of the NVFP4 projection path on one GPU.

Covers the named shapes of the benchmark configurations: the single 0.8B gate_proj projection, the 0.8B and 4B-class
decode steps at M = 1, 2, 4, 8 (work-list launch), the 4B-class prefill GEMMs at M = 512 and 4096 (GEMM alone and
activation quantisation + GEMM), the 4B-class prefill MLP block with and without the NVFP4-writing gate/up epilogue, and the (K, N) x M sweep with 1 % of weight rows scaled x8.  Every entry gives
microseconds, GB/s of algorithmic bytes (decode) or TFLOP/s (prefill), and the fraction of the HBM or FP4-tensor
roofline.  Inputs are seeded synthetic tensors quantised on the GPU; weights are rotated through enough copies that
no launch finds its operands in L2.

    python bench.py --report shape_report.json
"""
from __future__ import annotations

import json
import statistics

L2_BYTES = 126 * 1024 * 1024
FP4_NOMINAL_TFLOPS = 9000.0


def _alg_bytes(n, k, m):
    return n * k // 2 + n * k // 16 + m * k * 2 + m * n * 2 + 4


def _copies_for(nbytes: int, limit: int = 96) -> int:
    return max(2, min(limit, -(-int(1.5 * L2_BYTES) // max(nbytes, 1))))


def _make_weight(q, torch, device, gen, n, k, row_outliers=False):
    w = torch.randn((n, k), generator=gen, device=device, dtype=torch.float32) * 0.02
    if row_outliers:
        idx = torch.randperm(n, generator=gen, device=device)[: max(1, -(-n // 100))]
        w[idx] *= 8.0
    codes, scales, s2 = q.quantize_weight(w)
    return codes, scales, s2


def _time_graphs(torch, stream, graphs, reps: int) -> float:
    """Median microseconds per replay, cycling through `graphs`, CUDA events on the launching stream."""
    with torch.cuda.stream(stream):
        for i in range(max(3, len(graphs))):
            graphs[i % len(graphs)].replay()
        stream.synchronize()
        times = []
        for block in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(reps):
                graphs[(block * reps + i) % len(graphs)].replay()
            e1.record(stream)
            stream.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3 / reps)
    return statistics.median(times)


def _time_launches(torch, stream, fns, reps: int) -> float:
    """Median microseconds per call, cycling through `fns` as back-to-back launches on `stream` (the work-list kernel
    is launched with programmatic stream serialisation, so consecutive launches overlap head and tail)."""
    with torch.cuda.stream(stream):
        for i in range(max(3, len(fns))):
            fns[i % len(fns)]()
        stream.synchronize()
        times = []
        for block in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(reps):
                fns[(block * reps + i) % len(fns)]()
            e1.record(stream)
            stream.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3 / reps)
    return statistics.median(times)


def _capture(torch, stream, fn):
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
    return g


def decode_entries(q, torch, device, peaks, shapes, layers, ms, label, row_outliers=False):
    """Work-list launch over `layers` x `shapes` projections for every M in `ms`."""
    out = []
    gen = torch.Generator(device=device).manual_seed(4242)
    step_weight_bytes = layers * sum(n * k // 2 + n * k // 16 for n, k in shapes)
    sets = 2 if step_weight_bytes < 2 * L2_BYTES else 1
    weights = []
    for _ in range(sets):
        ws = []
        for _layer in range(layers):
            for n, k in shapes:
                codes, scales, s2 = _make_weight(q, torch, device, gen, n, k, row_outliers)
                ws.append(q.Nvfp4Weight.from_device(codes, scales, s2))
                del codes, scales
        weights.append(ws)
    stream = torch.cuda.Stream(device=device)
    for m in ms:
        xs = [torch.randn((m, k), generator=gen, device=device).to(torch.bfloat16) for _ in range(layers) for _, k in shapes]
        ys = [torch.empty((m, n), dtype=torch.bfloat16, device=device) for _ in range(layers) for n, _ in shapes]
        kernel = "gemv_w4a16_stream_kernel (work list)"
        graphs = None
        try:
            batches = [q.GemvBatch(list(zip(ws, xs, ys)), m) for ws in weights]
        except q.Q35bError as e:
            # activations too large for the streaming kernel's shared memory: per-projection SIMT launches
            kernel = f"gemv_w4a16_simt_kernel per projection ({e})"
            batches = []

            def run_set(ws):
                for w, x, y in zip(ws, xs, ys):
                    q.gemv_w4a16(w, x, out=y, kernel=q.GEMV_SIMT)

            graphs = [_capture(torch, stream, lambda ws=ws: run_set(ws)) for ws in weights]
        if graphs is None:
            us = _time_launches(torch, stream, [b.run for b in batches], reps=20)
        else:
            us = _time_graphs(torch, stream, graphs, reps=10)
        nbytes = layers * sum(_alg_bytes(n, k, m) for n, k in shapes)
        gbs = nbytes / us / 1e3
        for b in batches:
            if b.status() != 0:
                raise RuntimeError(f"device-side wait expired, code {b.status()}")
        out.append({"workload": label, "M": m, "projections": layers * len(shapes), "bytes": nbytes, "us": round(us, 2),
                    "GB/s": round(gbs, 1), "hbm_frac": round(gbs / peaks["hbm_gbs"], 4), "kernel": kernel})
        del batches, graphs
    return out


def single_projection_entries(q, torch, device, peaks, n, k, ms, label, row_outliers=False):
    """One projection per launch: SIMT and streaming kernels, weights rotated through > L2 worth of copies."""
    out = []
    gen = torch.Generator(device=device).manual_seed(99)
    wbytes = n * k // 2 + n * k // 16
    copies = _copies_for(wbytes)
    codes, scales, s2 = _make_weight(q, torch, device, gen, n, k, row_outliers)
    weights = [q.Nvfp4Weight.from_device(codes, scales, s2) for _ in range(copies)]
    stream = torch.cuda.Stream(device=device)
    for m in ms:
        x = torch.randn((m, k), generator=gen, device=device).to(torch.bfloat16)
        y = torch.empty((m, n), dtype=torch.bfloat16, device=device)
        for kernel, name in ((q.GEMV_SIMT, "gemv_w4a16_simt_kernel"), (q.GEMV_STREAM, "gemv_w4a16_stream_kernel")):
            try:
                graphs = [_capture(torch, stream, lambda w=w: q.gemv_w4a16(w, x, out=y, kernel=kernel)) for w in weights]
            except q.Q35bError:
                continue
            us = _time_graphs(torch, stream, graphs, reps=copies)
            nbytes = _alg_bytes(n, k, m)
            gbs = nbytes / us / 1e3
            out.append({"workload": label, "M": m, "N": n, "K": k, "bytes": nbytes, "us": round(us, 2),
                        "GB/s": round(gbs, 1), "hbm_frac": round(gbs / peaks["hbm_gbs"], 4), "kernel": name,
                        "l2": f"{copies} weight copies rotated"})
    return out


def _check_gemm_rows(torch, w, codes, scales, s2, a_codes, a_scales, g, m, k, y, rows=8):
    """A few output rows of one timed cell against the CPU oracle (relative L2 <= 1e-3), outside the timed region."""
    import numpy as np

    from oracle import q35oracle as o

    idx = torch.randperm(codes.shape[0], device=codes.device)[:rows].sort().values
    r = np.arange(m)[:, None]
    c = np.arange(k // 16)[None, :]
    slots = (k // 16 + 3) // 4 * 4
    tiled = a_scales.cpu().numpy()
    a_s = tiled[(((r // 128) * (slots // 4) + c // 4) * 32 + (r % 32)) * 16 + ((r % 128) // 32) * 4 + (c % 4)]
    eb, _ = o.gemm_w4a4(codes[idx].cpu().numpy(), scales[idx].cpu().numpy(), s2, a_codes.cpu().numpy(), a_s, float(g.item()),
                        threads=8)
    got = y[:, idx].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    return bool(o.rel_l2(o.bf16_to_f32(got), o.bf16_to_f32(eb)) <= 1e-3)


def gemm_entries(q, torch, device, peaks, n, k, ms, label, row_outliers=False):
    out = []
    gen = torch.Generator(device=device).manual_seed(7 + n + k)
    stream = torch.cuda.Stream(device=device)
    for m in ms:
        per_set = n * k * 9 // 16 + m * k * 9 // 16 + m * n * 2
        sets = max(2, min(6, -(-int(1.3 * L2_BYTES) // per_set)))
        data = []
        checked = None
        for i in range(sets):
            codes, scales, s2 = _make_weight(q, torch, device, gen, n, k, row_outliers)
            w = q.Nvfp4Weight.from_device(codes, scales, s2)
            x = torch.randn((m, k), generator=gen, device=device)
            x[:, torch.randperm(k, generator=gen, device=device)[: max(1, -(-k // 1000))]] *= 20.0
            x = x.to(torch.bfloat16)
            scratch = q.act_scratch(m, k, device)
            y = torch.empty((m, n), dtype=torch.bfloat16, device=device)
            q.project_prefill(w, x, out=y, scratch=scratch)
            if i == 0:
                torch.cuda.synchronize()
                checked = _check_gemm_rows(torch, w, codes, scales, s2, scratch[0].view(m, k // 2), scratch[1], scratch[2], m, k, y)
            del codes, scales
            data.append((w, x, scratch, y))
        torch.cuda.synchronize()

        def gemm_only(d):
            w, x, scratch, y = d
            q.gemm_w4a4(w, scratch[0].view(m, k // 2), scratch[1], scratch[2], m, out=y)

        def quant_gemm(d):
            w, x, scratch, y = d
            q.project_prefill(w, x, out=y, scratch=scratch)

        flops = 2.0 * m * n * k
        row = {"workload": label, "M": m, "N": n, "K": k, "GFLOP": round(flops / 1e9, 1), "l2": f"{sets} operand sets rotated",
               "checked": checked}
        alg_bytes = n * k * 9 // 16 + m * k * 9 // 16 + m * n * 2
        for name, fn in (("gemm_only", gemm_only), ("quant_gemm", quant_gemm)):
            graphs = [_capture(torch, stream, lambda d=d: fn(d)) for d in data]
            us = _time_graphs(torch, stream, graphs, reps=sets * 2)
            tf = flops / us / 1e6
            row[name] = {"us": round(us, 2), "TFLOP/s": round(tf, 1), "fp4_nominal_frac": round(tf / FP4_NOMINAL_TFLOPS, 4),
                         "frac_of_4x_measured_bf16": round(tf / (4 * peaks["bf16_tflops"]), 4)}
            if m <= 128 and name == "gemm_only":
                # few tokens: the weight stream bounds the cell, not the tensor pipe
                row[name]["hbm_frac"] = round(alg_bytes / us / 1e3 / peaks["hbm_gbs"], 4)
        row["kernel"] = ("gemm_w4a4_2cta_kernel" if (m >= 256 and n >= 192) else
                         "gemm_wstream_kernel" if (m <= 32 and not ((n + 127) // 128 < 24 and k // 256 > 16)) else "gemm_w4a4_tcgen05_kernel")
        out.append(row)
        del data
        torch.cuda.empty_cache()
    return out


def sharded_gemm_entries(q, torch, dist, rank, world, device, peaks, n, k, ms, label, row_outliers=False):
    """Prefill cells N-sharded over the ranks of a torchrun job (one process per GPU): every rank builds the same seeded
    weight, keeps the rows q35b_shard_range gives it, quantises the replicated activations itself and computes its
    columns.  Times are the maximum over ranks; TFLOP/s is the whole projection's FLOPs over that time.  The
    exchange that would follow is not part of the cell (bench.py times it on the gate/up shape): its lower bound,
    the bytes every rank takes in at the measured peer-copy rate, is printed beside the compute time."""
    from qwen35x_b200 import sharding

    out = []
    stream = torch.cuda.Stream(device=device)
    row_begin, row_count = sharding.shard_layout(n, world)[rank]
    for m in ms:
        gen = torch.Generator(device=device).manual_seed(7 + n + k + m)  # the same tensors on every rank
        per_set = (n // world) * k * 9 // 16 + m * k * 9 // 16 + m * (n // world) * 2
        sets = max(2, min(6, -(-int(1.3 * L2_BYTES) // per_set)))
        data = []
        checked = True
        for i in range(sets):
            codes, scales, s2 = _make_weight(q, torch, device, gen, n, k, row_outliers)
            w = q.Nvfp4Weight.from_device(codes, scales, s2, shard_index=rank, shard_count=world)
            x = torch.randn((m, k), generator=gen, device=device)
            x[:, torch.randperm(k, generator=gen, device=device)[: max(1, -(-k // 1000))]] *= 20.0
            x = x.to(torch.bfloat16)
            scratch = q.act_scratch(m, k, device)
            y = torch.empty((m, max(row_count, 1)), dtype=torch.bfloat16, device=device)
            if row_count > 0:
                q.project_prefill(w, x, out=y, scratch=scratch)
            if i == 0 and row_count > 0:
                torch.cuda.synchronize()
                sl = slice(row_begin, row_begin + row_count)
                checked = _check_gemm_rows(torch, w, codes[sl], scales[sl], s2, scratch[0].view(m, k // 2), scratch[1],
                                           scratch[2], m, k, y)
            del codes, scales
            data.append((w, x, scratch, y))
        torch.cuda.synchronize()

        def gemm_only(d):
            w, x, scratch, y = d
            if row_count > 0:
                q.gemm_w4a4(w, scratch[0].view(m, k // 2), scratch[1], scratch[2], m, out=y)

        def quant_gemm(d):
            w, x, scratch, y = d
            if row_count > 0:
                q.project_prefill(w, x, out=y, scratch=scratch)

        flops = 2.0 * m * n * k
        gather_in = m * (n - row_count) * 2
        row = {"workload": label, "M": m, "N": n, "K": k, "GPUs": world, "rows_of_rank0": sharding.shard_layout(n, world)[0][1],
               "GFLOP": round(flops / 1e9, 1),
               "gather_us_at_peer_copy_rate": round(gather_in / 770e9 * 1e6, 1)}
        for name, fn in (("gemm_only", gemm_only), ("quant_gemm", quant_gemm)):
            graphs = [_capture(torch, stream, lambda d=d: fn(d)) for d in data]
            dist.barrier()
            us = _time_graphs(torch, stream, graphs, reps=sets * 2)
            t = torch.tensor([us], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            us = float(t.item())
            tf = flops / us / 1e6
            row[name] = {"us": round(us, 2), "TFLOP/s": round(tf, 1),
                         "fp4_nominal_frac": round(tf / (world * FP4_NOMINAL_TFLOPS), 4)}
        ok = torch.tensor([1 if checked else 0], dtype=torch.int32, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        row["checked"] = bool(ok.item())
        out.append(row)
        del data
        torch.cuda.empty_cache()
    return out


def run_sharded(q, torch, dist, rank, world, device, peaks) -> dict:
    """The prefill cells with M >= 128 of the 4B-class prefill and of the sweep, N-sharded over `world` GPUs."""
    report = {"peaks": peaks, "gpus": world, "sharded_prefill": []}
    for (n, k) in ((18432, 2560), (2560, 9216)):
        report["sharded_prefill"] += sharded_gemm_entries(q, torch, dist, rank, world, device, peaks, n, k, [512, 4096],
                                                          "config 4: 4B-class prefill")
    for (n, k) in ((3584, 1024), (9216, 2560), (2560, 9216), (32768, 2560)):
        report["sharded_prefill"] += sharded_gemm_entries(q, torch, dist, rank, world, device, peaks, n, k, [128, 1024, 4096],
                                                          "config 5 sweep (1% rows x8)", row_outliers=True)
    return report


def sharded_to_markdown(report: dict) -> str:
    w = report["gpus"]
    out = [f"# Per-shape throughput report, prefill cells N-sharded over {w} x B200", "",
           f"Command: `python -m torch.distributed.run --nproc-per-node {w} --master-addr 127.0.0.1 bench.py --gpus {w} "
           "--report <path>.json` (CUDA-graph replays over rotating operand sets, CUDA events, maximum over ranks; every "
           "rank checks sampled rows of its shard against the CPU port). TFLOP/s = FLOPs of the whole projection / that "
           f"time; fraction of {w} x 9000 TFLOP/s nominal dense FP4. Activations are replicated and quantised on every "
           "rank. The exchange is not in these cells: the last column is what taking in the other ranks' BF16 columns "
           "costs at the measured 770 GB/s peer-copy rate.", "",
           "| workload | M | N | K | rows per rank | shard GEMM us (max) | TFLOP/s | of nominal | quantise+GEMM us | checked | "
           "BF16 gather at peer-copy rate us |", "|---|---|---|---|---|---|---|---|---|---|---|"]
    for r in report["sharded_prefill"]:
        g, qg = r["gemm_only"], r["quant_gemm"]
        out.append(f"| {r['workload']} | {r['M']} | {r['N']} | {r['K']} | {r['rows_of_rank0']} | {g['us']:.2f} | {g['TFLOP/s']:.1f} | "
                   f"{g['fp4_nominal_frac']:.3f} | {qg['us']:.2f} | {'yes' if r['checked'] else 'NO'} | "
                   f"{r['gather_us_at_peer_copy_rate']:.1f} |")
    return "\n".join(out) + "\n"


def mlp_entries(q, torch, device, peaks, hidden, inter, ms, label):
    """Prefill MLP block x -> down(silu(gate x) * up x) + residual: the chain with the gate/up GEMM writing BF16 and a
    separate quantise pass before the down projection, and the chain whose gate/up epilogue writes NVFP4 directly."""
    out = []
    gen = torch.Generator(device=device).manual_seed(31)
    stream = torch.cuda.Stream(device=device)
    for m in ms:
        per_set = (3 * hidden * inter) * 9 // 16 + m * inter * 2 + 3 * m * hidden * 2
        sets = max(2, min(6, -(-int(1.3 * L2_BYTES) // per_set)))
        data = []
        for _ in range(sets):
            g_c, g_s, g_s2 = _make_weight(q, torch, device, gen, inter, hidden)
            u_c, u_s, u_s2 = _make_weight(q, torch, device, gen, inter, hidden)
            gu = q.Nvfp4Weight.gate_up_from_host(g_c.cpu().numpy(), g_s.cpu().numpy(), float(g_s2), u_c.cpu().numpy(),
                                                 u_s.cpu().numpy(), float(u_s2))
            d_c, d_s, d_s2 = _make_weight(q, torch, device, gen, hidden, inter)
            down = q.Nvfp4Weight.from_device(d_c, d_s, d_s2)
            del g_c, g_s, u_c, u_s, d_c, d_s
            x = torch.randn((m, hidden), generator=gen, device=device).to(torch.bfloat16)
            res = torch.randn((m, hidden), generator=gen, device=device).to(torch.bfloat16)
            sx = q.act_scratch(m, hidden, device)
            sh = q.act_scratch(m, inter, device)
            h = torch.empty((m, inter), dtype=torch.bfloat16, device=device)
            y = torch.empty((m, hidden), dtype=torch.bfloat16, device=device)
            # calibrate the intermediate activation's scale once
            q.project_prefill(gu, x, out=h, scratch=sx)
            h_scale = (h.float().abs().max() / (6.0 * 448.0)).reshape(1).to(torch.float32)
            data.append((gu, down, x, res, sx, sh, h, y, h_scale))
        torch.cuda.synchronize()

        def two_pass(d):
            gu, down, x, res, sx, sh, h, y, h_scale = d
            q.project_prefill(gu, x, out=h, scratch=sx)
            q.project_prefill(down, h, out=y, scratch=sh, residual=res)

        def fused(d):
            gu, down, x, res, sx, sh, h, y, h_scale = d
            codes, scales, g = q.quantize_activations(x, scratch=sx)
            hc, hs, hg = q.gemm_w4a4_gate_up_quant(gu, codes, scales, g, m, h_scale, scratch=sh)
            q.gemm_w4a4(down, hc, hs, hg, m, out=y, residual=res)

        flops = 2.0 * m * hidden * inter * 3
        row = {"workload": label, "M": m, "hidden": hidden, "intermediate": inter, "GFLOP": round(flops / 1e9, 1),
               "l2": f"{sets} weight/activation sets rotated"}
        for name, fn in (("bf16_intermediate_then_quantise", two_pass), ("nvfp4_intermediate_from_epilogue", fused)):
            graphs = [_capture(torch, stream, lambda d=d: fn(d)) for d in data]
            us = _time_graphs(torch, stream, graphs, reps=sets * 2)
            row[name] = {"us": round(us, 2), "TFLOP/s": round(flops / us / 1e6, 1)}
        out.append(row)
        del data
        torch.cuda.empty_cache()
    return out


def run(path: str, q, torch, device, peaks) -> dict:
    shapes_0p8b = [(4096, 1024), (1024, 2048), (7168, 1024), (1024, 3584)]
    shapes_4b = [(18432, 2560), (2560, 9216), (10240, 2560), (2560, 4096)]
    sweep = [(3584, 1024), (9216, 2560), (2560, 9216), (32768, 2560)]  # (N, K)
    report = {"peaks": peaks, "decode": [], "single_projection": [], "prefill": [], "prefill_mlp": [], "sweep_decode": [],
              "sweep_prefill": []}
    report["single_projection"] += single_projection_entries(q, torch, device, peaks, 3584, 1024, [1],
                                                             "config 1: 0.8B gate_proj, single projection")
    report["decode"] += decode_entries(q, torch, device, peaks, shapes_0p8b, 24, [1, 2, 4, 8], "config 2: 0.8B-class decode step")
    report["decode"] += decode_entries(q, torch, device, peaks, shapes_4b, 32, [1, 2, 4, 8], "config 3: 4B-class decode step")
    torch.cuda.empty_cache()
    for n, k in ((18432, 2560), (2560, 9216)):
        report["prefill"] += gemm_entries(q, torch, device, peaks, n, k, [512, 4096], "config 4: 4B-class prefill")
    report["prefill_mlp"] += mlp_entries(q, torch, device, peaks, 2560, 9216, [512, 4096], "4B-class prefill MLP block")
    for n, k in sweep:
        report["sweep_decode"] += single_projection_entries(q, torch, device, peaks, n, k, [1], "config 5 sweep (1% rows x8)",
                                                            row_outliers=True)
        report["sweep_prefill"] += gemm_entries(q, torch, device, peaks, n, k, [16, 128, 1024, 4096],
                                                "config 5 sweep (1% rows x8)", row_outliers=True)
    if path:
        with open(path, "w") as f:
            json.dump(report, f, indent=1)
    return report


def to_markdown(report: dict) -> str:
    """The report as the tables kept under profiles/ (written next to the JSON by `bench.py --report`)."""
    pk = report["peaks"]
    out = ["# Per-shape throughput report (1 x B200)", "",
           "Command: `python bench.py --report <path>.json` (decode work lists as back-to-back launches, everything else "
           "as CUDA-graph replays; CUDA events on the launching stream, "
           "median of 5 blocks; weights/operands rotated through more than L2-size worth of copies; synthetic seeded "
           f"tensors quantised on the GPU). Peaks: measured HBM copy {pk['hbm_gbs']:.0f} GB/s; FP4 tensor: nominal "
           f"{FP4_NOMINAL_TFLOPS:.0f} TFLOP/s dense (no measured FP4 peak exists; 4 x measured BF16 burst = "
           f"{4 * pk['bf16_tflops']:.0f} TFLOP/s is shown beside it).", ""]

    def decode_table(title, rows, shape_cols):
        out.extend([f"## {title}", ""])
        head = ["workload", "M"] + (["N", "K"] if shape_cols else ["projections"]) + ["MB", "us", "GB/s", "of HBM peak", "kernel"]
        out.append("| " + " | ".join(head) + " |")
        out.append("|" + "---|" * len(head))
        for r in rows:
            mid = [str(r["N"]), str(r["K"])] if shape_cols else [str(r["projections"])]
            out.append("| " + " | ".join([r["workload"], str(r["M"])] + mid + [f"{r['bytes'] / 1e6:.1f}", f"{r['us']:.2f}",
                                          f"{r['GB/s']:.1f}", f"{r['hbm_frac']:.3f}", "`" + r["kernel"].split(" ")[0] + "`"]) + " |")
        out.append("")

    def gemm_table(title, rows):
        out.extend([f"## {title}", ""])
        head = ["workload", "M", "N", "K", "GFLOP", "GEMM us", "TFLOP/s", "of 9 PF nominal", "of 4xBF16 measured",
                "of HBM peak (M<=128)", "quantise+GEMM us", "checked", "kernel"]
        out.append("| " + " | ".join(head) + " |")
        out.append("|" + "---|" * len(head))
        for r in rows:
            g, qg = r["gemm_only"], r["quant_gemm"]
            out.append("| " + " | ".join([r["workload"], str(r["M"]), str(r["N"]), str(r["K"]), str(r["GFLOP"]), f"{g['us']:.2f}",
                                          f"{g['TFLOP/s']:.1f}", f"{g['fp4_nominal_frac']:.3f}", f"{g['frac_of_4x_measured_bf16']:.3f}",
                                          f"{g['hbm_frac']:.3f}" if "hbm_frac" in g else "-",
                                          f"{qg['us']:.2f}", {True: "yes", False: "NO", None: "-"}[r.get("checked")],
                                          "`" + r["kernel"] + "`"]) + " |")
        out.append("")

    decode_table("Decode (W4A16, one work-list launch over all projections of a step)", report["decode"], False)
    decode_table("Single projection per launch (decode)", report["single_projection"] + report["sweep_decode"], True)
    gemm_table("Prefill (W4A4 tcgen05 GEMM)", report["prefill"] + report["sweep_prefill"])
    if report.get("prefill_mlp"):
        out.extend(["## Prefill MLP block: down(silu(gate x) * up x) + residual", "",
                    "| workload | M | hidden | intermediate | GFLOP | BF16 intermediate + quantise pass us | TFLOP/s | "
                    "NVFP4 intermediate from the gate/up epilogue us | TFLOP/s |", "|" + "---|" * 9])
        for r in report["prefill_mlp"]:
            a, b = r["bf16_intermediate_then_quantise"], r["nvfp4_intermediate_from_epilogue"]
            out.append(f"| {r['workload']} | {r['M']} | {r['hidden']} | {r['intermediate']} | {r['GFLOP']} | {a['us']:.2f} | "
                       f"{a['TFLOP/s']:.1f} | {b['us']:.2f} | {b['TFLOP/s']:.1f} |")
        out.append("")
    if report.get("cpu_reference"):
        out.extend(["## Reference CPU path (oracle port of the scalar loop), same box", "",
                    "| shape (N, K, M) | 1 thread us (extrapolated) | all threads us (extrapolated) | cores | sample |",
                    "|---|---:|---:|---:|---|"])
        for r in report["cpu_reference"]:
            allk = [k for k in r if k.startswith("cpu_us_") and not k.startswith("cpu_us_1_")][0]
            out.append(f"| ({r['N']}, {r['K']}, {r['M']}) | {r['cpu_us_1_thread_extrapolated']:.0f} | {r[allk]:.0f} | {r['cores']} | {r['sample']} |")
        out.append("")
    return "\n".join(out)
