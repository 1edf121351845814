"""libq35b.so loads without a GPU and exports every function include/q35b_nvfp4.h declares."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "q35b_nvfp4.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"Q35B_API\s+[\w\s\*]+?\b(q35b_\w+)\s*\(", text)))


def test_header_lists_functions():
    names = declared_functions()
    assert "q35b_gemv_w4a16_bf16" in names and "q35b_gemm_w4a4_bf16" in names and len(names) >= 20


def test_every_symbol_exported(engine):
    L = engine.lib()
    missing = [n for n in declared_functions() if not hasattr(L, n)]
    assert not missing, missing
    assert b"q35b" in L.q35b_version()


def test_argument_errors_without_gpu(engine):
    L = engine.lib()
    h = ctypes.c_void_p()
    assert L.q35b_weight_create(None, None, 1.0, 1.0, 8, 16, 0, 1, ctypes.byref(h)) == 1
    assert b"null" in L.q35b_last_error()
    buf = (ctypes.c_uint8 * 64)()
    assert L.q35b_weight_create(buf, buf, 1.0, 1.0, 8, 24, 0, 1, ctypes.byref(h)) == 2  # cols % 16 != 0
    assert L.q35b_weight_create(buf, buf, 1.0, 1.0, 8, 16, 3, 2, ctypes.byref(h)) == 1  # bad shard
    assert L.q35b_gemv_w4a16_bf16(None, None, 1, None, -1, None) == 1


def test_shard_ranges(engine):
    for n in (2560, 3584, 18432, 9216, 32768, 100, 129):
        for g in (1, 2, 4, 8):
            spans = [engine.shard_range(n, i, g) for i in range(g)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == n
            for (b0, c0), (b1, _) in zip(spans, spans[1:]):
                assert b0 + c0 == b1
            for b, c in spans[:-1]:
                assert b % 128 == 0
            counts = [c for _, c in spans]
            if n % 128 == 0:
                assert max(counts) - min(counts) <= 128


def test_no_cpu_fallback(engine):
    import torch

    if torch.cuda.is_available():
        return
    import numpy as np
    import pytest

    with pytest.raises(engine.Q35bError):
        engine.Nvfp4Weight.from_host(np.zeros((8, 8), np.uint8), np.zeros((8, 1), np.uint8), 1.0)


def test_shape_report_renders_markdown():
    """The per-shape report's table renderer (no GPU): every section of a report dict appears with its rows."""
    import shape_report

    gemm = {"us": 10.0, "TFLOP/s": 100.0, "fp4_nominal_frac": 0.011, "frac_of_4x_measured_bf16": 0.015}
    report = {
        "peaks": {"hbm_gbs": 6545.0, "bf16_tflops": 1699.0},
        "decode": [{"workload": "step", "M": 1, "projections": 96, "bytes": 234578304, "us": 50.0, "GB/s": 4691.6,
                    "hbm_frac": 0.7168, "kernel": "gemv_w4a16_stream_kernel (work list)"}],
        "single_projection": [{"workload": "one", "M": 1, "N": 3584, "K": 1024, "bytes": 2073604, "us": 5.0, "GB/s": 414.7,
                               "hbm_frac": 0.063, "kernel": "gemv_w4a16_simt_kernel", "l2": "96 weight copies rotated"}],
        "sweep_decode": [],
        "prefill": [{"workload": "gemm", "M": 512, "N": 18432, "K": 2560, "GFLOP": 48.3, "gemm_only": gemm,
                     "quant_gemm": gemm, "kernel": "gemm_w4a4_2cta_kernel"}],
        "sweep_prefill": [],
        "prefill_mlp": [{"workload": "mlp", "M": 4096, "hidden": 2560, "intermediate": 9216, "GFLOP": 579.8,
                         "bf16_intermediate_then_quantise": {"us": 248.3, "TFLOP/s": 2335.1},
                         "nvfp4_intermediate_from_epilogue": {"us": 205.4, "TFLOP/s": 2823.4}}],
        "cpu_reference": [{"N": 3584, "K": 1024, "M": 1, "cpu_us_1_thread_extrapolated": 39418.5,
                           "cpu_us_16_threads_extrapolated": 4599.8, "cores": 16, "sample": "1024 rows"}],
    }
    md = shape_report.to_markdown(report)
    for needle in ("| step | 1 | 96 | 234.6 | 50.00 | 4691.6 | 0.717 | `gemv_w4a16_stream_kernel` |", "| one | 1 | 3584 | 1024 |",
                   "| gemm | 512 | 18432 | 2560 | 48.3 | 10.00 | 100.0 | 0.011 | 0.015 | - | 10.00 | - | `gemm_w4a4_2cta_kernel` |",
                   "| mlp | 4096 | 2560 | 9216 | 579.8 | 248.30 | 2335.1 | 205.40 | 2823.4 |", "| (3584, 1024, 1) | 39418 | 4600 | 16 | 1024 rows |"):
        assert needle in md, needle


def test_sharded_shape_report_renders_markdown():
    """The N-sharded report's table (no GPU): one row per cell with the maximum-over-ranks time and the gather bound."""
    import shape_report

    report = {"peaks": {"hbm_gbs": 6545.0, "bf16_tflops": 1699.0}, "gpus": 4, "sharded_prefill": [
        {"workload": "cell", "M": 4096, "N": 18432, "K": 2560, "GPUs": 4, "rows_of_rank0": 4608, "GFLOP": 386.5,
         "gather_us_at_peer_copy_rate": 147.1, "checked": True,
         "gemm_only": {"us": 33.0, "TFLOP/s": 11712.0, "fp4_nominal_frac": 0.3253},
         "quant_gemm": {"us": 55.0, "TFLOP/s": 7027.0, "fp4_nominal_frac": 0.1952}}]}
    md = shape_report.sharded_to_markdown(report)
    assert "N-sharded over 4 x B200" in md
    assert "| cell | 4096 | 18432 | 2560 | 4608 | 33.00 | 11712.0 | 0.325 | 55.00 | yes | 147.1 |" in md


def test_decode_work_list_plans_without_gpu():
    """The shared-memory plan of the decode work list (host arithmetic): which of the two CTA shapes a list gets and
    how deep its ring is, for the token counts and column counts of the benchmark configurations."""
    import pytest

    from qwen35x_b200 import engine

    # 0.8B-class step (largest K = 3584): two CTAs per SM up to seven tokens, the whole SM for eight
    for m in (1, 2, 3, 4):
        p = engine.gemv_plan(m, 3584)
        assert p["ctas_per_sm"] == 2 and p["ring_stages"] >= 3 and p["smem_bytes"] <= 112 * 1024, (m, p)
    assert engine.gemv_plan(1, 3584)["activation_buffers"] == 2
    p8 = engine.gemv_plan(8, 3584)
    assert p8["ctas_per_sm"] == 1 and p8["ring_stages"] >= 5 and p8["activation_buffers"] == 2 and p8["smem_bytes"] <= 227 * 1024
    # 4B-class step (largest K = 9216): one and two tokens fit half an SM, eight tokens leave the whole SM three stages
    assert engine.gemv_plan(1, 9216)["ctas_per_sm"] == 2
    assert engine.gemv_plan(2, 9216)["ctas_per_sm"] == 2
    p = engine.gemv_plan(8, 9216)
    assert p == {"ctas_per_sm": 1, "ring_stages": 3, "activation_buffers": 1, "smem_bytes": p["smem_bytes"]} and p["smem_bytes"] <= 227 * 1024
    # every plan respects its budget; more tokens never get a deeper ring at the same shape
    for k in (1024, 2560, 4096, 9216):
        last = None
        for m in range(1, 9):
            p = engine.gemv_plan(m, k)
            assert p["smem_bytes"] <= (112 if p["ctas_per_sm"] == 2 else 227) * 1024
            assert p["ring_stages"] >= 3
            if last is not None and last["ctas_per_sm"] == p["ctas_per_sm"] and last["activation_buffers"] == p["activation_buffers"]:
                assert p["ring_stages"] <= last["ring_stages"]
            last = p
    with pytest.raises(engine.Q35bError):
        engine.gemv_plan(9, 1024)
    with pytest.raises(engine.Q35bError):
        engine.gemv_plan(1, 1000)
    with pytest.raises(engine.Q35bError):
        engine.gemv_plan(8, 16384)  # 8 x 16384 fp16 activations do not fit an SM

