"""`bench.py --impl reference`: the reference's CPU implementation of the decode projections (the oracle port) timed
on the host cores.  No GPU involved: alone it prints one JSON line; under torchrun rank 0 prints it and the other
ranks exit 0 without work."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
KEYS = {"impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
        "config", "cpu_baseline", "e2e"}


def _lines(out: str):
    return [json.loads(ln) for ln in out.splitlines() if ln.startswith("{")]


def test_single_process(oracle):
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "1"],
                       capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    (line,) = _lines(r.stdout)
    assert KEYS <= set(line) and line["impl"] == "reference" and line["metric"] == "nvfp4_decode_step_bandwidth"
    assert line["value"] > 0 and line["cpu_baseline"]["kind"] == "port"
    assert line["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))
    assert "unavailable" in line["reference_gpu"] or "decode_step_scale_group" in line["reference_gpu"]
    assert line["e2e"]["value"] == line["value"] and line["e2e"]["h2d_bytes_per_step"] == 0


def test_two_ranks_only_rank_zero_reports(oracle):
    # torch.distributed.run sets OMP_NUM_THREADS=1 for its workers: the arm must not take its thread count from there
    env = dict(os.environ)
    env.pop("OMP_NUM_THREADS", None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29641", str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = _lines(r.stdout)
    assert len(lines) == 1 and lines[0]["impl"] == "reference" and lines[0]["n_gpus"] == 2
    assert lines[0]["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))
