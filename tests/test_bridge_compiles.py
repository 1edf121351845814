"""The binding a maintainer of the reference would add (qwen35x_b200/csrc/host/q35b_bridge.cpp) is compiled, syntax and
types only, against the reference's own headers and include/q35b_nvfp4.h: a drift of either interface fails here.
Skipped where no reference checkout or no CUDA headers are present."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_bridge_compiles_against_reference_headers():
    from oracle.build_oracle import reference_root  # $QWEN35X_REFERENCE_ROOT, else a checkout beside this repository

    REFERENCE = reference_root()
    if REFERENCE is None:
        pytest.skip("needs a reference checkout")
    header = REFERENCE / "include" / "qwen35x" / "runtime" / "cuda_bench.h"
    cuda_inc = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"
    gxx = shutil.which("g++")
    if not header.is_file() or not (cuda_inc / "cuda_runtime.h").is_file() or gxx is None:
        pytest.skip("needs a reference checkout, CUDA headers and g++")
    cmd = [gxx, "-std=c++20", "-fsyntax-only", "-Wall", "-Werror", f"-I{REFERENCE / 'include'}", f"-I{ROOT / 'include'}",
           f"-I{cuda_inc}", str(ROOT / "qwen35x_b200" / "csrc" / "host" / "q35b_bridge.cpp")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-4000:]
