"""Build the CPU oracle (gcc) and, when a reference checkout is present, the
reference shim (nvcc) into oracle/_ref/.

Test infrastructure only: the product library never depends on anything here.

  python oracle/build_oracle.py            # both (shim skipped without a checkout)

The reference checkout is looked up in $QWEN35X_REFERENCE_ROOT, else in a
directory named `reference` beside this repository.  Its sources are compiled
from where they lie; only binaries are written, and only under oracle/_ref/.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_OUT = HERE / "_ref"
ORACLE_SO = REF_OUT / "libq35oracle.so"
REF_SO = REF_OUT / "libq35ref.so"


def reference_root() -> Path | None:
    env = os.environ.get("QWEN35X_REFERENCE_ROOT")
    root = Path(env) if env else HERE.parent.parent / "reference"
    if (root / "src" / "runtime" / "cuda_bench.cu").is_file():
        return root
    return None


def _stale(out: Path, srcs: list[Path]) -> bool:
    if not out.is_file():
        return True
    t = out.stat().st_mtime
    return any(s.stat().st_mtime > t for s in srcs)


def build_oracle(force: bool = False) -> Path:
    """gcc build of the C restatement; works on any box with gcc."""
    src = HERE / "nvfp4_oracle.c"
    REF_OUT.mkdir(exist_ok=True)
    if force or _stale(ORACLE_SO, [src]):
        cmd = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-shared", "-fPIC",
               "-fvisibility=hidden", "-o", str(ORACLE_SO), str(src), "-lm"]
        subprocess.run(cmd, check=True)
    return ORACLE_SO


def build_reference_shim(force: bool = False) -> Path | None:
    """nvcc build of the reference's cuda_bench.cu behind extern "C" wrappers.
    Returns None when there is no reference checkout (the prebuilt file, if
    any, is left in place and still usable)."""
    root = reference_root()
    if root is None:
        return REF_SO if REF_SO.is_file() else None
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    src = HERE / "ref_shim.cu"
    ref_cu = root / "src" / "runtime" / "cuda_bench.cu"
    REF_OUT.mkdir(exist_ok=True)
    if force or _stale(REF_SO, [src, ref_cu]):
        cmd = [nvcc, "-std=c++20", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
               "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared",
               f"-DQWEN35X_REF_CUDA_BENCH_CU=\"{ref_cu}\"", f"-I{root / 'include'}",
               "-o", str(REF_SO), str(src), "-lcublasLt", "-lcudart"]
        subprocess.run(cmd, check=True)
    return REF_SO


def build_all(force: bool = False) -> dict:
    return {"oracle": build_oracle(force), "reference_shim": build_reference_shim(force)}


if __name__ == "__main__":
    out = build_all(force="--force" in sys.argv)
    for k, v in out.items():
        print(f"{k}: {v}")
