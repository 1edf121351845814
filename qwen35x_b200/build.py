"""Build libq35b.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m qwen35x_b200.build [--force] [--verbose]

The library links the CUDA runtime statically and resolves the few driver
entry points it needs at run time, so it loads on a machine without a GPU
(every compute call then fails with Q35B_ERR_CUDA)."""
from __future__ import annotations

import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "_lib"
LIB = LIB_DIR / "libq35b.so"
CLI = LIB_DIR / "q35b"

SOURCES = ["api.cu", "gemv_w4a16.cu", "gemv_stream.cu", "act_quant.cu", "gemm_w4a4_tcgen05.cu", "gemm_w4a4_2cta.cu", "gemm_wstream.cu", "static_prefill.cu", "peer_gather.cu"]
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-O2", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _stale(out: Path, deps: list[Path]) -> bool:
    if not out.is_file():
        return True
    t = out.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    LIB_DIR.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "q35b_nvfp4.h"]
    objs = []
    procs = []
    for name in SOURCES:
        src = CSRC / name
        obj = LIB_DIR / (src.stem + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            procs.append((name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for name, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            print(f"--- {name}\n{out}")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or not LIB.is_file():
        cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static", "-lpthread", "-ldl"]
        subprocess.run(cmd, check=True)
    build_cli(force=force or bool(procs))
    return LIB


def build_cli(force: bool = False) -> Path:
    """The C++ host mirror of the reference entry points and its command line (qwen35x_b200/_lib/q35b)."""
    host = CSRC / "host"
    srcs = [host / "nvfp4_runtime.cpp", host / "nvfp4_checkpoint.cpp", host / "q35b_main.cpp"]
    deps = srcs + [host / "nvfp4_runtime.h", host / "nvfp4_checkpoint.h", CSRC / "nvfp4_codec.cuh", PKG.parent / "include" / "q35b_nvfp4.h", LIB]
    if force or _stale(CLI, deps):
        cmd = [_nvcc(), "-std=c++17", "-O2", "-x", "cu", "-gencode", "arch=compute_100a,code=sm_100a", *map(str, srcs),
               "-o", str(CLI), f"-L{LIB_DIR}", "-lq35b", "-Xlinker", "-rpath,$ORIGIN", "-cudart", "static"]
        subprocess.run(cmd, check=True)
    return CLI


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
