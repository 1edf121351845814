"""Generate tests/golden/nvfp4_golden.npz from the reference itself.

Needs a reference checkout (see oracle/build_oracle.py): the reference's own
host codecs, encoders and layout helpers are called through oracle/_ref's shim,
and the two composite fixtures (a W4A16 projection and the cuBLASLt-recipe
activation quantisation of the reference's fixed input) are assembled in numpy
fp32 from those reference functions, following the loops at
src/runtime/cuda_bench.cu:2085-2100 and :2221-2235.

    python tests/golden/make_golden.py
"""
from __future__ import annotations

import ctypes as C
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))

from oracle import q35oracle as o  # noqa: E402


def main() -> None:
    R = o.ref_lib()
    if R is None:
        raise SystemExit("no reference checkout: cannot regenerate the golden vectors")
    rng = np.random.default_rng(20240607)
    f32 = np.float32

    e4m3_table = np.array([R.ref_decode_e4m3(i) for i in range(256)], dtype=f32)
    e2m1_table = np.array([R.ref_decode_e2m1(i) for i in range(16)], dtype=f32)

    # encoder inputs: every representable value, every midpoint, +-1 ulp around both, and random magnitudes
    pos = np.unique(np.abs(e4m3_table))
    mids = (pos[:-1] + pos[1:]) / 2
    pts = np.concatenate([pos, mids]).astype(f32)
    around = np.concatenate([pts, np.nextafter(pts, f32(np.inf)), np.nextafter(pts, f32(-np.inf))])
    rand = np.concatenate([np.abs(rng.standard_normal(4000)).astype(f32) * s for s in (1e-3, 1e-1, 1.0, 30.0, 600.0)])
    special = np.array([0.0, -1.0, 1e-8, 1e-30, 463.99, 464.0, 464.01, 480.0, 495.9, 496.0, 1e4, 1e9, 3e38, np.inf,
                        -np.inf, np.nan], dtype=f32)
    ue4m3_in = np.concatenate([around, rand, special]).astype(f32)
    ue4m3_out = np.array([R.ref_encode_ue4m3(float(v)) for v in ue4m3_in], dtype=np.uint8)

    lv = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], dtype=f32)
    lmid = (lv[:-1] + lv[1:]) / 2
    pts = np.concatenate([lv, lmid]).astype(f32)
    around = np.concatenate([pts, np.nextafter(pts, f32(np.inf)), np.nextafter(pts, f32(-np.inf))])
    around = np.concatenate([around, -around])
    rand = (rng.standard_normal(8000) * 2.5).astype(f32)
    special = np.array([0.0, -0.0, 7.0, -7.0, 100.0, -1e6, 1e30, np.inf, -np.inf, np.nan], dtype=f32)
    e2m1_in = np.concatenate([around, rand, special]).astype(f32)
    e2m1_out = np.array([R.ref_encode_e2m1(float(v)) for v in e2m1_in], dtype=np.uint8)

    # layout helpers
    sw_in = rng.integers(0, 127, size=(130, 9), dtype=np.uint8)
    sw_out = np.zeros(256 * 12, dtype=np.uint8)
    n = R.ref_swizzle_scales(sw_in.ctypes.data, 130, 9, sw_out.ctypes.data, sw_out.size)
    assert n == sw_out.size
    nib_in = rng.integers(0, 256, size=64, dtype=np.uint8)
    nib_out = np.zeros_like(nib_in)
    R.ref_swap_nibbles(nib_in.ctypes.data, nib_in.size, nib_out.ctypes.data)

    # composite 1: W4A16 projection of the reference's fixed input x[i] = ((i%17)-8)/17 (cuda_bench.cu:2085-2100)
    rows, cols = 24, 256
    codes = rng.integers(0, 256, size=(rows, cols // 2), dtype=np.uint8)
    scales = rng.integers(0x20, 0x58, size=(rows, cols // 16), dtype=np.uint8)
    s2, input_scale = f32(3.1e-4), f32(0.75)
    x = np.array([f32((i % 17) - 8) / f32(17.0) for i in range(cols)], dtype=f32)
    y = np.zeros(rows, dtype=f32)
    for r in range(rows):
        acc = f32(0)
        for c in range(cols):
            p = codes[r, c // 2]
            nib = (p & 0xF) if (c & 1) == 0 else (p >> 4)
            scale = f32(e4m3_table[scales[r, c // 16]] * s2)
            acc = f32(acc + f32(f32(e2m1_table[nib] * scale) * f32(x[c] * input_scale)))
        y[r] = acc

    # composite 2: cuBLASLt-recipe activation quantisation of the same input (cuda_bench.cu:2221-2237)
    kq = 1024
    xq = np.array([f32((i % 17) - 8) / f32(17.0) for i in range(kq)], dtype=f32)
    q_codes = np.zeros(kq // 2, dtype=np.uint8)
    q_scales = np.zeros(kq // 16, dtype=np.uint8)
    for g in range(kq // 16):
        blk = xq[g * 16:(g + 1) * 16]
        scale = max(f32(np.max(np.abs(blk)) / f32(6.0)), f32(1.0e-8))
        q_scales[g] = R.ref_encode_ue4m3(float(scale))
        for i in range(16):
            nib = R.ref_encode_e2m1(float(f32(blk[i] / scale)))
            col = g * 16 + i
            q_codes[col // 2] |= nib if (col & 1) == 0 else (nib << 4)
    q_swapped = np.zeros_like(q_codes)
    R.ref_swap_nibbles(q_codes.ctypes.data, q_codes.size, q_swapped.ctypes.data)
    q_tiled = np.zeros(128 * 64, dtype=np.uint8)
    n = R.ref_swizzle_scales(q_scales.ctypes.data, 1, kq // 16, q_tiled.ctypes.data, q_tiled.size)
    assert n == q_tiled.size

    out = Path(__file__).resolve().parent / "nvfp4_golden.npz"
    np.savez_compressed(
        out, e4m3_table=e4m3_table, e2m1_table=e2m1_table, ue4m3_in=ue4m3_in.view(np.uint32), ue4m3_out=ue4m3_out,
        e2m1_in=e2m1_in.view(np.uint32), e2m1_out=e2m1_out, sw_in=sw_in, sw_out=sw_out, nib_in=nib_in,
        nib_out=nib_out, mv_codes=codes, mv_scales=scales, mv_s2=s2, mv_input_scale=input_scale, mv_x=x, mv_y=y,
        q_x=xq, q_codes=q_codes, q_codes_swapped=q_swapped, q_scales=q_scales, q_scales_tiled=q_tiled)
    print(f"wrote {out} ({out.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
