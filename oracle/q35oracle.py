"""numpy front-end of the C oracle (oracle/nvfp4_oracle.c) and, when built, of
the reference shim (oracle/ref_shim.cu).  Test infrastructure only: imported
by tests/, by the smoke test and by the benchmark's CPU-baseline leg."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from . import build_oracle as _b

_u8p = C.POINTER(C.c_uint8)
_u16p = C.POINTER(C.c_uint16)
_f32p = C.POINTER(C.c_float)

_lib = None
_ref = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = _b.build_oracle()
        L = C.CDLL(str(path))
        L.q35o_decode_e2m1.restype = C.c_float
        L.q35o_decode_e2m1.argtypes = [C.c_uint8]
        L.q35o_decode_e4m3.restype = C.c_float
        L.q35o_decode_e4m3.argtypes = [C.c_uint8]
        L.q35o_encode_ue4m3.restype = C.c_uint8
        L.q35o_encode_ue4m3.argtypes = [C.c_float]
        L.q35o_encode_e2m1.restype = C.c_uint8
        L.q35o_encode_e2m1.argtypes = [C.c_float]
        L.q35o_tiled_scale_offset.restype = C.c_int64
        L.q35o_tiled_scale_offset.argtypes = [C.c_int, C.c_int, C.c_int]
        L.q35o_tiled_scale_bytes.restype = C.c_int64
        L.q35o_tiled_scale_bytes.argtypes = [C.c_int, C.c_int]
        L.q35o_swizzle_scales.restype = None
        L.q35o_swizzle_scales.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.q35o_matvec_f32.restype = None
        L.q35o_matvec_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.c_int, C.c_int, C.c_void_p,
                                      C.c_int, C.c_int, C.c_void_p]
        L.q35o_matvec_f32_omp.restype = None
        L.q35o_matvec_f32_omp.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.c_int, C.c_int,
                                          C.c_void_p, C.c_void_p, C.c_int]
        L.q35o_gemv_bf16.restype = None
        L.q35o_gemv_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                     C.c_void_p, C.c_void_p, C.c_int]
        L.q35o_dequant_weights_bf16.restype = None
        L.q35o_dequant_weights_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int, C.c_void_p]
        L.q35o_act_quant_reference.restype = None
        L.q35o_act_quant_reference.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.q35o_global_scale_from_amax.restype = C.c_float
        L.q35o_global_scale_from_amax.argtypes = [C.c_float]
        L.q35o_quantize_nvfp4.restype = None
        L.q35o_quantize_nvfp4.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p,
                                          C.c_void_p]
        L.q35o_gemm_w4a4.restype = None
        L.q35o_gemm_w4a4.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                     C.c_float, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int]
        L.q35o_max_threads.restype = C.c_int
        L.q35o_bf16_to_f32.restype = C.c_float
        L.q35o_bf16_to_f32.argtypes = [C.c_uint16]
        L.q35o_f32_to_bf16.restype = C.c_uint16
        L.q35o_f32_to_bf16.argtypes = [C.c_float]
        _lib = L
    return _lib


def ref_lib() -> C.CDLL | None:
    """The reference shim, or None when it has never been built on this tree."""
    global _ref
    if _ref is None:
        path = _b.build_reference_shim()
        if path is None:
            return None
        R = C.CDLL(str(path))
        R.ref_last_error.restype = C.c_char_p
        R.ref_decode_e2m1.restype = C.c_float
        R.ref_decode_e2m1.argtypes = [C.c_uint8]
        R.ref_decode_e4m3.restype = C.c_float
        R.ref_decode_e4m3.argtypes = [C.c_uint8]
        R.ref_encode_ue4m3.restype = C.c_uint8
        R.ref_encode_ue4m3.argtypes = [C.c_float]
        R.ref_encode_e2m1.restype = C.c_uint8
        R.ref_encode_e2m1.argtypes = [C.c_float]
        R.ref_swizzle_scales.restype = C.c_longlong
        R.ref_swizzle_scales.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_longlong]
        R.ref_swap_nibbles.restype = None
        R.ref_swap_nibbles.argtypes = [C.c_void_p, C.c_longlong, C.c_void_p]
        R.ref_w4a16_projection.restype = C.c_int
        R.ref_w4a16_projection.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.c_void_p,
                                           C.c_int, C.c_int, C.c_int]
        R.ref_custom_projection_benchmark.restype = C.c_int
        R.ref_custom_projection_benchmark.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.c_int, C.c_int,
                                                      C.c_int, C.c_int, C.c_int, C.POINTER(C.c_double),
                                                      C.POINTER(C.c_double)]
        R.ref_quantize_bf16_matrix.restype = C.c_int
        R.ref_quantize_bf16_matrix.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        R.ref_cublaslt_prefill_bf16.restype = C.c_int
        R.ref_cublaslt_prefill_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                                C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_double)]
        _ref = R
    return _ref


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


# ---------------------------------------------------------------- codecs
def decode_e2m1_table() -> np.ndarray:
    return np.array([lib().q35o_decode_e2m1(i) for i in range(16)], dtype=np.float32)


def decode_e4m3_table() -> np.ndarray:
    return np.array([lib().q35o_decode_e4m3(i) for i in range(256)], dtype=np.float32)


def encode_ue4m3(v) -> np.ndarray:
    v = _c(np.atleast_1d(v), np.float32)
    L = lib()
    return np.array([L.q35o_encode_ue4m3(float(x)) for x in v], dtype=np.uint8)


def encode_e2m1(v) -> np.ndarray:
    v = _c(np.atleast_1d(v), np.float32)
    L = lib()
    return np.array([L.q35o_encode_e2m1(float(x)) for x in v], dtype=np.uint8)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns (uint16), round to nearest even."""
    u = _c(x, np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (_c(h, np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---------------------------------------------------------------- layout
def tiled_scale_bytes(rows: int, scale_cols: int) -> int:
    return int(lib().q35o_tiled_scale_bytes(rows, scale_cols))


def tiled_scale_offset(row: int, col: int, scale_cols: int) -> int:
    return int(lib().q35o_tiled_scale_offset(row, col, scale_cols))


def swizzle_scales(scales: np.ndarray) -> np.ndarray:
    s = _c(scales, np.uint8)
    rows, cols = s.shape
    out = np.zeros(tiled_scale_bytes(rows, cols), dtype=np.uint8)
    lib().q35o_swizzle_scales(_p(s), rows, cols, _p(out))
    return out


# ---------------------------------------------------------------- W4A16
def matvec_f32(codes, scales, input_scale, s2, x, row_begin=0, row_end=None) -> np.ndarray:
    codes = _c(codes, np.uint8)
    scales = _c(scales, np.uint8)
    x = _c(x, np.float32)
    rows, cols = codes.shape[0], codes.shape[1] * 2
    row_end = rows if row_end is None else row_end
    y = np.zeros(row_end - row_begin, dtype=np.float32)
    lib().q35o_matvec_f32(_p(codes), _p(scales), input_scale, s2, rows, cols, _p(x), row_begin, row_end, _p(y))
    return y


def matvec_f32_omp(codes, scales, input_scale, s2, x, threads) -> np.ndarray:
    codes = _c(codes, np.uint8)
    scales = _c(scales, np.uint8)
    x = _c(x, np.float32)
    rows, cols = codes.shape[0], codes.shape[1] * 2
    y = np.zeros(rows, dtype=np.float32)
    lib().q35o_matvec_f32_omp(_p(codes), _p(scales), input_scale, s2, rows, cols, _p(x), _p(y), threads)
    return y


def gemv_bf16(codes, scales, s2, x_bf16, threads=1):
    """x_bf16: uint16 [m, K].  Returns (y_bf16 uint16 [m, N], y_f32 [m, N])."""
    codes = _c(codes, np.uint8)
    scales = _c(scales, np.uint8)
    x = _c(np.atleast_2d(x_bf16), np.uint16)
    rows, cols = codes.shape[0], codes.shape[1] * 2
    m = x.shape[0]
    assert x.shape[1] == cols
    yb = np.zeros((m, rows), dtype=np.uint16)
    yf = np.zeros((m, rows), dtype=np.float32)
    lib().q35o_gemv_bf16(_p(codes), _p(scales), s2, rows, cols, _p(x), m, _p(yb), _p(yf), threads)
    return yb, yf


def dequant_weights_bf16(codes, scales, s2) -> np.ndarray:
    codes = _c(codes, np.uint8)
    scales = _c(scales, np.uint8)
    rows, cols = codes.shape[0], codes.shape[1] * 2
    w = np.zeros((rows, cols), dtype=np.uint16)
    lib().q35o_dequant_weights_bf16(_p(codes), _p(scales), s2, rows, cols, _p(w))
    return w


# ---------------------------------------------------------------- quantisers
def act_quant_reference(x_f32, swap_nibbles=False):
    x = _c(np.atleast_2d(x_f32), np.float32)
    rows, cols = x.shape
    codes = np.zeros((rows, cols // 2), dtype=np.uint8)
    scales = np.zeros((rows, cols // 16), dtype=np.uint8)
    lib().q35o_act_quant_reference(_p(x), rows, cols, int(swap_nibbles), _p(codes), _p(scales))
    return codes, scales


def quantize_nvfp4(x, global_scale=0.0):
    """x: float32 [rows, cols] or uint16 (bf16 bits) [rows, cols].
    Returns (codes [rows, cols/2], scales [rows, cols/16] row-major, g)."""
    x = np.atleast_2d(x)
    is_bf16 = x.dtype == np.uint16
    x = _c(x, np.uint16 if is_bf16 else np.float32)
    rows, cols = x.shape
    codes = np.zeros((rows, cols // 2), dtype=np.uint8)
    scales = np.zeros((rows, cols // 16), dtype=np.uint8)
    g = C.c_float(0)
    lib().q35o_quantize_nvfp4(_p(x), int(is_bf16), rows, cols, float(global_scale), _p(codes), _p(scales),
                              C.byref(g))
    return codes, scales, float(g.value)


# ---------------------------------------------------------------- W4A4
def gemm_w4a4(w_codes, w_scales, s2, a_codes, a_scales, input_scale, n_begin=0, n_end=None, threads=1):
    """Returns (c_bf16 uint16 [m, n], c_f32 [m, n])."""
    w_codes = _c(w_codes, np.uint8)
    w_scales = _c(w_scales, np.uint8)
    a_codes = _c(a_codes, np.uint8)
    a_scales = _c(a_scales, np.uint8)
    rows, cols = w_codes.shape[0], w_codes.shape[1] * 2
    m = a_codes.shape[0]
    n_end = rows if n_end is None else n_end
    cf = np.zeros((m, n_end - n_begin), dtype=np.float32)
    cb = np.zeros((m, n_end - n_begin), dtype=np.uint16)
    lib().q35o_gemm_w4a4(_p(w_codes), _p(w_scales), s2, rows, cols, _p(a_codes), _p(a_scales), input_scale, m,
                         n_begin, n_end, _p(cf), _p(cb), threads)
    return cb, cf


def max_threads() -> int:
    return int(lib().q35o_max_threads())


def rel_l2(actual: np.ndarray, expected: np.ndarray) -> float:
    a = np.asarray(actual, dtype=np.float64).ravel()
    e = np.asarray(expected, dtype=np.float64).ravel()
    den = np.linalg.norm(e)
    return float(np.linalg.norm(a - e) / (den if den > 0 else 1.0))
