"""ctypes binding of libq35b.so plus thin torch helpers.

torch is used for device memory and streams only; every computation goes
through the C ABI.  There is no CPU fallback: if the library is missing or no
CUDA device is present, calls raise."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

_PKG = Path(__file__).resolve().parent
_LIB_PATH = _PKG / "_lib" / "libq35b.so"
_lib = None

GEMV_AUTO, GEMV_SIMT, GEMV_STREAM = -1, 10, 11


class Q35bError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"q35b status {status}: {message}")
        self.status = status


class _PeerRegion(C.Structure):
    _fields_ = [("offset", C.c_size_t), ("row_bytes", C.c_size_t), ("ld_bytes", C.c_size_t), ("rows", C.c_int)]


def lib() -> C.CDLL:
    """Load libq35b.so (built by `python -m qwen35x_b200.build`); raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.is_file():
        raise FileNotFoundError(f"{_LIB_PATH} is missing: run `python -m qwen35x_b200.build` (needs nvcc)")
    L = C.CDLL(str(_LIB_PATH))
    vp, i, f, sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
    L.q35b_last_error.restype = C.c_char_p
    L.q35b_version.restype = C.c_char_p
    L.q35b_launch_count.restype = C.c_ulonglong
    L.q35b_weight_create.restype = i
    L.q35b_weight_create.argtypes = [vp, vp, f, f, i, i, i, i, C.POINTER(vp)]
    L.q35b_weight_create_from_device.restype = i
    L.q35b_weight_create_from_device.argtypes = [vp, vp, f, f, i, i, i, i, vp, C.POINTER(vp)]
    L.q35b_weight_create_gate_up.restype = i
    L.q35b_weight_create_gate_up.argtypes = [vp, vp, f, vp, vp, f, i, i, C.POINTER(vp)]
    L.q35b_weight_create_gate_up_shard.restype = i
    L.q35b_weight_create_gate_up_shard.argtypes = [vp, vp, f, vp, vp, f, i, i, i, i, C.POINTER(vp)]
    L.q35b_weight_is_gate_up.restype = i
    L.q35b_weight_is_gate_up.argtypes = [vp]
    L.q35b_weight_dequant_bf16.restype = i
    L.q35b_weight_dequant_bf16.argtypes = [vp, vp, vp]
    L.q35b_weight_destroy.restype = None
    L.q35b_weight_destroy.argtypes = [vp]
    for name in ("q35b_weight_row_begin", "q35b_weight_rows", "q35b_weight_cols"):
        getattr(L, name).restype = i
        getattr(L, name).argtypes = [vp]
    L.q35b_weight_stream_bytes.restype = sz
    L.q35b_weight_stream_bytes.argtypes = [vp]
    L.q35b_shard_range.restype = i
    L.q35b_shard_range.argtypes = [i, i, i, C.POINTER(i), C.POINTER(i)]
    L.q35b_gemv_w4a16_bf16.restype = i
    L.q35b_gemv_w4a16_bf16.argtypes = [vp, vp, i, vp, i, vp]
    L.q35b_gemv_w4a16_f32.restype = i
    L.q35b_gemv_w4a16_f32.argtypes = [vp, vp, f, vp, i, vp]
    L.q35b_gemv_batch_create.restype = i
    L.q35b_gemv_batch_create.argtypes = [vp, i, i, C.POINTER(vp)]
    L.q35b_gemv_batch_create_tensor.restype = i
    L.q35b_gemv_batch_create_tensor.argtypes = [vp, i, i, i, C.POINTER(vp)]
    L.q35b_gemv_batch_run.restype = i
    L.q35b_gemv_batch_run.argtypes = [vp, vp]
    L.q35b_gemv_batch_destroy.restype = None
    L.q35b_gemv_batch_destroy.argtypes = [vp]
    L.q35b_gemv_batch_status.restype = i
    L.q35b_gemv_batch_status.argtypes = [vp, C.POINTER(C.c_uint)]
    L.q35b_debug_gemv_plan.restype = i
    L.q35b_debug_gemv_plan.argtypes = [i, i, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]
    L.q35b_debug_gemv_batch_wait.restype = i
    L.q35b_debug_gemv_batch_wait.argtypes = [vp, C.c_uint, C.c_uint]
    L.q35b_gemv_batch_stream_bytes.restype = sz
    L.q35b_gemv_batch_stream_bytes.argtypes = [vp]
    L.q35b_act_codes_bytes.restype = sz
    L.q35b_act_codes_bytes.argtypes = [i, i]
    L.q35b_act_scales_bytes.restype = sz
    L.q35b_act_scales_bytes.argtypes = [i, i]
    L.q35b_quant_workspace_bytes.restype = sz
    L.q35b_quantize_nvfp4_bf16.restype = i
    L.q35b_quantize_nvfp4_bf16.argtypes = [vp, i, i, f, vp, vp, vp, vp, vp]
    L.q35b_quantize_nvfp4_f32.restype = i
    L.q35b_quantize_nvfp4_f32.argtypes = [vp, i, i, f, vp, vp, vp, vp, vp]
    L.q35b_gemm_default_status.restype = i
    L.q35b_gemm_default_status.argtypes = [C.POINTER(C.c_uint)]
    L.q35b_static_prefill_status.restype = i
    L.q35b_static_prefill_status.argtypes = [C.POINTER(C.c_uint)]
    L.q35b_quantize_nvfp4_bf16_reference_recipe.restype = i
    L.q35b_quantize_nvfp4_bf16_reference_recipe.argtypes = [vp, i, i, i, vp, vp, vp]
    L.q35b_quantize_weight_f32.restype = i
    L.q35b_quantize_weight_f32.argtypes = [vp, i, i, vp, vp, vp, vp, vp]
    L.q35b_gemm_w4a4_bf16.restype = i
    L.q35b_gemm_w4a4_bf16.argtypes = [vp, vp, vp, vp, i, vp, i, vp, vp]
    L.q35b_static_prefill_capacity_bytes.restype = sz
    L.q35b_project_prefill_bf16_static.restype = i
    L.q35b_project_prefill_bf16_static.argtypes = [vp, vp, i, f, vp, i, vp]
    L.q35b_gemm_w4a4_bf16_residual.restype = i
    L.q35b_gemm_w4a4_bf16_residual.argtypes = [vp, vp, vp, vp, i, vp, i, vp, i, vp, vp]
    L.q35b_gemv_item_bytes.restype = C.c_size_t
    L.q35b_gemv_item_bytes.argtypes = []
    if int(L.q35b_gemv_item_bytes()) != C.sizeof(_GemvItem):
        raise Q35bError(1, "q35b_gemv_item layout of this binding does not match the library.")
    L.q35b_peer_buffer_create.restype = i
    L.q35b_peer_buffer_create.argtypes = [C.c_size_t, C.POINTER(vp)]
    L.q35b_peer_buffer_handle_bytes.restype = C.c_size_t
    L.q35b_peer_buffer_handle_bytes.argtypes = []
    L.q35b_peer_buffer_export.restype = i
    L.q35b_peer_buffer_export.argtypes = [vp, vp]
    L.q35b_peer_buffer_open.restype = i
    L.q35b_peer_buffer_open.argtypes = [vp, C.c_size_t, C.POINTER(vp)]
    L.q35b_peer_buffer_data.restype = vp
    L.q35b_peer_buffer_data.argtypes = [vp]
    L.q35b_peer_buffer_destroy.restype = None
    L.q35b_peer_buffer_destroy.argtypes = [vp]
    L.q35b_gemm_w4a4_bf16_allgather.restype = i
    L.q35b_gemm_w4a4_bf16_allgather.argtypes = [vp, vp, vp, vp, i, C.POINTER(vp), i, i, i, C.c_uint, vp, vp]
    L.q35b_peer_gather_wait.restype = i
    L.q35b_peer_gather_wait.argtypes = [C.POINTER(vp), i, i, C.c_uint, vp, vp]
    L.q35b_peer_push.restype = i
    L.q35b_peer_push.argtypes = [C.POINTER(vp), i, i, C.POINTER(_PeerRegion), i, C.c_uint, vp]
    L.q35b_gemm_w4a4_gate_up_nvfp4.restype = i
    L.q35b_gemm_w4a4_gate_up_nvfp4.argtypes = [vp, vp, vp, vp, i, vp, vp, vp, vp, vp]
    L.q35b_debug_encode_ue4m3.restype = C.c_uint8
    L.q35b_debug_encode_ue4m3.argtypes = [f]
    L.q35b_debug_encode_e2m1.restype = C.c_uint8
    L.q35b_debug_encode_e2m1.argtypes = [f]
    L.q35b_debug_decode_e4m3.restype = f
    L.q35b_debug_decode_e4m3.argtypes = [C.c_uint8]
    L.q35b_debug_decode_e2m1.restype = f
    L.q35b_debug_decode_e2m1.argtypes = [C.c_uint8]
    L.q35b_debug_tiled_scale_offset.restype = C.c_longlong
    L.q35b_debug_tiled_scale_offset.argtypes = [i, i, i]
    _lib = L
    return L


def _check(status: int) -> None:
    if status != 0:
        raise Q35bError(status, lib().q35b_last_error().decode("utf-8", "replace"))


def launch_count() -> int:
    return int(lib().q35b_launch_count())


def shard_range(n: int, shard_index: int, shard_count: int) -> tuple[int, int]:
    b, c = C.c_int(0), C.c_int(0)
    _check(lib().q35b_shard_range(n, shard_index, shard_count, C.byref(b), C.byref(c)))
    return b.value, c.value


def _torch():
    import torch

    if not torch.cuda.is_available():
        raise Q35bError(3, "no CUDA device: the NVFP4 projection engine has no CPU fallback")
    return torch


def _stream_ptr(torch) -> int:
    return int(torch.cuda.current_stream().cuda_stream)


class Nvfp4Weight:
    """One projection weight (or one row shard of it) repacked on the current CUDA device.

    Mirrors the role of the reference's PackedNvfp4Weight
    (src/runtime/qwen35x_cuda_backend.cpp:194-210)."""

    def __init__(self, handle: int, n: int, k: int, s2: float, input_scale: float):
        self._h = C.c_void_p(handle)
        self.n_total, self.k, self.s2, self.input_scale = n, k, s2, input_scale
        L = lib()
        self.row_begin = L.q35b_weight_row_begin(self._h)
        self.rows = L.q35b_weight_rows(self._h)
        self.stream_bytes = int(L.q35b_weight_stream_bytes(self._h))
        self.gate_up = bool(L.q35b_weight_is_gate_up(self._h))

    @classmethod
    def from_host(cls, codes: np.ndarray, scales: np.ndarray, weight_scale_2: float, input_scale: float = 1.0,
                  shard_index: int = 0, shard_count: int = 1) -> "Nvfp4Weight":
        _torch()
        codes = np.ascontiguousarray(codes, dtype=np.uint8)
        scales = np.ascontiguousarray(scales, dtype=np.uint8)
        n, k = codes.shape[0], codes.shape[1] * 2
        if scales.shape != (n, k // 16):
            raise Q35bError(2, "NVFP4 packed weight or scale size does not match matrix dimensions.")
        h = C.c_void_p()
        _check(lib().q35b_weight_create(codes.ctypes.data, scales.ctypes.data, weight_scale_2, input_scale, n, k,
                                        shard_index, shard_count, C.byref(h)))
        return cls(h.value, n, k, weight_scale_2, input_scale)

    @classmethod
    def gate_up_from_host(cls, gate_codes, gate_scales, gate_s2: float, up_codes, up_scales, up_s2: float,
                          shard_index: int = 0, shard_count: int = 1) -> "Nvfp4Weight":
        """gate_proj + up_proj as one weight with rows alternating in groups of eight (for the fused SiLU epilogue);
        with shard_count > 1 the row shard `shard_index` of that interleaved matrix."""
        _torch()
        arrs = [np.ascontiguousarray(a, dtype=np.uint8) for a in (gate_codes, gate_scales, up_codes, up_scales)]
        n_half, k = arrs[0].shape[0], arrs[0].shape[1] * 2
        if arrs[2].shape != arrs[0].shape or arrs[1].shape != (n_half, k // 16) or arrs[3].shape != (n_half, k // 16):
            raise Q35bError(2, "NVFP4 packed weight or scale size does not match matrix dimensions.")
        h = C.c_void_p()
        _check(lib().q35b_weight_create_gate_up_shard(arrs[0].ctypes.data, arrs[1].ctypes.data, gate_s2, arrs[2].ctypes.data,
                                                      arrs[3].ctypes.data, up_s2, n_half, k, shard_index, shard_count,
                                                      C.byref(h)))
        return cls(h.value, 2 * n_half, k, gate_s2, 1.0)

    def dequant_bf16(self):
        """The whole weight as BF16 [rows, K] on the device (the reference's load-time NVFP4 -> BF16 conversion)."""
        torch = _torch()
        out = torch.empty((self.rows, self.k), dtype=torch.bfloat16, device="cuda")
        _check(lib().q35b_weight_dequant_bf16(self._h, out.data_ptr(), _stream_ptr(torch)))
        return out

    @classmethod
    def from_device(cls, codes, scales, weight_scale_2: float, input_scale: float = 1.0, shard_index: int = 0,
                    shard_count: int = 1) -> "Nvfp4Weight":
        torch = _torch()
        assert codes.is_cuda and scales.is_cuda and codes.dtype == torch.uint8 and scales.dtype == torch.uint8
        codes, scales = codes.contiguous(), scales.contiguous()
        n, k = codes.shape[0], codes.shape[1] * 2
        if tuple(scales.shape) != (n, k // 16):
            raise Q35bError(2, "NVFP4 packed weight or scale size does not match matrix dimensions.")
        h = C.c_void_p()
        _check(lib().q35b_weight_create_from_device(codes.data_ptr(), scales.data_ptr(), weight_scale_2, input_scale,
                                                    n, k, shard_index, shard_count, _stream_ptr(torch), C.byref(h)))
        return cls(h.value, n, k, weight_scale_2, input_scale)

    @property
    def handle(self) -> C.c_void_p:
        return self._h

    def close(self) -> None:
        if self._h is not None and self._h.value:
            lib().q35b_weight_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def gemv_w4a16(weight: Nvfp4Weight, x, out=None, kernel: int = GEMV_AUTO):
    """Decode projection: x [m, K] bf16 (m = 1..8) -> y [m, rows] bf16."""
    torch = _torch()
    if x.dim() == 1:
        x = x.unsqueeze(0)
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[1] == weight.k
    m = x.shape[0]
    if out is None:
        out = torch.empty((m, weight.rows), dtype=torch.bfloat16, device=x.device)
    _check(lib().q35b_gemv_w4a16_bf16(weight.handle, x.data_ptr(), m, out.data_ptr(), kernel, _stream_ptr(torch)))
    return out


def gemv_w4a16_f32(weight: Nvfp4Weight, x, input_scale: float = 1.0, out=None, kernel: int = GEMV_AUTO):
    """The reference benchmark's contract: fp32 x [K], fp32 y [rows], x scaled by input_scale."""
    torch = _torch()
    assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and x.numel() == weight.k
    if out is None:
        out = torch.empty((weight.rows,), dtype=torch.float32, device=x.device)
    _check(lib().q35b_gemv_w4a16_f32(weight.handle, x.data_ptr(), input_scale, out.data_ptr(), kernel,
                                     _stream_ptr(torch)))
    return out


class _GemvItem(C.Structure):
    _fields_ = [("weight", C.c_void_p), ("x_bf16", C.c_void_p), ("y_bf16", C.c_void_p), ("residual_bf16", C.c_void_p),
                ("after", C.c_int)]


class GemvBatch:
    """A prepared work list of decode projections run by one persistent launch (q35b_gemv_batch_* in
    include/q35b_nvfp4.h).  items: sequence of (Nvfp4Weight, x [m,K] bf16, y [m,out_rows] bf16),
    (weight, x, y, residual [m,rows] bf16) or (weight, x, y, residual-or-None, after): with a residual the projection
    is added to it before the BF16 rounding; a gate/up weight (Nvfp4Weight.gate_up_from_host) yields silu(gate)*up
    with out_rows = rows/2; `after` = index of an earlier item whose y this item's x is (the down projection after
    gate/up) -- items without it are independent.  The tensors must stay alive and in place for the life of the batch."""

    def __init__(self, items, m: int, digits: int = 0):
        """digits > 0: run the list on the tensor cores with every token's activations expanded into that many NVFP4
        digit rows (q35b_gemv_batch_create_tensor; 5 is the intended setting); 0: BF16 activations carried exactly."""
        torch = _torch()
        self._keep = list(items)
        arr = (_GemvItem * len(self._keep))()
        for j, item in enumerate(self._keep):
            w, x, y = item[0], item[1], item[2]
            res = item[3] if len(item) > 3 else None
            after = item[4] if len(item) > 4 and item[4] is not None else -1
            assert -1 <= after < j
            out_rows = w.rows // 2 if w.gate_up else w.rows
            assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and tuple(x.shape) == (m, w.k)
            assert y.is_cuda and y.dtype == torch.bfloat16 and y.is_contiguous() and tuple(y.shape) == (m, out_rows)
            if res is not None:
                assert res.is_cuda and res.dtype == torch.bfloat16 and res.is_contiguous() and tuple(res.shape) == (m, w.rows)
            arr[j] = _GemvItem(w.handle.value, x.data_ptr(), y.data_ptr(), res.data_ptr() if res is not None else None,
                               after + 1)
        h = C.c_void_p()
        if digits > 0:
            _check(lib().q35b_gemv_batch_create_tensor(arr, len(self._keep), m, digits, C.byref(h)))
        else:
            _check(lib().q35b_gemv_batch_create(arr, len(self._keep), m, C.byref(h)))
        self._h = h
        self.digits = digits
        self.m = m
        self.stream_bytes = int(lib().q35b_gemv_batch_stream_bytes(h))

    def run(self) -> None:
        _check(lib().q35b_gemv_batch_run(self._h, _stream_ptr(_torch())))

    def status(self) -> int:
        out = C.c_uint(0)
        _check(lib().q35b_gemv_batch_status(self._h, C.byref(out)))
        return int(out.value)

    def debug_wait(self, wait_limit_polls: int, extra_completions: int) -> None:
        """Test hook (q35b_debug_gemv_batch_wait): short wait limit and extra completions demanded of dependencies."""
        _check(lib().q35b_debug_gemv_batch_wait(self._h, wait_limit_polls, extra_completions))

    def close(self) -> None:
        if self._h is not None and self._h.value:
            lib().q35b_gemv_batch_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_workspaces: dict = {}


def _workspace(torch, device):
    key = (device.index, int(torch.cuda.current_stream().cuda_stream))
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.zeros(int(lib().q35b_quant_workspace_bytes()), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def act_scratch(m: int, k: int, device):
    """Caller-owned scratch for an [m, k] activation: (codes, tiled scales, input-scale word)."""
    torch = _torch()
    L = lib()
    codes = torch.empty(int(L.q35b_act_codes_bytes(m, k)), dtype=torch.uint8, device=device)
    scales = torch.empty(int(L.q35b_act_scales_bytes(m, k)), dtype=torch.uint8, device=device)
    g = torch.empty(1, dtype=torch.float32, device=device)
    return codes, scales, g


def quantize_activations(x, global_scale: float = 0.0, scratch=None):
    """BF16 (or fp32) [m, k] -> (codes [m, k/2] u8, tiled scales u8, g fp32[1]) on the device."""
    torch = _torch()
    assert x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and x.is_contiguous() and x.dim() == 2
    m, k = x.shape
    codes, scales, g = scratch if scratch is not None else act_scratch(m, k, x.device)
    ws = _workspace(torch, x.device)
    fn = lib().q35b_quantize_nvfp4_bf16 if x.dtype == torch.bfloat16 else lib().q35b_quantize_nvfp4_f32
    _check(fn(x.data_ptr(), m, k, global_scale, codes.data_ptr(), scales.data_ptr(), g.data_ptr(), ws.data_ptr(),
              _stream_ptr(torch)))
    return codes.view(m, k // 2), scales, g


def gemv_plan(m: int, max_k: int) -> dict:
    """Shared-memory plan of a decode work list (q35b_debug_gemv_plan): host arithmetic, needs no device."""
    v = [C.c_int(0) for _ in range(4)]
    _check(lib().q35b_debug_gemv_plan(m, max_k, *[C.byref(x) for x in v]))
    return {"ctas_per_sm": v[0].value, "ring_stages": v[1].value, "activation_buffers": v[2].value, "smem_bytes": v[3].value}


def gemm_default_status() -> int:
    """The library's own GEMM status word of the current device (used when a call passes no status word)."""
    out = C.c_uint(0)
    _check(lib().q35b_gemm_default_status(C.byref(out)))
    return int(out.value)


def static_prefill_status() -> int:
    """Status word of the built-in prefill scratch of the current device (see project_prefill_static)."""
    out = C.c_uint(0)
    _check(lib().q35b_static_prefill_status(C.byref(out)))
    return int(out.value)


def quantize_activations_reference_recipe(x, swap_nibbles: bool = True):
    torch = _torch()
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.dim() == 2
    m, k = x.shape
    codes, scales, _ = act_scratch(m, k, x.device)
    _check(lib().q35b_quantize_nvfp4_bf16_reference_recipe(x.data_ptr(), m, k, int(swap_nibbles), codes.data_ptr(),
                                                           scales.data_ptr(), _stream_ptr(torch)))
    return codes.view(m, k // 2), scales


def quantize_weight(w_f32):
    """fp32 [n, k] on the device -> (codes [n, k/2], scales [n, k/16] row-major, s2 float)."""
    torch = _torch()
    assert w_f32.is_cuda and w_f32.dtype == torch.float32 and w_f32.is_contiguous() and w_f32.dim() == 2
    n, k = w_f32.shape
    codes = torch.empty((n, k // 2), dtype=torch.uint8, device=w_f32.device)
    scales = torch.empty((n, k // 16), dtype=torch.uint8, device=w_f32.device)
    s2 = torch.empty(1, dtype=torch.float32, device=w_f32.device)
    ws = _workspace(torch, w_f32.device)
    _check(lib().q35b_quantize_weight_f32(w_f32.data_ptr(), n, k, codes.data_ptr(), scales.data_ptr(), s2.data_ptr(),
                                          ws.data_ptr(), _stream_ptr(torch)))
    return codes, scales, float(s2.item())


def gemm_w4a4(weight: Nvfp4Weight, a_codes, a_scales_tiled, g, m: int, out=None, status=None, residual=None):
    """Prefill projection on quantised activations: -> c [m, rows] bf16; with `residual` [m, rows] bf16 the sum is
    rounded once; a gate/up weight gives silu(gate) * up, [m, rows/2]."""
    torch = _torch()
    out_cols = weight.rows // 2 if weight.gate_up else weight.rows
    if out is None:
        out = torch.empty((m, out_cols), dtype=torch.bfloat16, device=a_codes.device)
    assert out.dtype == torch.bfloat16 and out.stride(1) == 1
    st = status.data_ptr() if status is not None else None
    if residual is None:
        _check(lib().q35b_gemm_w4a4_bf16(weight.handle, a_codes.data_ptr(), a_scales_tiled.data_ptr(), g.data_ptr(), m,
                                         out.data_ptr(), out.stride(0), st, _stream_ptr(torch)))
    else:
        assert residual.dtype == torch.bfloat16 and residual.stride(1) == 1 and tuple(residual.shape) == (m, weight.rows)
        _check(lib().q35b_gemm_w4a4_bf16_residual(weight.handle, a_codes.data_ptr(), a_scales_tiled.data_ptr(),
                                                  g.data_ptr(), m, residual.data_ptr(), residual.stride(0),
                                                  out.data_ptr(), out.stride(0), st, _stream_ptr(torch)))
    return out


def gemm_w4a4_gate_up_quant(weight: Nvfp4Weight, a_codes, a_scales_tiled, g, m: int, out_scale, scratch=None, status=None):
    """Gate/up prefill projection whose epilogue quantises silu(gate) * up to NVFP4 with the given per-tensor scale
    (`out_scale`: 1-element fp32 device tensor) -> (codes [m, n_half/2] uint8, tiled scales, out_scale), the A operand
    of the down projection's gemm_w4a4.  `scratch` = act_scratch(m, n_half, device) to reuse buffers; a row shard of
    the gate/up weight writes only its own columns of that whole-width activation."""
    torch = _torch()
    assert weight.gate_up and out_scale.dtype == torch.float32 and out_scale.is_cuda
    inter = weight.n_total // 2
    codes, scales, _ = scratch if scratch is not None else act_scratch(m, inter, a_codes.device)
    st = status.data_ptr() if status is not None else None
    _check(lib().q35b_gemm_w4a4_gate_up_nvfp4(weight.handle, a_codes.data_ptr(), a_scales_tiled.data_ptr(), g.data_ptr(), m,
                                              codes.data_ptr(), scales.data_ptr(), out_scale.data_ptr(), st,
                                              _stream_ptr(torch)))
    return codes.reshape(-1)[:m * (inter // 2)].view(m, inter // 2), scales, out_scale


class PeerBuffer:
    """One rank's full output matrix [m, n] BF16 in memory the other ranks can store into (q35b_peer_buffer_*):
    `PeerBuffer.create(m, n)` on the owning rank, `export()` -> bytes for the other ranks, `PeerBuffer.open(handle, m, n)`
    there.  `tensor()` views the matrix as a torch tensor (owner and openers alike)."""

    def __init__(self, handle, m: int, n: int, device):
        self._h = handle
        self.m, self.n, self.device = m, n, device

    @classmethod
    def create(cls, m: int, n: int) -> "PeerBuffer":
        torch = _torch()
        h = C.c_void_p()
        _check(lib().q35b_peer_buffer_create(m * n * 2, C.byref(h)))
        return cls(h, m, n, torch.device("cuda", torch.cuda.current_device()))

    @classmethod
    def create_bytes(cls, nbytes: int) -> "PeerBuffer":
        """A buffer of raw bytes (several regions of different kinds, see peer_push); `tensor()` views it as
        [1, nbytes / 2] BF16, `bytes()` as uint8."""
        assert nbytes % 2 == 0
        return cls.create(1, nbytes // 2)

    @classmethod
    def open_bytes(cls, handle: bytes, nbytes: int) -> "PeerBuffer":
        return cls.open(handle, 1, nbytes // 2)

    def bytes(self):
        torch = _torch()
        return self.tensor().view(torch.uint8).reshape(-1)

    @classmethod
    def open(cls, handle: bytes, m: int, n: int) -> "PeerBuffer":
        torch = _torch()
        assert len(handle) == int(lib().q35b_peer_buffer_handle_bytes())
        h = C.c_void_p()
        buf = C.create_string_buffer(handle, len(handle))
        _check(lib().q35b_peer_buffer_open(buf, m * n * 2, C.byref(h)))
        return cls(h, m, n, torch.device("cuda", torch.cuda.current_device()))

    def export(self) -> bytes:
        buf = C.create_string_buffer(int(lib().q35b_peer_buffer_handle_bytes()))
        _check(lib().q35b_peer_buffer_export(self._h, buf))
        return buf.raw

    @property
    def handle(self):
        return self._h

    @property
    def __cuda_array_interface__(self):
        return {"shape": (self.m, self.n), "typestr": "<u2", "data": (int(lib().q35b_peer_buffer_data(self._h)), False),
                "version": 3, "strides": None}

    def tensor(self):
        torch = _torch()
        return torch.as_tensor(self, device=self.device).view(torch.bfloat16)

    def close(self) -> None:
        if self._h:
            lib().q35b_peer_buffer_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def gemm_w4a4_allgather(weight: Nvfp4Weight, a_codes, a_scales_tiled, g, m: int, buffers, rank: int, epoch: int, status,
                        wait: bool = True):
    """The shard's GEMM storing into every rank's matrix (buffers: PeerBuffer per rank, buffers[rank] local), then
    (wait=True) the bounded wait for the other ranks' parts; after it, buffers[rank].tensor() holds the whole [m, n]."""
    torch = _torch()
    world = len(buffers)
    arr = (C.c_void_p * world)(*[b.handle for b in buffers])
    assert status is not None and status.is_cuda
    _check(lib().q35b_gemm_w4a4_bf16_allgather(weight.handle, a_codes.data_ptr(), a_scales_tiled.data_ptr(), g.data_ptr(), m,
                                               arr, world, rank, buffers[rank].n, epoch, status.data_ptr(), _stream_ptr(torch)))
    if wait:
        peer_gather_wait(buffers, rank, epoch, status)


def peer_push(buffers, rank: int, regions, epoch: int) -> None:
    """Copy regions [(offset, rows, row_bytes, ld_bytes)] of buffers[rank] to the same place in every other rank's
    buffer and signal `epoch` (q35b_peer_push); the receivers wait with peer_gather_wait(.., epoch, ..)."""
    torch = _torch()
    world = len(buffers)
    arr = (C.c_void_p * world)(*[b.handle for b in buffers])
    regs = (_PeerRegion * len(regions))(*[_PeerRegion(o, rb, ld, r) for (o, r, rb, ld) in regions])
    _check(lib().q35b_peer_push(arr, world, rank, regs, len(regions), epoch, _stream_ptr(torch)))


def peer_gather_wait(buffers, rank: int, epoch: int, status) -> None:
    """Bounded device-side wait until every other rank's part of epoch `epoch` is in buffers[rank]."""
    torch = _torch()
    world = len(buffers)
    arr = (C.c_void_p * world)(*[b.handle for b in buffers])
    _check(lib().q35b_peer_gather_wait(arr, world, rank, epoch, status.data_ptr(), _stream_ptr(torch)))


def project_prefill(weight: Nvfp4Weight, x, out=None, scratch=None, global_scale: float = 0.0, residual=None):
    """BF16 [m, K] -> BF16 [m, rows]: activation quantisation followed by the W4A4 GEMM (and its fused epilogue)."""
    codes, scales, g = quantize_activations(x, global_scale, scratch)
    return gemm_w4a4(weight, codes, scales, g, x.shape[0], out, residual=residual)


def project_prefill_static(weight: Nvfp4Weight, x, out=None, global_scale: float = 0.0):
    """project_prefill for hosts that cannot allocate: the activation scratch is the library's built-in device
    array (see q35b_project_prefill_bf16_static in include/q35b_nvfp4.h).  Calls sharing a device must not overlap."""
    torch = _torch()
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.dim() == 2 and x.shape[1] == weight.k
    m = x.shape[0]
    if out is None:
        out = torch.empty((m, weight.rows), dtype=torch.bfloat16, device=x.device)
    _check(lib().q35b_project_prefill_bf16_static(weight.handle, x.data_ptr(), m, global_scale, out.data_ptr(),
                                                  out.stride(0), _stream_ptr(torch)))
    return out
