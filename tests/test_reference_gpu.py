"""The reference's own CUDA kernels, compiled unmodified into oracle/_ref and run on this GPU, against the oracle
and the engine.  This is what pins the oracle to outputs of the reference itself."""
import ctypes as C

import numpy as np
import pytest

from helpers import from_torch_bf16, make_activations, make_weight, to_torch_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref(oracle):
    R = oracle.ref_lib()
    if R is None:
        pytest.skip("reference shim not built")
    return R


@pytest.mark.parametrize("variant", [0, 1, 2, 4])
def test_reference_w4a16_kernels_match_oracle(engine, oracle, ref, variant):
    import torch

    n, k = 3584, 1024
    _, codes, scales, s2 = make_weight(n, k, seed=42)
    x = np.array([np.float32((i % 17) - 8) / np.float32(17.0) for i in range(k)], dtype=np.float32)
    d_codes, d_scales = torch.from_numpy(codes).cuda(), torch.from_numpy(scales).cuda()
    d_x = torch.from_numpy(x).cuda()
    d_y = torch.zeros(n, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    assert ref.ref_w4a16_projection(d_codes.data_ptr(), d_scales.data_ptr(), d_x.data_ptr(), 0.5, s2, d_y.data_ptr(),
                                    n, k, variant) == 0, ref.ref_last_error()
    torch.cuda.synchronize()
    y_ref = d_y.cpu().numpy()
    exp = oracle.matvec_f32(codes, scales, 0.5, s2, x)
    # the reference reports max_abs_error ~1e-9 for its kernels (docs/development_plan.md:410)
    assert np.max(np.abs(y_ref - exp)) < 1e-6
    assert oracle.rel_l2(y_ref, exp) < 1e-5
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    y_eng = engine.gemv_w4a16_f32(w, d_x, input_scale=0.5).cpu().numpy()
    assert oracle.rel_l2(y_eng, y_ref) < 1e-5


def test_reference_benchmark_self_check(oracle, ref):
    """run_nvfp4_custom_projection_benchmark on synthetic tensors: its embedded CPU check passes on this GPU."""
    n, k = 3584, 1024
    _, codes, scales, s2 = make_weight(n, k, seed=42)
    ms, err = C.c_double(0), C.c_double(0)
    rc = ref.ref_custom_projection_benchmark(codes.ctypes.data, scales.ctypes.data, 1.0, s2, n, k, 2, 2, 5,
                                             C.byref(ms), C.byref(err))
    assert rc == 0, ref.ref_last_error()
    assert err.value < 1e-6 and ms.value > 0


def test_reference_activation_quantiser_bytes(engine, oracle, ref):
    """nvfp4_quantize_bf16_matrix_for_cublaslt_kernel output == oracle restatement == engine's reference-recipe mode."""
    import torch

    m, k = 40, 1024
    xb = make_activations(m, k, seed=9, outlier_frac=0.001)
    x = to_torch_bf16(xb)
    codes = torch.zeros((m, k // 2), dtype=torch.uint8, device="cuda")
    scales = torch.zeros(oracle.tiled_scale_bytes(m, k // 16), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    assert ref.ref_quantize_bf16_matrix(x.data_ptr(), codes.data_ptr(), scales.data_ptr(), m, k) == 0
    torch.cuda.synchronize()
    e_codes, e_scales = oracle.act_quant_reference(oracle.bf16_to_f32(xb), swap_nibbles=True)
    assert np.array_equal(codes.cpu().numpy(), e_codes)
    assert np.array_equal(scales.cpu().numpy(), oracle.swizzle_scales(e_scales))
    c2, s2 = engine.quantize_activations_reference_recipe(x, swap_nibbles=True)
    assert torch.equal(c2, codes) and torch.equal(s2, scales)


def test_w4a4_gemm_matches_the_reference_cublaslt_bridge(engine, oracle, ref):
    """Pins the W4A4 projection to an output of the reference itself: run_nvfp4_cublaslt_prefill_projection_device_bf16
    (src/runtime/cuda_bench.cu:1056-1167 behind include/qwen35x/runtime/cuda_bench.h:70-83: the reference's
    quantiser + cuBLASLt FP4 matmul, fp32 output) against the engine's tcgen05 GEMM fed with activations quantised
    by the reference's own recipe (no per-tensor scale: g = 1).  Same codes, same scale bytes, same formula: the
    outputs may differ by accumulation order and by the BF16 rounding of the engine's output only."""
    import ctypes as C

    import torch

    for (m, n, k) in ((300, 1024, 1024), (64, 512, 2560), (16, 3584, 1024)):
        _, codes, scales, s2 = make_weight(n, k, seed=n + k)
        xb = make_activations(m, k, seed=m, outlier_frac=0.001)
        x = to_torch_bf16(xb)
        swapped = ((codes & 0x0F) << 4) | (codes >> 4)
        d_w = torch.from_numpy(swapped).cuda()
        d_ws = torch.from_numpy(oracle.swizzle_scales(scales)).cuda()
        d_s2 = torch.tensor([s2], dtype=torch.float32, device="cuda")
        d_ac = torch.zeros(m * k // 2, dtype=torch.uint8, device="cuda")
        d_as = torch.zeros(oracle.tiled_scale_bytes(m, k // 16), dtype=torch.uint8, device="cuda")
        d_c = torch.zeros((m, n), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        rc = ref.ref_cublaslt_prefill_bf16(x.data_ptr(), d_w.data_ptr(), d_ws.data_ptr(), d_s2.data_ptr(), m, n, k,
                                           d_ac.data_ptr(), d_as.data_ptr(), d_c.data_ptr(), None)
        if rc != 0:
            pytest.skip(f"the reference's cuBLASLt FP4 bridge does not run here: {ref.ref_last_error().decode()}")
        torch.cuda.synchronize()
        expected = d_c.cpu().numpy()
        w = engine.Nvfp4Weight.from_host(codes, scales, s2)
        a_codes, a_scales = engine.quantize_activations_reference_recipe(x, swap_nibbles=False)
        one = torch.ones(1, dtype=torch.float32, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        c = engine.gemm_w4a4(w, a_codes, a_scales, one, m, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        got = oracle.bf16_to_f32(from_torch_bf16(c))
        exp_bf16 = oracle.bf16_to_f32(oracle.bf16_round(expected))
        assert oracle.rel_l2(got, exp_bf16) <= 1e-3, (m, n, k, oracle.rel_l2(got, exp_bf16))
        assert oracle.rel_l2(got, expected) <= 3e-3  # against the unrounded fp32 output: BF16 rounding of ours on top
