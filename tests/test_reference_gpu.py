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
