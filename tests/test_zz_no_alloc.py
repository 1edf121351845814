"""The prefill projection that allocates nothing (q35b_project_prefill_bf16_static) against the ordinary path
(q35b_quantize_nvfp4_bf16 + q35b_gemm_w4a4_bf16 with caller-owned scratch).

Some hosts of this library cannot call cudaMalloc where they need a projection: they own the whole device through
their own arena, or run under a fixed memory budget, or must avoid the device-wide synchronisation an allocation
brings.  For them the activation scratch is an array built into the library.  This test goes through the C ABI,
twice in a row with different shapes, because the built-in array keeps the first call's bytes while the second runs.
It is collected last so that a failure here cannot hide any other test's result."""
import ctypes as C

import pytest

from helpers import make_activations, make_weight, to_torch_bf16

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-3  # the tolerance of tests/test_gemm_gpu.py; the two paths run the same kernels, so they also match exactly


def _both_paths(engine, w, x):
    import torch

    L = engine.lib()
    m = x.shape[0]
    expected = engine.project_prefill(w, x)
    got = torch.full((m, w.rows), float("nan"), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc = L.q35b_project_prefill_bf16_static(w.handle, C.c_void_p(x.data_ptr()), m, C.c_float(0.0),
                                            C.c_void_p(got.data_ptr()), got.stride(0),
                                            C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, L.q35b_last_error()
    torch.cuda.synchronize()
    # the call took no device memory (the driver's free-memory figure is what any allocation would move) ...
    assert torch.cuda.mem_get_info()[0] == free_before
    # ... and none of its bounded device-side waits expired
    assert engine.static_prefill_status() == 0
    return got, expected


def test_static_scratch_matches_caller_scratch_twice(engine, oracle):
    import torch

    _, codes, scales, s2 = make_weight(640, 2560, seed=31)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    # the set-up call (first on this device): it resolves the built-in array, which is when the driver materialises
    # the library's 24 MiB of static device data; from then on a call must leave the free-memory figure alone
    engine.project_prefill_static(w, torch.zeros((8, 2560), dtype=torch.bfloat16, device="cuda"))
    torch.cuda.synchronize()
    # first call: a large activation fills the built-in scratch; second call: a smaller one with other values
    for m, seed in ((300, 1), (130, 2)):
        x = to_torch_bf16(make_activations(m, 2560, seed, outlier_frac=0.001))
        got, expected = _both_paths(engine, w, x)
        err = oracle.rel_l2(got.float().cpu().numpy(), expected.float().cpu().numpy())
        assert err <= REL_L2_TOL, err
        assert torch.equal(got, expected)


def test_static_scratch_rejects_oversized_activation(engine):
    import torch

    L = engine.lib()
    _, codes, scales, s2 = make_weight(128, 9216, seed=3)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    cap = int(L.q35b_static_prefill_capacity_bytes())
    m = cap // (9216 // 2) + 200  # codes alone exceed the capacity
    x = torch.zeros((m, 9216), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((m, 128), dtype=torch.bfloat16, device="cuda")
    rc = L.q35b_project_prefill_bf16_static(w.handle, C.c_void_p(x.data_ptr()), m, C.c_float(0.0),
                                            C.c_void_p(out.data_ptr()), out.stride(0), None)
    assert rc == 2
    assert b"built-in scratch holds" in L.q35b_last_error()
