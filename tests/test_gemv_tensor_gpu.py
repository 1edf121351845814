"""The decode work list on the tensor cores (q35b_gemv_batch_create_tensor): weights streamed through tcgen05.mma, the
BF16 activations of every token entering as an NVFP4 digit expansion.  Against the CPU oracle's exact W4A16 result:
relative L2 <= 1e-3 per output matrix (the bound of the exact decode kernels), and with five digits the fp32 error of
the expansion itself stays below 2e-4."""
import numpy as np
import pytest

from helpers import from_torch_bf16, make_activations, make_weight, to_torch_bf16

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-3


def _run_list(engine, torch, shapes, m, digits, seed, residual_on=(), outliers=0.001):
    items, host = [], []
    for j, (n, k) in enumerate(shapes):
        _, codes, scales, s2 = make_weight(n, k, seed=seed + j)
        xb = make_activations(m, k, seed=seed + 50 + j, outlier_frac=outliers)
        w = engine.Nvfp4Weight.from_host(codes, scales, s2)
        y = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
        rb = make_activations(m, n, seed=seed + 90 + j) if j in residual_on else None
        items.append((w, to_torch_bf16(xb), y) + ((to_torch_bf16(rb),) if rb is not None else ()))
        host.append((codes, scales, s2, xb, rb))
    batch = engine.GemvBatch(items, m, digits=digits)
    batch.run()
    batch.run()  # the digit buffers are rewritten by every run
    torch.cuda.synchronize()
    assert batch.status() == 0
    return items, host


@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8])
def test_decode_layer_shapes(engine, oracle, m):
    import torch

    shapes = [(4096, 1024), (1024, 2048), (7168, 1024), (1024, 3584), (1000, 256), (130, 512)]
    items, host = _run_list(engine, torch, shapes, m, 5, seed=300 + m, residual_on=(1, 3))
    for item, (codes, scales, s2, xb, rb) in zip(items, host):
        eb, ef = oracle.gemv_bf16(codes, scales, s2, xb, threads=8)
        if rb is not None:
            eb = oracle.bf16_round(ef + oracle.bf16_to_f32(rb))
        err = oracle.rel_l2(oracle.bf16_to_f32(from_torch_bf16(item[2])), oracle.bf16_to_f32(eb))
        assert err <= REL_L2_TOL, (codes.shape, m, err)


@pytest.mark.parametrize("digits,bound", [(3, 2e-2), (4, 4e-3), (5, 1e-3), (6, 1e-3)])
def test_error_shrinks_with_the_number_of_digits(engine, oracle, digits, bound):
    import torch

    items, host = _run_list(engine, torch, [(2048, 2560)], 4, digits, seed=77)
    codes, scales, s2, xb, _ = host[0]
    eb, _ = oracle.gemv_bf16(codes, scales, s2, xb, threads=8)
    err = oracle.rel_l2(oracle.bf16_to_f32(from_torch_bf16(items[0][2])), oracle.bf16_to_f32(eb))
    assert err <= bound, (digits, err)


def test_gate_up_pair_and_4b_shapes(engine, oracle):
    import torch

    m, k, half = 4, 2560, 1152
    g = make_weight(half, k, seed=1)
    u = make_weight(half, k, seed=2)
    d = make_weight(2560, 9216, seed=3)
    xb = make_activations(m, k, seed=4, outlier_frac=0.001)
    xd = make_activations(m, 9216, seed=5, outlier_frac=0.001)
    gu = engine.Nvfp4Weight.gate_up_from_host(g[1], g[2], g[3], u[1], u[2], u[3])
    dn = engine.Nvfp4Weight.from_host(d[1], d[2], d[3])
    y_gu = torch.zeros((m, half), dtype=torch.bfloat16, device="cuda")
    y_dn = torch.zeros((m, 2560), dtype=torch.bfloat16, device="cuda")
    batch = engine.GemvBatch([(gu, to_torch_bf16(xb), y_gu), (dn, to_torch_bf16(xd), y_dn)], m, digits=5)
    batch.run()
    torch.cuda.synchronize()
    assert batch.status() == 0
    _, gate = oracle.gemv_bf16(g[1], g[2], g[3], xb, threads=8)
    _, up = oracle.gemv_bf16(u[1], u[2], u[3], xb, threads=8)
    exp = oracle.bf16_round((gate / (1 + np.exp(-gate)) * up).astype(np.float32))
    assert oracle.rel_l2(oracle.bf16_to_f32(from_torch_bf16(y_gu)), oracle.bf16_to_f32(exp)) <= 2e-3  # two projections' error
    eb, _ = oracle.gemv_bf16(d[1], d[2], d[3], xd, threads=8)
    assert oracle.rel_l2(oracle.bf16_to_f32(from_torch_bf16(y_dn)), oracle.bf16_to_f32(eb)) <= REL_L2_TOL


def test_special_activations_and_argument_errors(engine, oracle):
    import torch

    n, k = 512, 1024
    _, codes, scales, s2 = make_weight(n, k, seed=9)
    x = np.random.default_rng(1).standard_normal((2, k)).astype(np.float32)
    x[0, :256] = 0.0
    x[1, 300:316] *= 1e-6
    x[1, 7] = 250.0
    xb = oracle.bf16_round(x)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    y = torch.zeros((2, n), dtype=torch.bfloat16, device="cuda")
    batch = engine.GemvBatch([(w, to_torch_bf16(xb), y)], 2, digits=5)
    batch.run()
    torch.cuda.synchronize()
    assert batch.status() == 0
    eb, _ = oracle.gemv_bf16(codes, scales, s2, xb, threads=4)
    assert oracle.rel_l2(oracle.bf16_to_f32(from_torch_bf16(y)), oracle.bf16_to_f32(eb)) <= REL_L2_TOL
    # all-zero activations give exact zeros
    z = torch.zeros((2, k), dtype=torch.bfloat16, device="cuda")
    batch0 = engine.GemvBatch([(w, z, y)], 2, digits=5)
    batch0.run()
    torch.cuda.synchronize()
    assert float(y.float().abs().max()) == 0.0
    with pytest.raises(engine.Q35bError):
        engine.GemvBatch([(w, z, y)], 2, digits=9)
    y2 = torch.zeros((2, n), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(engine.Q35bError) as e:
        engine.GemvBatch([(w, z, y), (w, z, y2, None, 0)], 2, digits=5)  # an item that runs after another one
    assert e.value.status == 1
