"""W4A16 decode projection on the GPU (through the C ABI) against the CPU oracle.
Tolerance: relative L2 error <= 1e-3 per output matrix (the BF16 output rounding alone is ~2e-3 per element max,
~1.1e-3/sqrt(3) in L2, so the fp32 result is compared through the same BF16 rounding as the oracle's)."""
import numpy as np
import pytest

from helpers import from_torch_bf16, make_activations, make_weight, to_torch_bf16

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-3


def _check(engine, oracle, n, k, m, seed, kernel=-1, **wkw):
    _, codes, scales, s2 = make_weight(n, k, seed, **wkw)
    xb = make_activations(m, k, seed + 1, outlier_frac=0.001)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    y = engine.gemv_w4a16(w, to_torch_bf16(xb), kernel=kernel)
    yb = from_torch_bf16(y)
    eb, ef = oracle.gemv_bf16(codes, scales, s2, xb, threads=8)
    err = oracle.rel_l2(oracle.bf16_to_f32(yb), oracle.bf16_to_f32(eb))
    assert err <= REL_L2_TOL, (n, k, m, err)
    # element-wise: within one BF16 ulp of the oracle (different fp32 summation order only)
    yf32, ef32 = oracle.bf16_to_f32(yb), oracle.bf16_to_f32(eb)
    rms = float(np.sqrt(np.mean(ef.astype(np.float64) ** 2)))
    assert np.all(np.abs(yf32 - ef32) <= np.abs(ef32) * 2.0 ** -7 + 1e-4 * rms + 1e-30)
    w.close()
    return err


@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 6, 7, 8])
def test_config1_shape_all_m(engine, oracle, m):
    _check(engine, oracle, 3584, 1024, m, seed=10 + m)


@pytest.mark.parametrize("n,k", [(4096, 1024), (1024, 2048), (7168, 1024), (1024, 3584)])
def test_decode_step_shapes_0p8b(engine, oracle, n, k):
    _check(engine, oracle, n, k, 1, seed=n + k)


@pytest.mark.parametrize("n,k,m", [(2560, 9216, 1), (2560, 4096, 4), (1024, 2560, 8), (512, 2560, 2)])
def test_4b_class_shapes(engine, oracle, n, k, m):
    _check(engine, oracle, n, k, m, seed=n + k + m)


@pytest.mark.parametrize("n,k,m", [(1, 32, 1), (3, 64, 2), (17, 96, 1), (257, 160, 3), (129, 1056, 8), (16, 2560, 1),
                                   (5, 48, 1), (33, 16, 2), (7, 80, 8)])
def test_ragged_and_small_shapes(engine, oracle, n, k, m):
    _check(engine, oracle, n, k, m, seed=n * 7 + k)


def test_row_outliers(engine, oracle):
    _check(engine, oracle, 512, 2560, 1, seed=99, row_outlier_frac=0.01)


def test_all_codes_and_scale_bytes(engine, oracle):
    """Every E2M1 code and every E4M3 byte the reference decodes (sign bit and 0x7f included)."""
    rng = np.random.default_rng(0)
    n, k = 256, 512
    codes = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    scales = rng.integers(0, 256, size=(n, k // 16), dtype=np.uint8)
    scales[:8] = np.arange(256, dtype=np.uint8).reshape(8, 32)
    s2 = 1.0 / 1024
    xb = make_activations(2, k, 3)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    yb = from_torch_bf16(engine.gemv_w4a16(w, to_torch_bf16(xb)))
    eb, _ = oracle.gemv_bf16(codes, scales, s2, xb, threads=8)
    assert oracle.rel_l2(oracle.bf16_to_f32(yb), oracle.bf16_to_f32(eb)) <= REL_L2_TOL


@pytest.mark.parametrize("m", [1, 4, 5, 8])
def test_every_unsigned_scale_byte_through_the_streaming_kernel(engine, oracle, m):
    """All 128 unsigned E4M3 bytes (zero, the subnormals 0x01..0x07, 0x7f = 480) as block scales of the streaming
    kernel, which for five to eight tokens folds the scale into its fp16 operand: every block's byte is its index
    modulo 128, so each row meets every byte, with every E2M1 code around it."""
    rng = np.random.default_rng(m)
    n, k = 384, 2048
    codes = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    scales = ((np.arange(n)[:, None] * 5 + np.arange(k // 16)[None, :]) % 128).astype(np.uint8)
    s2 = 1.0 / 4096
    xb = make_activations(m, k, 30 + m, outlier_frac=0.002)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    yb = from_torch_bf16(engine.gemv_w4a16(w, to_torch_bf16(xb), kernel=engine.GEMV_STREAM))
    eb, _ = oracle.gemv_bf16(codes, scales, s2, xb, threads=8)
    assert oracle.rel_l2(oracle.bf16_to_f32(yb), oracle.bf16_to_f32(eb)) <= REL_L2_TOL
    # blocks whose scale is a subnormal or zero only: the small products must not be flushed
    tiny = scales.copy()
    tiny[:] = (np.arange(n)[:, None] + np.arange(k // 16)[None, :]) % 8
    w2 = engine.Nvfp4Weight.from_host(codes, tiny, 1.0)
    yb2 = from_torch_bf16(engine.gemv_w4a16(w2, to_torch_bf16(xb), kernel=engine.GEMV_STREAM))
    eb2, _ = oracle.gemv_bf16(codes, tiny, 1.0, xb, threads=8)
    assert oracle.rel_l2(oracle.bf16_to_f32(yb2), oracle.bf16_to_f32(eb2)) <= REL_L2_TOL
    w.close()
    w2.close()


def test_f32_contract_of_reference_benchmark(engine, oracle):
    """fp32 input x[i] = ((i%17)-8)/17 scaled by input_scale, fp32 output: the reference bench's check
    (src/runtime/cuda_bench.cu:2085-2100) on its first 64 rows, max_abs_error style."""
    import torch

    n, k = 3584, 1024
    _, codes, scales, s2 = make_weight(n, k, seed=42)
    x = np.array([np.float32((i % 17) - 8) / np.float32(17.0) for i in range(k)], dtype=np.float32)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2, input_scale=0.5)
    y = engine.gemv_w4a16_f32(w, torch.from_numpy(x).cuda(), input_scale=0.5).cpu().numpy()
    exp = oracle.matvec_f32(codes, scales, 0.5, s2, x)
    assert np.max(np.abs(y[:64] - exp[:64])) < 1e-6
    assert oracle.rel_l2(y, exp) < 1e-5


def test_sharded_rows_concatenate(engine, oracle):
    n, k = 2560, 1024
    _, codes, scales, s2 = make_weight(n, k, seed=7)
    xb = make_activations(2, k, 8)
    x = to_torch_bf16(xb)
    full = engine.Nvfp4Weight.from_host(codes, scales, s2)
    y_full = from_torch_bf16(engine.gemv_w4a16(full, x))
    for g in (2, 8):
        parts = []
        for i in range(g):
            w = engine.Nvfp4Weight.from_host(codes, scales, s2, shard_index=i, shard_count=g)
            assert (w.row_begin, w.rows) == engine.shard_range(n, i, g)
            parts.append(from_torch_bf16(engine.gemv_w4a16(w, x)))
        assert np.array_equal(np.concatenate(parts, axis=1), y_full)


def test_errors(engine):
    import torch

    _, codes, scales, s2 = make_weight(16, 64, seed=1)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    x9 = torch.zeros((9, 64), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(engine.Q35bError) as e:
        engine.gemv_w4a16(w, x9)
    assert e.value.status == 2
    with pytest.raises(engine.Q35bError):
        engine.gemv_w4a16(w, x9[:1].contiguous(), kernel=12345)
    with pytest.raises(engine.Q35bError):
        engine.Nvfp4Weight.from_host(codes, scales[:, :3], s2)
