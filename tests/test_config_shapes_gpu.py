"""Every shape the benchmark times, at its full size, against the CPU oracle on sampled output rows.

Decode (W4A16): the 4B-class projections gate+up [18432, 2560] (plain, not fused), down [2560, 9216], in-projection
[10240, 2560], out-projection [2560, 4096] and the sweep's [32768, 2560], M = 1, 2, 4, 8, run as one work list per M
(the launch the benchmark times) and as single projections through both decode kernels.
Prefill (W4A4): the sweep's four (K, N) shapes at M = 16, 128, 1024, 4096 with 1 % of the weight rows scaled x8.

Weights are quantised on the GPU (bit-exactness of that quantiser against the oracle is covered elsewhere); the
oracle then recomputes a random sample of output rows from the very bytes the kernels read.
Tolerance: relative L2 <= 1e-3 over the sampled rows of each output matrix."""
import numpy as np
import pytest

from helpers import from_torch_bf16

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-3
DECODE_SHAPES = [(18432, 2560), (2560, 9216), (10240, 2560), (2560, 4096), (32768, 2560)]  # (N, K)
SWEEP_SHAPES = [(3584, 1024), (9216, 2560), (2560, 9216), (32768, 2560)]  # (N, K)


def _gpu_weight(engine, torch, n, k, seed, row_outliers):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn((n, k), generator=gen, device="cuda") * 0.02
    if row_outliers:
        w[torch.randperm(n, generator=gen, device="cuda")[: max(1, -(-n // 100))]] *= 8.0
    codes, scales, s2 = engine.quantize_weight(w)
    return codes, scales, s2


def _activations(torch, m, k, seed, channel_outliers=True):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((m, k), generator=gen, device="cuda")
    if channel_outliers:
        x[:, torch.randperm(k, generator=gen, device="cuda")[: max(1, -(-k // 1000))]] *= 20.0
    return x.to(torch.bfloat16)


def _tiled_to_rowmajor(tiled, rows, scale_cols):
    r = np.arange(rows)[:, None]
    c = np.arange(scale_cols)[None, :]
    padded = (scale_cols + 3) // 4 * 4
    off = (((r // 128) * (padded // 4) + c // 4) * 32 + (r % 32)) * 16 + ((r % 128) // 32) * 4 + (c % 4)
    return tiled[off]


@pytest.fixture(scope="module")
def decode_weights(engine):
    import torch

    out = []
    for j, (n, k) in enumerate(DECODE_SHAPES):
        codes, scales, s2 = _gpu_weight(engine, torch, n, k, seed=900 + j, row_outliers=(n == 32768))
        rows = np.sort(np.random.default_rng(j).choice(n, size=48, replace=False))
        out.append({"n": n, "k": k, "s2": s2, "w": engine.Nvfp4Weight.from_device(codes, scales, s2), "rows": rows,
                    "codes": codes[rows].cpu().numpy(), "scales": scales[rows].cpu().numpy()})
    return out


def _check_decode(oracle, entry, xb, yb):
    eb, _ = oracle.gemv_bf16(entry["codes"], entry["scales"], entry["s2"], xb, threads=8)
    err = oracle.rel_l2(oracle.bf16_to_f32(yb[:, entry["rows"]]), oracle.bf16_to_f32(eb))
    assert err <= REL_L2_TOL, (entry["n"], entry["k"], xb.shape[0], err)


@pytest.mark.parametrize("m", [1, 2, 4, 8])
def test_decode_work_list_at_full_size(engine, oracle, decode_weights, m):
    import torch

    items = []
    for j, e in enumerate(decode_weights):
        x = _activations(torch, m, e["k"], seed=50 + 10 * m + j)
        y = torch.zeros((m, e["n"]), dtype=torch.bfloat16, device="cuda")
        items.append((e["w"], x, y))
    batch = engine.GemvBatch(items, m)
    batch.run()
    torch.cuda.synchronize()
    assert batch.status() == 0
    for e, (_, x, y) in zip(decode_weights, items):
        _check_decode(oracle, e, from_torch_bf16(x), from_torch_bf16(y))


@pytest.mark.parametrize("m", [1, 8])
def test_decode_single_projection_kernels_at_full_size(engine, oracle, decode_weights, m):
    import torch

    for j, e in enumerate(decode_weights):
        x = _activations(torch, m, e["k"], seed=70 + m + j)
        for kernel in (engine.GEMV_SIMT, engine.GEMV_STREAM):
            y = engine.gemv_w4a16(e["w"], x, kernel=kernel)
            _check_decode(oracle, e, from_torch_bf16(x), from_torch_bf16(y))


@pytest.mark.parametrize("m", [16, 128, 1024, 4096])
@pytest.mark.parametrize("n,k", SWEEP_SHAPES)
def test_prefill_sweep_with_row_outliers(engine, oracle, m, n, k):
    import torch

    codes, scales, s2 = _gpu_weight(engine, torch, n, k, seed=n + k + m, row_outliers=True)
    w = engine.Nvfp4Weight.from_device(codes, scales, s2)
    x = _activations(torch, m, k, seed=3 * m + n, channel_outliers=False)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    a_codes, a_scales, g = engine.quantize_activations(x)
    c = engine.gemm_w4a4(w, a_codes, a_scales, g, m, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    rng = np.random.default_rng(n + m)
    n_rows = 16 if m * k > 2 ** 22 else 48
    # the x8 rows are what stresses the block scales: always sample some of them
    big = torch.nonzero(scales.max(dim=1).values >= 0x70).flatten().cpu().numpy()
    rows = np.unique(np.concatenate([rng.choice(n, size=n_rows, replace=False), big[:8]]))
    h_codes, h_scales = codes[rows].cpu().numpy(), scales[rows].cpu().numpy()
    a_c = a_codes.cpu().numpy()
    a_s = _tiled_to_rowmajor(a_scales.cpu().numpy(), m, k // 16)
    eb, _ = oracle.gemm_w4a4(h_codes, h_scales, s2, a_c, a_s, float(g.item()), threads=8)
    err = oracle.rel_l2(oracle.bf16_to_f32(from_torch_bf16(c)[:, rows]), oracle.bf16_to_f32(eb))
    assert err <= REL_L2_TOL, (m, n, k, err)


def test_misaligned_activations_are_rejected(engine):
    """The vector decode kernel reads activations with 16-byte loads: a pointer that is not 16-byte aligned must come
    back as an argument error, not as a launch."""
    import ctypes as C

    import torch

    codes, scales, s2 = _gpu_weight(engine, torch, 256, 1024, seed=1, row_outliers=False)
    w = engine.Nvfp4Weight.from_device(codes, scales, s2)
    x = torch.zeros(1024 + 8, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(256, dtype=torch.bfloat16, device="cuda")
    L = engine.lib()
    before = engine.launch_count()
    for kernel in (engine.GEMV_SIMT, engine.GEMV_STREAM, engine.GEMV_AUTO):
        rc = L.q35b_gemv_w4a16_bf16(w.handle, C.c_void_p(x.data_ptr() + 2), 1, C.c_void_p(y.data_ptr()), kernel, None)
        if kernel == engine.GEMV_AUTO:
            assert rc == 1  # falls to the vector kernel, which rejects it
        else:
            assert rc == 1, L.q35b_last_error()
        assert b"aligned" in L.q35b_last_error()
    assert engine.launch_count() == before
    xf = torch.zeros(1024 + 4, dtype=torch.float32, device="cuda")
    yf = torch.zeros(256, dtype=torch.float32, device="cuda")
    assert L.q35b_gemv_w4a16_f32(w.handle, C.c_void_p(xf.data_ptr() + 4), C.c_float(1.0), C.c_void_p(yf.data_ptr()),
                                 engine.GEMV_SIMT, None) == 1


def test_fp32_activations_quantise_like_the_oracle(engine, oracle):
    """q35b_quantize_nvfp4_f32 (the reference prefill benchmark's input type): bytes equal to the oracle's."""
    import torch

    rng = np.random.default_rng(8)
    x = rng.standard_normal((130, 1024)).astype(np.float32)
    x[:, 7] *= 20.0
    x[3, :64] = 0.0
    codes, scales, g = engine.quantize_activations(torch.from_numpy(x).cuda())
    e_codes, e_scales, e_g = oracle.quantize_nvfp4(x)
    assert np.float32(g.item()) == np.float32(e_g)
    assert np.array_equal(codes.cpu().numpy(), e_codes)
    assert np.array_equal(scales.cpu().numpy(), oracle.swizzle_scales(e_scales))
