"""W4A4 prefill GEMM (tcgen05 block-scaled FP4) through the C ABI against the CPU oracle, which quantises the
activations with the identical NVFP4 recipe.  Tolerance: relative L2 error <= 1e-3 per output matrix."""
import numpy as np
import pytest

from helpers import from_torch_bf16, make_activations, make_weight, to_torch_bf16

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-3


def _tiled_to_rowmajor(tiled, rows, scale_cols):
    r = np.arange(rows)[:, None]
    c = np.arange(scale_cols)[None, :]
    padded = (scale_cols + 3) // 4 * 4
    off = (((r // 128) * (padded // 4) + c // 4) * 32 + (r % 32)) * 16 + ((r % 128) // 32) * 4 + (c % 4)
    return tiled[off]


def _run(engine, oracle, m, n, k, seed, **wkw):
    import torch

    _, codes, scales, s2 = make_weight(n, k, seed, **wkw)
    xb = make_activations(m, k, seed + 1, outlier_frac=0.001)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    a_codes, a_scales, g = engine.quantize_activations(to_torch_bf16(xb))
    c = engine.gemm_w4a4(w, a_codes, a_scales, g, m, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"device-side wait expired, code {int(status.item())}"
    e_codes, e_scales, e_g = oracle.quantize_nvfp4(xb)
    eb, ef = oracle.gemm_w4a4(codes, scales, s2, e_codes, e_scales, e_g, threads=8)
    cb = from_torch_bf16(c)
    err = oracle.rel_l2(oracle.bf16_to_f32(cb), oracle.bf16_to_f32(eb))
    assert err <= REL_L2_TOL, (m, n, k, err)
    return err


@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (128, 128, 64), (1, 128, 64), (16, 256, 1024)])
def test_single_tile(engine, oracle, m, n, k):
    _run(engine, oracle, m, n, k, seed=m + n + k)


@pytest.mark.parametrize("m,n,k", [(130, 384, 512), (300, 1000, 1024), (257, 520, 320), (64, 2560, 2560), (512, 640, 9216)])
def test_ragged_tiles(engine, oracle, m, n, k):
    _run(engine, oracle, m, n, k, seed=m * 3 + n + k)


def test_row_outliers_stress_block_scales(engine, oracle):
    _run(engine, oracle, 128, 512, 1024, seed=77, row_outlier_frac=0.01)


def test_k_not_multiple_of_64_is_rejected(engine):
    import torch

    _, codes, scales, s2 = make_weight(128, 80, seed=1)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    x = torch.zeros((4, 80), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(engine.Q35bError) as e:
        engine.project_prefill(w, x)
    assert e.value.status == 2


@pytest.mark.parametrize("m", [512, 4096])
@pytest.mark.parametrize("n,k", [(18432, 2560), (2560, 9216)])
def test_full_size_sampled_rows_and_linearity(engine, oracle, m, n, k):
    """Benchmark sizes: weights quantised on the GPU; 24 sampled output rows (all tokens) against the oracle fed with
    the GPU quantiser's bytes (bit-exactness of those is covered in test_quant_gpu), plus the scaling property
    C(2^3 * g) == 2^3 * C(g) which holds exactly in BF16."""
    import torch

    gen = torch.Generator(device="cuda").manual_seed(n + k + m)
    wf = torch.randn((n, k), generator=gen, device="cuda") * 0.02
    codes, scales, s2 = engine.quantize_weight(wf)
    w = engine.Nvfp4Weight.from_device(codes, scales, s2)
    x = torch.randn((m, k), generator=gen, device="cuda")
    x[:, torch.randperm(k, generator=gen, device="cuda")[: max(1, -(-k // 1000))]] *= 20
    x = x.to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    a_codes, a_scales, g = engine.quantize_activations(x)
    c = engine.gemm_w4a4(w, a_codes, a_scales, g, m, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    rng = np.random.default_rng(0)
    rows = np.sort(rng.choice(n, size=24, replace=False))
    h_codes, h_scales = codes.cpu().numpy(), scales.cpu().numpy()
    a_c = a_codes.cpu().numpy()
    a_s = _tiled_to_rowmajor(a_scales.cpu().numpy(), m, k // 16)
    gval = float(g.item())
    cb = from_torch_bf16(c)
    exp = np.zeros((m, len(rows)), dtype=np.uint16)
    for j, r in enumerate(rows):
        eb, _ = oracle.gemm_w4a4(h_codes[r:r + 1], h_scales[r:r + 1], s2, a_c, a_s, gval, threads=8)
        exp[:, j] = eb[:, 0]
    err = oracle.rel_l2(oracle.bf16_to_f32(cb[:, rows]), oracle.bf16_to_f32(exp))
    assert err <= REL_L2_TOL, err
    g8 = (g * 8.0).contiguous()
    c8 = engine.gemm_w4a4(w, a_codes, a_scales, g8, m)
    assert torch.equal(c8.float(), c.float() * 8.0)


def test_matches_w4a16_within_activation_noise(engine, oracle):
    """Sanity of the whole prefill path against the unquantised-activation projection (what the reference's own
    prefill check compares with, cuda_bench.cu:2571-2585): FP4 activation noise only."""
    m, n, k = 8, 512, 2560
    _, codes, scales, s2 = make_weight(n, k, seed=5)
    xb = make_activations(m, k, 6)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    c = from_torch_bf16(engine.project_prefill(w, to_torch_bf16(xb)))
    y = from_torch_bf16(engine.gemv_w4a16(w, to_torch_bf16(xb)))
    assert oracle.rel_l2(oracle.bf16_to_f32(c), oracle.bf16_to_f32(y)) < 0.15


def test_gemm_without_a_status_word_reports_into_the_library_word(engine):
    """A call that passes no status word uses the library's own (nothing is launched in front of the kernel for it);
    after clean runs on all three GEMM kernels the getter reads 0."""
    import torch

    for (m, n, k) in ((300, 1024, 512), (64, 512, 512), (16, 3584, 1024)):
        _, codes, scales, s2 = make_weight(n, k, seed=n + m)
        w = engine.Nvfp4Weight.from_host(codes, scales, s2)
        a_codes, a_scales, g = engine.quantize_activations(to_torch_bf16(make_activations(m, k, seed=m)))
        before = engine.launch_count()
        c = engine.gemm_w4a4(w, a_codes, a_scales, g, m)
        assert engine.launch_count() == before + 1
        torch.cuda.synchronize()
        assert c.shape == (m, n)
        assert engine.gemm_default_status() == 0
        w.close()

