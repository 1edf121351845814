"""NVFP4 quantisation on the GPU against the CPU oracle: codes, block scales and the per-tensor scale are bit-exact."""
import numpy as np
import pytest

from helpers import make_activations, to_torch_bf16

pytestmark = pytest.mark.gpu


def _tiled_to_rowmajor(oracle, tiled, rows, scale_cols):
    out = np.zeros((rows, scale_cols), dtype=np.uint8)
    for r in range(rows):
        for c in range(scale_cols):
            out[r, c] = tiled[oracle.tiled_scale_offset(r, c, scale_cols)]
    return out


def _run(engine, oracle, xb, global_scale=0.0):
    m, k = xb.shape
    codes, scales, g = engine.quantize_activations(to_torch_bf16(xb), global_scale)
    e_codes, e_scales, e_g = oracle.quantize_nvfp4(xb, global_scale)
    assert np.float32(g.item()).view(np.uint32) == np.float32(e_g).view(np.uint32)
    assert np.array_equal(codes.cpu().numpy(), e_codes)
    tiled = scales.cpu().numpy()
    assert np.array_equal(tiled, oracle.swizzle_scales(e_scales))  # padding bytes are zero as well
    return codes, scales, g


@pytest.mark.parametrize("m,k", [(1, 1024), (8, 2560), (128, 1024), (130, 2560), (512, 2560), (257, 9216)])
def test_bit_exact_dynamic_scale(engine, oracle, m, k):
    _run(engine, oracle, make_activations(m, k, seed=m + k, outlier_frac=0.001))


@pytest.mark.parametrize("m,k", [(1, 16), (3, 48), (5, 80), (127, 16), (2, 4112)])
def test_ragged_k(engine, oracle, m, k):
    _run(engine, oracle, make_activations(m, k, seed=m * 3 + k))


def test_static_scale_and_saturation(engine, oracle):
    xb = make_activations(16, 512, seed=4)
    _run(engine, oracle, xb, global_scale=0.01)
    _run(engine, oracle, xb, global_scale=1e-7)  # block scales saturate at 0x7e, codes at +-6


def test_special_values(engine, oracle):
    x = np.zeros((4, 256), dtype=np.float32)
    x[1, :16] = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0]
    x[2, 17] = 3e38
    x[3, 40] = -1e-30
    _run(engine, oracle, oracle.bf16_round(x))
    _run(engine, oracle, np.zeros((2, 64), dtype=np.uint16))  # all zero: g = 1, everything zero


def test_repeated_calls_keep_workspace_clean(engine, oracle):
    a = make_activations(64, 1024, seed=1)
    b = make_activations(64, 1024, seed=2) 
    for xb in (a, b, a):
        _run(engine, oracle, xb)


def test_reference_recipe_bytes(engine, oracle):
    """The reference's own recipe (unrounded divisor, even element in the high nibble) reproduces the oracle's
    restatement of cuda_bench.cu:2221-2237 byte for byte."""
    xb = make_activations(40, 1024, seed=9, outlier_frac=0.001)
    codes, scales = engine.quantize_activations_reference_recipe(to_torch_bf16(xb), swap_nibbles=True)
    e_codes, e_scales = oracle.act_quant_reference(oracle.bf16_to_f32(xb), swap_nibbles=True)
    assert np.array_equal(codes.cpu().numpy(), e_codes)
    assert np.array_equal(scales.cpu().numpy(), oracle.swizzle_scales(e_scales))


def test_weight_quantiser(engine, oracle):
    import torch

    rng = np.random.default_rng(21)
    w = (rng.standard_normal((300, 1024)) * 0.02).astype(np.float32)
    w[::100] *= 8
    codes, scales, s2 = engine.quantize_weight(torch.from_numpy(w).cuda())
    e_codes, e_scales, e_s2 = oracle.quantize_nvfp4(w)
    assert np.float32(s2).view(np.uint32) == np.float32(e_s2).view(np.uint32)
    assert np.array_equal(codes.cpu().numpy(), e_codes) and np.array_equal(scales.cpu().numpy(), e_scales)
    # device-side repack gives the same projection as the host-side one
    xb = make_activations(1, 1024, 5)
    w_dev = engine.Nvfp4Weight.from_device(codes, scales, s2)
    w_host = engine.Nvfp4Weight.from_host(e_codes, e_scales, e_s2)
    y1 = engine.gemv_w4a16(w_dev, to_torch_bf16(xb))
    y2 = engine.gemv_w4a16(w_host, to_torch_bf16(xb))
    assert torch.equal(y1, y2)


def test_full_size_round_trip_property(engine, oracle):
    """Full benchmark size (M=4096, K=2560): dequantised codes reproduce the input to within half a code step of
    each block's scale, and re-quantising the dequantised tensor with the same g is idempotent."""
    import torch

    m, k = 4096, 2560
    g0 = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((m, k), generator=g0, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    codes, scales, g = engine.quantize_activations(x)
    gval = float(g.item())
    assert gval == pytest.approx(float(x.abs().max().float()) / (6 * 448), rel=1e-6)
    e2 = torch.tensor(oracle.decode_e2m1_table(), device="cuda")
    e4 = torch.tensor(oracle.decode_e4m3_table(), device="cuda")
    # row-major view of the tiled scales via the offset function
    r = torch.arange(m, device="cuda")[:, None]
    c = torch.arange(k // 16, device="cuda")[None, :]
    off = (((r // 128) * ((k // 16) // 4) + c // 4) * 32 + (r % 32)) * 16 + ((r % 128) // 32) * 4 + (c % 4)
    sc = e4[scales[off.reshape(-1)].long()].reshape(m, k // 16)
    vals = torch.empty((m, k), device="cuda")
    vals[:, 0::2] = e2[(codes & 0xF).long()]
    vals[:, 1::2] = e2[(codes >> 4).long()]
    blk = sc.repeat_interleave(16, dim=1) * gval
    deq = vals * blk
    assert torch.all((deq - x.float()).abs() <= blk * 1.0 + 1e-12)
    codes2, scales2, _ = engine.quantize_activations(deq.to(torch.bfloat16), global_scale=gval)
    same = (codes2 == codes).float().mean().item()
    # not exactly idempotent: rounding the dequantised values to BF16 moves some across a code boundary
    assert same > 0.9


@pytest.mark.parametrize("spread", [3, 24])
def test_division_at_every_rounding_boundary(engine, oracle, spread):
    """The block quantiser does not run sixteen IEEE divisions and sixteen threshold scans: it multiplies by a shared
    refined reciprocal and hands the products to the hardware E2M1 converter unless one of them lies within 8 ulp of
    a rounding boundary, in which case the block is redone with correctly rounded quotients and the ties-down
    encoder.  Values are placed -spread..+spread ulp around d times every E2M1 rounding boundary (0.25 .. 5.0) - 3
    keeps every probe on the exact path, 24 straddles the hand-over between the two - for thousands of divisors d
    spread over 60 binary orders of magnitude (so that the plain-division path for extreme exponents runs as well):
    codes must equal the oracle's, which divides with the host's IEEE division."""
    import torch

    rng = np.random.default_rng(77)
    e4 = oracle.decode_e4m3_table().astype(np.float32)
    bounds = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    n, k = 64, 1024
    for trial in range(12):
        top = np.float32(10.0 ** rng.uniform(-25, 25))
        w = np.zeros((n, k), dtype=np.float32)
        amax = (top * 10.0 ** rng.uniform(-6, 0, size=(n, k // 16))).astype(np.float32)
        amax[0, 0] = top
        w[:, 0::16] = amax * rng.choice(np.array([-1.0, 1.0], dtype=np.float32), size=amax.shape)
        _, scales0, g = oracle.quantize_nvfp4(w)
        d = (np.maximum(e4[scales0], np.float32(1e-8)) * np.float32(g)).astype(np.float32)  # [n, k/16]
        for j in range(1, 16):
            target = (bounds[rng.integers(0, 7, size=d.shape)] * d).astype(np.float32)
            bits = target.view(np.int32) + rng.integers(-spread, spread + 1, size=d.shape, dtype=np.int32)
            w[:, j::16] = bits.view(np.float32) * rng.choice(np.array([-1.0, 1.0], dtype=np.float32), size=d.shape)
        e_codes, e_scales, e_g = oracle.quantize_nvfp4(w)
        assert np.array_equal(e_scales, scales0) and e_g == g  # the probes did not move any amax
        codes, scales, s2 = engine.quantize_weight(torch.from_numpy(w).cuda())
        assert np.float32(s2).view(np.uint32) == np.float32(e_g).view(np.uint32)
        assert np.array_equal(scales.cpu().numpy(), e_scales)
        assert np.array_equal(codes.cpu().numpy(), e_codes), f"trial {trial}: {(codes.cpu().numpy() != e_codes).sum()} code bytes differ"


def test_zeros_signed_zeros_and_values_that_round_to_zero(engine, oracle):
    """Exact zeros and -0 encode as code 0; a negative value too small for the first level keeps its sign bit
    (code 8), as (value < 0) does in the reference's encoder; blocks mixing them with ordinary values included."""
    rng = np.random.default_rng(5)
    x = rng.standard_normal((64, 1024)).astype(np.float32)
    x[rng.random(x.shape) < 0.3] = 0.0
    x[rng.random(x.shape) < 0.1] = -0.0
    tiny = rng.random(x.shape) < 0.1
    x[tiny] = (-1e-4 * rng.random(x.shape).astype(np.float32))[tiny]
    x[5] = 0.0
    x[6] = -0.0
    xb = oracle.bf16_round(x)
    codes, _, _ = _run(engine, oracle, xb)
    assert (codes.cpu().numpy() & 0x08).any()  # some negative zeros were produced, and matched the oracle
    _run(engine, oracle, xb, global_scale=2.0 ** -9)  # a power-of-two scale: many quotients land exactly on boundaries
    q = (rng.integers(-24, 25, size=(32, 512)) * 0.25).astype(np.float32)  # multiples of 0.25: ties everywhere
    _run(engine, oracle, oracle.bf16_round(q), global_scale=0.125)  # blocks holding a +-6 get the divisor 1.0
