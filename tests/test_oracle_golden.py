"""The CPU oracle against the committed golden vectors (generated from the reference's own host functions by
tests/golden/make_golden.py)."""
from pathlib import Path

import numpy as np
import pytest

G = np.load(Path(__file__).parent / "golden" / "nvfp4_golden.npz")


def test_decode_tables(oracle):
    assert np.array_equal(oracle.decode_e4m3_table().view(np.uint32), G["e4m3_table"].view(np.uint32))
    assert np.array_equal(oracle.decode_e2m1_table().view(np.uint32), G["e2m1_table"].view(np.uint32))
    # facts the engine relies on: 0x7f is 480 (not NaN), subnormals are m * 2^-9, sign bit honoured
    t = oracle.decode_e4m3_table()
    assert t[0x7F] == 480.0 and t[0x7E] == 448.0 and t[1] == 2.0 ** -9 and t[0x81] == -(2.0 ** -9)


def test_encode_ue4m3(oracle):
    v = G["ue4m3_in"].view(np.float32)
    assert np.array_equal(oracle.encode_ue4m3(v), G["ue4m3_out"])


def test_encode_e2m1(oracle):
    v = G["e2m1_in"].view(np.float32)
    assert np.array_equal(oracle.encode_e2m1(v), G["e2m1_out"])


def test_encode_tie_rules(oracle):
    # ties go to the smaller magnitude / lower byte (strict '<' in the reference scan)
    assert list(oracle.encode_e2m1(np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32))) == [0, 1, 2, 3, 4, 5, 6]
    assert list(oracle.encode_e2m1(np.array([-0.25, -5.0, -7.0, 100.0], np.float32))) == [8, 14, 15, 7]
    assert list(oracle.encode_ue4m3(np.array([464.0, 464.5, 1e-8, 2.0 ** -10, 2.0 ** -10 * 1.01], np.float32))) == [0x7E, 0x7F, 0, 0, 1]


def test_swizzle(oracle):
    assert np.array_equal(oracle.swizzle_scales(G["sw_in"]), G["sw_out"])
    rows, cols = G["sw_in"].shape
    sw = G["sw_out"]
    for r in (0, 1, 31, 32, 127, 128, 129):
        for c in range(cols):
            assert sw[oracle.tiled_scale_offset(r, c, cols)] == G["sw_in"][r, c]


def test_matvec_fixture(oracle):
    y = oracle.matvec_f32(G["mv_codes"], G["mv_scales"], float(G["mv_input_scale"]), float(G["mv_s2"]), G["mv_x"])
    assert np.array_equal(y.view(np.uint32), G["mv_y"].view(np.uint32))


def test_reference_recipe_quantiser(oracle):
    codes, scales = oracle.act_quant_reference(G["q_x"][None, :])
    assert np.array_equal(codes[0], G["q_codes"])
    assert np.array_equal(scales[0], G["q_scales"])
    codes_sw, _ = oracle.act_quant_reference(G["q_x"][None, :], swap_nibbles=True)
    assert np.array_equal(codes_sw[0], G["q_codes_swapped"])
    assert np.array_equal(oracle.swizzle_scales(scales), G["q_scales_tiled"])


def test_engine_recipe_properties(oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 256)).astype(np.float32)
    x[:, 7] *= 20
    x[2, 32:48] = 0.0  # an all-zero block
    codes, scales, g = oracle.quantize_nvfp4(x)
    assert g == pytest.approx(np.abs(x).max() / (6 * 448), rel=1e-6)
    assert scales.max() <= 0x7E
    assert scales[2, 2] == 0 and not codes[2, 16:24].any()
    # dequantised values stay within half a code step of the input, block by block
    e2 = oracle.decode_e2m1_table()
    e4 = oracle.decode_e4m3_table()
    lo, hi = codes & 0xF, codes >> 4
    vals = np.empty_like(x)
    vals[:, 0::2], vals[:, 1::2] = e2[lo], e2[hi]
    deq = vals * np.repeat(e4[scales], 16, axis=1) * g
    blk_scale = np.repeat(e4[scales], 16, axis=1) * g
    assert np.all(np.abs(deq - x) <= 1.0 * blk_scale + 1e-12)
    # bf16 input path gives the same bytes as the fp32 path on bf16-representable data
    xb = oracle.bf16_round(x)
    c1, s1, g1 = oracle.quantize_nvfp4(xb)
    c2, s2, g2 = oracle.quantize_nvfp4(oracle.bf16_to_f32(xb))
    assert np.array_equal(c1, c2) and np.array_equal(s1, s2) and g1 == g2
    # a supplied global scale is used verbatim; saturation at 0x7e
    _, s3, g3 = oracle.quantize_nvfp4(x, global_scale=1e-6)
    assert g3 == pytest.approx(1e-6) and s3.max() == 0x7E


def test_gemv_bf16_matches_matvec(oracle):
    from helpers import make_activations, make_weight

    _, codes, scales, s2 = make_weight(40, 512, seed=1)
    xb = make_activations(3, 512, seed=2)
    yb, yf = oracle.gemv_bf16(codes, scales, s2, xb)
    for t in range(3):
        ref = oracle.matvec_f32(codes, scales, 1.0, s2, oracle.bf16_to_f32(xb[t]))
        assert np.array_equal(ref.view(np.uint32), yf[t].view(np.uint32))
    assert np.array_equal(yb, oracle.bf16_round(yf))
    yb4, yf4 = oracle.gemv_bf16(codes, scales, s2, xb, threads=4)
    assert np.array_equal(yf4, yf) and np.array_equal(yb4, yb)


def test_w4a4_close_to_w4a16(oracle):
    from helpers import make_activations, make_weight

    _, codes, scales, s2 = make_weight(32, 512, seed=5)
    xb = make_activations(4, 512, seed=6, outlier_frac=0.01)
    a_codes, a_scales, g = oracle.quantize_nvfp4(xb)
    cb, cf = oracle.gemm_w4a4(codes, scales, s2, a_codes, a_scales, g)
    _, yf = oracle.gemv_bf16(codes, scales, s2, xb)
    # activation quantisation noise only: FP4 with per-16 scales is a few percent in relative L2
    assert oracle.rel_l2(cf, yf) < 0.15
    # shard slicing is exact
    cb2, cf2 = oracle.gemm_w4a4(codes, scales, s2, a_codes, a_scales, g, n_begin=8, n_end=24)
    assert np.array_equal(cf2, cf[:, 8:24]) and np.array_equal(cb2, cb[:, 8:24])
