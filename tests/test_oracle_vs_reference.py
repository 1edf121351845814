"""The CPU oracle against the reference's own host functions, compiled unmodified into oracle/_ref (skipped where
neither a reference checkout nor a prebuilt shim exists)."""
import numpy as np
import pytest


@pytest.fixture(scope="module")
def ref(oracle):
    R = oracle.ref_lib()
    if R is None:
        pytest.skip("reference shim not built (no reference checkout)")
    return R


def test_decoders_all_bytes(oracle, ref):
    L = oracle.lib()
    for b in range(256):
        assert L.q35o_decode_e4m3(b) == ref.ref_decode_e4m3(b)
    for c in range(16):
        assert L.q35o_decode_e2m1(c) == ref.ref_decode_e2m1(c)


def test_encoders_dense_sweep(oracle, ref):
    L = oracle.lib()
    rng = np.random.default_rng(11)
    # log-uniform magnitudes over the whole useful range plus signed noise
    mags = np.exp(rng.uniform(np.log(1e-6), np.log(2e3), size=30000)).astype(np.float32)
    for v in mags:
        assert L.q35o_encode_ue4m3(float(v)) == ref.ref_encode_ue4m3(float(v))
    vals = (rng.standard_normal(30000) * 3).astype(np.float32)
    for v in vals:
        assert L.q35o_encode_e2m1(float(v)) == ref.ref_encode_e2m1(float(v))


def test_swizzle_shapes(oracle, ref):
    rng = np.random.default_rng(12)
    for rows, cols in [(1, 64), (1, 1), (127, 3), (128, 4), (129, 5), (300, 160)]:
        s = rng.integers(0, 256, size=(rows, cols), dtype=np.uint8)
        mine = oracle.swizzle_scales(s)
        out = np.zeros_like(mine)
        n = ref.ref_swizzle_scales(s.ctypes.data, rows, cols, out.ctypes.data, out.size)
        assert n == mine.size and np.array_equal(mine, out)
