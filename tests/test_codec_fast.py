"""The engine's constant-time encoders (host twins of the device code, exported by libq35b) against the oracle's
restatement of the reference scan: every switch point of the scan is located by bisection over fp32 bit patterns and
the fast encoder must switch at exactly the same pattern."""
import numpy as np


def _f(bits: int) -> float:
    return float(np.array([bits], dtype=np.uint32).view(np.float32)[0])


def _switch_points(fn, lo_bits: int, hi_bits: int):
    """All bit patterns b in (lo, hi] where fn(b) != fn(b-1), assuming fn is monotone in b."""
    out = []

    def rec(lo, hi, flo, fhi):
        if flo == fhi:
            return
        if hi - lo == 1:
            out.append(hi)
            return
        mid = (lo + hi) // 2
        fm = fn(_f(mid))
        rec(lo, mid, flo, fm)
        rec(mid, hi, fm, fhi)

    rec(lo_bits, hi_bits, fn(_f(lo_bits)), fn(_f(hi_bits)))
    return out


def test_ue4m3_switch_points(oracle, engine):
    L, E = oracle.lib(), engine.lib()
    lo, hi = 0x00000001, 0x4B7FFFFF  # smallest denormal .. just below 2^24
    pts = _switch_points(lambda v: L.q35o_encode_ue4m3(v), lo, hi)
    assert len(pts) == 127
    for b in pts:
        for d in (-2, -1, 0, 1, 2):
            v = _f(b + d)
            assert E.q35b_debug_encode_ue4m3(v) == L.q35o_encode_ue4m3(v), hex(b + d)
    assert _switch_points(lambda v: E.q35b_debug_encode_ue4m3(v), lo, hi) == pts


def test_ue4m3_specials_and_samples(oracle, engine):
    L, E = oracle.lib(), engine.lib()
    rng = np.random.default_rng(5)
    vals = list(np.exp(rng.uniform(np.log(1e-12), np.log(1e12), size=20000)).astype(np.float32))
    vals += [0.0, -0.0, -3.0, float("nan"), float("inf"), -float("inf"), 1e-45, 2.0 ** 24, 2.0 ** 24 * 1.5, 1e30, 3.4e38]
    for v in vals:
        assert E.q35b_debug_encode_ue4m3(float(v)) == L.q35o_encode_ue4m3(float(v)), v


def test_e2m1_switch_points(oracle, engine):
    L, E = oracle.lib(), engine.lib()
    lo, hi = 0x00000000, 0x497FFFFF  # 0 .. just below 2^20
    pts = _switch_points(lambda v: L.q35o_encode_e2m1(v), lo, hi)
    assert len(pts) == 7
    for b in pts:
        for d in (-1, 0, 1):
            for sign in (0, 0x80000000):
                v = _f((b + d) | sign)
                assert E.q35b_debug_encode_e2m1(v) == L.q35o_encode_e2m1(v), hex(b + d)
    assert _switch_points(lambda v: E.q35b_debug_encode_e2m1(v), lo, hi) == pts
    # every exponent of the encoder's range at a spread of mantissas, both signs
    for e in range(0, 147):
        for mant in (0, 1, 0x1FFFFF, 0x200000, 0x200001, 0x3FFFFF, 0x400000, 0x5FFFFF, 0x600000, 0x600001, 0x7FFFFF):
            for sign in (0, 0x80000000):
                v = _f((e << 23) | mant | sign)
                assert E.q35b_debug_encode_e2m1(v) == L.q35o_encode_e2m1(v), hex((e << 23) | mant)
    rng = np.random.default_rng(6)
    vals = list((rng.standard_normal(20000) * 4).astype(np.float32))
    vals += [0.0, -0.0, float("nan"), float("inf"), -float("inf"), 2.0 ** 20, -(2.0 ** 27), 1e30, -3e38]
    for v in vals:
        assert E.q35b_debug_encode_e2m1(float(v)) == L.q35o_encode_e2m1(float(v)), v


def test_decoders(oracle, engine):
    L, E = oracle.lib(), engine.lib()
    for b in range(256):
        assert E.q35b_debug_decode_e4m3(b) == L.q35o_decode_e4m3(b)
    for c in range(16):
        assert E.q35b_debug_decode_e2m1(c) == L.q35o_decode_e2m1(c)


def test_tiled_offset(oracle, engine):
    E = engine.lib()
    for cols in (1, 4, 9, 64, 160):
        padded = (cols + 3) // 4 * 4
        for r in (0, 5, 31, 32, 100, 127, 128, 300):
            for c in range(0, cols, max(1, cols // 7)):
                assert E.q35b_debug_tiled_scale_offset(r, c, padded) == oracle.tiled_scale_offset(r, c, cols)
