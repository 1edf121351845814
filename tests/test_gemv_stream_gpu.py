"""The streaming (persistent, TMA-fed, mma.sync) decode projection against the CPU oracle: single projections through
q35b_gemv_w4a16_bf16(kernel=STREAM) and whole work lists through q35b_gemv_batch_*.
Tolerance: relative L2 <= 1e-3 per output matrix, and element-wise within one BF16 ulp."""
import numpy as np
import pytest

from helpers import from_torch_bf16, make_activations, make_weight, to_torch_bf16

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-3


def _compare(oracle, yb, codes, scales, s2, xb):
    eb, ef = oracle.gemv_bf16(codes, scales, s2, xb, threads=8)
    err = oracle.rel_l2(oracle.bf16_to_f32(yb), oracle.bf16_to_f32(eb))
    assert err <= REL_L2_TOL, err
    rms = float(np.sqrt(np.mean(ef.astype(np.float64) ** 2)))
    assert np.all(np.abs(oracle.bf16_to_f32(yb) - oracle.bf16_to_f32(eb)) <= np.abs(ef) * 2.0 ** -7 + 1e-4 * rms + 1e-30)


@pytest.mark.parametrize("n,k,m", [(3584, 1024, 1), (4096, 1024, 1), (1024, 2048, 1), (7168, 1024, 1), (1024, 3584, 1),
                                   (3584, 1024, 2), (3584, 1024, 3), (3584, 1024, 4), (3584, 1024, 5), (3584, 1024, 8),
                                   (2560, 9216, 1), (2560, 4096, 4), (1000, 2560, 7), (130, 256, 1), (1, 256, 2),
                                   (257, 512, 8)])
def test_single_projection(engine, oracle, n, k, m):
    _, codes, scales, s2 = make_weight(n, k, seed=n + k + m)
    xb = make_activations(m, k, seed=m + 1, outlier_frac=0.001)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    y = engine.gemv_w4a16(w, to_torch_bf16(xb), kernel=engine.GEMV_STREAM)
    _compare(oracle, from_torch_bf16(y), codes, scales, s2, xb)
    # a second call reuses the cached work list and gives identical bits
    y2 = engine.gemv_w4a16(w, to_torch_bf16(xb), kernel=engine.GEMV_STREAM)
    assert np.array_equal(from_torch_bf16(y), from_torch_bf16(y2))


def test_activation_dynamic_range(engine, oracle):
    """Per-K-step power-of-two activation scaling: huge, tiny and zero steps side by side."""
    n, k = 512, 1024
    _, codes, scales, s2 = make_weight(n, k, seed=3)
    rng = np.random.default_rng(4)
    x = rng.standard_normal((2, k)).astype(np.float32)
    x[0, :256] *= 1e20
    x[0, 256:512] *= 1e-20
    x[0, 512:768] = 0.0
    x[1, 5] = 3e4
    xb = oracle.bf16_round(x)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    y = engine.gemv_w4a16(w, to_torch_bf16(xb), kernel=engine.GEMV_STREAM)
    _compare(oracle, from_torch_bf16(y), codes, scales, s2, xb)


def test_work_list_of_a_decode_layer(engine, oracle):
    import torch

    shapes = [(4096, 1024), (1024, 2048), (7168, 1024), (1024, 3584)] * 2
    for m in (1, 4):
        items, host = [], []
        for j, (n, k) in enumerate(shapes):
            _, codes, scales, s2 = make_weight(n, k, seed=100 + j)
            xb = make_activations(m, k, seed=200 + j)
            w = engine.Nvfp4Weight.from_host(codes, scales, s2)
            y = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
            items.append((w, to_torch_bf16(xb), y))
            host.append((codes, scales, s2, xb))
        batch = engine.GemvBatch(items, m)
        assert batch.stream_bytes == sum(n * k // 2 + n * k // 16 for n, k in shapes)
        batch.run()
        batch.run()
        torch.cuda.synchronize()
        assert batch.status() == 0
        for (w, x, y), (codes, scales, s2, xb) in zip(items, host):
            _compare(oracle, from_torch_bf16(y), codes, scales, s2, xb)


def test_ineligible_shapes_are_rejected(engine):
    import torch

    _, codes, scales, s2 = make_weight(64, 96, seed=1)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    x = torch.zeros((1, 96), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(engine.Q35bError) as e:
        engine.gemv_w4a16(w, x, kernel=engine.GEMV_STREAM)
    assert e.value.status == 2
    rng = np.random.default_rng(0)
    neg = rng.integers(0x80, 0xFF, size=(64, 16), dtype=np.uint8)
    w2 = engine.Nvfp4Weight.from_host(rng.integers(0, 256, size=(64, 128), dtype=np.uint8), neg, 1.0)
    with pytest.raises(engine.Q35bError) as e:
        engine.gemv_w4a16(w2, torch.zeros((1, 256), dtype=torch.bfloat16, device="cuda"), kernel=engine.GEMV_STREAM)
    assert e.value.status == 5


def test_auto_selection(engine, oracle):
    """AUTO runs the streaming kernel for a weight of 24 MiB or more and the SIMT kernel below that; on a capturing
    stream it never allocates (first use of the streaming kernel would), so it stays on the SIMT kernel there."""
    import torch

    n, k = 20480, 4096  # 47 MB of codes + scales
    _, codes, scales, s2 = make_weight(n, k, seed=11)
    xb = make_activations(2, k, seed=12)
    x = to_torch_bf16(xb)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    # capture before the streaming work list exists: must succeed (SIMT) and replay correctly
    y_graph = torch.empty((2, n), dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            engine.gemv_w4a16(w, x, out=y_graph, kernel=engine.GEMV_AUTO)
        graph.replay()
        stream.synchronize()
    y_simt = engine.gemv_w4a16(w, x, kernel=engine.GEMV_SIMT)
    assert np.array_equal(from_torch_bf16(y_graph), from_torch_bf16(y_simt))
    # outside a capture the large weight goes to the streaming kernel
    y_auto = engine.gemv_w4a16(w, x, kernel=engine.GEMV_AUTO)
    y_stream = engine.gemv_w4a16(w, x, kernel=engine.GEMV_STREAM)
    assert np.array_equal(from_torch_bf16(y_auto), from_torch_bf16(y_stream))
    _compare(oracle, from_torch_bf16(y_auto), codes, scales, s2, xb)
    # a small weight stays on the SIMT kernel
    _, c2, sc2, s22 = make_weight(3584, 1024, seed=13)
    x2 = to_torch_bf16(make_activations(1, 1024, seed=14))
    w2 = engine.Nvfp4Weight.from_host(c2, sc2, s22)
    assert np.array_equal(from_torch_bf16(engine.gemv_w4a16(w2, x2, kernel=engine.GEMV_AUTO)),
                          from_torch_bf16(engine.gemv_w4a16(w2, x2, kernel=engine.GEMV_SIMT)))
