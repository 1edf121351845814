"""Fused epilogues of the decode work list and the NVFP4 -> BF16 weight dequantisation, against the CPU oracle.
Tolerance: relative L2 <= 1e-3 (BF16 outputs)."""
import numpy as np
import pytest

from helpers import from_torch_bf16, make_activations, make_weight, to_torch_bf16

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-3


@pytest.mark.parametrize("m", [1, 3, 8])
def test_projection_plus_residual(engine, oracle, m):
    """y = bf16(projection + residual): matvec_down_residual_nvfp4 (src/kernels/cuda/decode_layers.cuh:404-428)."""
    import torch

    n, k = 1024, 3584
    _, codes, scales, s2 = make_weight(n, k, seed=11)
    xb = make_activations(m, k, seed=12)
    rb = make_activations(m, n, seed=13)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    y = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    batch = engine.GemvBatch([(w, to_torch_bf16(xb), y, to_torch_bf16(rb))], m)
    batch.run()
    torch.cuda.synchronize()
    assert batch.status() == 0
    _, yf = oracle.gemv_bf16(codes, scales, s2, xb, threads=8)
    exp = oracle.bf16_round(yf + oracle.bf16_to_f32(rb))
    got = from_torch_bf16(y)
    assert oracle.rel_l2(oracle.bf16_to_f32(got), oracle.bf16_to_f32(exp)) <= REL_L2_TOL


@pytest.mark.parametrize("m", [1, 2, 5])
def test_gate_up_silu(engine, oracle, m):
    """y = bf16(silu(gate . x) * (up . x)), silu(g) = g / (1 + exp(-g)): matvec_gate_up_silu_nvfp4
    (decode_layers.cuh:339-365) with the exact sigmoid of silu_multiply_kernel (src/runtime/cuda_bench.cu:215-222)."""
    import torch

    n_half, k = 3584, 1024
    _, g_codes, g_scales, g_s2 = make_weight(n_half, k, seed=21, std=0.05)
    _, u_codes, u_scales, u_s2 = make_weight(n_half, k, seed=22, std=0.03)
    xb = make_activations(m, k, seed=23)
    w = engine.Nvfp4Weight.gate_up_from_host(g_codes, g_scales, g_s2, u_codes, u_scales, u_s2)
    assert w.gate_up and w.rows == 2 * n_half
    y = torch.zeros((m, n_half), dtype=torch.bfloat16, device="cuda")
    batch = engine.GemvBatch([(w, to_torch_bf16(xb), y)], m)
    batch.run()
    torch.cuda.synchronize()
    assert batch.status() == 0
    _, gate = oracle.gemv_bf16(g_codes, g_scales, g_s2, xb, threads=8)
    _, up = oracle.gemv_bf16(u_codes, u_scales, u_s2, xb, threads=8)
    exp = (gate / (np.float32(1.0) + np.exp(-gate, dtype=np.float32)) * up).astype(np.float32)
    got = oracle.bf16_to_f32(from_torch_bf16(y))
    assert oracle.rel_l2(got, oracle.bf16_to_f32(oracle.bf16_round(exp))) <= REL_L2_TOL
    # a gate/up weight is only meaningful with its epilogue
    with pytest.raises(engine.Q35bError):
        engine.gemv_w4a16(w, to_torch_bf16(xb))


def test_mlp_work_list(engine, oracle):
    """gate+up+SiLU and an independent down+residual in one launch, mixed with a plain projection."""
    import torch

    k, inter = 1024, 512
    _, g_codes, g_scales, g_s2 = make_weight(inter, k, seed=31)
    _, u_codes, u_scales, u_s2 = make_weight(inter, k, seed=32)
    _, d_codes, d_scales, d_s2 = make_weight(k, inter * 2, seed=33)
    x1 = make_activations(2, k, 34)
    x2 = make_activations(2, inter * 2, 35)
    res = make_activations(2, k, 36)
    gu = engine.Nvfp4Weight.gate_up_from_host(g_codes, g_scales, g_s2, u_codes, u_scales, u_s2)
    down = engine.Nvfp4Weight.from_host(d_codes, d_scales, d_s2)
    y1 = torch.zeros((2, inter), dtype=torch.bfloat16, device="cuda")
    y2 = torch.zeros((2, k), dtype=torch.bfloat16, device="cuda")
    y3 = torch.zeros((2, k), dtype=torch.bfloat16, device="cuda")
    batch = engine.GemvBatch([(gu, to_torch_bf16(x1), y1), (down, to_torch_bf16(x2), y2, to_torch_bf16(res)),
                              (down, to_torch_bf16(x2), y3)], 2)
    batch.run()
    torch.cuda.synchronize()
    assert batch.status() == 0
    _, gate = oracle.gemv_bf16(g_codes, g_scales, g_s2, x1, threads=8)
    _, up = oracle.gemv_bf16(u_codes, u_scales, u_s2, x1, threads=8)
    e1 = oracle.bf16_round((gate / (1 + np.exp(-gate)) * up).astype(np.float32))
    eb, ef = oracle.gemv_bf16(d_codes, d_scales, d_s2, x2, threads=8)
    e2 = oracle.bf16_round(ef + oracle.bf16_to_f32(res))
    for got, exp in ((y1, e1), (y2, e2), (y3, eb)):
        assert oracle.rel_l2(oracle.bf16_to_f32(from_torch_bf16(got)), oracle.bf16_to_f32(exp)) <= REL_L2_TOL


def test_weight_dequant_bf16_bit_exact(engine, oracle):
    """bf16(e2m1 * (e4m3 * s2)) per element, bit-exact with the oracle's restatement of
    src/runtime/qwen35x_cuda_backend.cpp:742-755; all codes and (non-negative and negative) scale bytes."""
    rng = np.random.default_rng(2)
    n, k = 130, 512
    codes = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    scales = rng.integers(0, 256, size=(n, k // 16), dtype=np.uint8)
    s2 = 3.0e-4
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    got = from_torch_bf16(w.dequant_bf16())
    exp = oracle.dequant_weights_bf16(codes, scales, s2)
    assert np.array_equal(got, exp)


@pytest.mark.parametrize("m", [7, 300])
def test_prefill_gemm_plus_residual(engine, oracle, m):
    """c = bf16(W4A4 projection + residual) in the GEMM epilogue (1-CTA kernel for m = 7, 2-CTA for m = 300)."""
    import torch

    n, k = 520, 1024
    _, codes, scales, s2 = make_weight(n, k, seed=41)
    xb = make_activations(m, k, seed=42, outlier_frac=0.001)
    rb = make_activations(m, n, seed=43)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    a_codes, a_scales, g = engine.quantize_activations(to_torch_bf16(xb))
    c = engine.gemm_w4a4(w, a_codes, a_scales, g, m, status=status, residual=to_torch_bf16(rb))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    e_codes, e_scales, e_g = oracle.quantize_nvfp4(xb)
    _, cf = oracle.gemm_w4a4(codes, scales, s2, e_codes, e_scales, e_g, threads=8)
    exp = oracle.bf16_round(cf + oracle.bf16_to_f32(rb))
    assert oracle.rel_l2(oracle.bf16_to_f32(from_torch_bf16(c)), oracle.bf16_to_f32(exp)) <= REL_L2_TOL


@pytest.mark.parametrize("m,n_half", [(5, 256), (300, 1000), (256, 9216)])
def test_prefill_gate_up_silu(engine, oracle, m, n_half):
    """c = bf16(silu(gate) * up) straight from the GEMM epilogue, [m, n_half] (half the output bytes)."""
    import torch

    k = 512 if n_half > 2000 else 1024
    _, g_codes, g_scales, g_s2 = make_weight(n_half, k, seed=51, std=0.05)
    _, u_codes, u_scales, u_s2 = make_weight(n_half, k, seed=52, std=0.03)
    xb = make_activations(m, k, seed=53, outlier_frac=0.001)
    w = engine.Nvfp4Weight.gate_up_from_host(g_codes, g_scales, g_s2, u_codes, u_scales, u_s2)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    c = engine.project_prefill(w, to_torch_bf16(xb))
    a_codes, a_scales, g = engine.quantize_activations(to_torch_bf16(xb))
    c2 = engine.gemm_w4a4(w, a_codes, a_scales, g, m, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and tuple(c.shape) == (m, n_half) and torch.equal(c, c2)
    e_codes, e_scales, e_g = oracle.quantize_nvfp4(xb)
    rows = np.arange(n_half) if n_half <= 1000 else np.sort(np.random.default_rng(0).choice(n_half, 64, replace=False))
    got = oracle.bf16_to_f32(from_torch_bf16(c))[:, rows]
    exp = np.zeros((m, len(rows)), dtype=np.float32)
    for j, r in enumerate(rows):
        _, gate = oracle.gemm_w4a4(g_codes[r:r + 1], g_scales[r:r + 1], g_s2, e_codes, e_scales, e_g, threads=8)
        _, up = oracle.gemm_w4a4(u_codes[r:r + 1], u_scales[r:r + 1], u_s2, e_codes, e_scales, e_g, threads=8)
        exp[:, j] = (gate / (1 + np.exp(-gate)) * up)[:, 0]
    assert oracle.rel_l2(got, oracle.bf16_to_f32(oracle.bf16_round(exp))) <= REL_L2_TOL


def _untile(oracle, tiled: np.ndarray, rows: int, scale_cols: int) -> np.ndarray:
    """Row-major [rows, scale_cols] view of a tiled scale array (padding dropped)."""
    out = np.zeros((rows, scale_cols), dtype=np.uint8)
    for r in range(rows):
        for c in range(scale_cols):
            out[r, c] = tiled[oracle.tiled_scale_offset(r, c, scale_cols)]
    return out


@pytest.mark.parametrize("m,n_half,shrink", [(300, 384, 1.0), (100, 384, 1.0), (257, 192, 8.0), (64, 64, 1.0)])
def test_prefill_gate_up_to_nvfp4(engine, oracle, m, n_half, shrink):
    """The gate/up GEMM that writes silu(gate) * up as an NVFP4 activation: its codes and block scales equal the
    stand-alone quantiser applied, with the same per-tensor scale, to the BF16 output of the plain gate/up GEMM
    (bit for bit, also when the scale is too small and values saturate), and the down projection on that activation
    meets the oracle within relative L2 <= 1e-3."""
    import torch

    k = 512
    _, g_codes, g_scales, g_s2 = make_weight(n_half, k, seed=61, std=0.05)
    _, u_codes, u_scales, u_s2 = make_weight(n_half, k, seed=62, std=0.03)
    xb = make_activations(m, k, seed=63, outlier_frac=0.001)
    w = engine.Nvfp4Weight.gate_up_from_host(g_codes, g_scales, g_s2, u_codes, u_scales, u_s2)
    a_codes, a_scales, g = engine.quantize_activations(to_torch_bf16(xb))
    c = engine.gemm_w4a4(w, a_codes, a_scales, g, m)
    scale = float(c.float().abs().max().item()) / (6.0 * 448.0) / shrink
    out_scale = torch.tensor([scale], dtype=torch.float32, device="cuda")
    scale = float(out_scale.item())  # the fp32 value both paths see
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    f_codes, f_scales, _ = engine.gemm_w4a4_gate_up_quant(w, a_codes, a_scales, g, m, out_scale, status=status)
    u_codes_q, u_scales_q, u_g = engine.quantize_activations(c, global_scale=scale)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and float(u_g.item()) == scale
    assert torch.equal(f_codes.reshape(-1), u_codes_q.reshape(-1)[: m * n_half // 2])
    f_rm = _untile(oracle, f_scales.cpu().numpy(), m, n_half // 16)
    assert np.array_equal(f_rm, _untile(oracle, u_scales_q.cpu().numpy(), m, n_half // 16))
    # and against the oracle's quantiser on the same BF16 values
    e_codes, e_scales, _ = oracle.quantize_nvfp4(from_torch_bf16(c), global_scale=scale)
    assert np.array_equal(f_codes.cpu().numpy().reshape(m, n_half // 2), e_codes) and np.array_equal(f_rm, e_scales)
    # down projection fed by the fused output
    n_out = 256
    _, d_codes, d_scales, d_s2 = make_weight(n_out, n_half, seed=64)
    wd = engine.Nvfp4Weight.from_host(d_codes, d_scales, d_s2)
    y = engine.gemm_w4a4(wd, f_codes, f_scales, out_scale, m, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    eb, _ = oracle.gemm_w4a4(d_codes, d_scales, d_s2, e_codes, e_scales, scale, threads=8)
    assert oracle.rel_l2(oracle.bf16_to_f32(from_torch_bf16(y)), oracle.bf16_to_f32(eb)) <= REL_L2_TOL


def test_prefill_gate_up_to_nvfp4_rejects(engine):
    import torch

    _, codes, scales, s2 = make_weight(256, 256, seed=1)
    plain = engine.Nvfp4Weight.from_host(codes, scales, s2)
    a_codes, a_scales, g = engine.quantize_activations(torch.zeros((8, 256), dtype=torch.bfloat16, device="cuda"))
    one = torch.ones(1, dtype=torch.float32, device="cuda")
    with pytest.raises(AssertionError):
        engine.gemm_w4a4_gate_up_quant(plain, a_codes, a_scales, g, 8, one)
    odd = engine.Nvfp4Weight.gate_up_from_host(codes[:48], scales[:48], s2, codes[48:96], scales[48:96], s2)
    with pytest.raises(engine.Q35bError) as e:
        engine.gemm_w4a4_gate_up_quant(odd, a_codes, a_scales, g, 8, one)
    assert e.value.status == 2


@pytest.mark.parametrize("m", [1, 4])
def test_work_list_with_dependencies(engine, oracle, m):
    """Two MLP blocks chained in ONE launch: gate/up -> down(+residual) -> gate/up -> down(+residual); each item
    names the item whose output it reads, and the kernel holds its activations back until that item is stored.
    Replayed through a CUDA graph to check that the completion counts are reset per run."""
    import torch

    hidden, inter = 1024, 3584
    weights, items, expect = [], [], []
    x0 = make_activations(m, hidden, seed=70)
    x_host = oracle.bf16_to_f32(x0)
    x_dev = to_torch_bf16(x0)
    cur_dev, cur_bits = x_dev, x0
    for layer in range(2):
        _, g_codes, g_scales, g_s2 = make_weight(inter, hidden, seed=71 + 3 * layer, std=0.05)
        _, u_codes, u_scales, u_s2 = make_weight(inter, hidden, seed=72 + 3 * layer, std=0.03)
        _, d_codes, d_scales, d_s2 = make_weight(hidden, inter, seed=73 + 3 * layer, std=0.05)
        gu = engine.Nvfp4Weight.gate_up_from_host(g_codes, g_scales, g_s2, u_codes, u_scales, u_s2)
        down = engine.Nvfp4Weight.from_host(d_codes, d_scales, d_s2)
        weights += [gu, down]
        h = torch.zeros((m, inter), dtype=torch.bfloat16, device="cuda")
        y = torch.zeros((m, hidden), dtype=torch.bfloat16, device="cuda")
        items.append((gu, cur_dev, h, None, len(items) - 1 if layer > 0 else None))
        items.append((down, h, y, cur_dev, len(items) - 1))
        # oracle chain on the BF16 values the kernel sees
        _, gate = oracle.gemv_bf16(g_codes, g_scales, g_s2, cur_bits, threads=8)
        _, up = oracle.gemv_bf16(u_codes, u_scales, u_s2, cur_bits, threads=8)
        h_bits = oracle.bf16_round((gate / (np.float32(1.0) + np.exp(-gate, dtype=np.float32)) * up).astype(np.float32))
        _, d = oracle.gemv_bf16(d_codes, d_scales, d_s2, h_bits, threads=8)
        y_bits = oracle.bf16_round(d + oracle.bf16_to_f32(cur_bits))
        expect.append((h, h_bits, y, y_bits))
        cur_dev, cur_bits = y, y_bits
    del x_host
    batch = engine.GemvBatch(items, m)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        batch.run()
        stream.synchronize()
        assert batch.status() == 0
        first = [t[2].clone() for t in expect]
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            batch.run()
        for t in expect:
            t[0].zero_()
            t[2].zero_()
        for _ in range(3):
            graph.replay()
        stream.synchronize()
    assert batch.status() == 0
    for (h, h_bits, y, y_bits), y_first in zip(expect, first):
        assert torch.equal(y, y_first)
        assert oracle.rel_l2(oracle.bf16_to_f32(from_torch_bf16(h)), oracle.bf16_to_f32(h_bits)) <= 2 * REL_L2_TOL
        assert oracle.rel_l2(oracle.bf16_to_f32(from_torch_bf16(y)), oracle.bf16_to_f32(y_bits)) <= 2 * REL_L2_TOL


def test_work_list_dependency_without_activation_ring(engine, oracle):
    """4B-class MLP block at M = 8: the down projection's activations (8 x 9216) leave no room for the raw-activation
    ring, so the activation warp reads the gate/up output straight from global memory once it is complete."""
    import torch

    m, hidden, inter = 8, 2560, 9216
    _, g_codes, g_scales, g_s2 = make_weight(inter, hidden, seed=81, std=0.05)
    _, u_codes, u_scales, u_s2 = make_weight(inter, hidden, seed=82, std=0.03)
    _, d_codes, d_scales, d_s2 = make_weight(hidden, inter, seed=83, std=0.05)
    xb = make_activations(m, hidden, seed=84)
    gu = engine.Nvfp4Weight.gate_up_from_host(g_codes, g_scales, g_s2, u_codes, u_scales, u_s2)
    down = engine.Nvfp4Weight.from_host(d_codes, d_scales, d_s2)
    x = to_torch_bf16(xb)
    h = torch.zeros((m, inter), dtype=torch.bfloat16, device="cuda")
    y = torch.zeros((m, hidden), dtype=torch.bfloat16, device="cuda")
    batch = engine.GemvBatch([(gu, x, h), (down, h, y, x, 0)], m)
    for _ in range(2):
        batch.run()
    torch.cuda.synchronize()
    assert batch.status() == 0
    _, gate = oracle.gemv_bf16(g_codes, g_scales, g_s2, xb, threads=8)
    _, up = oracle.gemv_bf16(u_codes, u_scales, u_s2, xb, threads=8)
    h_bits = oracle.bf16_round((gate / (np.float32(1.0) + np.exp(-gate, dtype=np.float32)) * up).astype(np.float32))
    _, d = oracle.gemv_bf16(d_codes, d_scales, d_s2, h_bits, threads=8)
    y_bits = oracle.bf16_round(d + oracle.bf16_to_f32(xb))
    assert oracle.rel_l2(oracle.bf16_to_f32(from_torch_bf16(h)), oracle.bf16_to_f32(h_bits)) <= 2 * REL_L2_TOL
    assert oracle.rel_l2(oracle.bf16_to_f32(from_torch_bf16(y)), oracle.bf16_to_f32(y_bits)) <= 2 * REL_L2_TOL


def test_work_list_dependency_must_point_backwards(engine):
    import torch

    _, codes, scales, s2 = make_weight(256, 256, seed=1)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    x = torch.zeros((1, 256), dtype=torch.bfloat16, device="cuda")
    y = torch.zeros((1, 256), dtype=torch.bfloat16, device="cuda")
    arr = (engine.engine._GemvItem * 1)(engine.engine._GemvItem(w.handle.value, x.data_ptr(), y.data_ptr(), None, 1))
    import ctypes

    h = ctypes.c_void_p()
    assert engine.lib().q35b_gemv_batch_create(arr, 1, 1, ctypes.byref(h)) == 1  # item 0 cannot run after item 0


def test_dependency_wait_that_cannot_be_met_expires(engine, oracle):
    """A dependent item whose producer never delivers the completions it waits for: with the test hook's short limit
    on every device-side wait the dependency poll runs out, 15 lands in the status word, the other roles run out on
    their own waits and the kernel returns within milliseconds; the context stays usable and, with the hook switched
    off again, the same list computes the right result."""
    import time

    import torch

    m, hidden, inter = 2, 512, 1024
    _, g_codes, g_scales, g_s2 = make_weight(inter, hidden, seed=1)
    _, u_codes, u_scales, u_s2 = make_weight(inter, hidden, seed=2)
    _, d_codes, d_scales, d_s2 = make_weight(hidden, inter, seed=3)
    gu = engine.Nvfp4Weight.gate_up_from_host(g_codes, g_scales, g_s2, u_codes, u_scales, u_s2)
    down = engine.Nvfp4Weight.from_host(d_codes, d_scales, d_s2)
    xb = make_activations(m, hidden, seed=4)
    x = to_torch_bf16(xb)
    h = torch.zeros((m, inter), dtype=torch.bfloat16, device="cuda")
    y = torch.zeros((m, hidden), dtype=torch.bfloat16, device="cuda")
    batch = engine.GemvBatch([(gu, x, h), (down, h, y, None, 0)], m)
    batch.run()
    torch.cuda.synchronize()
    assert batch.status() == 0
    good = y.clone()
    batch.debug_wait(4096, 1)  # one completion more than item 0 can ever report
    t0 = time.perf_counter()
    batch.run()
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 2.0
    assert batch.status() == 15
    assert float(torch.ones(8, device="cuda").sum().item()) == 8.0  # the context is alive
    batch.debug_wait(1 << 22, 0)
    y.zero_()
    batch.run()
    torch.cuda.synchronize()
    assert batch.status() == 0 and torch.equal(y, good)
