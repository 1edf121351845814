"""The N-sharded prefill MLP block (sharding.PeerMlp): gate/up shards write their columns of the NVFP4 intermediate,
q35b_peer_push carries them (and later the BF16 output shards) to every rank.  Ranks are emulated in one process on
one GPU, stage by stage, so that no launch ever waits for a later one; the result on every rank must equal, bit for
bit, the unsharded chain of the same library (which other tests hold against the oracle)."""
import numpy as np
import pytest

from helpers import make_activations, make_weight, to_torch_bf16

pytestmark = pytest.mark.gpu


def _unsharded(engine, torch, m, gate, up, down, a_codes, a_scales, g, h_scale, res):
    gu = engine.Nvfp4Weight.gate_up_from_host(gate[1], gate[2], gate[3], up[1], up[2], up[3])
    dn = engine.Nvfp4Weight.from_host(down[1], down[2], down[3])
    hc, hs, hg = engine.gemm_w4a4_gate_up_quant(gu, a_codes, a_scales, g, m, h_scale)
    return hc.clone(), hs.clone(), engine.gemm_w4a4(dn, hc, hs, hg, m, residual=res)


@pytest.mark.parametrize("world,m,hidden,inter", [(2, 300, 512, 1024), (4, 257, 768, 1536), (8, 130, 512, 2048),
                                                   (8, 512, 2560, 9216), (3, 64, 256, 384)])
def test_emulated_ranks_compute_the_same_block(engine, oracle, world, m, hidden, inter):
    import torch

    from qwen35x_b200 import sharding

    gate = make_weight(inter, hidden, seed=world + 1)
    up = make_weight(inter, hidden, seed=world + 2)
    down = make_weight(hidden, inter, seed=world + 3)
    x = to_torch_bf16(make_activations(m, hidden, seed=9, outlier_frac=0.001))
    res = to_torch_bf16(make_activations(m, hidden, seed=10))
    a_codes, a_scales, g = engine.quantize_activations(x)
    # calibrate the intermediate's per-tensor scale on the BF16 output of the same GEMM
    gu_full = engine.Nvfp4Weight.gate_up_from_host(gate[1], gate[2], gate[3], up[1], up[2], up[3])
    h = engine.gemm_w4a4(gu_full, a_codes, a_scales, g, m)
    h_scale = (h.float().abs().max() / (6.0 * 448.0)).reshape(1).to(torch.float32)
    exp_codes, exp_scales, exp_out = _unsharded(engine, torch, m, gate, up, down, a_codes, a_scales, g, h_scale, res)

    # scale bytes of real rows and columns (the epilogue leaves the padding of the tiled layout alone)
    r = torch.arange(m, device="cuda")[:, None]
    c = torch.arange(inter // 16, device="cuda")[None, :]
    slots = (inter // 16 + 3) // 4 * 4
    valid = ((((r // 128) * (slots // 4) + c // 4) * 32 + (r % 32)) * 16 + ((r % 128) // 32) * 4 + (c % 4)).reshape(-1)

    layout = sharding.MlpLayout(m, hidden, inter)
    buffers = [engine.PeerBuffer.create_bytes(layout.total) for _ in range(world)]
    for b in buffers:
        b.bytes().fill_(0x5a)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ranks = []
    for r in range(world):
        gu = engine.Nvfp4Weight.gate_up_from_host(gate[1], gate[2], gate[3], up[1], up[2], up[3], shard_index=r,
                                                  shard_count=world)
        dn = engine.Nvfp4Weight.from_host(down[1], down[2], down[3], shard_index=r, shard_count=world)
        ranks.append(sharding.PeerMlp(layout, buffers, r, gu, dn, h_scale, status))
    for rounds in range(2):  # the second round checks that epochs, counters and flags are reusable
        for stage in range(4):
            for p in ranks:
                p.stage(stage, a_codes, a_scales, g, residual=res)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for p in ranks:
            assert torch.equal(p.h_codes.view(m, inter // 2), exp_codes)
            assert torch.equal(p.h_scales[valid], exp_scales[valid])
            assert torch.equal(p.out, exp_out)
        for b in buffers:
            b.bytes()[:layout.total].fill_(0xa5)


def test_row_groups_of_the_pipelined_block(engine, oracle):
    """PeerMlp.run(chunks=c) cuts the tokens into groups of whole 128-row blocks and pushes each group while the next
    one computes.  Here the same per-group steps are issued rank by rank on one GPU (no launch waits for a later
    one): offsets of every group into codes, scale tiles and output must land exactly where the unsharded block
    puts them."""
    import torch

    from qwen35x_b200 import sharding

    world, m, hidden, inter = 4, 600, 512, 1024
    gate = make_weight(inter, hidden, seed=21)
    up = make_weight(inter, hidden, seed=22)
    down = make_weight(hidden, inter, seed=23)
    x = to_torch_bf16(make_activations(m, hidden, seed=24))
    res = to_torch_bf16(make_activations(m, hidden, seed=25))
    a_codes, a_scales, g = engine.quantize_activations(x)
    h_scale = torch.tensor([0.004], dtype=torch.float32, device="cuda")
    _, _, exp_out = _unsharded(engine, torch, m, gate, up, down, a_codes, a_scales, g, h_scale, res)
    layout = sharding.MlpLayout(m, hidden, inter)
    buffers = [engine.PeerBuffer.create_bytes(layout.total) for _ in range(world)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ranks = [sharding.PeerMlp(layout, buffers, r,
                              engine.Nvfp4Weight.gate_up_from_host(gate[1], gate[2], gate[3], up[1], up[2], up[3],
                                                                   shard_index=r, shard_count=world),
                              engine.Nvfp4Weight.from_host(down[1], down[2], down[3], shard_index=r, shard_count=world),
                              h_scale, status) for r in range(world)]
    groups = [(0, 256), (256, 256), (512, 88)]
    for (r0, rows) in groups:
        for p in ranks:
            p._gate_up(a_codes, a_scales, g, r0, rows)
            p._push_h(r0, rows)
    for p in ranks:
        for _ in groups:
            p._wait()
    for (r0, rows) in groups:
        for p in ranks:
            p._down(res, r0, rows)
            p._push_out(r0, rows)
    for p in ranks:
        for _ in groups:
            p._wait()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for p in ranks:
        assert torch.equal(p.out, exp_out)
