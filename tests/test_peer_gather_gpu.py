"""The N-sharded prefill projection whose GEMM stores are the all-gather (q35b_gemm_w4a4_bf16_allgather).
On one GPU the ranks are emulated in one process: every rank's shard GEMM is launched first, the waits afterwards,
so no launch ever waits for a later one.  With two or more GPUs a torchrun job runs the real thing over CUDA IPC.
Reference: the unsharded GEMM of the same library (bit-identical columns) and the oracle (relative L2 <= 1e-3).
N = 1000 and N = 200 give a last shard and a row stride that are not multiples of 16 elements: the remote stores
then go lane by lane instead of as whole forwarded rows."""
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import from_torch_bf16, make_activations, make_weight, to_torch_bf16

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-3


@pytest.mark.parametrize("world,m,n,k", [(2, 300, 1024, 512), (3, 64, 1152, 256), (4, 257, 2560, 512), (8, 130, 2048, 256),
                                         (8, 300, 3584, 512), (2, 300, 1000, 512), (3, 40, 200, 256)])
def test_emulated_ranks_fill_every_matrix(engine, oracle, world, m, n, k):
    import torch

    _, codes, scales, s2 = make_weight(n, k, seed=world + n)
    xb = make_activations(m, k, seed=7, outlier_frac=0.001)
    a_codes, a_scales, g = engine.quantize_activations(to_torch_bf16(xb))
    full = engine.gemm_w4a4(engine.Nvfp4Weight.from_host(codes, scales, s2), a_codes, a_scales, g, m)
    buffers = [engine.PeerBuffer.create(m, n) for _ in range(world)]
    for b in buffers:
        b.tensor().zero_()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    shards = [engine.Nvfp4Weight.from_host(codes, scales, s2, shard_index=r, shard_count=world) for r in range(world)]
    for epoch in (1, 2):  # the second round checks that counters and flags are reusable
        for r in range(world):
            engine.gemm_w4a4_allgather(shards[r], a_codes, a_scales, g, m, buffers, r, epoch, status, wait=False)
        for r in range(world):
            engine.peer_gather_wait(buffers, r, epoch, status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for b in buffers:
            assert torch.equal(b.tensor(), full)
            b.tensor().zero_()
    e_codes, e_scales, e_g = oracle.quantize_nvfp4(xb)
    eb, _ = oracle.gemm_w4a4(codes, scales, s2, e_codes, e_scales, e_g, threads=8)
    assert oracle.rel_l2(oracle.bf16_to_f32(from_torch_bf16(full)), oracle.bf16_to_f32(eb)) <= REL_L2_TOL


def test_wait_for_a_rank_that_never_stores_expires(engine):
    """A flag nothing sets: the bounded wait gives up, records 31, and the context stays usable."""
    import torch

    buffers = [engine.PeerBuffer.create(8, 128) for _ in range(2)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    engine.peer_gather_wait(buffers, 0, 5, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 31
    assert float(torch.ones(4, device="cuda").sum().item()) == 4.0


def test_buffer_too_small_is_rejected(engine):
    import torch

    _, codes, scales, s2 = make_weight(256, 256, seed=1)
    w = engine.Nvfp4Weight.from_host(codes, scales, s2)
    a_codes, a_scales, g = engine.quantize_activations(torch.zeros((8, 256), dtype=torch.bfloat16, device="cuda"))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    small = [engine.PeerBuffer.create(8, 128)]
    with pytest.raises(engine.Q35bError) as e:
        engine.gemm_w4a4_allgather(w, a_codes, a_scales, g, 8, small, 0, 1, status)
    assert e.value.status in (1, 2)


def test_two_processes_over_ipc():
    """Two ranks on two GPUs: every rank ends with the full matrix (checked inside the worker against its own
    unsharded GEMM)."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29631", os.path.join(here, "peer_gather_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
