"""Multi-rank host logic on CPU: two gloo ranks shard a projection by rows and all-gather the slabs."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, n: int, m: int):
    sys.path.insert(0, str(ROOT))
    from qwen35x_b200 import sharding

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(123)
        full = torch.randn((m, n), generator=gen).to(torch.bfloat16)  # same on every rank
        begin, count = sharding.shard_layout(n, world)[rank]
        local = full[:, begin:begin + count].contiguous()
        out = sharding.all_gather_rows(local, n)
        assert out.shape == (m, n) and torch.equal(out, full), f"rank {rank}: gathered matrix differs"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n", [2560, 3584, 1000, 128])
def test_two_ranks_gather_row_shards(n):
    mp.spawn(_worker, args=(2, _free_port(), n, 5), nprocs=2, join=True)


def test_layout_matches_c_abi(engine):
    from qwen35x_b200 import sharding

    for n in (2560, 3584, 18432, 9216, 100, 129, 32768):
        for world in (1, 2, 4, 8):
            assert sharding.shard_layout(n, world) == [engine.shard_range(n, i, world) for i in range(world)]
