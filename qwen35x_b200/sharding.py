"""Row sharding of a projection across ranks and the one exchange step of the prefill path.

A weight [N, K] is cut into contiguous row slabs on 128-row boundaries (q35b_shard_range); every rank computes
C[:, slab] for the same, replicated activations; one all-gather of the BF16 slabs rebuilds C[M, N] on every rank.
Slabs can differ by one 128-row block, so they are padded to the widest slab for the collective."""
from __future__ import annotations


def shard_layout(n: int, world: int):
    """[(row_begin, row_count)] per rank; pure Python twin of q35b_shard_range (include/q35b_nvfp4.h)."""
    blocks = (n + 127) // 128
    out = []
    for i in range(world):
        b0 = blocks * i // world
        b1 = blocks * (i + 1) // world
        begin, end = min(b0 * 128, n), min(b1 * 128, n)
        out.append((begin, end - begin))
    return out


def all_gather_slabs(local, n: int, group=None, out=None):
    """local: [M, rows_of_this_rank] -> the slabs of all ranks as [world, M, widest] (rank i's slab is
    result[i, :, :shard_layout(n, world)[i][1]]).  This is the exchange step itself: one collective, and no copy at
    all when every rank holds the same number of rows."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    layout = shard_layout(n, world)
    m = local.shape[0]
    assert local.shape[1] == layout[rank][1]
    widest = max(c for _, c in layout)
    padded = local if local.shape[1] == widest else torch.nn.functional.pad(local, (0, widest - local.shape[1]))
    if out is None:
        out = torch.empty((world * m, widest), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out.view(torch.uint8), padded.contiguous().view(torch.uint8), group=group)
    return out.view(world, m, widest)


def all_gather_rows(local, n: int, group=None):
    """local: [M, rows_of_this_rank] on any device -> [M, N] on every rank (NCCL on GPUs, gloo on CPU):
    all_gather_slabs followed by a copy into row-major [M, N]."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    layout = shard_layout(n, world)
    m = local.shape[0]
    assert local.shape[1] == layout[rank][1]
    widest = max(c for _, c in layout)
    padded = local if local.shape[1] == widest else torch.nn.functional.pad(local, (0, widest - local.shape[1]))
    # rank slabs are concatenated along dim 0; the collective moves bytes (uint8 is taken by every backend)
    gathered = torch.empty((world * m, widest), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(gathered.view(torch.uint8), padded.contiguous().view(torch.uint8), group=group)
    return assemble(gathered.view(world, m, widest), n)


def assemble(gathered, n: int):
    """[world, M, widest] slabs -> [M, N]."""
    import torch

    world, m, _ = gathered.shape
    out = torch.empty((m, n), dtype=gathered.dtype, device=gathered.device)
    for (begin, count), slab in zip(shard_layout(n, world), gathered):
        out[:, begin:begin + count] = slab[:, :count]
    return out
