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


class PeerGather:
    """The exchange step fused into the GEMM's stores (q35b_gemm_w4a4_bf16_allgather): every rank owns a full
    [m, n] BF16 matrix the others can store into; handles travel once through the process group at construction.

        gather = PeerGather(m, n)                       # collective: every rank of the group calls it
        gather.project(weight_shard, codes, scales, g)  # GEMM + stores to all ranks + bounded wait
        c = gather.tensor()                             # [m, n] on this rank

    Ranks must call `project` the same number of times (each call is one epoch).  Before reusing the matrix for the
    next projection every rank must have finished reading it: call `dist.barrier()` or order the work otherwise."""

    def __init__(self, m: int, n: int, group=None):
        import torch
        import torch.distributed as dist

        from . import engine

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.m, self.n = m, n
        device = torch.device("cuda", torch.cuda.current_device())

        def agree(error):
            """Every rank learns whether any rank failed the last local step, so that all raise or none does."""
            flag = torch.tensor([0 if error is None else 1], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
            if int(flag.item()) != 0:
                raise RuntimeError(f"peer buffer set-up failed: {error if error is not None else 'on another rank'}")

        error, self.local = None, None
        nbytes = int(engine.lib().q35b_peer_buffer_handle_bytes())
        try:
            self.local = engine.PeerBuffer.create(m, n)
            mine = torch.frombuffer(bytearray(self.local.export()), dtype=torch.uint8).to(device)
        except Exception as e:  # noqa: BLE001 - turned into one error on every rank
            error = e
            mine = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        agree(error)
        handles = torch.empty((self.world, nbytes), dtype=torch.uint8, device=device)
        dist.all_gather_into_tensor(handles, mine, group=group)
        handles = handles.cpu().numpy()
        try:
            self.buffers = [self.local if r == self.rank else engine.PeerBuffer.open(handles[r].tobytes(), m, n)
                            for r in range(self.world)]
        except Exception as e:  # noqa: BLE001
            error = e
        agree(error)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = 0
        dist.barrier(group)

    def project(self, weight_shard, a_codes, a_scales_tiled, g):
        from . import engine

        self.epoch += 1
        engine.gemm_w4a4_allgather(weight_shard, a_codes, a_scales_tiled, g, self.m, self.buffers, self.rank, self.epoch,
                                   self.status)
        return self.local.tensor()

    def tensor(self):
        return self.local.tensor()

    def check(self) -> None:
        code = int(self.status.item())
        if code != 0:
            raise RuntimeError(f"device-side wait expired in the gathering projection, code {code}")
