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


def _round_up(v: int, m: int) -> int:
    return (v + m - 1) // m * m


class MlpLayout:
    """Byte layout of one rank's peer buffer for the N-sharded prefill MLP block (hidden -> intermediate -> hidden):

        [h codes  m x inter/2][h tiled scales  ceil128(m) x ceil4(inter/16)][out  m x hidden BF16]

    h = silu(gate x) * up x as an NVFP4 activation, written shard by shard: rank r's gate/up GEMM fills its own
    columns locally, `push` regions carry them to the other ranks.  Pure arithmetic, no GPU needed."""

    def __init__(self, m: int, hidden: int, inter: int):
        assert inter % 64 == 0 and hidden % 8 == 0
        self.m, self.hidden, self.inter = m, hidden, inter
        self.codes_off = 0
        self.codes_ld = inter // 2
        self.scales_off = _round_up(m * self.codes_ld, 256)
        self.scale_slots = _round_up(inter // 16, 4)
        self.row_blocks = _round_up(m, 128) // 128
        self.scales_bytes = self.row_blocks * 128 * self.scale_slots
        self.out_off = _round_up(self.scales_off + self.scales_bytes, 256)
        self.out_ld = hidden * 2
        self.total = _round_up(self.out_off + m * self.out_ld, 256)

    def h_regions(self, col0: int, cols: int):
        """Regions (offset, rows, row_bytes, ld_bytes) holding columns [col0, col0 + cols) of h: the code bytes of
        every row, and per 128-row block the run of 512-byte scale tiles of those columns."""
        assert col0 % 64 == 0 and cols % 64 == 0
        if cols == 0:
            return []
        return [(self.codes_off + col0 // 2, self.m, cols // 2, self.codes_ld),
                (self.scales_off + (col0 // 64) * 512, self.row_blocks, (cols // 64) * 512, (self.scale_slots // 4) * 512)]

    def out_regions(self, col0: int, cols: int):
        assert col0 % 8 == 0 and cols % 8 == 0
        return [(self.out_off + col0 * 2, self.m, cols * 2, self.out_ld)] if cols else []


class PeerMlp:
    """One N-sharded prefill MLP block per call, out = down(silu(gate x) * up x) + residual on every rank:

        quantise x (replicated)  ->  gate/up GEMM on this rank's shard, epilogue writes NVFP4 h columns
        ->  push h columns to all ranks, wait  ->  down GEMM on this rank's row shard (+ residual)
        ->  push the BF16 output columns to all ranks, wait.

    The exchange moves 0.5625 bytes per element of h and 2 bytes per element of the output instead of the BF16
    all-gather of gate/up (4 bytes per element of h).  `buffers` lists every rank's PeerBuffer (buffers[rank] local);
    in one process all of them can be local (emulated ranks: call `stage(i)` for all ranks in turn)."""

    def __init__(self, layout: MlpLayout, buffers, rank: int, gate_up_shard, down_shard, h_scale, status):
        self.layout, self.buffers, self.rank = layout, buffers, rank
        self.gate_up, self.down, self.h_scale, self.status = gate_up_shard, down_shard, h_scale, status
        self.world = len(buffers)
        self.epoch = 0
        raw = buffers[rank].bytes()
        L = layout
        self.h_codes = raw[L.codes_off:L.codes_off + L.m * L.codes_ld]
        self.h_scales = raw[L.scales_off:L.scales_off + L.scales_bytes]
        self.out = buffers[rank].tensor().reshape(-1)[L.out_off // 2:L.out_off // 2 + L.m * L.hidden].view(L.m, L.hidden)

    def stage(self, i: int, a_codes=None, a_scales=None, g=None, residual=None):
        """Stage 0: gate/up GEMM + push of h; 1: wait for h; 2: down GEMM + push of the output; 3: wait for it."""
        from . import engine

        L = self.layout
        if i == 0:
            self.epoch += 2
            engine.gemm_w4a4_gate_up_quant(self.gate_up, a_codes, a_scales, g, L.m, self.h_scale,
                                           scratch=(self.h_codes, self.h_scales, None), status=self.status)
            regs = L.h_regions(self.gate_up.row_begin // 2, self.gate_up.rows // 2)
            engine.peer_push(self.buffers, self.rank, regs or [(0, 0, 16, 16)], self.epoch - 1)
        elif i == 1:
            engine.peer_gather_wait(self.buffers, self.rank, self.epoch - 1, self.status)
        elif i == 2:
            col0, cols = self.down.row_begin, self.down.rows
            if cols:
                res = residual[:, col0:col0 + cols] if residual is not None else None
                engine.gemm_w4a4(self.down, self.h_codes.view(L.m, L.codes_ld), self.h_scales, self.h_scale, L.m,
                                 out=self.out[:, col0:col0 + cols], status=self.status, residual=res)
            engine.peer_push(self.buffers, self.rank, L.out_regions(col0, cols) or [(0, 0, 16, 16)], self.epoch)
        else:
            engine.peer_gather_wait(self.buffers, self.rank, self.epoch, self.status)

    def run(self, a_codes, a_scales, g, residual=None):
        self.stage(0, a_codes, a_scales, g)
        self.stage(1)
        self.stage(2, residual=residual)
        self.stage(3)
        return self.out
