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

    Ranks must call `project` the same number of times: the epochs are counted on the device (epoch argument 0 of
    the C ABI), so a captured `project` can be replayed as a CUDA graph.  Before reusing the matrix for the next
    projection every rank must have finished reading it: call `dist.barrier()` or order the work otherwise."""

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
        dist.barrier(group)

    def project(self, weight_shard, a_codes, a_scales_tiled, g):
        from . import engine

        engine.gemm_w4a4_allgather(weight_shard, a_codes, a_scales_tiled, g, self.m, self.buffers, self.rank, 0, self.status)
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
        self.scales_ld = (self.scale_slots // 4) * 512   # bytes of scale tiles per 128-row block
        self.out_off = _round_up(self.scales_off + self.scales_bytes, 256)
        self.out_ld = hidden * 2
        self.total = _round_up(self.out_off + m * self.out_ld, 256)

    def h_regions(self, col0: int, cols: int, row0: int = 0, rows: int | None = None):
        """Regions (offset, rows, row_bytes, ld_bytes) holding columns [col0, col0 + cols) of rows [row0, row0 + rows)
        of h: the code bytes of every row, and per 128-row block the run of 512-byte scale tiles of those columns.
        row0 must be a multiple of 128 (a scale tile is 128 rows high)."""
        rows = self.m - row0 if rows is None else rows
        assert col0 % 64 == 0 and cols % 64 == 0 and row0 % 128 == 0
        if cols == 0 or rows == 0:
            return []
        blocks = _round_up(rows, 128) // 128
        return [(self.codes_off + row0 * self.codes_ld + col0 // 2, rows, cols // 2, self.codes_ld),
                (self.scales_off + (row0 // 128) * self.scales_ld + (col0 // 64) * 512, blocks, (cols // 64) * 512, self.scales_ld)]

    def out_regions(self, col0: int, cols: int, row0: int = 0, rows: int | None = None):
        rows = self.m - row0 if rows is None else rows
        assert col0 % 8 == 0 and cols % 8 == 0
        return [(self.out_off + row0 * self.out_ld + col0 * 2, rows, cols * 2, self.out_ld)] if cols and rows else []


class PeerMlp:
    """One N-sharded prefill MLP block per call, out = down(silu(gate x) * up x) + residual on every rank:

        quantise x (replicated)  ->  gate/up GEMM on this rank's shard, epilogue writes NVFP4 h columns
        ->  push h columns to all ranks, wait  ->  down GEMM on this rank's row shard (+ residual)
        ->  push the BF16 output columns to all ranks, wait.

    The exchange moves 0.5625 bytes per element of h and 2 bytes per element of the output instead of the BF16
    all-gather of gate/up (4 bytes per element of h).  `buffers` lists every rank's PeerBuffer (buffers[rank] local);
    in one process all of them can be local (emulated ranks: call `stage(i)` for all ranks in turn).  Epochs are
    counted on the device, so `run` can be captured in a CUDA graph and replayed; every rank must run the same
    sequence of blocks with the same `chunks`.

    `run(..., chunks=c)` cuts the tokens into c groups (multiples of 128 rows) and issues the pushes on a second
    stream, so that the transfer of one group runs under the GEMM of the next."""

    def __init__(self, layout: MlpLayout, buffers, rank: int, gate_up_shard, down_shard, h_scale, status):
        self.layout, self.buffers, self.rank = layout, buffers, rank
        self.gate_up, self.down, self.h_scale, self.status = gate_up_shard, down_shard, h_scale, status
        self.world = len(buffers)
        raw = buffers[rank].bytes()
        L = layout
        self.h_codes = raw[L.codes_off:L.codes_off + L.m * L.codes_ld]
        self.h_scales = raw[L.scales_off:L.scales_off + L.scales_bytes]
        self.out = buffers[rank].tensor().reshape(-1)[L.out_off // 2:L.out_off // 2 + L.m * L.hidden].view(L.m, L.hidden)
        self._comm = None

    # -- the four steps on a group of rows [r0, r0 + rows) -------------------------------------------------------
    def _gate_up(self, a_codes, a_scales, g, r0, rows):
        from . import engine

        L = self.layout
        k = a_codes.shape[1] * 2
        a_slots = _round_up(k // 16, 4)
        engine.gemm_w4a4_gate_up_quant(
            self.gate_up, a_codes[r0:r0 + rows], a_scales[(r0 // 128) * 128 * a_slots:], g, rows, self.h_scale,
            scratch=(self.h_codes[r0 * L.codes_ld:], self.h_scales[(r0 // 128) * L.scales_ld:], None), status=self.status)

    def _push_h(self, r0, rows):
        from . import engine

        regs = self.layout.h_regions(self.gate_up.row_begin // 2, self.gate_up.rows // 2, r0, rows)
        engine.peer_push(self.buffers, self.rank, regs or [(0, 0, 16, 16)], 0)

    def _down(self, residual, r0, rows):
        from . import engine

        L = self.layout
        col0, cols = self.down.row_begin, self.down.rows
        if cols:
            res = residual[r0:r0 + rows, col0:col0 + cols] if residual is not None else None
            engine.gemm_w4a4(self.down, self.h_codes.view(L.m, L.codes_ld)[r0:r0 + rows], self.h_scales[(r0 // 128) * L.scales_ld:],
                             self.h_scale, rows, out=self.out[r0:r0 + rows, col0:col0 + cols], status=self.status, residual=res)

    def _push_out(self, r0, rows):
        from . import engine

        regs = self.layout.out_regions(self.down.row_begin, self.down.rows, r0, rows)
        engine.peer_push(self.buffers, self.rank, regs or [(0, 0, 16, 16)], 0)

    def _wait(self):
        from . import engine

        engine.peer_gather_wait(self.buffers, self.rank, 0, self.status)

    def stage(self, i: int, a_codes=None, a_scales=None, g=None, residual=None):
        """Stage 0: gate/up GEMM + push of h; 1: wait for h; 2: down GEMM + push of the output; 3: wait for it."""
        m = self.layout.m
        if i == 0:
            self._gate_up(a_codes, a_scales, g, 0, m)
            self._push_h(0, m)
        elif i == 1:
            self._wait()
        elif i == 2:
            self._down(residual, 0, m)
            self._push_out(0, m)
        else:
            self._wait()

    def run(self, a_codes, a_scales, g, residual=None, chunks: int = 1):
        import torch

        m = self.layout.m
        if chunks <= 1 or self.world == 1:
            for i in range(4):
                self.stage(i, a_codes, a_scales, g, residual)
            return self.out
        # row groups of whole 128-row blocks
        blocks = _round_up(m, 128) // 128
        cuts = [min(m, 128 * (blocks * c // chunks)) for c in range(chunks + 1)]
        groups = [(cuts[c], cuts[c + 1] - cuts[c]) for c in range(chunks) if cuts[c + 1] > cuts[c]]
        main = torch.cuda.current_stream()
        if self._comm is None:
            self._comm = torch.cuda.Stream(device=self.out.device)
        comm = self._comm
        comm.wait_stream(main)
        # pushes go to the second stream in the order h(0), h(1), ..., out(0), out(1), ...; the waits on the main
        # stream come in the same order, which is what the device-counted epochs match
        for (r0, rows) in groups:
            self._gate_up(a_codes, a_scales, g, r0, rows)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(comm):
                comm.wait_event(done)
                self._push_h(r0, rows)
        for (r0, rows) in groups:
            self._wait()
            self._down(residual, r0, rows)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(comm):
                comm.wait_event(done)
                self._push_out(r0, rows)
        for _ in groups:
            self._wait()
        main.wait_stream(comm)
        return self.out
