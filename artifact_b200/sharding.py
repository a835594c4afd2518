"""Row-block sharding of the aggregation over the GPUs of one node.

Destinations are independent, so rank r owns a block of destination rows and a plan built for
that block only; what the ranks exchange per pass is the feature matrix: every rank contributes
its block of rows and receives all the others (NCCL over NVLink) into a full [N, D] buffer in its
own HBM.  Kernels only ever read local memory.  Upstream is single-GPU (no collective anywhere in
its tree); this module is new.
"""
import ctypes

import numpy as np
import torch
import torch.distributed as dist

from . import _native


def row_blocks(num_nodes, world, indptr=None, row_cost=8):
    """-> (block_rows, [(r0, r1)] per rank).

    Without `indptr`: equal-sized blocks (the last may be short or empty), block_rows = their
    size, so that one all_gather_into_tensor moves the whole matrix.
    With `indptr` (the destination CSR's row pointers): contiguous blocks of about equal *work*,
    work(v) = in-degree(v) + row_cost — on a power-law graph whose hubs sit next to each other equal
    row counts would give one rank most of the edges.  block_rows is None (blocks differ)."""
    if world <= 0:
        return num_nodes, [(0, num_nodes)]
    if indptr is None:
        blk = (num_nodes + world - 1) // world
        return blk, [(min(r * blk, num_nodes), min((r + 1) * blk, num_nodes)) for r in range(world)]
    ip = np.asarray(indptr, dtype=np.int64)
    if ip.shape[0] != num_nodes + 1:
        raise ValueError("indptr must have num_nodes + 1 entries")
    work = (ip - ip[0]) + row_cost * np.arange(num_nodes + 1, dtype=np.int64)     # cumulative work before row v
    cuts = [0]
    for r in range(1, world):
        cuts.append(int(np.searchsorted(work, work[-1] * r / world, side="left")))
    cuts.append(num_nodes)
    cuts = np.maximum.accumulate(np.minimum(cuts, num_nodes))
    return None, [(int(cuts[r]), int(cuts[r + 1])) for r in range(world)]


class ShardedFeatures:
    """The receive buffer of one feature matrix and its all-gather.

    Equal blocks (bounds=None): a padded [world*block, D] buffer filled by one
    all_gather_into_tensor.  Given `bounds` ([(r0, r1)] per rank, e.g. from row_blocks(...,
    indptr)): an exact [N, D] buffer whose blocks travel as grouped sends/receives.
    The rows are stored with a stride padded to a multiple of 4 floats (so that the gather kernels
    use 128-bit loads whatever D is); `full` is the [rows, D] view, and whole padded rows travel."""

    def __init__(self, num_nodes, dim, rank, world, device, dtype=torch.float32, group=None, bounds=None,
                 shared=False):
        """shared: allocate the buffer as a SharedStore, so that peers can map it (copy transport)"""
        self.n, self.dim, self.rank, self.world, self.group = num_nodes, dim, rank, world, group
        if bounds is None:
            self.block, self.blocks = row_blocks(num_nodes, world)
            self.equal = True
            rows = self.block * world
        else:
            self.blocks = [(int(a), int(b)) for a, b in bounds]
            if len(self.blocks) != world or self.blocks[0][0] != 0 or self.blocks[-1][1] != num_nodes or any(
                    self.blocks[i][1] != self.blocks[i + 1][0] for i in range(world - 1)):
                raise ValueError("bounds must be `world` contiguous blocks covering [0, num_nodes)")
            self.block, self.equal = None, False
            rows = num_nodes
        self.shared = SharedStore(rows, (dim + 3) // 4 * 4, device) if shared else None
        self._store = (self.shared.tensor if shared else
                       torch.zeros((rows, (dim + 3) // 4 * 4), dtype=dtype, device=device))
        self.full = self._store[:, :dim]

    @property
    def local_rows(self):
        r0, r1 = self.blocks[self.rank]
        return r1 - r0

    def _block_rows(self, b):
        if self.equal:
            return b * self.block, (b + 1) * self.block
        return self.blocks[b]

    def block_view(self, b):
        """the rows of the buffer that rank b's block occupies (padding rows included for equal blocks)"""
        r0, r1 = self._block_rows(b)
        return self.full[r0:r1]

    def _block_store(self, b):
        """the same rows with their padding columns: contiguous, this is what travels"""
        r0, r1 = self._block_rows(b)
        return self._store[r0:r1]

    def local_view(self):
        """this rank's block inside the full buffer"""
        return self.block_view(self.rank)

    def exchange_ops(self, offsets):
        """grouped point-to-point operations that bring in the blocks of ranks (rank + k) % world, k in
        `offsets`, and send this rank's block to ranks (rank - k) % world"""
        ops = []
        for k in offsets:
            if k % self.world == 0:
                continue                             # the rank's own block is already in place
            src = (self.rank + k) % self.world
            dst = (self.rank - k) % self.world
            if self.local_view().numel():
                ops.append(dist.P2POp(dist.isend, self._block_store(self.rank), dst, group=self.group))
            if self.block_view(src).numel():
                ops.append(dist.P2POp(dist.irecv, self._block_store(src), src, group=self.group))
        return ops

    def all_gather(self, x_local=None):
        """x_local: this rank's block (padded to [block, D] for equal blocks) or None to send the rows
        already in local_view().  Returns the full [N, D] matrix (a view without padding rows)."""
        src = self.local_view() if x_local is None else x_local
        if tuple(src.shape) != tuple(self.local_view().shape):
            raise RuntimeError(f"local block must be {tuple(self.local_view().shape)}, got {tuple(src.shape)}")
        if x_local is not None and x_local.data_ptr() != self.local_view().data_ptr():
            self.local_view().copy_(x_local)
        if self.world > 1:
            if self.equal:
                dist.all_gather_into_tensor(self._store, self._block_store(self.rank), group=self.group)
            else:
                ops = self.exchange_ops(range(1, self.world))
                if ops:
                    for w in dist.batch_isend_irecv(ops):
                        w.wait()
        return self.full[:self.n]


class ShardedAggregator:
    """plan for this rank's row block + the all-gather in front of it"""

    def __init__(self, plan, features: ShardedFeatures):
        r0, r1 = features.blocks[features.rank]
        if (plan.info["row_begin"], plan.info["row_end"]) != (r0, r1):
            raise RuntimeError("the plan does not cover this rank's row block")
        self.plan, self.features = plan, features

    def aggregate(self, x_local, degrees, mode, out=None, phases=7):
        x_full = self.features.all_gather(x_local)
        return self.plan.aggregate(x_full, degrees, mode, out=out, phases=phases)


def stage_schedule(world):
    """Which peers' blocks travel in which stage, as lists of ring offsets k (the block of rank
    (r + k) % world).  Stage 0 is the rank's own block; the peers are cut into two groups, the
    nearer (world-1)//2 first, so that a pass is three stages whatever the world size: the
    aggregation of one stage covers the transfer of the next, while the number of kernel launches
    and NCCL calls per pass stays fixed.  [[0], [1, 2, 3], [4, 5, 6, 7]] for 8 ranks, [[0], [1],
    [2, 3]] for 4.  Measured on B200s, 114.6M-edge graph, D=256, ms per forward+backward step —
    8 GPUs: [[0],[1,2,3],[4..7]] 2.57; [[0],[1..7]] 2.66; no overlap 2.77; [[0,1,2,3],[4..7]] 2.77;
    [[0],[1],[2,3,4],[5,6,7]] 3.03; one stage per peer 5.7 (launch-bound);
    4 GPUs: [[0],[1],[2,3]] 3.63; [[0],[1,2,3]] 3.96."""
    if world <= 1:
        return [[0]]
    first = max(1, (world - 1) // 2)
    stages = [[0], list(range(1, 1 + first))]
    if 1 + first < world:
        stages.append(list(range(1 + first, world)))
    return stages


def piece_rows(lo, hi, piece, pieces):
    """rows of piece `piece` when [lo, hi) is cut into `pieces` contiguous parts of about equal size"""
    n = hi - lo
    return lo + n * piece // pieces, lo + n * (piece + 1) // pieces


def transfer_pieces(world, received_bytes_per_pass, piece_bytes=256e6, max_pieces=4):
    """How many pieces a peer group's transfer would be cut into if pieces of about `piece_bytes` were
    wanted (PipelinedAggregator(pieces=...)).  Pieces let the aggregation of one piece cover the transfer
    of the next: a large transfer beside a memory-bound gather is slowed down by it (2 B200s, 2.45M-node
    graph, D=256: 1.25 GB arrive in 1.97 ms alone and in ~5.9 ms beside the gather), and a stage cannot
    start before all it reads has landed.  But every piece is one more compute stage, i.e. one more
    pass over every destination row, and on that graph (mean degree 50) this costs more than the overlap
    returns: 19.8 / 21.0 / 23.7 ms per step with 1 / 2 / 4 pieces.  The pipeline therefore defaults to
    one piece; this helper is for callers whose rows are long enough to afford more."""
    if world <= 1:
        return 1
    groups = max(1, len(stage_schedule(world)) - 1)
    return int(min(max_pieces, max(1, round(received_bytes_per_pass / groups / piece_bytes))))


def compute_stages(ranges_per_stage, n, dim, entries_per_row, tile_bytes=64e6, min_entries_per_tile=48):
    """Cuts every transfer stage into compute stages whose source rows fit L2.

    ranges_per_stage[s]: the feature-row ranges [(r0, r1), ...] that transfer stage s makes readable
    (stage 0: the rank's own block).  -> (range_bounds, stage_of_range,
    transfer_stage_of_compute_stage).  When a stage's rows hold more than `tile_bytes` of features
    they are cut into tiles (contiguous row ranges of about equal size) that are aggregated one after
    the other, so that the gathers of a tile hit L2 (126 MB) — unless a destination would then gather
    fewer than `min_entries_per_tile` rows per tile, where the extra passes over the output cost more
    than the misses."""
    pieces = []                       # (r0, r1, compute stage)
    transfer_of = []
    for s, ranges in enumerate(ranges_per_stage):
        rng = sorted((int(a), int(b)) for a, b in ranges if b > a)
        rows = sum(b - a for a, b in rng)
        tiles = 1
        if rows > 0:
            tiles = max(1, int(np.ceil(rows * dim * 4 / tile_bytes)))
            while tiles > 1 and entries_per_row * (rows / max(n, 1)) / tiles < min_entries_per_tile:
                tiles -= 1
        per_tile = int(np.ceil(rows / tiles)) if rows else 0
        first = len(transfer_of)
        transfer_of.extend([s] * tiles)
        done = 0
        for a, b in rng:
            while a < b:
                t = min(done // per_tile, tiles - 1) if per_tile else 0
                take = min(b - a, (t + 1) * per_tile - done) if t < tiles - 1 else b - a
                pieces.append((a, a + take, first + t))
                a += take
                done += take
    pieces.sort()
    bounds, stage_of = [0], []
    for a, b, k in pieces:
        if a != bounds[-1]:
            raise RuntimeError("the stages' ranges do not tile the rows")
        bounds.append(b)
        stage_of.append(k)
    if bounds[-1] != n:
        raise RuntimeError("the stages' ranges do not cover every row")
    return bounds, stage_of, transfer_of


class _DeviceArray:
    """a raw device pointer behind the array interface torch.as_tensor reads (no copy is made)"""

    def __init__(self, ptr, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f4", "data": (int(ptr), False), "version": 2}


class SharedStore:
    """A [rows, ld] fp32 buffer on this GPU that the other processes of the box can map: its own
    device allocation (rof_shared_alloc), exported by a 64-byte handle, wrapped as a torch tensor."""

    def __init__(self, rows, ld, device):
        self.device = torch.device(device)
        ptr = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        self.bytes = max(int(rows) * int(ld) * 4, 4)
        with torch.cuda.device(self.device):
            _native.check(_native.cuda().rof_shared_alloc(self.bytes, ctypes.byref(ptr), handle))
        self.ptr, self.handle = ptr.value, bytes(handle)
        self.tensor = torch.as_tensor(_DeviceArray(self.ptr, (max(int(rows), 1), int(ld))), device=self.device)[:rows]
        if self.tensor.data_ptr() != self.ptr and rows:
            raise RuntimeError("torch copied the shared buffer instead of wrapping it")
        self.tensor.zero_()

    def close(self):
        if self.ptr:
            torch.cuda.synchronize(self.device)
            with torch.cuda.device(self.device):
                _native.cuda().rof_shared_free(ctypes.c_void_p(self.ptr))
            self.ptr = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class PeerWindows:
    """Every rank's feature buffer mapped into this process (CUDA interprocess handles), for
    copy-engine transfers.

    An SM-driven collective next to a gather kernel that saturates HBM gets a fraction of its
    bandwidth (2 B200s, 2.45M nodes x 256 floats: 3.9 ms of transfers and 16.5 ms of kernels take
    19.8 ms together).  A `cudaMemcpyAsync` out of the peer's buffer is carried out by the copy
    engines instead: no SMs, and its requests reach the memory system beside the kernel's.
    The constructor is collective over the group: every rank publishes the handle of its SharedStore
    and maps the others'.  `base[r]` is the device address of rank r's buffer in this process; it is
    only ever the source of rof_copy_async, never a kernel operand.  One process per GPU."""

    def __init__(self, store: SharedStore, rank, world, group=None):
        self.rank, self.world, self.device, self.store = rank, world, store.device, store
        everyone = [None] * world
        dist.all_gather_object(everyone, (store.handle, store.bytes), group=group)
        self.base = {}
        err = None
        try:
            with torch.cuda.device(self.device):
                for r, (handle, nbytes) in enumerate(everyone):
                    if r == rank:
                        continue
                    if nbytes != store.bytes:
                        raise RuntimeError(f"rank {r}'s buffer has another size than this rank's")
                    ptr = ctypes.c_void_p()
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(handle)
                    _native.check(_native.cuda().rof_shared_open(buf, ctypes.byref(ptr)))
                    self.base[r] = ptr.value
        except Exception as ex:                   # every rank must learn of it: they fail together below
            err = repr(ex)
        status = [None] * world
        dist.all_gather_object(status, err, group=group)
        bad = [(r, e) for r, e in enumerate(status) if e]
        if bad:
            self.close()
            raise RuntimeError(f"rank {bad[0][0]} could not map its peers' buffers: {bad[0][1]}")

    def pull(self, dst, peer, byte_offset, stream):
        """`dst` (contiguous rows of the local buffer) <- the bytes at `byte_offset` of rank `peer`'s
        buffer, as one asynchronous copy on `stream` (a torch stream)"""
        if not dst.is_contiguous():
            raise RuntimeError("peer copies move whole contiguous row ranges")
        nbytes = dst.numel() * dst.element_size()
        if byte_offset < 0 or byte_offset + nbytes > self.store.bytes:
            raise RuntimeError("peer copy outside the peer's buffer")
        with torch.cuda.device(self.device):
            _native.check(_native.cuda().rof_copy_async(ctypes.c_void_p(dst.data_ptr()),
                                                        ctypes.c_void_p(self.base[peer] + byte_offset), nbytes,
                                                        ctypes.c_void_p(stream.cuda_stream)))

    def close(self):
        if self.base:
            torch.cuda.synchronize(self.device)
            with torch.cuda.device(self.device):
                for p in self.base.values():
                    _native.cuda().rof_shared_close(ctypes.c_void_p(p))
            self.base = {}

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class PipelinedAggregator:
    """All-gather overlapped with aggregation, stage by stage.

    Rank r reads its own block in stage 0 and the blocks of ranks (r + k) % world, k in the
    stage's offsets (see stage_schedule), in the later stages; with `pieces` > 1 each group's transfer
    is cut further into that many stages (see transfer_pieces for when that pays).  A stage's rows travel as one group of paired
    sends/receives on a high-priority side stream (send a piece of the own block to rank r-k, receive
    the same piece of the block of rank r+k; NVSwitch gives every pair full bandwidth), and the
    per-stage plans run on the compute stream as soon as their rows have landed, adding into `out`.
    A stage whose rows exceed L2 is aggregated as several compute stages (compute_stages).  The result
    equals the whole-plan aggregate up to the order of the fp32 adds.  Every kernel reads this GPU's
    memory only.
    """

    def __init__(self, plan, features: ShardedFeatures, stage_plans=None, schedule=None, tile_bytes=64e6,
                 like=None, pieces=None, transport="nccl"):
        """transport: "nccl" (grouped send/receive) or "copy" (copy engines pull the peers' blocks out of
        their buffers, PeerWindows; collective: every rank must construct its aggregator at the same
        point)."""
        f = features
        r0, r1 = f.blocks[f.rank]
        if (plan.info["row_begin"], plan.info["row_end"]) != (r0, r1):
            raise RuntimeError("the plan does not cover this rank's row block")
        self.features, self.whole = f, plan
        if like is not None:          # a second feature buffer over the same plans (e.g. the gradient's)
            self.schedule, self.pieces, self.transfers = like.schedule, like.pieces, like.transfers
            self.stage_plans, self.transfer_of = like.stage_plans, like.transfer_of
        else:
            self.schedule = schedule or stage_schedule(f.world)
            self.pieces = max(1, int(pieces or 1))
            # transfer stages: the own block, then every group of peers, piece by piece
            self.transfers = []
            for offs in self.schedule:
                if all(k % f.world == 0 for k in offs):
                    self.transfers.append([(k, 0, 1) for k in offs])
                else:
                    for pc in range(self.pieces):
                        self.transfers.append([(k, pc, self.pieces) for k in offs])
            if f.world > 1:
                rows = max(r1 - r0, 1)
                ranges = []
                for st in self.transfers:
                    rs = []
                    for k, pc, npc in st:
                        lo, hi = piece_rows(*f._block_rows((f.rank + k) % f.world), pc, npc)
                        rs.append((min(lo, f.n), min(hi, f.n)))       # padding rows hold no features
                    ranges.append(rs)
                bounds, stage_of, self.transfer_of = compute_stages(
                    ranges, f.n, f.dim, plan.info["gather_entries"] / rows, tile_bytes)
                self.stage_plans = stage_plans or plan.stages_by_ranges(bounds, stage_of)
            else:
                self.stage_plans, self.transfer_of = stage_plans or [plan], [0]
        dev = f.full.device
        # the transfers run at high priority: their few blocks must get onto SMs that a gather kernel
        # with hundreds of thousands of short blocks would otherwise keep full
        self.comm_stream = torch.cuda.Stream(dev, priority=-1) if f.world > 1 else None
        self.ready = torch.cuda.Event() if f.world > 1 else None
        self.landed = [torch.cuda.Event() for _ in self.transfers]
        self.launches = 0
        self._prepared = None          # (key, [(fn, args)] per compute stage) of the last validated pass
        self.transport = transport if f.world > 1 else "nccl"
        if self.transport not in ("nccl", "copy"):
            raise ValueError("transport must be 'nccl' or 'copy'")
        if self.transport == "copy":
            if f.shared is None:
                raise RuntimeError("the copy transport needs ShardedFeatures(..., shared=True)")
            self.windows = PeerWindows(f.shared, f.rank, f.world, f.group)
            self._token = torch.zeros(1, device=dev)
            self.released = torch.cuda.Event()

    def _stage_ops(self, stage):
        f = self.features
        ops = []
        for k, pc, npc in stage:
            if k % f.world == 0:
                continue                                  # the rank's own block is already in place
            src, dst = (f.rank + k) % f.world, (f.rank - k) % f.world
            s0, s1 = piece_rows(*f._block_rows(f.rank), pc, npc)
            d0, d1 = piece_rows(*f._block_rows(src), pc, npc)
            if s1 > s0:
                ops.append(dist.P2POp(dist.isend, f._store[s0:s1], dst, group=f.group))
            if d1 > d0:
                ops.append(dist.P2POp(dist.irecv, f._store[d0:d1], src, group=f.group))
        return ops

    def _transfer_by_copies(self, cur):
        """Every rank pulls the blocks it needs out of the peers' buffers.  Two one-float all-reduces on
        the transfer stream order the ranks: the first says that every rank's own block is written (it
        follows this rank's `ready` event in stream order), the second that every rank has finished
        reading — the current stream waits for it at the end of the pass, so nothing that is enqueued
        after the pass can overwrite a block a peer is still reading."""
        f = self.features
        self.ready.record(cur)
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(self.ready)
            dist.all_reduce(self._token, group=f.group)
            for s, stage in enumerate(self.transfers):
                for k, pc, npc in stage:
                    if k % f.world == 0:
                        continue
                    src = (f.rank + k) % f.world
                    d0, d1 = piece_rows(*f._block_rows(src), pc, npc)
                    if d1 > d0:
                        self.windows.pull(f._store[d0:d1], src, d0 * f._store.stride(0) * 4, self.comm_stream)
                self.landed[s].record(self.comm_stream)
            dist.all_reduce(self._token, group=f.group)
            self.released.record(self.comm_stream)

    def _transfer(self, cur):
        if self.transport == "copy":
            return self._transfer_by_copies(cur)
        self.ready.record(cur)
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(self.ready)
            for s, stage in enumerate(self.transfers):
                ops = self._stage_ops(stage)
                if ops:
                    for w in dist.batch_isend_irecv(ops):
                        w.wait()
                self.landed[s].record(self.comm_stream)

    def _compute(self, cur, degrees, mode, out, wait=True):
        f = self.features
        x_full = f.full[:f.n]
        # a pass is several small launches: after the first, fully checked pass over the same buffers the
        # stages are re-issued through prepared C-ABI calls, without the Python-side checks
        key = (x_full.data_ptr(), out.data_ptr(), tuple(out.shape), out.stride(0),
               degrees.data_ptr() if degrees is not None else 0, mode)
        fast = self._prepared[1] if (self._prepared is not None and self._prepared[0] == key) else None
        launches = 0
        waited = set()
        prepared = []
        for k, p in enumerate(self.stage_plans):
            s = self.transfer_of[k]
            if wait and f.world > 1 and s not in waited and any(o % f.world for o, _, _ in self.transfers[s]):
                cur.wait_event(self.landed[s])
                waited.add(s)
            if fast is not None:
                fn, args = fast[k]
                args[-1] = ctypes.c_void_p(cur.cuda_stream)
                with torch.cuda.device(f.full.device):
                    _native.check(fn(*args))
            else:
                p.aggregate(x_full, degrees, mode, out=out, accumulate=k > 0)
                launches += p.last_launch_count()
                prepared.append(p.prepared_call(x_full, degrees, mode, out, k > 0))
        if fast is None:
            self.launches = launches
            self._prepared = (key, prepared)
        return out

    def aggregate(self, x_local, degrees, mode, out):
        f = self.features
        cur = torch.cuda.current_stream(f.full.device)
        if x_local is not None and x_local.data_ptr() != f.local_view().data_ptr():
            f.local_view().copy_(x_local)
        if f.world > 1:
            self._transfer(cur)
        self._compute(cur, degrees, mode, out)
        if self.transport == "copy":
            cur.wait_event(self.released)
        return out

    def transfer_only(self):
        """the pass's transfers without its kernels (timing breakdown); the current stream waits for them"""
        f = self.features
        if f.world <= 1:
            return
        cur = torch.cuda.current_stream(f.full.device)
        self._transfer(cur)
        for ev in self.landed:
            cur.wait_event(ev)
        if self.transport == "copy":
            cur.wait_event(self.released)

    def aggregate_only(self, degrees, mode, out):
        """the pass's kernels over whatever the buffer holds, without transfers (timing breakdown)"""
        return self._compute(torch.cuda.current_stream(self.features.full.device), degrees, mode, out, wait=False)


def column_chunks(dim, chunks=None):
    """[(c0, c1)] column ranges a feature matrix of width `dim` is exchanged in.  Default: four chunks
    from 256 floats, two from 128, one below (chunks narrower than 64 floats cost more in the gather
    than the overlap returns); chunk widths are multiples of 4 floats except possibly the last."""
    if chunks is None:
        chunks = 4 if dim >= 256 else (2 if dim >= 128 else 1)
    chunks = max(1, min(int(chunks), max(1, dim // 4)))
    per = ((dim + chunks - 1) // chunks + 3) // 4 * 4
    out = []
    c = 0
    while c < dim:
        out.append((c, min(dim, c + per)))
        c += per
    return out


class ColumnChunkedFeatures:
    """A feature matrix stored as K column chunks, each a contiguous [world*block, width_k] buffer of its
    own, so that every chunk is exchanged by ONE all_gather_into_tensor and can be aggregated (into the
    matching columns of the output) while the next chunk is still travelling.  Row blocks are of equal
    size (the collective needs that); rows are padded to a multiple of 4 floats."""

    def __init__(self, num_nodes, dim, rank, world, device, chunks=None, dtype=torch.float32, group=None):
        self.n, self.dim, self.rank, self.world, self.group = num_nodes, dim, rank, world, group
        self.block, self.blocks = row_blocks(num_nodes, world)
        self.cols = column_chunks(dim, chunks)
        self._stores = [torch.zeros((self.block * world, (c1 - c0 + 3) // 4 * 4), dtype=dtype, device=device)
                        for c0, c1 in self.cols]
        self.device = self._stores[0].device

    def chunk_full(self, k):
        """[N, width_k] view of chunk k holding every rank's rows (valid after its all-gather)"""
        c0, c1 = self.cols[k]
        return self._stores[k][:self.n, :c1 - c0]

    def chunk_local(self, k):
        """this rank's [block, width_k] rows of chunk k (padding rows beyond N included)"""
        c0, c1 = self.cols[k]
        return self._stores[k][self.rank * self.block:(self.rank + 1) * self.block, :c1 - c0]

    def _local_store(self, k):
        return self._stores[k][self.rank * self.block:(self.rank + 1) * self.block]

    def set_local(self, x_local):
        """copy this rank's [rows <= block, dim] features into the chunk buffers"""
        rows = x_local.size(0)
        for k, (c0, c1) in enumerate(self.cols):
            self.chunk_local(k)[:rows].copy_(x_local[:, c0:c1])

    def fill_normal_(self, generator):
        for s in self._stores:
            s.normal_(generator=generator)

    def rows(self, index):
        """the full-width rows `index` (a LongTensor on this device) gathered from the chunks"""
        return torch.cat([self.chunk_full(k)[index] for k in range(len(self.cols))], dim=1)

    def all_gather_chunk(self, k):
        if self.world > 1:
            dist.all_gather_into_tensor(self._stores[k], self._local_store(k), group=self.group)


class ColumnPipelinedAggregator:
    """All-gather overlapped with aggregation, column chunk by column chunk.

    The features travel as K column chunks, one all_gather_into_tensor each, on a high-priority side
    stream; chunk k is aggregated — the whole block plan over a [N, width_k] matrix, writing columns
    [c0, c1) of `out` — as soon as it has landed, while chunk k+1 is still on its way.  Compared with
    staging by source block (PipelinedAggregator) nothing is added to an existing output row and no
    destination row is visited once per stage with a fraction of its entries: a chunk re-reads only
    the 4-byte column entries, so short rows keep their efficiency, the transfers are plain collectives
    (one NCCL call each, in-network replication where NCCL uses it), and a chunk of up to ~64 MB needs
    no source tiling to stay in L2.  Every kernel reads this GPU's memory only.
    """

    def __init__(self, plan, features: ColumnChunkedFeatures):
        f = features
        r0, r1 = f.blocks[f.rank]
        if (plan.info["row_begin"], plan.info["row_end"]) != (r0, r1):
            raise RuntimeError("the plan does not cover this rank's row block")
        self.plan, self.features = plan, f
        self.comm_stream = torch.cuda.Stream(f.device, priority=-1) if f.world > 1 else None
        self.ready = torch.cuda.Event() if f.world > 1 else None
        self.landed = [torch.cuda.Event() for _ in f.cols]
        self.tiles = [plan.auto_tiles(c1 - c0) for c0, c1 in f.cols]
        self.launches = 0

    def _transfer(self, cur):
        f = self.features
        self.ready.record(cur)
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(self.ready)
            for k in range(len(f.cols)):
                f.all_gather_chunk(k)
                self.landed[k].record(self.comm_stream)

    def _compute(self, cur, degrees, mode, out, wait=True):
        f = self.features
        self.launches = 0
        for k, (c0, c1) in enumerate(f.cols):
            if wait and f.world > 1:
                cur.wait_event(self.landed[k])
            self.plan.aggregate(f.chunk_full(k), degrees, mode, out=out[:, c0:c1], tiles=self.tiles[k])
            self.launches += self.plan.last_launch_count()
        return out

    def aggregate(self, x_local, degrees, mode, out):
        f = self.features
        cur = torch.cuda.current_stream(f.device)
        if x_local is not None:
            f.set_local(x_local)
        if f.world > 1:
            self._transfer(cur)
        return self._compute(cur, degrees, mode, out)

    def transfer_only(self):
        """the pass's transfers without its kernels (timing breakdown); the current stream waits for them"""
        if self.features.world <= 1:
            return
        cur = torch.cuda.current_stream(self.features.device)
        self._transfer(cur)
        for ev in self.landed:
            cur.wait_event(ev)

    def aggregate_only(self, degrees, mode, out):
        """the pass's kernels over whatever the buffers hold, without transfers (timing breakdown)"""
        return self._compute(torch.cuda.current_stream(self.features.device), degrees, mode, out, wait=False)


class PieceMajorFeatures:
    """A feature matrix stored piece-major: every rank's row block is cut into P pieces of `pb` rows, and
    buffer piece p holds piece p of every rank — rows [p*world*pb, (p+1)*world*pb) of one [P*world*pb, D]
    matrix — so that ONE all_gather_into_tensor per piece moves a P-th of every block into place, and
    the pieces are exactly the source tiles the single-GPU pass walks (an L2-sized slice of the matrix
    each).  Global row r of rank b (offset o = r - b*block inside its block) lives in buffer row
    (o // pb) * world*pb + b*pb + o % pb; `perm` maps global ids to buffer rows, and a plan for this
    layout is built from index tensors whose *source* ids went through it (PieceMajorPipeline.plan_from_v2).
    Rows are padded to a multiple of 4 floats."""

    def __init__(self, num_nodes, dim, rank, world, device, pieces, dtype=torch.float32, group=None):
        self.n, self.dim, self.rank, self.world, self.group = num_nodes, dim, rank, world, group
        self.pieces = max(1, int(pieces))
        self.block, self.blocks = row_blocks(num_nodes, world)
        self.pb = (self.block + self.pieces - 1) // self.pieces          # rows of one rank's piece
        self.size = self.pieces * world * self.pb                         # rows of the buffer (>= num_nodes)
        self._store = torch.zeros((self.size, (dim + 3) // 4 * 4), dtype=dtype, device=device)
        self.full = self._store[:, :dim]
        self.device = self._store.device

    def perm(self, ids):
        """buffer rows of global row ids (numpy array or LongTensor in, same kind out)"""
        if isinstance(ids, torch.Tensor):
            b = torch.div(ids, self.block, rounding_mode="floor")
            o = ids - b * self.block
            return torch.div(o, self.pb, rounding_mode="floor") * (self.world * self.pb) + b * self.pb + o % self.pb
        ids = np.asarray(ids, dtype=np.int64)
        b, o = ids // self.block, ids % self.block
        return (o // self.pb) * (self.world * self.pb) + b * self.pb + o % self.pb

    def piece_store(self, p):
        """the contiguous rows of piece p (all ranks)"""
        return self._store[p * self.world * self.pb:(p + 1) * self.world * self.pb]

    def local_piece(self, p):
        """this rank's [pb, D] slot inside piece p"""
        r0 = p * self.world * self.pb + self.rank * self.pb
        return self._store[r0:r0 + self.pb]

    def set_local(self, x_local, degrees_local=None, op="copy"):
        """scatter this rank's [rows <= block, dim] features into its slots, optionally scaled per row
        (op 'rsqrt': the GCN factor of the source rows, applied before they travel)"""
        from .plan import scale_rows
        rows = x_local.size(0)
        for p in range(self.pieces):
            a, b = p * self.pb, min((p + 1) * self.pb, rows)
            if b <= a:
                break
            dst = self.local_piece(p)[:b - a, :self.dim]
            if op == "copy":
                dst.copy_(x_local[a:b])
            else:
                scale_rows(x_local[a:b], degrees_local[a:b], op, out=dst)

    def rows(self, index):
        """the rows with global ids `index` (a LongTensor on this device)"""
        return self.full[self.perm(index)]

    def all_gather_piece(self, p):
        if self.world > 1:
            dist.all_gather_into_tensor(self.piece_store(p), self.local_piece(p), group=self.group)


class PieceMajorPipeline:
    """All-gather overlapped with aggregation over a piece-major feature matrix.

    Piece p of every block travels in one all_gather_into_tensor on a high-priority side stream, and the
    rank's plan, split by source piece exactly like a single-GPU pass is split into source tiles, adds
    piece p's entries into `out` as soon as it has landed.  The compute side is therefore the single-GPU
    tiled pass (an L2-sized piece at a time), the transfer side is P plain collectives, and the two
    overlap piece by piece.  GCN passes travel pre-scaled: each rank multiplies its own rows by
    rsqrt(degrees) on the way into its slots and the kernels run ROF_MODE_GCN_PRESCALED, because source
    rows are addressed by buffer row while `degrees` stays indexed by node id.
    """

    @staticmethod
    def default_pieces(num_nodes, dim, world, entries_per_row=None, piece_bytes=64e6, min_entries_per_piece=48):
        """pieces of about `piece_bytes` of features (L2-sized), but no more than leave a destination
        `min_entries_per_piece` gathered rows per piece: every piece is one more pass over the destination
        rows, and short rows lose more to that than the overlap returns (2 B200s, community graph, 21
        entries per row: 1.30 ms per step with one piece, 1.71 ms with two).  One piece = one all-gather,
        then the whole plan."""
        pieces = max(1, round(num_nodes * dim * 4 / piece_bytes))
        if entries_per_row is not None:
            pieces = min(pieces, max(1, int(entries_per_row // min_entries_per_piece)))
        return int(min(8, max(1, pieces)))

    @staticmethod
    def plan_from_v2(features, uniqpart_column_index, uniqpart_pointers, part2Node_ptr, part2Node_col, device=None):
        """the rank's ROF_v2 plan over the piece-major matrix: source ids mapped to buffer rows"""
        from .plan import AggregationPlan
        f = features
        col = f.perm(np.asarray(uniqpart_column_index)).astype(np.int32)
        i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32))
        return AggregationPlan.from_v2(f.size, i32(col), i32(uniqpart_pointers), i32(part2Node_ptr), i32(part2Node_col),
                                       rows=f.blocks[f.rank], device=device or f.device)

    @staticmethod
    def own_first_ranges(pieces, world, pb, rank):
        """(range_bounds, stage_of_range) of the own-first split: the rank's own slot of every piece is
        stage 0 (readable before any transfer), the rest of piece p is stage p + 1"""
        bounds, stage = [0], []
        for p in range(pieces):
            base = p * world * pb
            for end, st in ((base + rank * pb, p + 1), (base + (rank + 1) * pb, 0), (base + world * pb, p + 1)):
                bounds.append(end)
                stage.append(st)
        return bounds, stage

    def __init__(self, plan, features: PieceMajorFeatures, like=None, own_first=False):
        """own_first: one more stage in front, over the rank's own rows, which need no transfer: it runs
        while the first piece travels (otherwise nothing covers that all-gather) at the price of one more
        pass over the destination rows."""
        f = features
        if (plan.info["row_begin"], plan.info["row_end"]) != tuple(f.blocks[f.rank]) or plan.info["num_nodes"] != f.size:
            raise RuntimeError("the plan must cover this rank's row block over the piece-major matrix (plan_from_v2)")
        self.plan, self.features = plan, f
        self.own_first = bool(like.own_first if like is not None else (own_first and f.world > 1))
        if like is not None:
            self.stage_plans = like.stage_plans
        elif self.own_first:
            self.stage_plans = plan.stages_by_ranges(*self.own_first_ranges(f.pieces, f.world, f.pb, f.rank))
        else:
            self.stage_plans = plan.stages(f.world * f.pb, list(range(f.pieces))) if f.pieces > 1 else [plan]
        self.comm_stream = torch.cuda.Stream(f.device, priority=-1) if f.world > 1 else None
        self.ready = torch.cuda.Event() if f.world > 1 else None
        self.landed = [torch.cuda.Event() for _ in range(f.pieces)]
        self.launches = 0
        self._prepared = None

    def pad_degrees(self, degrees):
        """degrees ([num_nodes], indexed by node id) padded to the buffer's row count, as the plan expects"""
        f = self.features
        out = torch.ones(f.size, dtype=degrees.dtype, device=degrees.device)
        out[:f.n] = degrees
        return out

    def _transfer(self, cur):
        f = self.features
        self.ready.record(cur)
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(self.ready)
            for p in range(f.pieces):
                f.all_gather_piece(p)
                self.landed[p].record(self.comm_stream)

    def _compute(self, cur, degrees_padded, mode, out, wait=True):
        f = self.features
        kmode = "gcn_prescaled" if mode == "gcn" else mode
        key = (out.data_ptr(), tuple(out.shape), out.stride(0),
               degrees_padded.data_ptr() if degrees_padded is not None else 0, kmode)
        fast = self._prepared[1] if (self._prepared is not None and self._prepared[0] == key) else None
        launches, prepared = 0, []
        first = 1 if self.own_first else 0           # stage s reads piece s - first (stage 0 of own-first: none)
        for p, sp in enumerate(self.stage_plans):
            if wait and f.world > 1 and p >= first:
                cur.wait_event(self.landed[p - first])
            if fast is not None:
                fn, args = fast[p]
                args[-1] = ctypes.c_void_p(cur.cuda_stream)
                with torch.cuda.device(f.device):
                    _native.check(fn(*args))
            else:
                sp.aggregate(f.full, degrees_padded, kmode, out=out, accumulate=p > 0)
                launches += sp.last_launch_count()
                prepared.append(sp.prepared_call(f.full, degrees_padded, kmode, out, p > 0))
        if fast is None:
            self.launches = launches
            self._prepared = (key, prepared)
        return out

    def aggregate(self, x_local, degrees_padded, mode, out):
        """x_local: this rank's [rows, dim] features (unscaled), or None when its slots are already filled;
        degrees_padded: pad_degrees(degrees) (None for 'sum')"""
        f = self.features
        cur = torch.cuda.current_stream(f.device)
        if x_local is not None:
            r0, r1 = f.blocks[f.rank]
            if mode == "gcn":
                f.set_local(x_local, degrees_padded[r0:r1], "rsqrt")
            else:
                f.set_local(x_local)
        if f.world > 1:
            self._transfer(cur)
        return self._compute(cur, degrees_padded, mode, out)

    def transfer_only(self):
        if self.features.world <= 1:
            return
        cur = torch.cuda.current_stream(self.features.device)
        self._transfer(cur)
        for ev in self.landed:
            cur.wait_event(ev)

    def aggregate_only(self, degrees_padded, mode, out):
        return self._compute(torch.cuda.current_stream(self.features.device), degrees_padded, mode, out, wait=False)
