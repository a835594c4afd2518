"""Two-dimensional sharding of the aggregation: destinations x sources over an r x c grid of GPUs.

Row-block sharding (sharding.py) makes every rank receive the whole feature matrix but its own block:
(R-1)/R of N*D per pass, which bounds graphs with few edges per node (a rank's share of the gather is
over before the rows have arrived).  Here rank (i, j) = i*c + j computes, for the destinations of
*destination group* i (the row blocks of ranks i*c .. i*c+c-1, contiguous), the partial sums over the
sources of *column group* j (the row blocks of ranks j, c+j, 2c+j, ...):

  1. all-gather of the feature blocks inside the column group (r ranks): (r-1)/R of N*D received;
  2. the rank's plan: rows of group i, only the entries whose source lies in column group j;
  3. reduce-scatter of the partial rows inside the destination group (c ranks): (c-1)/R of N*D
     received, after which every rank holds the finished sums of its own row block;
  4. the per-row factor of the mean / GCN operator on the own rows.

Received per pass: (r + c - 2)/R of N*D — 0.5 at 2 x 4 against 0.875 for row blocks on 8 GPUs.  The
partial rows are produced in Q chunks of destinations, laid out so that each chunk is one
reduce_scatter_tensor, and chunk q travels while chunk q+1 is gathered.  GCN rows travel pre-scaled
by rsqrt(deg) of the source; the kernels run in sum mode and step 4 applies rsqrt(deg) (or 1/deg) of
the destination.  Steps 1 and 3 run either as NCCL collectives or as asynchronous copies out of the
peers' shared buffers (copy engines) followed by a local add (GridPipeline's `transport`).  Upstream
has no multi-GPU path (ROF_evaluation/ROF_main.py runs one process).

Reuse groups are not used here: a group's sources may lie in different column groups.  The plans are
built from the destination CSR (the `SAG` / `GNNA` layout of upstream, reuse_conv.cpp:132-205).
"""
import numpy as np
import torch
import torch.distributed as dist

from .plan import AggregationPlan, padded_width, scale_rows
from .sharding import PeerWindows, SharedStore, row_blocks


class GridLayout:
    """Index arithmetic of the r x c grid for one rank.  `cols` = c, `chunks` = Q."""

    def __init__(self, num_nodes, world, rank, cols, chunks=1):
        if world % cols:
            raise ValueError("the grid's column count must divide the world size")
        self.n, self.world, self.rank = int(num_nodes), int(world), int(rank)
        self.c, self.r = int(cols), world // int(cols)
        self.i, self.j = divmod(self.rank, self.c)
        self.blk, self.blocks = row_blocks(self.n, world)
        self.q = max(1, int(chunks))
        self.cb = (self.blk + self.q - 1) // self.q          # rows of one rank's chunk
        self.src_rows = self.r * self.blk                    # gathered source rows (column group j)
        self.dst_rows = self.q * self.c * self.cb            # partial rows, chunk-major (>= c * blk)
        self.m = max(self.src_rows, self.dst_rows)           # node count the local plans are built for
        self.d0 = min(self.i * self.c * self.blk, self.n)    # destination group i = global rows [d0, d1)
        self.d1 = min((self.i + 1) * self.c * self.blk, self.n)

    def column_group(self, j=None):
        j = self.j if j is None else j
        return [ii * self.c + j for ii in range(self.r)]

    def destination_group(self, i=None):
        i = self.i if i is None else i
        return [i * self.c + jj for jj in range(self.c)]

    def src_map(self, ids):
        """global source ids -> rows of the gathered buffer; -1 for sources of other column groups"""
        ids = np.asarray(ids, dtype=np.int64)
        b, o = ids // self.blk, ids % self.blk
        return np.where(b % self.c == self.j, (b // self.c) * self.blk + o, -1)

    def dst_map(self, ids):
        """global destination ids of group i -> rows of the chunk-major partial buffer:
        chunk q holds rows [q*cb, (q+1)*cb) of every rank of the group, rank after rank"""
        ids = np.asarray(ids, dtype=np.int64)
        b, o = ids // self.blk - self.i * self.c, ids % self.blk
        return (o // self.cb) * (self.c * self.cb) + b * self.cb + o % self.cb

    def local_csr(self, indptr_dst, indices_src):
        """(row_ptr [dst_rows + 1], col) of this rank's tile of the adjacency: rows in partial-buffer
        order, entries = gathered-buffer rows, only sources of column group j"""
        ip = np.asarray(indptr_dst, dtype=np.int64)
        e0, e1 = int(ip[self.d0]), int(ip[self.d1])
        src = self.src_map(np.asarray(indices_src[e0:e1]))
        deg = np.diff(ip[self.d0:self.d1 + 1])
        keep = src >= 0
        rows = self.dst_map(np.repeat(np.arange(self.d0, self.d1, dtype=np.int64), deg)[keep])
        src = src[keep]
        order = np.argsort(rows, kind="stable")
        counts = np.bincount(rows, minlength=self.dst_rows)
        ptr = np.zeros(self.dst_rows + 1, dtype=np.int64)
        np.cumsum(counts, out=ptr[1:])
        return ptr, src[order].astype(np.int32)

    def chunk_rows(self, q):
        return q * self.c * self.cb, (q + 1) * self.c * self.cb

    def chunk_plans(self, indptr_dst, indices_src, device=None):
        """one plan per chunk of destinations (rows = the chunk's slice of the partial buffer)"""
        ptr, col = self.local_csr(indptr_dst, indices_src)
        if ptr[-1] >= 2 ** 31:
            raise ValueError("more than 2^31 entries in one rank's tile")
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32))
        ci, pp, pn = t(col), t(ptr), t(np.arange(self.dst_rows))
        return [AggregationPlan.from_parts(self.m, ci, pp, pn, rows=self.chunk_rows(q), device=device)
                for q in range(self.q)]


class GridPipeline:
    """One rank of the r x c grid: buffers, groups and the pass (see the module docstring).

    `groups` = (column process group, destination process group) or None for a layout that is only
    computed with (tests that emulate the ranks on one GPU fill `sources` themselves and add the
    partial rows of a destination group on the host)."""

    @staticmethod
    def default_cols(world):
        """columns of the grid: received rows are (r + c - 2)/R, least for a square grid; the larger
        factor goes to the columns (the reduce-scatter overlaps the gather chunk by chunk, the
        all-gather in front of the pass does not)"""
        c = 1
        while c * c < world:
            c *= 2
        while world % c:
            c //= 2
        return max(1, c)

    @staticmethod
    def make_groups(layout):
        """the two process groups of this rank; every rank must call this (new_group is collective)"""
        L = layout
        col = dst = None
        for j in range(L.c):
            g = dist.new_group(L.column_group(j))
            if j == L.j:
                col = g
        for i in range(L.r):
            g = dist.new_group(L.destination_group(i))
            if i == L.i:
                dst = g
        return col, dst

    def __init__(self, layout, plans, dim, device, groups=None, like=None, transport="nccl"):
        """transport "nccl": all_gather_into_tensor and reduce_scatter_tensor.  transport "copy"
        (collective constructor): the source and the partial buffers are shared stores that the
        peers map; a rank pulls the other slots of its column group and, chunk by chunk, the partial
        rows of its own block from the other ranks of its destination group with asynchronous copies
        (copy engines), and adds them itself.  One-float all-reduces on the transfer stream tell the
        ranks when a slot or a chunk may be read and when the buffers may be written again."""
        L = layout
        self.layout, self.plans, self.dim, self.device = L, plans, int(dim), torch.device(device)
        ld = padded_width(dim)
        self.groups = groups if like is None else like.groups
        self.transport = transport if (self.groups is not None and L.world > 1) else "nccl"
        if self.transport not in ("nccl", "copy"):
            raise ValueError("transport must be 'nccl' or 'copy'")
        self.src_win = self.part_win = None
        if self.transport == "copy":
            self.src_store = SharedStore(L.m, ld, device)
            self.part_store = SharedStore(L.dst_rows, ld, device)
            self._src, self._partial = self.src_store.tensor, self.part_store.tensor
            if L.r > 1:
                self.src_win = PeerWindows(self.src_store, L.i, L.r, self.groups[0])
            if L.c > 1:
                self.part_win = PeerWindows(self.part_store, L.j, L.c, self.groups[1])
            # the partial rows of this rank's block as the other ranks of the destination group hold them
            self._incoming = torch.zeros((max(L.c - 1, 1), L.q * L.cb, ld), device=device)
            self._token = torch.zeros(1, device=device)
            self.released = torch.cuda.Event()
        else:
            self._src = torch.zeros((L.m, ld), device=device)       # rows [0, r*blk): the column group's features
            self._partial = torch.zeros((L.dst_rows, ld), device=device)
        self.sources = self._src[:, :dim]
        self.partial = self._partial[:, :dim]
        self._reduced = torch.zeros((L.q * L.cb, ld), device=device)
        self.comm = torch.cuda.Stream(device, priority=-1)
        self.ready = torch.cuda.Event()
        self.gathered = torch.cuda.Event()
        self.done = [torch.cuda.Event() for _ in range(L.q)]
        self.reduced = [torch.cuda.Event() for _ in range(L.q)]
        self.launches = 0

    def own_slot(self):
        L = self.layout
        return self._src[L.i * L.blk:(L.i + 1) * L.blk]

    def set_local(self, x_local, degrees_local, mode):
        """this rank's rows (scaled by rsqrt(deg) for GCN) into its slot of the source buffer"""
        rows = x_local.size(0)
        scale_rows(x_local, degrees_local, "rsqrt" if mode == "gcn" else "copy", out=self.own_slot()[:rows, :self.dim])

    def gather_sources(self, cur):
        L = self.layout
        if L.r > 1:
            self.ready.record(cur)
            with torch.cuda.stream(self.comm):
                self.comm.wait_event(self.ready)
                if self.transport == "copy":
                    dist.all_reduce(self._token, group=self.groups[0])       # every own slot of the group is written
                    row_bytes = self._src.stride(0) * 4
                    for ii in range(L.r):
                        if ii != L.i:
                            self.src_win.pull(self._src[ii * L.blk:(ii + 1) * L.blk], ii, ii * L.blk * row_bytes, self.comm)
                else:
                    dist.all_gather_into_tensor(self._src[:L.src_rows], self.own_slot(), group=self.groups[0])
                self.gathered.record(self.comm)
            cur.wait_event(self.gathered)

    def compute_chunk(self, q):
        a, b = self.layout.chunk_rows(q)
        p = self.plans[q]
        p.aggregate(self.sources, None, "sum", out=self._partial[a:b, :self.dim])
        return p.last_launch_count()

    def reduce_chunk(self, q, cur):
        """partial rows of chunk q -> this rank's rows [q*cb, (q+1)*cb) of the finished sums"""
        L = self.layout
        a, b = L.chunk_rows(q)
        out = self._reduced[q * L.cb:(q + 1) * L.cb]
        self.done[q].record(cur)
        with torch.cuda.stream(self.comm):
            self.comm.wait_event(self.done[q])
            if self.transport == "copy":
                if L.c > 1:
                    dist.all_reduce(self._token, group=self.groups[1])       # chunk q is complete on every rank of the group
                    row_bytes = self._partial.stride(0) * 4
                    k = 0
                    for jj in range(L.c):
                        if jj != L.j:
                            self.part_win.pull(self._incoming[k][q * L.cb:(q + 1) * L.cb], jj,
                                               (a + L.j * L.cb) * row_bytes, self.comm)
                            k += 1
            elif L.c > 1:
                dist.reduce_scatter_tensor(out, self._partial[a:b], group=self.groups[1])
            else:
                out.copy_(self._partial[a:b])
            self.reduced[q].record(self.comm)

    def _add_pulled(self):
        """finished sums of this rank's block = its own partial rows + the ones pulled from the peers"""
        L = self.layout
        ld = self._partial.shape[1]
        own = self._partial.view(L.q, L.c, L.cb, ld)[:, L.j]
        acc = self._reduced.view(L.q, L.cb, ld)
        if L.c > 1:
            torch.add(own, self._incoming[0].view(L.q, L.cb, ld), out=acc)
            for k in range(1, L.c - 1):
                acc.add_(self._incoming[k].view(L.q, L.cb, ld))
            return L.c - 1
        acc.copy_(own)
        return 1

    def aggregate(self, x_local, degrees_local, mode, out, transfers=True, kernels=True):
        """x_local: this rank's [rows, dim] features (None: the own slot is already filled);
        degrees_local: the degrees of the same rows (None for 'sum'); out: [rows, dim].
        transfers / kernels = False leave one side out (timing breakdown: the buffers then hold
        whatever the last full pass left)."""
        cur = torch.cuda.current_stream(self.device)
        launches = 0
        if kernels and x_local is not None:
            self.set_local(x_local, degrees_local, mode)
            launches += 1
        if transfers:
            self.gather_sources(cur)
        for q in range(self.layout.q):
            if kernels:
                launches += self.compute_chunk(q)
            if transfers:
                self.reduce_chunk(q, cur)
        if transfers:
            for ev in self.reduced:
                cur.wait_event(ev)
            if self.transport == "copy":
                with torch.cuda.stream(self.comm):       # every rank has pulled what it needs: buffers may be rewritten
                    dist.all_reduce(self._token)
                    self.released.record(self.comm)
        if kernels:
            if self.transport == "copy":
                launches += self._add_pulled()
            rows = out.size(0)
            op = {"sum": "copy", "mean": "reciprocal", "gcn": "rsqrt"}[mode]
            scale_rows(self._reduced[:rows, :self.dim], degrees_local, op, out=out)
            launches += 1
        if transfers and self.transport == "copy":
            cur.wait_event(self.released)
        self.launches = launches
        return out

    def close_windows(self):
        """unmap the peers' buffers (every rank, before any owner frees its stores)"""
        for w in (self.src_win, self.part_win):
            if w is not None:
                w.close()

    def transfer_only(self):
        """the pass's collectives without its kernels (timing breakdown)"""
        return self.aggregate(None, None, "sum", None, transfers=True, kernels=False)

    def aggregate_only(self, degrees_local, mode, out):
        """the pass's kernels over whatever the buffers hold, without collectives (timing breakdown)"""
        return self.aggregate(None, degrees_local, mode, out, transfers=False, kernels=True)

    def received_bytes_per_pass(self):
        L = self.layout
        ld = self._src.shape[1]
        return ((L.r - 1) * L.blk + (L.c - 1) * L.q * L.cb) * ld * 4
