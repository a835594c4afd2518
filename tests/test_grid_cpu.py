"""Destination x source grid sharding (artifact_b200/grid.py), host side: the index maps are
one-to-one, the tiles of the adjacency partition its entries, the partial rows of a destination
group add up to the operator, and the chunk plans (exported without a GPU) compute those partials."""
import numpy as np
import pytest
import torch

from artifact_b200.grid import GridLayout, GridPipeline
from conftest import load_golden
from test_sharding_cpu import eval_plan_numpy


def dense_sum(g, x):
    ip, idx = g["indptr_dst"], g["indices_src"]
    out = np.zeros((g["N"], x.shape[1]))
    for v in range(g["N"]):
        out[v] = x[idx[ip[v]:ip[v + 1]]].sum(0)
    return out


def test_default_grid_shapes():
    assert [GridPipeline.default_cols(w) for w in (1, 2, 4, 8, 16)] == [1, 2, 2, 4, 4]
    assert GridPipeline.default_cols(6) == 2
    with pytest.raises(ValueError):
        GridLayout(100, 8, 0, 3)


@pytest.mark.parametrize("name", ["c2_n640_ps2", "c5_n1024_ps2"])
@pytest.mark.parametrize("world,cols,chunks", [(2, 2, 1), (2, 1, 2), (4, 2, 3), (8, 4, 2), (8, 2, 4), (6, 3, 2)])
def test_grid_tiles_partition_the_operator(name, world, cols, chunks):
    g = load_golden(name)
    n = g["N"]
    x = np.random.default_rng(world * 10 + cols).standard_normal((n, 3))
    want = dense_sum(g, x)
    got = np.zeros_like(want)
    entries = 0
    for rank in range(world):
        L = GridLayout(n, world, rank, cols, chunks)
        assert sorted(L.column_group() + [r for j in range(L.c) if j != L.j for r in L.column_group(j)]) == list(range(world))
        # sources of the column group map one-to-one into the gathered buffer, the others to -1
        sm = L.src_map(np.arange(n))
        mine = sm >= 0
        assert len(np.unique(sm[mine])) == mine.sum() and sm[mine].max() < L.src_rows
        for rr in L.column_group():
            a, b = L.blocks[rr]
            assert mine[a:b].all() and (sm[a:b] == (rr // L.c) * L.blk + np.arange(b - a)).all()
        # destinations of the group map one-to-one into the chunk-major partial buffer; the rows of
        # rank (i, j') in chunk q are contiguous where reduce_scatter_tensor expects them
        dm = L.dst_map(np.arange(L.d0, L.d1))
        assert len(np.unique(dm)) == L.d1 - L.d0 and dm.max() < L.dst_rows
        for jj, rr in enumerate(L.destination_group()):
            a, b = L.blocks[rr]
            for q in range(L.q):
                lo, hi = a + q * L.cb, min(a + (q + 1) * L.cb, b)
                if hi > lo:
                    assert (L.dst_map(np.arange(lo, hi)) == q * L.c * L.cb + jj * L.cb + np.arange(hi - lo)).all()
        ptr, col = L.local_csr(g["indptr_dst"], g["indices_src"])
        entries += len(col)
        assert ptr[-1] == len(col) and (col >= 0).all() and (col < L.src_rows).all()
        # this rank's partial rows, added where a reduce-scatter inside the destination group puts them
        xs = np.zeros((L.src_rows, 3))
        xs[sm[mine]] = x[mine]
        part = np.zeros((L.dst_rows, 3))
        for row in range(L.dst_rows):
            part[row] = xs[col[ptr[row]:ptr[row + 1]]].sum(0)
        got[L.d0:L.d1] += part[dm]
    assert entries == len(g["indices_src"])
    assert np.allclose(got, want, rtol=1e-9, atol=1e-9)


@pytest.mark.parametrize("world,cols,chunks,rank", [(4, 2, 3, 1), (8, 4, 2, 6), (2, 2, 1, 0)])
def test_chunk_plans_compute_the_partials(world, cols, chunks, rank):
    g = load_golden("c2_n640_ps2")
    n = g["N"]
    L = GridLayout(n, world, rank, cols, chunks)
    plans = L.chunk_plans(g["indptr_dst"], g["indices_src"])
    assert len(plans) == chunks
    ptr, col = L.local_csr(g["indptr_dst"], g["indices_src"])
    xs = np.random.default_rng(rank).standard_normal((L.m, 4)).astype(np.float32)
    total = 0
    for q, p in enumerate(plans):
        a, b = L.chunk_rows(q)
        info = p.info
        assert (info["row_begin"], info["row_end"], info["num_nodes"]) == (a, b, L.m)
        got = eval_plan_numpy(p.export(), xs, L.m)
        want = np.stack([xs[col[ptr[r]:ptr[r + 1]]].astype(np.float64).sum(0) for r in range(a, b)])
        assert np.allclose(got, want, rtol=1e-6, atol=1e-6)
        total += info["gather_entries"]
    assert total == len(col)


def _grid_worker(rank, world, port, cols, chunks, q):
    import os
    import sys
    import torch.distributed as dist
    from conftest import ROOT
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = load_golden("c2_n640_ps2")
    n, dim = g["N"], 5
    x = np.random.default_rng(9).standard_normal((n, dim)).astype(np.float32)
    L = GridLayout(n, world, rank, cols, chunks)
    col_group, dst_group = GridPipeline.make_groups(L)
    r0, r1 = L.blocks[rank]
    # 1. all-gather inside the column group: slot order = position of the rank in the group
    own = torch.zeros((L.blk, dim))
    own[:r1 - r0] = torch.from_numpy(x[r0:r1])
    slots = [torch.zeros((L.blk, dim)) for _ in range(L.r)]
    dist.all_gather(slots, own, group=col_group)
    src = torch.cat(slots).numpy()
    # 2. this rank's partial rows
    ptr, col = L.local_csr(g["indptr_dst"], g["indices_src"])
    part = np.stack([src[col[ptr[r]:ptr[r + 1]]].astype(np.float64).sum(0) for r in range(L.dst_rows)])
    # 3. reduce-scatter inside the destination group (gloo has none: all-reduce, then this rank's rows)
    t = torch.from_numpy(part)
    dist.all_reduce(t, group=dst_group)
    mine = np.concatenate([t.numpy()[k * L.c * L.cb + L.j * L.cb:k * L.c * L.cb + (L.j + 1) * L.cb] for k in range(L.q)])
    gathered = [None] * world
    dist.all_gather_object(gathered, (r0, mine[:r1 - r0]))
    if rank == 0:
        q.put(gathered)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,cols,chunks", [(2, 2, 2), (4, 2, 3)])
def test_grid_pass_over_gloo(world, cols, chunks):
    """the communication pattern of the pass with gloo ranks on the CPU: process groups as
    make_groups builds them, slot order of the all-gather, row order of the reduce-scatter"""
    import os
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31000 + (os.getpid() + world * 7 + cols) % 2000
    procs = [ctx.Process(target=_grid_worker, args=(r, world, port, cols, chunks, q)) for r in range(world)]
    for p in procs:
        p.start()
    gathered = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    g = load_golden("c2_n640_ps2")
    x = np.random.default_rng(9).standard_normal((g["N"], 5)).astype(np.float32)
    got = np.concatenate([o for _, o in sorted(gathered, key=lambda t: t[0])])
    assert np.allclose(got, dense_sum(g, x.astype(np.float64)), rtol=1e-6, atol=1e-6)
