"""The multi-GPU host logic with two gloo ranks on CPU: equal row blocks, per-block plans built
from the same index tensors, and the all-gather of feature blocks.  The kernels cannot run
here, so each rank evaluates its exported plan with numpy; the concatenated blocks must equal
the oracle on the whole graph."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, layout_args, load_golden


def eval_plan_numpy(ex, x, n):
    """out[r] = sum over the row's entries; entries >= n are partial rows of the exported groups"""
    part = np.stack([x[ex["group_col"][ex["group_ptr"][g]:ex["group_ptr"][g + 1]]].astype(np.float64).sum(0)
                     for g in range(len(ex["group_ptr"]) - 1)]) if len(ex["group_ptr"]) > 1 else np.zeros((0, x.shape[1]))
    out = np.zeros((len(ex["row_ptr"]) - 1, x.shape[1]))
    for r in range(out.shape[0]):
        for c in ex["col"][ex["row_ptr"][r]:ex["row_ptr"][r + 1]]:
            out[r] += x[c] if c < n else part[c - n]
    return out


def _worker(rank, world, port, name, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from artifact_b200.plan import AggregationPlan
    from artifact_b200.sharding import ShardedFeatures
    g = load_golden(name)
    n, dim = g["N"], 6
    x = np.random.default_rng(4).standard_normal((n, dim)).astype(np.float32)
    feats = ShardedFeatures(n, dim, rank, world, torch.device("cpu"))
    r0, r1 = feats.blocks[rank]
    local = torch.zeros((feats.block, dim))
    local[:r1 - r0] = torch.from_numpy(x[r0:r1])
    x_full = feats.all_gather(local).numpy()
    assert np.array_equal(x_full, x)                                  # every rank now holds all rows
    plan = AggregationPlan.from_v2(n, *layout_args(g["layouts"], "v2"), rows=(r0, r1))
    out = eval_plan_numpy(plan.export(), x_full, n)
    gathered = [None] * world
    dist.all_gather_object(gathered, (r0, r1, out))
    if rank == 0:
        q.put(np.concatenate([o for _, _, o in sorted(gathered, key=lambda t: t[0])]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("name", ["c5_n1024_ps2", "shared_prefix_12_ps3"])
@pytest.mark.parametrize("world", [2, 3])
def test_two_rank_row_blocks_equal_whole_graph(name, world):
    import rof_oracle
    g = load_golden(name)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + world * 7 + len(name)) % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, name, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    x = np.random.default_rng(4).standard_normal((g["N"], 6)).astype(np.float32)
    L = g["layouts"]
    want = rof_oracle.aggregate_v2(x, L["uniqpart_column_index"], g["degrees"], L["uniqpart_pointers"],
                                   L["part2Node_ptr"], L["part2Node_col"], "sum", exact64=True)
    assert np.allclose(got, want, rtol=1e-6, atol=1e-6)


def test_row_blocks_cover_and_pad():
    from artifact_b200.sharding import row_blocks
    for n in (0, 1, 7, 8, 1000):
        for w in (1, 2, 3, 8):
            blk, blocks = row_blocks(n, w)
            assert blk * w >= n and len(blocks) == w
            assert blocks[0][0] == 0 and blocks[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(blocks, blocks[1:]))
            assert all(0 <= r1 - r0 <= blk for r0, r1 in blocks)


def test_row_blocks_balanced_by_edges_on_an_unpermuted_power_law_graph():
    """hubs first (in-degree falls with the node id): equal row counts would give rank 0 most of the
    edges; blocks cut by in-degree + row cost must be within 15 % of each other"""
    from artifact_b200.sharding import row_blocks
    n = 20000
    deg = np.maximum(1, (20000.0 * (np.arange(n) + 1.0) ** -0.7)).astype(np.int64)
    indptr = np.concatenate([[0], np.cumsum(deg)])
    for w in (2, 4, 8):
        _, eq = row_blocks(n, w)
        blk, bal = row_blocks(n, w, indptr=indptr)
        assert blk is None and bal[0][0] == 0 and bal[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(bal, bal[1:]))
        work = lambda blocks: np.array([indptr[b] - indptr[a] + 8 * (b - a) for a, b in blocks], dtype=np.float64)
        assert work(eq).max() / work(eq).mean() > 1.4              # the problem being solved
        assert work(bal).max() / work(bal).mean() < 1.15
    # one rank: everything
    assert row_blocks(n, 1, indptr=indptr)[1] == [(0, n)]


def _unequal_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from artifact_b200.sharding import ShardedFeatures
    n, dim = 50, 3
    bounds = [(0, 5), (5, 33), (33, 50)]
    x = torch.arange(n * dim, dtype=torch.float32).reshape(n, dim)
    feats = ShardedFeatures(n, dim, rank, world, torch.device("cpu"), bounds=bounds)
    r0, r1 = bounds[rank]
    assert tuple(feats.local_view().shape) == (r1 - r0, dim) and feats.full.shape[0] == n
    full = feats.all_gather(x[r0:r1].clone())
    q.put((rank, bool(torch.equal(full, x))))
    dist.barrier()
    dist.destroy_process_group()


def test_unequal_blocks_all_gather():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() * 5 + 91) % 2000
    procs = [ctx.Process(target=_unequal_worker, args=(r, 3, port, q)) for r in range(3)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in range(3))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == [(0, True), (1, True), (2, True)]


def test_stage_schedule_covers_every_peer_once():
    from artifact_b200.sharding import stage_schedule
    for w in (1, 2, 3, 4, 5, 8, 16):
        sch = stage_schedule(w)
        assert sch[0] == [0]
        flat = [k for s in sch for k in s]
        assert flat == list(range(w))
        assert len(sch) <= 3
    assert stage_schedule(8) == [[0], [1, 2, 3], [4, 5, 6, 7]] and stage_schedule(2) == [[0], [1]]
    assert stage_schedule(4) == [[0], [1], [2, 3]]


def _lonely_worker(rank, world, port, q):
    import datetime
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from artifact_b200.sharding import ShardedFeatures
    feats = ShardedFeatures(64, 4, rank, world, torch.device("cpu"))
    feats.all_gather(torch.ones((feats.block, 4)))          # a pass with every rank present works
    dist.barrier()
    if rank == 1:
        os._exit(0)                                         # rank 1 leaves between passes, nothing in flight
    try:
        feats.all_gather(torch.ones((feats.block, 4)))
        q.put("no error")
    except Exception as e:                                  # the survivor gets an error, not a hang
        q.put(type(e).__name__)


def test_a_rank_that_left_is_an_error_not_a_hang():
    """failure detection is the process group's: a pass after a peer has gone ends with an
    exception within the group's timeout (the device code itself never waits on a peer)"""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() * 3 + 17) % 2000
    procs = [ctx.Process(target=_lonely_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
    assert got != "no error", got
