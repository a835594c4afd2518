"""Staged plans (multi-GPU pipeline) on the host: the stages partition the whole plan's entries by
the arrival stage of their source block, groups land in the stage of their last source, and the
stage-by-stage sum equals the whole-plan sum."""
import numpy as np
import pytest

from artifact_b200.plan import AggregationPlan
from artifact_b200.sharding import row_blocks
from conftest import layout_args, load_golden
from test_sharding_cpu import eval_plan_numpy


@pytest.mark.parametrize("name", ["c5_n1024_ps2", "c2_n640_ps2", "shared_prefix_12_ps3"])
@pytest.mark.parametrize("world,rank", [(2, 0), (2, 1), (4, 2), (8, 5)])
def test_stages_partition_and_sum(name, world, rank):
    g = load_golden(name)
    n = g["N"]
    blk, blocks = row_blocks(n, world)
    r0, r1 = blocks[rank]
    whole = AggregationPlan.from_v2(n, *layout_args(g["layouts"], "v2"), rows=(r0, r1))
    sob = [(b - rank) % world for b in range(world)]
    stages = whole.stages(blk, sob)
    assert len(stages) == world
    x = np.random.default_rng(8).standard_normal((n, 5)).astype(np.float32)
    want = eval_plan_numpy(whole.export(), x, n)
    got = np.zeros_like(want)
    edges = 0
    for k, sp in enumerate(stages):
        ex = sp.export()
        assert (sp.info["row_begin"], sp.info["row_end"]) == (r0, r1)
        src = ex["col"][ex["col"] < n]
        assert all(sob[c // blk] == k for c in src)                       # only blocks that have arrived
        for gi in range(len(ex["group_ptr"]) - 1):
            gs = ex["group_col"][ex["group_ptr"][gi]:ex["group_ptr"][gi + 1]]
            assert max(sob[c // blk] for c in gs) == k                     # built when its last source lands
        got += eval_plan_numpy(ex, x, n)
        edges += sp.info["original_edges"]
    assert edges == whole.info["original_edges"]
    assert sum(s.info["num_groups"] for s in stages) == whole.info["num_groups"]
    assert np.allclose(got, want, rtol=1e-9, atol=1e-9)


def test_stage_arguments_are_checked():
    from artifact_b200 import _native
    g = load_golden("shared_prefix_12_ps3")
    whole = AggregationPlan.from_v2(12, *layout_args(g["layouts"], "v2"))
    with pytest.raises(_native.RofError):
        whole.stages(2, [0, 1])            # 2 blocks of 2 rows do not cover 12 nodes
    with pytest.raises(_native.RofError):
        whole.stages(0, [0])


@pytest.mark.parametrize("name", ["c5_n1024_ps2", "c2_n640_ps2"])
@pytest.mark.parametrize("world,rank", [(2, 1), (4, 0), (8, 3)])
def test_compute_stages_tile_the_transfer_stages(name, world, rank):
    """unequal row blocks (balanced by edges), every transfer stage cut into L2-sized compute
    stages: the ranges cover every row once, a compute stage only names rows of its transfer
    stage, and the stage-by-stage sum equals the whole plan"""
    from artifact_b200.sharding import compute_stages, stage_schedule
    g = load_golden(name)
    n = g["N"]
    _, blocks = row_blocks(n, world, indptr=g["indptr_dst"])
    assert blocks[0][0] == 0 and blocks[-1][1] == n
    r0, r1 = blocks[rank]
    whole = AggregationPlan.from_v2(n, *layout_args(g["layouts"], "v2"), rows=(r0, r1))
    sched = stage_schedule(world)
    dim = 5
    # a tiny "L2" so that stages really are cut, and no minimum of entries per tile
    ranges = [[blocks[(rank + k) % world] for k in offs] for offs in sched]
    bounds, stage_of, transfer_of = compute_stages(ranges, n, dim, 1e9, tile_bytes=n * dim * 4 / 5,
                                                   min_entries_per_tile=0)
    assert bounds[0] == 0 and bounds[-1] == n and all(a < b for a, b in zip(bounds, bounds[1:]))
    assert len(transfer_of) == max(stage_of) + 1 > len(sched)
    assert transfer_of == sorted(transfer_of)
    owner = np.zeros(n, np.int64)
    for b, (a, e) in enumerate(blocks):
        owner[a:e] = b
    stage_of_offset = {k: s for s, ks in enumerate(sched) for k in ks}
    for (a, e), k in zip(zip(bounds, bounds[1:]), stage_of):
        assert {stage_of_offset[(int(o) - rank) % world] for o in np.unique(owner[a:e])} == {transfer_of[k]}
    stages = whole.stages_by_ranges(bounds, stage_of)
    x = np.random.default_rng(3).standard_normal((n, dim)).astype(np.float32)
    want = eval_plan_numpy(whole.export(), x, n)
    got = np.zeros_like(want)
    row_stage = np.zeros(n, np.int64)
    for (a, e), k in zip(zip(bounds, bounds[1:]), stage_of):
        row_stage[a:e] = k
    for k, sp in enumerate(stages):
        ex = sp.export()
        src = ex["col"][ex["col"] < n]
        assert (row_stage[src] == k).all()
        got += eval_plan_numpy(ex, x, n)
    assert np.allclose(got, want, rtol=1e-9, atol=1e-9)
    # default tile size and the real minimum: these small graphs need no cut
    b2, s2, t2 = compute_stages(ranges, n, dim, whole.info["gather_entries"] / max(r1 - r0, 1))
    assert t2 == list(range(len(sched)))


def test_transfer_pieces_follow_the_bytes():
    from artifact_b200.sharding import piece_rows, transfer_pieces
    assert transfer_pieces(1, 1e12) == 1
    assert transfer_pieces(2, 119e6) == 1 and transfer_pieces(8, 208e6) == 1      # small transfers stay whole
    assert transfer_pieces(2, 1.25e9) == 4 and transfer_pieces(8, 2.19e9) == 4     # large ones are cut (capped)
    for lo, hi in ((0, 10), (7, 7), (100, 1003)):
        for pcs in (1, 3, 4):
            cuts = [piece_rows(lo, hi, p, pcs) for p in range(pcs)]
            assert cuts[0][0] == lo and cuts[-1][1] == hi
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))


def test_stage_ranges_are_checked():
    from artifact_b200 import _native
    g = load_golden("shared_prefix_12_ps3")
    whole = AggregationPlan.from_v2(12, *layout_args(g["layouts"], "v2"))
    with pytest.raises(_native.RofError):
        whole.stages_by_ranges([0, 6, 11], [0, 1])      # does not reach num_nodes
    with pytest.raises(_native.RofError):
        whole.stages_by_ranges([0, 8, 6, 12], [0, 1, 0])  # not ascending
    with pytest.raises(ValueError):
        whole.stages_by_ranges([0, 12], [0, 1])


@pytest.mark.parametrize("name", ["c5_n1024_ps2", "c2_n640_ps2"])
@pytest.mark.parametrize("world,rank,pieces", [(2, 1, 2), (4, 0, 3), (8, 5, 4)])
def test_piece_major_layout_and_its_plans(name, world, rank, pieces):
    """piece-major feature layout (one all-gather per piece): the map from node ids to buffer rows is
    one-to-one, each rank's piece is contiguous where the collective puts it, and the rank's plan over
    the permuted matrix — whole, and split by piece — gives the same sums as the plan over the
    row-major matrix"""
    import torch
    from artifact_b200.sharding import PieceMajorFeatures, PieceMajorPipeline
    g = load_golden(name)
    n, L = g["N"], g["layouts"]
    f = PieceMajorFeatures(n, 5, rank, world, torch.device("cpu"), pieces)
    q = f.perm(np.arange(n))
    assert len(np.unique(q)) == n and q.max() < f.size
    for b, (a, e) in enumerate(f.blocks):
        for p in range(pieces):
            lo, hi = a + p * f.pb, min(a + (p + 1) * f.pb, e)
            if hi > lo:
                assert (q[lo:hi] == p * world * f.pb + b * f.pb + np.arange(hi - lo)).all()
    r0, r1 = f.blocks[rank]
    plain = AggregationPlan.from_v2(n, *layout_args(L, "v2"), rows=(r0, r1))
    perm_plan = PieceMajorPipeline.plan_from_v2(f, *layout_args(L, "v2"))
    assert perm_plan.info["num_nodes"] == f.size and perm_plan.info["original_edges"] == plain.info["original_edges"]
    x = np.random.default_rng(1).standard_normal((n, 5)).astype(np.float32)
    xp = np.zeros((f.size, 5), np.float32)
    xp[q] = x
    want = eval_plan_numpy(plain.export(), x, n)
    assert np.allclose(eval_plan_numpy(perm_plan.export(), xp, f.size), want, rtol=1e-9, atol=1e-9)
    got = np.zeros_like(want)
    stages = perm_plan.stages(world * f.pb, list(range(pieces)))
    for p, sp in enumerate(stages):
        ex = sp.export()
        src = ex["col"][ex["col"] < f.size]
        assert ((src // (world * f.pb)) == p).all()          # stage p reads piece p only
        got += eval_plan_numpy(ex, xp, f.size)
    assert np.allclose(got, want, rtol=1e-9, atol=1e-9)
    # own rows first: stage 0 reads only the rank's own slots, stage p + 1 the rest of piece p
    bounds, stage_of = PieceMajorPipeline.own_first_ranges(pieces, world, f.pb, rank)
    own_rows = set(f.perm(np.arange(r0, r1)).tolist())
    got = np.zeros_like(want)
    own_stages = perm_plan.stages_by_ranges(bounds, stage_of)
    assert len(own_stages) == pieces + 1
    for s, sp in enumerate(own_stages):
        ex = sp.export()
        src = ex["col"][ex["col"] < f.size]
        if s == 0:
            assert set(src.tolist()) <= own_rows
        else:
            assert ((src // (world * f.pb)) == s - 1).all() and not (set(src.tolist()) & own_rows)
        got += eval_plan_numpy(ex, xp, f.size)
    assert np.allclose(got, want, rtol=1e-9, atol=1e-9)
