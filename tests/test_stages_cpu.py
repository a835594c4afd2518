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
