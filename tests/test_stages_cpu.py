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
