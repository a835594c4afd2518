"""Plan builder (host part of the CUDA library) on the fixtures: the destination-major plan
must expand back to exactly the original CSR, for all three layouts; bad layouts are
rejected with a status, not a crash.  Runs without a GPU (host-only plans)."""
import numpy as np
import pytest

from artifact_b200 import _native
from artifact_b200.plan import AggregationPlan
from conftest import layout_args

BUILDERS = {"parts": AggregationPlan.from_parts, "v1": AggregationPlan.from_v1, "v2": AggregationPlan.from_v2}


def expand_rows(ex, N):
    rows = []
    for r in range(len(ex["row_ptr"]) - 1):
        ent = ex["col"][ex["row_ptr"][r]:ex["row_ptr"][r + 1]]
        src = []
        for c in ent:
            if c < N:
                src.append(int(c))
            else:
                g = c - N
                src.extend(int(s) for s in ex["group_col"][ex["group_ptr"][g]:ex["group_ptr"][g + 1]])
        rows.append(sorted(src))
    return rows


@pytest.mark.parametrize("which", ["parts", "v1", "v2"])
def test_plan_round_trip(golden, which):
    N = golden["N"]
    plan = BUILDERS[which](N, *layout_args(golden["layouts"], which))
    ex = plan.export()
    rows = expand_rows(ex, N)
    ip, ix = golden["indptr_dst"], golden["indices_src"]
    for v in range(N):
        assert rows[v] == list(ix[ip[v]:ip[v + 1]]), (which, v)
    info = plan.info
    assert info["original_edges"] == len(ix)
    assert info["gather_entries"] == len(ex["col"])
    # the reuse accounting of upstream's scripts (small-main.py:176-188): every group saves
    # (fan-out - 1) * part_size gathered rows and costs fan-out partial rows
    if which != "parts":
        fan = golden["layouts"]["picked_fanout"].astype(np.int64)
        ps = golden["layouts"]["part_size"]
        assert info["num_groups"] == len(fan)
        assert info["partial_entries"] == fan.sum()
        assert info["gather_entries"] == len(ix) - ps * fan.sum() + fan.sum()
        assert info["group_sources"] == ps * len(fan)


@pytest.mark.parametrize("which", ["parts", "v2"])
def test_items_cover_every_entry_once(golden, which):
    N = golden["N"]
    plan = BUILDERS[which](N, *layout_args(golden["layouts"], which))
    ex = plan.export()
    covered = np.zeros(len(ex["col"]), np.int32)
    seen_rows = set()
    lens = []
    for b, e, dst, mid in ex["items"]:
        covered[b:e] += 1
        assert b <= mid <= e and (ex["col"][b:mid] >= N).all() and (ex["col"][mid:e] < N).all()
        lens.append(e - b)
        assert e - b <= plan.info["segment_edges"]
        if dst >= 0:
            assert dst not in seen_rows
            seen_rows.add(int(dst))
            assert (b, e) == (ex["row_ptr"][dst], ex["row_ptr"][dst + 1])
    assert (covered == 1).all()
    assert lens == sorted(lens, reverse=True)            # longest first
    split = {int(r) for r, _, _, _ in ex["split_rows"]}
    assert seen_rows | split == set(range(N)) and not (seen_rows & split)
    for row, first, count, _ in ex["split_rows"]:
        segs = sorted((b, e) for b, e, dst, _ in ex["items"] if dst < 0 and first <= -dst - 1 < first + count)
        assert segs[0][0] == ex["row_ptr"][row] and segs[-1][1] == ex["row_ptr"][row + 1]
        assert all(a[1] == b[0] for a, b in zip(segs, segs[1:]))


def test_row_block_plans_tile_the_graph(golden):
    N = golden["N"]
    L = golden["layouts"]
    full = AggregationPlan.from_v2(N, *layout_args(L, "v2")).export()
    full_rows = expand_rows(full, N)
    cuts = [0, N // 3, N // 3, (2 * N) // 3, N]
    got = []
    for r0, r1 in zip(cuts[:-1], cuts[1:]):
        p = AggregationPlan.from_v2(N, *layout_args(L, "v2"), rows=(r0, r1))
        assert (p.info["row_begin"], p.info["row_end"]) == (r0, r1)
        got += expand_rows(p.export(), N)
    assert got == full_rows


def test_empty_graph_and_no_groups():
    z = np.zeros(0, np.int32)
    p = AggregationPlan.from_parts(0, z, z, z)
    assert p.info["num_items"] == 0
    p = AggregationPlan.from_v1(5, np.array([1, 2], np.int32), np.array([0, 2], np.int32), np.array([3], np.int32),
                                np.array([0], np.int32), np.array([0], np.int32), z)
    assert p.info["num_groups"] == 0 and p.info["num_items"] == 5
    assert p.workspace_bytes(64) == 0


@pytest.mark.parametrize("case", ["col_range", "ptr_order", "dst_range", "flag_range", "ptr_overrun"])
def test_bad_layouts_are_rejected(case):
    col = np.array([0, 1, 2, 3], np.int32)
    pp = np.array([0, 2, 4], np.int32)
    p2n = np.array([1, 2], np.int32)
    flag = np.array([0, 0], np.int32)
    ppc = np.array([0, 2], np.int32)
    cic = np.array([0, 1], np.int32)
    if case == "col_range":
        col = np.array([0, 1, 9, 3], np.int32)
    elif case == "ptr_order":
        pp = np.array([0, 3, 2], np.int32)
    elif case == "dst_range":
        p2n = np.array([1, -1], np.int32)
    elif case == "flag_range":
        flag = np.array([0, 2], np.int32)
    elif case == "ptr_overrun":
        pp = np.array([0, 2, 5], np.int32)
    with pytest.raises(_native.RofError) as e:
        AggregationPlan.from_v1(4, col, pp, p2n, flag, ppc, cic)
    assert e.value.status == 2 and "bad layout" in str(e.value)


def test_bad_arguments():
    z = np.zeros(0, np.int32)
    with pytest.raises(_native.RofError) as e:
        AggregationPlan.from_parts(4, z, z, z, rows=(3, 2))
    assert e.value.status == 1
    with pytest.raises(TypeError):
        AggregationPlan.from_parts(4, np.zeros(2, np.float32), z, z)


def test_auto_tiles_heuristic():
    """source tiling only when the feature matrix exceeds L2 and rows stay long per tile"""
    from conftest import load_golden
    g = load_golden("c2_n640_ps2")                      # 640 nodes, mean degree ~160
    plan = AggregationPlan.from_parts(g["N"], *layout_args(g["layouts"], "parts"))
    assert plan.auto_tiles(256) == 1                    # 640 x 256 x 4 B is far below L2
    # the same row length on a matrix of 10^6 rows x 256: tiles until ~64 MB blocks, at most 8,
    # but never fewer than 48 entries per row and tile
    plan.info = dict(plan.info, num_nodes=1_000_000, row_begin=0, row_end=1000, gather_entries=1000 * 160)
    assert plan.auto_tiles(256) == 2
    plan.info = dict(plan.info, gather_entries=1000 * 2000)
    assert plan.auto_tiles(256) == 8
    plan.info = dict(plan.info, gather_entries=1000 * 40)
    assert plan.auto_tiles(256) == 1
    assert plan.auto_tiles(16) == 1


def test_segment_length_follows_plan_size():
    z = np.zeros(0, np.int32)
    n = 300
    big = np.arange(n, dtype=np.int32)
    col = np.concatenate([big] * 3)                     # three rows of 300 entries
    plan = AggregationPlan.from_parts(n, col, np.array([0, 300, 600, 900], np.int32), np.array([0, 1, 2], np.int32))
    assert plan.info["segment_edges"] == 256            # small plan: shortest segments
    assert plan.info["split_rows"] == 3 and plan.info["num_slots"] == 6


def test_fuzz_plans_and_oracle_on_random_graphs():
    """random small graphs through the product's search, then: every layout's plan expands back to the
    CSR, staged plans partition it, and the oracle gives the same sums over all three layouts"""
    import rof_oracle
    from artifact_b200 import graphs, search
    rng = np.random.default_rng(77)
    for trial in range(40):
        n = int(rng.integers(5, 80))
        p = float(rng.choice([0.05, 0.2, 0.5, 0.85]))
        ps = int(rng.integers(2, 6))
        a = rng.random((n, n)) < p
        rows = [np.flatnonzero(a[v]).astype(np.int32) for v in range(n)]
        ip = np.concatenate([[0], np.cumsum([len(r) for r in rows])]).astype(np.int64)
        ix = np.concatenate(rows).astype(np.int32) if ip[-1] else np.zeros(0, np.int32)
        t_ip, t_ix = graphs.transpose_csr(n, ip, ix)
        L = search.reuse_search(ip, ix, t_ip, t_ix, ps)
        want = [list(r) for r in rows]
        for which in ("parts", "v1", "v2"):
            plan = BUILDERS[which](n, *layout_args(L, which))
            assert expand_rows(plan.export(), n) == want, (trial, which)
        whole = AggregationPlan.from_v2(n, *layout_args(L, "v2"))
        tiles = int(rng.integers(2, 5))
        blk = (n + tiles - 1) // tiles
        got = [[] for _ in range(n)]
        for sp in whole.stages(blk, list(range(tiles))):
            for v, r in enumerate(expand_rows(sp.export(), n)):
                got[v] += r
        assert [sorted(r) for r in got] == want
        x = rng.standard_normal((n, 3)).astype(np.float32)
        deg = np.maximum(np.diff(ip), 1).astype(np.float32)
        base = rof_oracle.aggregate_parts(x, L["original_column_index"], deg, L["part_pointers"], L["part2Node"], "gcn", True)
        cache = np.zeros((len(L["part_pointers_cache"]) - 1, 4), np.float32)
        v1 = rof_oracle.aggregate_v1(x, L["column_index"], deg, L["part_pointers"], L["part2Node"], cache,
                                     L["part_cache_flagindex"], L["part_pointers_cache"], L["column_index_cache"], "gcn", True)
        v2 = rof_oracle.aggregate_v2(x, L["uniqpart_column_index"], deg, L["uniqpart_pointers"], L["part2Node_ptr"],
                                     L["part2Node_col"], "gcn", True)
        assert np.allclose(v1, base, rtol=1e-6, atol=1e-6) and np.allclose(v2, base, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("which", ["parts", "v2"])
def test_tiles_hold_the_same_rows(golden, which, monkeypatch):
    """shared-memory tiles (forced on): every tiled row must expand to exactly the entries of the
    plan's row — staged slots through the tile's stage list plus the rows read from global
    memory — every staged id must occur at least twice in its tile, and rows and tiles must be
    covered once"""
    monkeypatch.setenv("ROF_TILES", "1")
    N = golden["N"]
    plan = BUILDERS[which](N, *layout_args(golden["layouts"], which))
    ex, tl = plan.export(), plan.export_tiles()
    info = plan.info
    assert info["num_tiles"] == len(tl["tiles"]) > 0
    lens = np.diff(ex["row_ptr"])
    short = np.flatnonzero(lens <= 256)
    assert info["tile_items"] == len(short)
    seen, shared = [], 0
    for t, (first, count, sb, sc) in enumerate(tl["tiles"]):
        assert 0 < count <= 32 and 0 <= sc <= 64 and sb == t * 64
        stage = tl["stage_col"][sb:sb + sc]
        assert len(set(stage.tolist())) == sc
        occurrences = {}
        for b, e, dst, mid in tl["titems"][first:first + count]:
            seen.append(dst)
            slots, glob = tl["tcol"][b:mid], tl["tcol"][mid:e]
            assert (slots >= 0).all() and (slots < sc).all()
            assert not set(glob.tolist()) & set(stage.tolist()), "a staged id is also read from global memory"
            got = sorted(stage[slots].tolist() + glob.tolist())
            want = sorted(ex["col"][ex["row_ptr"][dst]:ex["row_ptr"][dst + 1]].tolist())
            assert got == want, (which, dst)
            shared += len(slots)
            for c in stage[slots]:
                occurrences[int(c)] = occurrences.get(int(c), 0) + 1
        assert all(v >= 2 for v in occurrences.values()) and len(occurrences) == sc
    assert sorted(seen) == short.tolist()
    assert info["tile_shared_entries"] == shared and info["tile_entries"] == int(lens[short].sum())


def test_tiles_are_built_only_where_rows_share_entries(monkeypatch):
    """unset ROF_TILES: the community fixture (neighbouring rows share a pool of sources) gets tiles,
    the power-law fixture does not; ROF_TILES=0 never builds them"""
    from conftest import load_golden
    monkeypatch.delenv("ROF_TILES", raising=False)
    c5, c2 = load_golden("c5_n1024_ps2"), load_golden("c2_n640_ps2")
    assert AggregationPlan.from_v2(c5["N"], *layout_args(c5["layouts"], "v2")).info["num_tiles"] > 0
    assert AggregationPlan.from_parts(c5["N"], *layout_args(c5["layouts"], "parts")).info["num_tiles"] > 0
    assert AggregationPlan.from_v2(c2["N"], *layout_args(c2["layouts"], "v2")).info["num_tiles"] == 0
    monkeypatch.setenv("ROF_TILES", "0")
    assert AggregationPlan.from_v2(c5["N"], *layout_args(c5["layouts"], "v2")).info["num_tiles"] == 0


def test_reuse_groups_are_used_only_where_they_pay(monkeypatch):
    """the library's own rule (ROF_REUSE_MIN unset): the community fixture saves about a third of its
    gathered rows and keeps its groups; the power-law fixture saves a few per cent and is run without
    partial rows — same rows either way"""
    from conftest import load_golden
    monkeypatch.delenv("ROF_REUSE_MIN", raising=False)
    c5, c2 = load_golden("c5_n1024_ps2"), load_golden("c2_n640_ps2")
    p5 = AggregationPlan.from_v2(c5["N"], *layout_args(c5["layouts"], "v2"))
    p2 = AggregationPlan.from_v2(c2["N"], *layout_args(c2["layouts"], "v2"))
    assert p5.info["num_groups"] > 0 and p5.info["gather_entries"] < 0.8 * p5.info["original_edges"]
    assert p2.info["num_groups"] == 0 and p2.info["gather_entries"] == p2.info["original_edges"]
    for g, p in ((c5, p5), (c2, p2)):
        rows = expand_rows(p.export(), g["N"])
        ip, ix = g["indptr_dst"], g["indices_src"]
        assert all(rows[v] == list(ix[ip[v]:ip[v + 1]]) for v in range(g["N"]))
    # kept groups all have a positive benefit: fan-out x (size - 1) > size + 1
    ex = p5.export()
    fan = np.bincount(ex["col"][ex["col"] >= c5["N"]] - c5["N"], minlength=p5.info["num_groups"])
    size = np.diff(ex["group_ptr"])
    assert (fan * (size - 1) > size + 1).all()
