"""The product's reuse search must return, array for array, what upstream's reuse_search_ext
returns: against the committed fixtures (upstream's real output) everywhere, and against the
live upstream module on fresh random graphs where oracle/_ref/ holds it."""
import numpy as np
import pytest

import ref_search
from artifact_b200 import graphs, search

ARRAYS = ["part_pointers", "part2Node", "num_parts_per_node_acc", "intersection_num_per_part", "index_picked",
          "picked_fanout", "column_index", "part_pointers_cache", "column_index_cache", "part_cache_flagindex",
          "uniqpart_column_index", "uniqpart_pointers", "part2Node_ptr", "part2Node_col"]


def compare(mine, ref):
    for k in ARRAYS:
        assert np.array_equal(mine[k], np.asarray(ref[k]).astype(np.int32)), k


def test_search_equals_upstream_fixture(golden):
    mine = search.reuse_search(golden["indptr_dst"], golden["indices_src"], golden["indptr_src"],
                               golden["indices_dst"], golden["layouts"]["part_size"])
    compare(mine, golden["layouts"])


@pytest.mark.parametrize("budget", [0, 1 << 20])
def test_search_without_and_with_small_bitmap_budget(budget):
    from conftest import load_golden
    g = load_golden("c2_n640_ps2")
    mine = search.reuse_search(g["indptr_dst"], g["indices_src"], g["indptr_src"], g["indices_dst"], 2,
                               bitmap_budget_bytes=budget)
    compare(mine, g["layouts"])


CASES = [("c2", 1500 / 232965, 2), ("c2", 1500 / 232965, 3), ("c2", 900 / 232965, 5), ("c5", 4096 / 1048576, 2),
         ("c5", 4096 / 1048576, 3), ("c3", 0.05, 2), ("c4", 0.002, 2), ("c4", 0.002, 4), ("c1", 1.0, 4)]


@pytest.mark.parametrize("cfg,scale,ps", CASES)
def test_search_equals_live_upstream(cfg, scale, ps):
    mod = ref_search.load_module()
    if mod is None:
        pytest.skip("upstream preprocessor not built here (oracle/_ref)")
    g = graphs.CONFIGS[cfg](scale)
    ref = ref_search.run(g.indptr_dst, g.indices_src, g.indptr_src, g.indices_dst, ps, mod)
    for threads in (1, 0):
        mine = search.search_graph(g, ps, num_threads=threads)
        compare(mine, ref)


def test_thread_count_does_not_change_the_result():
    g = graphs.config5(8192 / 1048576)
    a = search.search_graph(g, 2, num_threads=1)
    b = search.search_graph(g, 2, num_threads=8)
    compare(a, b)


def test_bad_arguments():
    g = graphs.config5(128 / 1048576)
    with pytest.raises(ValueError):
        search.search_graph(g, 0)
    with pytest.raises(ValueError):
        search.reuse_search(g.indptr_dst, g.indices_src[::-1].copy(), g.indptr_src, g.indices_dst, 2)


def test_cached_search_round_trips(tmp_path):
    g = graphs.config5(2048 / 1048576)
    a, hit_a = search.cached_search_graph(g, 2, str(tmp_path))
    b, hit_b = search.cached_search_graph(g, 2, str(tmp_path))
    assert (hit_a, hit_b) == (False, True)
    compare(a, b)
    assert b["part_size"] == 2 and np.array_equal(b["original_column_index"], g.indices_src)
    g2 = graphs.config5(4096 / 1048576)                    # another graph: another cache entry
    _, hit_c = search.cached_search_graph(g2, 2, str(tmp_path))
    assert not hit_c and len(list(tmp_path.glob("reuse_*_ps2.npz"))) == 2


def _random_graph(rng, n, p):
    a = rng.random((n, n)) < p
    ip = np.zeros(n + 1, np.int64)
    idx = []
    for v in range(n):
        r = np.flatnonzero(a[v]).astype(np.int32)
        idx.append(r)
        ip[v + 1] = ip[v] + len(r)
    ix = np.concatenate(idx) if idx else np.zeros(0, np.int32)
    t_ip, t_ix = graphs.transpose_csr(n, ip, ix.astype(np.int32))
    return ip, ix.astype(np.int32), t_ip, t_ix


def test_fuzz_small_graphs_against_live_upstream():
    """many small random graphs (dense ones make long tie runs in the fan-out sort, sparse ones empty
    rows and zero groups), every part size: all 14 arrays equal upstream's"""
    mod = ref_search.load_module()
    if mod is None:
        pytest.skip("upstream preprocessor not built here (oracle/_ref)")
    rng = np.random.default_rng(2024)
    checked = groups = 0
    for trial in range(150):
        n = int(rng.integers(10, 70))
        p = float(rng.choice([0.03, 0.1, 0.3, 0.6, 0.9]))
        ps = int(rng.integers(1, 6))
        ip, ix, t_ip, t_ix = _random_graph(rng, n, p)
        if len(ix) == 0:
            continue
        ref = ref_search.run(ip, ix, t_ip, t_ix, ps, mod)
        mine = search.reuse_search(ip, ix, t_ip, t_ix, ps, num_threads=int(rng.integers(1, 4)))
        compare(mine, ref)
        checked += 1
        groups += len(ref["index_picked"])
    assert checked > 120 and groups > 200
