"""Seeded synthetic graph generators: determinism, CSR validity, config shapes."""
import numpy as np
import pytest

from artifact_b200 import graphs


def check_csr(g):
    n = g.num_nodes
    assert g.indptr_dst.shape == (n + 1,) and g.indptr_dst[0] == 0 and g.indptr_dst[-1] == g.num_edges
    assert (np.diff(g.indptr_dst) >= 0).all()
    assert g.indices_src.min() >= 0 and g.indices_src.max() < n
    for v in np.random.default_rng(0).integers(0, n, 200):
        r = g.indices_src[g.indptr_dst[v]:g.indptr_dst[v + 1]]
        assert (np.diff(r) > 0).all()                      # ascending, no duplicates
    # the transposed CSR describes the same edge set
    dst = np.repeat(np.arange(n), np.diff(g.indptr_dst))
    src2 = np.repeat(np.arange(n), np.diff(g.indptr_src))
    a = np.sort(dst.astype(np.int64) * n + g.indices_src)
    b = np.sort(g.indices_dst.astype(np.int64) * n + src2)
    assert np.array_equal(a, b)


def test_config1_exact_shape():
    g = graphs.config1()
    assert g.num_nodes == 2708 and g.num_edges == 2 * 5278 + 2708 and g.symmetric
    check_csr(g)
    assert (g.indices_src[g.indptr_dst[:-1]] <= np.arange(2708)).all()      # every row holds its self-loop


@pytest.mark.parametrize("cfg,scale", [("c2", 0.01), ("c3", 0.05), ("c4", 0.002), ("c5", 0.004)])
def test_configs_are_valid_and_deterministic(cfg, scale):
    a = graphs.CONFIGS[cfg](scale)
    b = graphs.CONFIGS[cfg](scale)
    check_csr(a)
    assert np.array_equal(a.indptr_dst, b.indptr_dst) and np.array_equal(a.indices_src, b.indices_src)


def test_config2_mean_degree_and_cap():
    g = graphs.config2(0.02)
    assert abs(g.num_edges / g.num_nodes - 492) < 25
    assert g.in_degree.max() <= g.num_nodes


def test_config5_structure():
    g = graphs.config5(1024 / 1048576)
    assert (g.in_degree == 32).all()
    rows = g.indices_src.reshape(g.num_nodes, 32)
    for c in range(0, g.num_nodes, 64):
        common = set(rows[c]).intersection(*[set(r) for r in rows[c + 1:c + 64]])
        assert len(common) >= 24                              # the per-cluster shared pool
