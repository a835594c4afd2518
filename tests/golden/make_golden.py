"""Generates the fixtures in this directory.  Run in a container where the upstream tree is
mounted and `make -C oracle ref_search` has been run:

    python tests/golden/make_golden.py

Each `<name>.npz` holds a small seeded graph (both CSRs), every index array upstream's own
preprocessor (compiled unmodified from its sources) returns for it, and the dense fp64 result
of D^-1/2 A D^-1/2 X, A X and D^-1 A X for a seeded X — so the GPU box, which has neither the
upstream tree nor a need to trust our own search, can pin the plan builder, the search
re-implementation and the oracle against upstream's real output.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import ref_search  # noqa: E402
from artifact_b200 import graphs  # noqa: E402


def shared_prefix_graph():
    """12 nodes; nodes 4..7 all have in-neighbours {0,1,2} (a reuse group for part_size 3),
    8..11 share {3,4}; node 11 has no in-edge at all (an empty row)."""
    rows = {0: [1, 5], 1: [0, 2, 9], 2: [1], 3: [0, 1, 2, 8, 10], 4: [0, 1, 2, 3], 5: [0, 1, 2], 6: [0, 1, 2, 7],
            7: [0, 1, 2, 4, 5, 6, 9], 8: [3, 4, 6], 9: [3, 4], 10: [3, 4, 5, 6, 7, 8, 9], 11: []}
    n = 12
    indptr = np.zeros(n + 1, np.int64)
    idx = []
    for v in range(n):
        idx += sorted(rows[v])
        indptr[v + 1] = len(idx)
    indices = np.array(idx, np.int32)
    t_indptr, t_indices = graphs.transpose_csr(n, indptr, indices)
    return graphs.Graph("shared_prefix_12", n, indptr, indices, t_indptr, t_indices, False, 0)


def dense_expected(g, x, mode):
    n = g.num_nodes
    A = np.zeros((n, n))
    A[np.repeat(np.arange(n), np.diff(g.indptr_dst)), g.indices_src] = 1.0
    deg = np.diff(g.indptr_dst).astype(np.float64)
    with np.errstate(divide="ignore", invalid="ignore"):
        if mode == "gcn":
            s = 1.0 / np.sqrt(deg)
            return ((s[:, None] * A * s[None, :]) @ x.astype(np.float64))
        if mode == "mean":
            inv = np.where(deg > 0, 1.0 / np.maximum(deg, 1), 0.0)
            return inv[:, None] * (A @ x.astype(np.float64))
    return A @ x.astype(np.float64)


CASES = [
    ("shared_prefix_12_ps3", shared_prefix_graph, 3, True),
    ("shared_prefix_12_ps2", shared_prefix_graph, 2, True),
    ("c1_full_ps3", lambda: graphs.config1(), 3, False),
    ("c1_full_ps2", lambda: graphs.config1(), 2, False),
    ("c5_n1024_ps2", lambda: graphs.config5(1024 / 1048576), 2, True),
    ("c5_n1024_ps4", lambda: graphs.config5(1024 / 1048576), 4, True),
    ("c2_n640_ps2", lambda: graphs.config2(640 / 232965), 2, False),
    ("c3_n1500_ps3", lambda: graphs.config3(1500 / 169343), 3, True),
]


def main():
    mod = ref_search.load_module()
    assert mod is not None, "build oracle/_ref first: make -C oracle ref_search"
    for name, make, ps, with_dense in CASES:
        g = make()
        L = ref_search.run(g.indptr_dst, g.indices_src, g.indptr_src, g.indices_dst, ps, mod)
        out = {"num_nodes": np.int64(g.num_nodes), "symmetric": np.int64(g.symmetric),
               "indptr_dst": g.indptr_dst.astype(np.int32), "indices_src": g.indices_src,
               "indptr_src": g.indptr_src.astype(np.int32), "indices_dst": g.indices_dst}
        for k, v in L.items():
            out["ref_" + k] = np.asarray(v)
        if with_dense:
            x = np.random.default_rng(7).standard_normal((g.num_nodes, 8)).astype(np.float32)
            out["x"] = x
            for mode in ("gcn", "sum", "mean"):
                out["dense_" + mode] = dense_expected(g, x, mode)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **out)
        print(f"{name}: N={g.num_nodes} E={g.num_edges} groups={len(L['index_picked'])} "
              f"fanout_sum={int(L['picked_fanout'].sum())} -> {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
