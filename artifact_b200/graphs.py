"""Seeded synthetic graphs with the shapes of the five benchmark configurations.

Every graph is returned as a destination-major CSR (``indptr_dst``, ``indices_src``: row v
lists the in-neighbours of v, ascending, no duplicates) plus the transposed CSR
(``indptr_src``, ``indices_dst``) — the four arrays the reuse preprocessor takes
(ROF_evaluation/ROF_main.py:59-64, ROF_evaluation/cuda/middle-main.py:184-198).

The configurations name public-dataset *shapes* only; nothing of any dataset is
reproduced here.  ``scale`` shrinks node and edge counts proportionally for tests.
"""
import ctypes
from dataclasses import dataclass

import numpy as np

from . import _native


@dataclass
class Graph:
    name: str
    num_nodes: int
    indptr_dst: np.ndarray   # int64 [n+1]
    indices_src: np.ndarray  # int32 [e]
    indptr_src: np.ndarray   # int64 [n+1]
    indices_dst: np.ndarray  # int32 [e]
    symmetric: bool
    seed: int

    @property
    def num_edges(self):
        return int(self.indices_src.shape[0])

    @property
    def in_degree(self):
        return np.diff(self.indptr_dst)

    def degrees_f32(self):
        """`degrees` as upstream builds it: float32(np.diff(indptr_dst)) (ROF_main.py:138,144)."""
        return self.in_degree.astype(np.float32)


def _fetch(handle, n):
    lib = _native.host()
    e = lib.rofh_graph_num_edges(handle)
    indptr = np.empty(n + 1, dtype=np.int64)
    indices = np.empty(e, dtype=np.int32)
    lib.rofh_graph_fetch(handle, indptr.ctypes.data_as(ctypes.c_void_p),
                         indices.ctypes.data_as(ctypes.c_void_p))
    lib.rofh_graph_free(handle)
    return indptr, indices


def transpose_csr(n, indptr, indices):
    lib = _native.host()
    t_indptr = np.empty(n + 1, dtype=np.int64)
    t_indices = np.empty(indices.shape[0], dtype=np.int32)
    lib.rofh_transpose_csr(n, indptr.ctypes.data_as(ctypes.c_void_p),
                           indices.ctypes.data_as(ctypes.c_void_p),
                           t_indptr.ctypes.data_as(ctypes.c_void_p),
                           t_indices.ctypes.data_as(ctypes.c_void_p))
    return t_indptr, t_indices


def power_law_weights(n, exponent, target_edges, cap=None):
    """Expected-degree sequence w_i = min(cap, c * (i+1)^(-1/(exponent-1))), descending, with
    c chosen so that the expected number of directed pairs sum_uv min(1, w_u w_v / sum(w))
    equals ``target_edges``."""
    shape = (np.arange(n, dtype=np.float64) + 1.0) ** (-1.0 / (exponent - 1.0))

    def expected(c):
        w = shape * c
        if cap is not None:
            w = np.minimum(w, cap)
        S = w.sum()
        # for destination weight b: sources with a >= S/b are certain
        asc = w[::-1]
        suffix = np.concatenate([[0.0], np.cumsum(asc)])  # suffix[k] = sum of k smallest
        thr = S / w
        k_sat = n - np.searchsorted(asc, thr, side="left")  # number with a >= thr
        tot = k_sat + (w / S) * suffix[n - k_sat]
        return float(tot.sum()), w

    lo, hi = 1e-9, 1e15
    for _ in range(100):
        mid = (lo * hi) ** 0.5
        e, _ = expected(mid)
        if e < target_edges:
            lo = mid
        else:
            hi = mid
    return expected(hi)[1]


def chung_lu_directed(name, n, target_edges, exponent, cap, seed, self_loops=False):
    """Directed Chung-Lu graph with power-law in- and out-weights (independent node orders)."""
    rng = np.random.default_rng(seed)
    w = power_law_weights(n, exponent, target_edges, cap)
    src_id = rng.permutation(n).astype(np.int32)      # rank -> node id (out-weights)
    dst_rank = rng.permutation(n)                     # node id -> rank (in-weights)
    b = np.ascontiguousarray(w[dst_rank])
    lib = _native.host()
    h = lib.rofh_chung_lu_rows(n, w.ctypes.data_as(ctypes.c_void_p),
                               src_id.ctypes.data_as(ctypes.c_void_p),
                               b.ctypes.data_as(ctypes.c_void_p), ctypes.c_double(float(w.sum())),
                               ctypes.c_uint64(seed), int(self_loops))
    indptr, indices = _fetch(h, n)
    t_indptr, t_indices = transpose_csr(n, indptr, indices)
    return Graph(name, n, indptr, indices, t_indptr, t_indices, False, seed)


def symmetrize(g, add_self_loops=False, name=None):
    """Union of the graph with its transpose (optionally plus i->i), rows ascending, no duplicates."""
    n = g.num_nodes
    lib = _native.host()
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    indptr = np.empty(n + 1, dtype=np.int64)
    lib.rofh_symmetrize(n, p(g.indptr_dst), p(g.indices_src), p(g.indptr_src), p(g.indices_dst),
                        int(add_self_loops), p(indptr), None)
    cols = np.empty(int(indptr[-1]), dtype=np.int32)
    lib.rofh_symmetrize(n, p(g.indptr_dst), p(g.indices_src), p(g.indptr_src), p(g.indices_dst),
                        int(add_self_loops), p(indptr), p(cols))
    return Graph(name or g.name, n, indptr, cols, indptr, cols, True, g.seed)


def _trim_undirected(g, undirected_edges, seed):
    """Drop random undirected pairs until exactly `undirected_edges` remain (small graphs only)."""
    n = g.num_nodes
    dst = np.repeat(np.arange(n, dtype=np.int64), np.diff(g.indptr_dst))
    src = g.indices_src.astype(np.int64)
    upper = np.flatnonzero(src < dst)
    if upper.shape[0] < undirected_edges:
        return None
    keep = np.sort(np.random.default_rng(seed).permutation(upper)[:undirected_edges])
    d, s = dst[keep], src[keep]
    key = np.unique(np.concatenate([d * n + s, s * n + d]))
    indptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(np.bincount(key // n, minlength=n), out=indptr[1:])
    cols = (key % n).astype(np.int32)
    return Graph(g.name, n, indptr, cols, indptr, cols, True, g.seed)


def chung_lu_undirected(name, n, undirected_edges, exponent, seed, cap=None, self_loops=False,
                        exact=False):
    """Undirected power-law graph: a directed Chung-Lu draw symmetrised.  With ``exact`` the
    draw is made slightly too dense and random pairs are dropped to hit the count exactly."""
    if not exact:
        g = symmetrize(chung_lu_directed(name, n, undirected_edges, exponent, cap, seed), name=name)
    else:
        g, target = None, undirected_edges
        while g is None:
            target = int(target * 1.05) + 1
            g = _trim_undirected(
                symmetrize(chung_lu_directed(name, n, target, exponent, cap, seed), name=name),
                undirected_edges, seed)
    return symmetrize(g, add_self_loops=True, name=name) if self_loops else g


def community(name, n, cluster, pool, extra, seed):
    lib = _native.host()
    h = lib.rofh_community_rows(n, cluster, pool, extra, ctypes.c_uint64(seed))
    indptr, indices = _fetch(h, n)
    t_indptr, t_indices = transpose_csr(n, indptr, indices)
    return Graph(name, n, indptr, indices, t_indptr, t_indices, False, seed)


# ---------------------------------------------------------------------------------------
# The five benchmark configurations (sizes from the benchmark definition; `scale` < 1
# shrinks nodes and edges together, keeping the mean degree).
# ---------------------------------------------------------------------------------------

def config1(scale=1.0):
    """2,708 nodes, 5,278 undirected edges, exponent 2.5, plus self-loops (GCN, F=1433->16->7)."""
    n = max(16, int(round(2708 * scale)))
    return chung_lu_undirected("c1_gcn_small", n, int(round(5278 * scale)), 2.5, 1001, self_loops=True,
                               exact=True)


def config2(scale=1.0):
    """232,965 nodes, ~114.6M directed edges, exponent 2.1, degree cap 20,000."""
    n = max(64, int(round(232965 * scale)))
    e = int(round(114.6e6 * scale))
    cap = min(20000, max(8, n // 4))
    return chung_lu_directed("c2_reuse_microbench", n, e, 2.1, cap, 1002)


def config3(scale=1.0):
    """169,343 nodes, ~1.17M directed edges symmetrised to ~2.33M, exponent 2.3 (GIN)."""
    n = max(64, int(round(169343 * scale)))
    g = chung_lu_directed("c3_gin", n, int(round(1.17e6 * scale)), 2.3, None, 1003)
    return symmetrize(g, name="c3_gin")


def config4(scale=1.0):
    """2,449,029 nodes, ~61.9M undirected (~123.7M directed) edges, exponent 2.2 (GCN, multi-GPU)."""
    n = max(64, int(round(2449029 * scale)))
    return chung_lu_undirected("c4_gcn_large", n, int(round(61.9e6 * scale)), 2.2, 1004)


def config5(scale=1.0):
    """1,048,576 nodes in clusters of 64; 24 shared + 8 random in-neighbours each."""
    n = max(128, int(round(1048576 * scale)) // 64 * 64)
    return community("c5_high_reuse", n, 64, 24, 8, 1005)


CONFIGS = {"c1": config1, "c2": config2, "c3": config3, "c4": config4, "c5": config5}
