"""Host-side reuse-group search (librof_host.so): same inputs and the same output arrays as
upstream's `reuse_search_ext` pipeline as its scripts drive it (ROF_evaluation/ROF_main.py:71-127,
part_size given, discard_remainder_part=True), computed by the parallel re-implementation in
csrc/host/reuse_search.cpp.  Index outputs are int32, ready for `ROF_inputInfo`."""
import ctypes
import os

import numpy as np

from . import _native

_ARRAYS = ["part_pointers", "part2Node", "num_parts_per_node_acc", "intersection_num_per_part", "index_picked",
           "picked_fanout", "column_index", "part_pointers_cache", "column_index_cache", "part_cache_flagindex",
           "uniqpart_column_index", "uniqpart_pointers", "part2Node_ptr", "part2Node_col"]
_STAGES = ["split", "count", "pick", "lists", "reorganise", "assemble"]


def _lib():
    lib = _native.host()
    if not getattr(lib, "_search_bound", False):
        lib.rofh_reuse_search.restype = ctypes.c_void_p
        lib.rofh_reuse_search.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 4 + [ctypes.c_int, ctypes.c_int,
                                                                                   ctypes.c_int64]
        lib.rofh_search_size.restype = ctypes.c_int64
        lib.rofh_search_size.argtypes = [ctypes.c_void_p, ctypes.c_int]
        lib.rofh_search_fetch.restype = None
        lib.rofh_search_fetch.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        lib.rofh_search_seconds.restype = ctypes.c_double
        lib.rofh_search_seconds.argtypes = [ctypes.c_void_p, ctypes.c_int]
        lib.rofh_search_free.restype = None
        lib.rofh_search_free.argtypes = [ctypes.c_void_p]
        lib._search_bound = True
    return lib


def reuse_search(indptr_dst, indices_src, indptr_src, indices_dst, part_size, num_threads=0,
                 bitmap_budget_bytes=4 << 30):
    """-> dict of int32 arrays named like upstream's variables, plus 'part_size', 'seconds'
    (per stage) and 'original_column_index'."""
    ip_d = np.ascontiguousarray(indptr_dst, dtype=np.int64)
    ix_s = np.ascontiguousarray(indices_src, dtype=np.int32)
    ip_s = np.ascontiguousarray(indptr_src, dtype=np.int64)
    ix_d = np.ascontiguousarray(indices_dst, dtype=np.int32)
    n = ip_d.shape[0] - 1
    if ip_s.shape[0] != n + 1 or ix_s.shape[0] != ix_d.shape[0]:
        raise ValueError("the two CSRs describe different graphs")
    lib = _lib()
    p = lambda a: ctypes.c_void_p(a.ctypes.data)
    h = lib.rofh_reuse_search(n, p(ip_d), p(ix_s), p(ip_s), p(ix_d), int(part_size), int(num_threads),
                              int(bitmap_budget_bytes))
    if not h:
        raise ValueError("reuse_search: bad arguments (part_size must be 1..16; rows must be ascending without "
                         "duplicates; fewer than 2^31 edges)")
    try:
        out = {"part_size": int(part_size)}
        for i, name in enumerate(_ARRAYS):
            a = np.empty(lib.rofh_search_size(h, i), dtype=np.int32)
            lib.rofh_search_fetch(h, i, p(a))
            out[name] = a
        out["seconds"] = {s: lib.rofh_search_seconds(h, i) for i, s in enumerate(_STAGES)}
    finally:
        lib.rofh_search_free(h)
    out["original_column_index"] = ix_s
    return out


def search_graph(g, part_size, **kw):
    return reuse_search(g.indptr_dst, g.indices_src, g.indptr_src, g.indices_dst, part_size, **kw)


def reuse_ratios(layouts):
    """The ratios upstream's scripts print (ROF_evaluation/cuda/small-main.py:176-188)."""
    fan = layouts["picked_fanout"].astype(np.int64)
    ps = layouts["part_size"]
    raw_parts = int(layouts["part2Node"].shape[0])
    raw_edges = int(layouts["original_column_index"].shape[0])
    return {
        "groups": int(fan.shape[0]),
        "reused_part_ratio": float(fan.sum() / max(raw_parts, 1)),
        "reused_part_reduction_ratio": float((fan - 1).sum() / max(raw_parts, 1)),
        "reused_edge_ratio": float(fan.sum() * ps / max(raw_edges, 1)),
        "reused_edge_reduction_ratio": float((fan - 1).sum() * ps / max(raw_edges, 1)),
    }


# ---- on-disk cache of search results -------------------------------------------------------
# The search takes tens of seconds at 10^8 edges (upstream's own takes hours), so its outputs
# are worth keeping between runs, like upstream's scripts keep their `inputInfo` with
# torch.save (ROF_evaluation/cuda/middle-main.py:440-452).  One .npz per (graph, part_size);
# the graph is identified by its shape and a digest of its CSR.

_SAVED = _ARRAYS + ["original_column_index"]


def graph_digest(indptr_dst, indices_src):
    import hashlib
    h = hashlib.sha256()
    ip = np.ascontiguousarray(indptr_dst, dtype=np.int64)
    ix = np.ascontiguousarray(indices_src, dtype=np.int32)
    h.update(np.int64([ip.shape[0], ix.shape[0]]).tobytes())
    h.update(ip.tobytes())
    h.update(ix.tobytes())
    return h.hexdigest()[:24]


def save_layouts(path, layouts):
    tmp = f"{path}.tmp{os.getpid()}.npz"
    np.savez(tmp, part_size=np.int64(layouts["part_size"]), **{k: layouts[k] for k in _SAVED})
    os.replace(tmp, path)


def load_layouts(path):
    z = np.load(path)
    out = {k: z[k] for k in _SAVED}
    out["part_size"] = int(z["part_size"])
    out["seconds"] = {}
    return out


def cached_search_graph(g, part_size, cache_dir, **kw):
    """search_graph() with results kept under `cache_dir`; returns (layouts, was_cached)."""
    os.makedirs(cache_dir, exist_ok=True)
    path = os.path.join(cache_dir, f"reuse_{graph_digest(g.indptr_dst, g.indices_src)}_ps{int(part_size)}.npz")
    if os.path.exists(path):
        try:
            return load_layouts(path), True
        except Exception:
            pass                                            # unreadable file: recompute and overwrite
    L = search_graph(g, part_size, **kw)
    try:
        save_layouts(path, L)
    except OSError:
        pass
    return L, False
