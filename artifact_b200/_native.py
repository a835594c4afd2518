"""ctypes loaders for the two in-tree shared libraries.

There is no fallback of any kind: if a library is missing the loader raises, and every
product entry point fails with it.
"""
import ctypes
import os
import threading

from . import build as _build

_lock = threading.Lock()
_host = None
_cuda = None

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_int64 = ctypes.c_int64
c_uint64 = ctypes.c_uint64
c_double = ctypes.c_double
c_char_p = ctypes.c_char_p


class NativeLibraryMissing(RuntimeError):
    pass


def _load(path, what):
    if not os.path.exists(path):
        raise NativeLibraryMissing(
            f"{what} not built: {path} is missing. Run `python -m artifact_b200.build` "
            "(nvcc for sm_100a is required; there is no CPU or eager fallback).")
    return ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)


def host():
    """librof_host.so: graph generators and the reuse-group search (host only)."""
    global _host
    with _lock:
        if _host is None:
            lib = _load(_build.host_lib_path(), "host helper library")
            lib.rofh_chung_lu_rows.restype = c_void_p
            lib.rofh_chung_lu_rows.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_double, c_uint64, c_int]
            lib.rofh_community_rows.restype = c_void_p
            lib.rofh_community_rows.argtypes = [c_int, c_int, c_int, c_int, c_uint64]
            lib.rofh_graph_num_edges.restype = c_int64
            lib.rofh_graph_num_edges.argtypes = [c_void_p]
            lib.rofh_graph_fetch.restype = None
            lib.rofh_graph_fetch.argtypes = [c_void_p, c_void_p, c_void_p]
            lib.rofh_graph_free.restype = None
            lib.rofh_graph_free.argtypes = [c_void_p]
            lib.rofh_transpose_csr.restype = None
            lib.rofh_transpose_csr.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_void_p]
            lib.rofh_symmetrize.restype = None
            lib.rofh_symmetrize.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]
            lib.rofh_set_num_threads.restype = None
            lib.rofh_set_num_threads.argtypes = [c_int]
            lib.rofh_max_threads.restype = c_int
            lib.rofh_max_threads.argtypes = []
            _host = lib
        return _host


class PlanInfo(ctypes.Structure):
    _fields_ = [(n, c_int64) for n in (
        "num_nodes", "row_begin", "row_end", "num_groups", "group_sources", "gather_entries",
        "partial_entries", "original_edges", "num_items", "split_rows", "num_slots", "segment_edges",
        "num_tiles", "tile_items", "tile_entries", "tile_shared_entries", "tile_staged_rows")]


# every symbol include/rof_b200.h declares: (name, restype, argtypes)
CUDA_ABI = [
    ("rof_plan_create_parts", c_int, [ctypes.POINTER(c_void_p), c_int, c_int, c_int, c_int, c_void_p, c_int64,
                                      c_void_p, c_void_p, c_int, c_void_p]),
    ("rof_plan_create_v1", c_int, [ctypes.POINTER(c_void_p), c_int, c_int, c_int, c_int, c_void_p, c_int64,
                                   c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    ("rof_plan_create_v2", c_int, [ctypes.POINTER(c_void_p), c_int, c_int, c_int, c_int, c_void_p, c_int64,
                                   c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    ("rof_plan_create_stages", c_int, [c_void_p, c_int, c_void_p, c_int, c_int, ctypes.POINTER(c_void_p), c_void_p]),
    ("rof_plan_create_stages_ranges", c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.POINTER(c_void_p),
                                              c_void_p]),
    ("rof_plan_destroy", None, [c_void_p]),
    ("rof_plan_get_info", c_int, [c_void_p, ctypes.POINTER(PlanInfo)]),
    ("rof_plan_export", c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    ("rof_plan_export_tiles", c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    ("rof_plan_workspace_bytes", c_int64, [c_void_p, c_int]),
    ("rof_plan_algorithmic_bytes", c_int64, [c_void_p, c_int, c_int]),
    ("rof_aggregate", c_int, [c_void_p, c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int64, c_void_p,
                              c_void_p, c_int64, c_void_p]),
    ("rof_aggregate_phases", c_int, [c_void_p, c_int, c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int64,
                                     c_void_p, c_void_p, c_int64, c_void_p]),
    ("rof_aggregate_fused", c_int, [c_void_p, c_int, c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int64,
                                    c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, ctypes.c_float, c_int,
                                    c_void_p]),
    ("rof_aggregate_static_scratch", c_int, [c_void_p, c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int64,
                                             c_void_p]),
    ("rof_scale_rows", c_int, [c_void_p, c_int64, c_int, c_void_p, c_int, c_void_p, c_int64, c_int64, c_void_p]),
    ("rof_probe_read", c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    ("rof_copy_async", c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    ("rof_shared_alloc", c_int, [c_int64, ctypes.POINTER(c_void_p), c_void_p]),
    ("rof_shared_open", c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    ("rof_shared_close", c_int, [c_void_p]),
    ("rof_shared_free", c_int, [c_void_p]),
    ("rof_plan_take_status", c_int, [c_void_p]),
    ("rof_last_launch_count", c_int, []),
    ("rof_last_error", c_char_p, []),
    ("rof_version", c_int, []),
    ("rof_compiled_arch", c_int, []),
]


def cuda():
    """librof_b200.so: plan builder, sm_100a kernels and the C ABI of include/rof_b200.h."""
    global _cuda
    with _lock:
        if _cuda is None:
            lib = _load(_build.cuda_lib_path(), "CUDA library")
            for name, res, args in CUDA_ABI:
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _cuda = lib
        return _cuda


class RofError(RuntimeError):
    """A C-ABI call returned a non-zero rof_status (raised like upstream's TORCH_CHECK failures,
    reuse_conv.cpp:121-123, instead of upstream's exit(-1))."""

    def __init__(self, status, message):
        super().__init__(f"rof_b200 status {status}: {message}")
        self.status = status


def check(status):
    if status != 0:
        raise RofError(status, cuda().rof_last_error().decode("utf-8", "replace"))


def host_cores():
    """cores this process may run on (not what OMP_NUM_THREADS says)"""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def use_all_host_cores():
    """let the host library's OpenMP regions use every core of the process's affinity mask"""
    n = host_cores()
    host().rofh_set_num_threads(n)
    return n
