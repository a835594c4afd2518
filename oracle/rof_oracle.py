"""CPU ORACLE — TEST INFRASTRUCTURE ONLY (numpy front-end of rof_oracle.c).

Mirrors upstream's seven operator entry points (ROF/reuse_conv/reuse_conv.cpp:355-364) on
host numpy arrays, so parity tests read like calls of upstream's module.  The dense X.W
products around the aggregation (reuse_conv_kernel.cu:302, 382-383) are numpy matmuls.
Nothing in the product imports this module.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_build", "librof_oracle.so")
MODE = {"gcn": 0, "sum": 1, "mean": 2}
_lib = None


def build(force=False):
    src = os.path.join(HERE, "rof_oracle.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", HERE, "oracle"])
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.oracle_rsqrt_rn.restype = ctypes.c_float
        _lib.oracle_rsqrt_rn.argtypes = [ctypes.c_float]
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def aggregate_parts(x, column_index, degrees, part_pointers, part2Node, mode="gcn", exact64=False):
    x = _f32(x)
    n, d = x.shape
    out = np.empty((n, d), dtype=np.float32)
    ci, deg, pp, p2n = _i32(column_index), _f32(degrees), _i32(part_pointers), _i32(part2Node)
    rc = lib().oracle_parts(_p(out), ctypes.c_int64(d), _p(x), ctypes.c_int64(d), n, d, _p(ci), _p(deg), _p(pp),
                            _p(p2n), int(p2n.shape[0]), MODE[mode], int(exact64))
    assert rc == 0
    return out


def aggregate_v1(x, column_index, degrees, part_pointers, part2Node, part_result_cache, part_cache_flagindex,
                 part_pointers_cache, column_index_cache, mode="gcn", exact64=False):
    x = _f32(x)
    n, d = x.shape
    out = np.empty((n, d), dtype=np.float32)
    ci, deg, pp, p2n = _i32(column_index), _f32(degrees), _i32(part_pointers), _i32(part2Node)
    fl, ppc, cic = _i32(part_cache_flagindex), _i32(part_pointers_cache), _i32(column_index_cache)
    g = int(ppc.shape[0]) - 1
    assert part_result_cache.dtype == np.float32 and part_result_cache.shape == (g, d + 1)
    assert part_result_cache.flags.c_contiguous
    rc = lib().oracle_v1(_p(out), ctypes.c_int64(d), _p(x), ctypes.c_int64(d), n, d, _p(ci), _p(deg), _p(pp), _p(p2n),
                         int(p2n.shape[0]), _p(part_result_cache), g, _p(fl), _p(ppc), _p(cic), MODE[mode],
                         int(exact64))
    assert rc == 0
    return out


def aggregate_v2(x, uniqpart_column_index, degrees, uniqpart_pointers, part2Node_ptr, part2Node_col, mode="gcn",
                 exact64=False):
    x = _f32(x)
    n, d = x.shape
    out = np.empty((n, d), dtype=np.float32)
    ci, deg, up = _i32(uniqpart_column_index), _f32(degrees), _i32(uniqpart_pointers)
    pnp, pnc = _i32(part2Node_ptr), _i32(part2Node_col)
    rc = lib().oracle_v2(_p(out), ctypes.c_int64(d), _p(x), ctypes.c_int64(d), n, d, _p(ci), _p(deg), _p(up), _p(pnp),
                         _p(pnc), int(up.shape[0]) - 1, MODE[mode], int(exact64))
    assert rc == 0
    return out


def plain_csr(x, indptr, indices, degrees, mode="sum", rows=None, num_threads=0, out=None):
    """Reuse-free CSR gather-sum with OpenMP (the timed CPU baseline)."""
    x = _f32(x)
    n, d = x.shape
    if out is None:
        out = np.zeros((n, d), dtype=np.float32)
    ip = np.ascontiguousarray(indptr, dtype=np.int64)
    ix, deg = _i32(indices), _f32(degrees)
    r0, r1 = rows if rows is not None else (0, n)
    rc = lib().oracle_plain_csr(_p(out), ctypes.c_int64(d), _p(x), ctypes.c_int64(d), int(r0), int(r1), d, _p(ip),
                                _p(ix), _p(deg), MODE[mode], int(num_threads))
    assert rc == 0
    return out


def max_threads():
    return int(lib().oracle_max_threads())


def rsqrt_rn(v):
    return float(lib().oracle_rsqrt_rn(ctypes.c_float(v)))


# ---- upstream's seven entry points, on numpy arrays --------------------------------------

def SAG(input, row_pointers, column_index, degrees, part_pointers, part2Node, partSize=0, dimWorker=0,
        warpPerBlock=0, exact64=False):
    return aggregate_parts(input, column_index, degrees, part_pointers, part2Node, "sum", exact64)


def _mm(a, b, exact64):
    if exact64:
        return (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
    return _f32(a) @ _f32(b)


def GNNA_forward(input, weight, column_index, degrees, part_pointers, part2Node, partSize=0, dimWorker=0,
                 warpPerBlock=0, exact64=False):
    return [aggregate_parts(_mm(input, weight, exact64), column_index, degrees, part_pointers, part2Node, "gcn",
                            exact64)]


def GNNA_backward(d_output, X, weight, column_index, degrees, part_pointers, part2Node, partSize=0, dimWorker=0,
                  warpPerBlock=0, exact64=False):
    dp = aggregate_parts(d_output, column_index, degrees, part_pointers, part2Node, "gcn", exact64)
    return [_mm(dp, weight.T, exact64), _mm(X.T, dp, exact64)]


def reuse_forward_v1(input, weight, column_index, degrees, part_pointers, part2Node, partSize, dimWorker,
                     warpPerBlock, part_result_cache, part_cache_flagindex, part_pointers_cache, column_index_cache,
                     exact64=False):
    return [aggregate_v1(_mm(input, weight, exact64), column_index, degrees, part_pointers, part2Node,
                         part_result_cache, part_cache_flagindex, part_pointers_cache, column_index_cache, "gcn",
                         exact64)]


def reuse_backward_v1(d_output, X, weight, column_index, degrees, part_pointers, part2Node, partSize, dimWorker,
                      warpPerBlock, part_result_cache, part_cache_flagindex, part_pointers_cache, column_index_cache,
                      exact64=False):
    dp = aggregate_v1(d_output, column_index, degrees, part_pointers, part2Node, part_result_cache,
                      part_cache_flagindex, part_pointers_cache, column_index_cache, "gcn", exact64)
    return [_mm(dp, weight.T, exact64), _mm(X.T, dp, exact64)]


def reuse_forward_v2(input, weight, uniqpart_column_index, degrees, uniqpart_pointers, part2Node_ptr, part2Node_col,
                     partSize=0, dimWorker=0, warpPerBlock=0, exact64=False):
    return [aggregate_v2(_mm(input, weight, exact64), uniqpart_column_index, degrees, uniqpart_pointers,
                         part2Node_ptr, part2Node_col, "gcn", exact64)]


def reuse_backward_v2(d_output, X, weight, uniqpart_column_index, degrees, uniqpart_pointers, part2Node_ptr,
                      part2Node_col, partSize=0, dimWorker=0, warpPerBlock=0, exact64=False):
    dp = aggregate_v2(d_output, uniqpart_column_index, degrees, uniqpart_pointers, part2Node_ptr, part2Node_col,
                      "gcn", exact64)
    return [_mm(dp, weight.T, exact64), _mm(X.T, dp, exact64)]
