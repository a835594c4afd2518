"""The seven operator entry points of upstream's extension module `ROF`
(ROF/reuse_conv/reuse_conv.cpp:355-364), same names, positional signatures and return
shapes, on top of the C ABI in include/rof_b200.h.

What differs from upstream, on purpose:
* `partSize`, `dimWorker` and `warpPerBlock` are accepted and ignored: the schedule is chosen
  by the plan (degree-sorted work items, lane groups sized from the feature width).
* work is enqueued on torch's *current* stream (upstream uses the legacy default stream and,
  for ROF_v1, a cudaDeviceSynchronize between its two kernels, reuse_conv_kernel.cu:689);
* a graph without any reuse group (G = 0) works (upstream: "invalid configuration argument"
  then exit(-1), reuse_conv_kernel.cu:650-652, 709-714);
* errors raise RuntimeError; the process is never killed;
* `tmp = X.W` is allocated with a row stride padded to a multiple of 4 floats, so widths such as 7,
  47 or 602 still run on 128-bit loads; a `d_output` whose rows are not 16-byte aligned is copied
  into such a buffer, and that copy applies upstream's per-neighbour factor rsqrt(degrees[n])
  (reuse_conv_kernel.cu:254, 914) on the way (`rof_scale_rows` + ROF_MODE_GCN_PRESCALED).  Aligned
  inputs keep the factor inside the gather kernel: hoisting it into a pass of its own measured
  slower on B200 (the kernel is bound by memory, not by the multiply).

Each distinct set of index tensors is turned into an AggregationPlan the first time it is
seen and cached; the cache holds the tensors, so their addresses cannot be reused while the
entry lives.  In-place edits of a cached index tensor are detected through `_version`.
"""
from collections import OrderedDict

import torch

from .plan import AggregationPlan, padded_width, scale_rows

_PLAN_CACHE = OrderedDict()
_PLAN_CACHE_SIZE = 32


def _check_input(t, name):
    # upstream CHECK_INPUT = CHECK_CUDA + CHECK_CONTIGUOUS (reuse_conv.cpp:121-123)
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _key(layout, num_nodes, tensors):
    return (layout, num_nodes) + tuple((t.data_ptr(), t.numel(), t._version, t.device.index) for t in tensors)


def _plan(layout, num_nodes, tensors, builder):
    k = _key(layout, num_nodes, tensors)
    p = _PLAN_CACHE.get(k)
    if p is None:
        p = builder()
        _PLAN_CACHE[k] = p
        while len(_PLAN_CACHE) > _PLAN_CACHE_SIZE:
            _PLAN_CACHE.popitem(last=False)
    else:
        _PLAN_CACHE.move_to_end(k)
    return p


def clear_plan_cache():
    _PLAN_CACHE.clear()


def plan_for_parts(num_nodes, column_index, part_pointers, part2Node):
    t = (column_index, part_pointers, part2Node)
    return _plan("parts", num_nodes, t, lambda: AggregationPlan.from_parts(num_nodes, *t))


def plan_for_v1(num_nodes, column_index, part_pointers, part2Node, part_cache_flagindex, part_pointers_cache,
                column_index_cache):
    t = (column_index, part_pointers, part2Node, part_cache_flagindex, part_pointers_cache, column_index_cache)
    return _plan("v1", num_nodes, t, lambda: AggregationPlan.from_v1(num_nodes, *t))


def plan_for_v2(num_nodes, uniqpart_column_index, uniqpart_pointers, part2Node_ptr, part2Node_col):
    t = (uniqpart_column_index, uniqpart_pointers, part2Node_ptr, part2Node_col)
    return _plan("v2", num_nodes, t, lambda: AggregationPlan.from_v2(num_nodes, *t))


def _cache_arg(plan, part_result_cache, dim):
    """upstream's caching kernel fills the caller's [reuse_size, dim+1] buffer; mirror that when
    the buffer has the documented shape, otherwise leave it alone."""
    if part_result_cache is None or part_result_cache.numel() == 0:
        return None
    c = part_result_cache.detach()
    if tuple(c.shape) != (plan.info["num_groups"], dim + 1):
        raise RuntimeError(f"part_result_cache must have shape [{plan.info['num_groups']}, {dim + 1}] "
                           f"(reuse_size x out_channels+1), got {tuple(c.shape)}")
    return c


def _transform(input, weight):
    """tmp = input @ weight with rows padded to a multiple of 4 floats (upstream: tmp =
    torch::mm(input, weight), reuse_conv_kernel.cu:302, 621, 971)"""
    d = weight.size(1)
    ld = padded_width(d)
    if ld == d:
        return torch.mm(input, weight)
    w = torch.zeros((weight.size(0), ld), dtype=weight.dtype, device=weight.device)
    w[:, :d] = weight
    return torch.mm(input, w)[:, :d]


def _gcn_rows(x, degrees):
    """-> (rows the gather kernels can read with 128-bit loads, mode): x itself in GCN mode when its
    rows are 16-byte aligned, else a padded copy already multiplied by rsqrt(degrees)"""
    if x.size(1) % 4 == 0 and x.data_ptr() % 16 == 0 and x.stride(0) % 4 == 0:
        return x, "gcn"
    return scale_rows(x, degrees, "rsqrt"), "gcn_prescaled"


def _aligned_rows(x):
    """x itself when its rows are 16-byte aligned, else a copy with a padded row stride"""
    if x.size(1) % 4 == 0 and x.data_ptr() % 16 == 0:
        return x
    return scale_rows(x, None, "copy")


def aggregate_gcn(kernel_type, info, x):
    """A_hat x for one of upstream's three kernel types, without a weight: the aggregation step of the
    seven entry points on its own (used by the layer when it aggregates before it transforms)."""
    n = x.size(0)
    if kernel_type == "GNNA":
        plan = plan_for_parts(n, info.column_index, info.part_pointers, info.part2Node)
    elif kernel_type == "ROF_v1":
        plan = plan_for_v1(n, info.column_index, info.part_pointers, info.part2Node, info.part_cache_flagindex,
                           info.part_pointers_cache, info.column_index_cache)
    elif kernel_type == "ROF_v2":
        plan = plan_for_v2(n, info.uniqpart_column_index, info.uniqpart_pointers, info.part2Node_ptr,
                           info.part2Node_col)
    else:
        raise NotImplementedError
    xs, mode = _gcn_rows(x.contiguous(), info.degrees)
    return plan.aggregate(xs, info.degrees, mode, tiles="auto")


def _backward_tail(d_input_prime, X, weight):
    # reuse_conv_kernel.cu:382-383 / 819-820 / 1050-1051
    d_input = torch.mm(d_input_prime, weight.transpose(0, 1))
    d_weight = torch.mm(X.transpose(0, 1), d_input_prime)
    return [d_input, d_weight]


# ---- reuse_conv.cpp:132-153 ---------------------------------------------------------------
def SAG(input, row_pointers, column_index, degrees, part_pointers, part2Node, partSize, dimWorker, warpPerBlock):
    for t, n in ((input, "input"), (row_pointers, "row_pointers"), (column_index, "column_index"),
                 (degrees, "degrees"), (part_pointers, "part_pointers"), (part2Node, "part2Node")):
        _check_input(t, n)
    plan = plan_for_parts(input.size(0), column_index, part_pointers, part2Node)
    return plan.aggregate(_aligned_rows(input), None, "sum", tiles="auto")


# ---- reuse_conv.cpp:158-205 ---------------------------------------------------------------
def GNNA_forward(input, weight, column_index, degrees, part_pointers, part2Node, partSize, dimWorker, warpPerBlock):
    for t, n in ((input, "input"), (weight, "weight"), (column_index, "column_index"), (degrees, "degrees"),
                 (part_pointers, "part_pointers"), (part2Node, "part2Node")):
        _check_input(t, n)
    plan = plan_for_parts(input.size(0), column_index, part_pointers, part2Node)
    tmp = _transform(input, weight)                                 # reuse_conv_kernel.cu:302
    return [plan.aggregate(tmp, degrees, "gcn", tiles="auto")]


def GNNA_backward(d_output, X, weight, column_index, degrees, part_pointers, part2Node, partSize, dimWorker,
                  warpPerBlock):
    for t, n in ((d_output, "d_output"), (X, "X"), (weight, "weight"), (column_index, "column_index"),
                 (degrees, "degrees"), (part_pointers, "part_pointers"), (part2Node, "part2Node")):
        _check_input(t, n)
    plan = plan_for_parts(d_output.size(0), column_index, part_pointers, part2Node)
    ds, mode = _gcn_rows(d_output, degrees)
    return _backward_tail(plan.aggregate(ds, degrees, mode, tiles="auto"), X, weight)


# ---- reuse_conv.cpp:208-285 ---------------------------------------------------------------
def reuse_forward_v1(input, weight, column_index, degrees, part_pointers, part2Node, partSize, dimWorker,
                     warpPerBlock, part_result_cache, part_cache_flagindex, part_pointers_cache, column_index_cache):
    for t, n in ((input, "input"), (weight, "weight"), (column_index, "column_index"), (degrees, "degrees"),
                 (part_pointers, "part_pointers"), (part2Node, "part2Node"), (part_result_cache, "part_result_cache"),
                 (part_cache_flagindex, "part_cache_flagindex"), (part_pointers_cache, "part_pointers_cache"),
                 (column_index_cache, "column_index_cache")):
        _check_input(t, n)
    plan = plan_for_v1(input.size(0), column_index, part_pointers, part2Node, part_cache_flagindex,
                       part_pointers_cache, column_index_cache)
    tmp = _transform(input, weight)                                 # reuse_conv_kernel.cu:621
    return [plan.aggregate(tmp, degrees, "gcn", tiles="auto",
                           cache_result=_cache_arg(plan, part_result_cache, tmp.size(1)))]


def reuse_backward_v1(d_output, X, W, column_index, degrees, part_pointers, part2Node, partSize, dimWorker,
                      warpPerBlock, part_result_cache, part_cache_flagindex, part_pointers_cache, column_index_cache):
    for t, n in ((d_output, "d_output"), (X, "X"), (W, "W"), (column_index, "column_index"), (degrees, "degrees"),
                 (part_pointers, "part_pointers"), (part2Node, "part2Node"), (part_result_cache, "part_result_cache"),
                 (part_cache_flagindex, "part_cache_flagindex"), (part_pointers_cache, "part_pointers_cache"),
                 (column_index_cache, "column_index_cache")):
        _check_input(t, n)
    plan = plan_for_v1(d_output.size(0), column_index, part_pointers, part2Node, part_cache_flagindex,
                       part_pointers_cache, column_index_cache)
    ds, mode = _gcn_rows(d_output, degrees)
    dp = plan.aggregate(ds, degrees, mode, tiles="auto",
                        cache_result=_cache_arg(plan, part_result_cache, d_output.size(1)))
    return _backward_tail(dp, X, W)


# ---- reuse_conv.cpp:288-346 ---------------------------------------------------------------
def reuse_forward_v2(input, weight, uniqpart_column_index, degrees, uniqpart_pointers, part2Node_ptr, part2Node_col,
                     partSize, dimWorker, warpPerBlock):
    for t, n in ((input, "input"), (weight, "weight"), (uniqpart_column_index, "uniqpart_column_index"),
                 (degrees, "degrees"), (uniqpart_pointers, "uniqpart_pointers"), (part2Node_ptr, "part2Node_ptr"),
                 (part2Node_col, "part2Node_col")):
        _check_input(t, n)
    plan = plan_for_v2(input.size(0), uniqpart_column_index, uniqpart_pointers, part2Node_ptr, part2Node_col)
    tmp = _transform(input, weight)                                 # reuse_conv_kernel.cu:971
    return [plan.aggregate(tmp, degrees, "gcn", tiles="auto")]


def reuse_backward_v2(d_output, X, W, uniqpart_column_index, degrees, uniqpart_pointers, part2Node_ptr, part2Node_col,
                      partSize, dimWorker, warpPerBlock):
    for t, n in ((d_output, "d_output"), (X, "X"), (W, "W"), (uniqpart_column_index, "uniqpart_column_index"),
                 (degrees, "degrees"), (uniqpart_pointers, "uniqpart_pointers"), (part2Node_ptr, "part2Node_ptr"),
                 (part2Node_col, "part2Node_col")):
        _check_input(t, n)
    plan = plan_for_v2(d_output.size(0), uniqpart_column_index, uniqpart_pointers, part2Node_ptr, part2Node_col)
    ds, mode = _gcn_rows(d_output, degrees)
    return _backward_tail(plan.aggregate(ds, degrees, mode, tiles="auto"), X, W)
