"""Autograd function and layer with upstream's interface (ROF/reuse_conv/reuse_conv.py).

`ROF_GCNConvFunc.apply(x, weight, inputInfo, add_self_loops, kernel_type)` and
`ROF_GCNConv(in_channels, out_channels, bias=True, **kwargs)` keep upstream's argument
meaning, defaults and error behaviour (reuse_conv.py:30-92, 96-150), so the call sites in
ROF_evaluation/ROF_main.py:192-200, 230 run unchanged.  The backward pass applies the same
operator to grad_output as the forward does (reuse_conv.py:76-92): exact for symmetric
graphs, upstream's convention otherwise.
"""
import math

import torch

from . import ops as ROF

_KERNEL_TYPES = ("GNNA", "ROF_v1", "ROF_v2")

_V1_FIELDS = ("column_index", "degrees", "part_pointers", "part2Node")
_V1_CACHE_FIELDS = ("part_result_cache", "part_cache_flagindex", "part_pointers_cache", "column_index_cache")
_V2_FIELDS = ("uniqpart_column_index", "uniqpart_pointers", "part2Node_ptr", "part2Node_col")


class ROF_GCNConvFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, inputInfo, add_self_loops=False, kernel_type="ROF_v1"):
        if add_self_loops:
            # upstream has no self-loop path either (reuse_conv.py:72-73): insert i->i edges into
            # the CSR before the reuse search instead
            raise NotImplementedError
        if kernel_type not in _KERNEL_TYPES:
            raise NotImplementedError
        info = inputInfo
        ctx.kernel_type = kernel_type
        ctx.launch = (info.partSize, info.dimWorker, info.warpPerBlock)
        ctx.info = info
        # the layer rebinds inputInfo.part_result_cache on every call (one buffer per layer), so the
        # one seen now is the one backward must use (upstream saves it with save_for_backward)
        ctx.cache = info.part_result_cache
        # Optional, off unless the layer asks for it: A_hat (x W) = (A_hat x) W, so when the input is
        # narrower than the output the aggregation — the memory-bound step — can run at the input
        # width, and the backward pass needs no second aggregation for dW (dW = (A_hat x)^T dY).
        # Upstream always transforms first (reuse_conv_kernel.cu:302, 621, 971).
        ctx.aggregate_first = (getattr(info, "transform_order", "reference") == "auto"
                               and x.size(1) < weight.size(1))
        if ctx.aggregate_first:
            ax = ROF.aggregate_gcn(kernel_type, info, x)
            ctx.save_for_backward(ax, weight)
            return torch.mm(ax, weight)
        ctx.save_for_backward(x, weight)
        ps, dw, wpb = ctx.launch
        if kernel_type == "GNNA":
            return ROF.GNNA_forward(x, weight, info.column_index, info.degrees, info.part_pointers, info.part2Node,
                                    ps, dw, wpb)[0]
        if kernel_type == "ROF_v1":
            return ROF.reuse_forward_v1(x, weight, info.column_index, info.degrees, info.part_pointers,
                                        info.part2Node, ps, dw, wpb, info.part_result_cache,
                                        info.part_cache_flagindex, info.part_pointers_cache,
                                        info.column_index_cache)[0]
        return ROF.reuse_forward_v2(x, weight, info.uniqpart_column_index, info.degrees, info.uniqpart_pointers,
                                    info.part2Node_ptr, info.part2Node_col, ps, dw, wpb)[0]

    @staticmethod
    def backward(ctx, grad_output):
        x, weight = ctx.saved_tensors
        # upstream aggregates grad_output with the forward operator, which is the true gradient
        # only for a symmetric graph (ROF_main.py:62).  When the caller attached the layouts of
        # the transposed graph as `inputInfo.transposed` (same `degrees`), they are used instead
        # and the gradient is exact for directed graphs too.
        info = getattr(ctx.info, "transposed", None) or ctx.info
        ps, dw, wpb = ctx.launch
        grad_output = grad_output.contiguous()
        if ctx.aggregate_first:
            ax = x                                      # what forward saved is A_hat x
            d_weight = torch.mm(ax.transpose(0, 1), grad_output)
            d_input = None
            if ctx.needs_input_grad[0]:
                d_input = ROF.aggregate_gcn(ctx.kernel_type, info, torch.mm(grad_output, weight.transpose(0, 1)))
            return d_input, d_weight, None, None, None
        if ctx.kernel_type == "GNNA":
            d_input, d_weight = ROF.GNNA_backward(grad_output, x, weight, info.column_index, info.degrees,
                                                  info.part_pointers, info.part2Node, ps, dw, wpb)
        elif ctx.kernel_type == "ROF_v1":
            d_input, d_weight = ROF.reuse_backward_v1(grad_output, x, weight, info.column_index, info.degrees,
                                                      info.part_pointers, info.part2Node, ps, dw, wpb,
                                                      ctx.cache if info is ctx.info else _scratch_cache(info, grad_output), info.part_cache_flagindex,
                                                      info.part_pointers_cache, info.column_index_cache)
        else:
            d_input, d_weight = ROF.reuse_backward_v2(grad_output, x, weight, info.uniqpart_column_index,
                                                      info.degrees, info.uniqpart_pointers, info.part2Node_ptr,
                                                      info.part2Node_col, ps, dw, wpb)
        return d_input, d_weight, None, None, None


def _scratch_cache(info, grad_output):
    """a [groups, dim+1] buffer for the ROF_v1 backward over the transposed layouts (its group count
    differs from the forward's, so the layer's own part_result_cache does not fit)"""
    groups = int(info.part_pointers_cache.shape[0]) - 1
    return torch.empty((groups, grad_output.size(1) + 1), dtype=grad_output.dtype, device=grad_output.device)


class ROF_GCNConv(torch.nn.Module):
    """GCN convolution out = A_hat (x W) + b.  kwargs (reuse_conv.py:102-125): add_self_loops
    (default True, which raises at call time exactly like upstream — pass False), kernel_type
    ('ROF_v1'), reuse_size (rows of part_result_cache = number of reuse groups), dimWorker
    (0 -> min(out_channels, 32)), weight_initializer ('glorot' | 'uniform' | 'he'); plus one kwarg
    upstream does not have, transform_order ('reference' | 'auto')."""

    def __init__(self, in_channels, out_channels, bias=True, **kwargs):
        super().__init__()
        self.in_channels, self.out_channels, self.kwargs = in_channels, out_channels, kwargs
        self.add_self_loops = kwargs.get("add_self_loops", True)
        self.kernel_type = kwargs.get("kernel_type", "ROF_v1")
        self.reuse_size = kwargs.get("reuse_size", 0)
        self.dimWorker = kwargs.get("dimWorker", 0) or min(out_channels, 32)
        # "reference": transform, then aggregate, like upstream; "auto": aggregate first when the input
        # is narrower than the output (same result up to fp32 rounding, fewer bytes gathered)
        self.transform_order = kwargs.get("transform_order", "reference")
        self.weight = torch.nn.Parameter(torch.empty(in_channels, out_channels))
        if bias:
            self.bias = torch.nn.Parameter(torch.empty(out_channels))
        else:
            self.register_parameter("bias", None)
        # upstream keeps the v1 scratch as a Parameter of shape [reuse_size, out_channels+1]
        self.part_result_cache = torch.nn.Parameter(torch.zeros(max(self.reuse_size, 0), out_channels + 1))
        self.reset_parameters()

    def reset_parameters(self):
        kind = self.kwargs.get("weight_initializer", "glorot")
        if kind == "glorot":
            torch.nn.init.xavier_uniform_(self.weight)
        elif kind == "uniform":
            bound = 1.0 / math.sqrt(self.in_channels)
            torch.nn.init.uniform_(self.weight, -bound, bound)
        elif kind == "he":
            bound = math.sqrt(6.0 / ((1.0 + 5.0) * self.in_channels))   # kaiming-uniform, a = sqrt(5)
            torch.nn.init.uniform_(self.weight, -bound, bound)
        else:
            raise NotImplementedError
        if self.bias is not None:
            torch.nn.init.zeros_(self.bias)
        with torch.no_grad():
            self.part_result_cache.zero_()

    def forward(self, x, inputInfo):
        inputInfo.part_result_cache = self.part_result_cache
        inputInfo.dimWorker = self.dimWorker
        inputInfo.transform_order = self.transform_order
        out = ROF_GCNConvFunc.apply(x, self.weight, inputInfo, self.add_self_loops, self.kernel_type)
        return out if self.bias is None else out + self.bias

    def forward_fused(self, x, inputInfo, relu=False):
        """Inference-only forward with the bias add (and optionally the ReLU that follows the layer
        in upstream's model) fused into the aggregation: act(A_hat (x W) + b) in one pass over the
        output instead of two or three.  No autograd graph is recorded."""
        if self.add_self_loops:
            raise NotImplementedError
        info = inputInfo
        n = x.size(0)
        if self.kernel_type == "GNNA":
            plan = ROF.plan_for_parts(n, info.column_index, info.part_pointers, info.part2Node)
        elif self.kernel_type == "ROF_v1":
            plan = ROF.plan_for_v1(n, info.column_index, info.part_pointers, info.part2Node,
                                   info.part_cache_flagindex, info.part_pointers_cache, info.column_index_cache)
        elif self.kernel_type == "ROF_v2":
            plan = ROF.plan_for_v2(n, info.uniqpart_column_index, info.uniqpart_pointers, info.part2Node_ptr,
                                   info.part2Node_col)
        else:
            raise NotImplementedError
        with torch.no_grad():
            tmp = ROF._transform(x, self.weight)
            return plan.aggregate(tmp, info.degrees, "gcn", tiles="auto",
                                  bias=self.bias.detach() if self.bias is not None else None, relu=relu)
