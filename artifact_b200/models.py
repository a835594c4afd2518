"""Stand-ins for the module upstream imports but does not ship (`ROF_models`:
ROF_evaluation/ROF_main.py:31): the `ROF_inputInfo` attribute bag, the `ROF_GCN` stack, and a
GIN stack for the sum-aggregation configuration.  Shapes and argument order are inferred from
the call sites (ROF_main.py:164-174, 192-200, 230; ROF_evaluation/cuda/middle-rof.py:496)."""
import numpy as np
import torch
import torch.nn.functional as F

from .plan import AggregationPlan, scale_rows
from .reuse_conv import ROF_GCNConv

_TENSOR_FIELDS = ("row_pointers", "column_index", "degrees", "part_pointers", "part2Node", "part_cache_flagindex",
                  "part_pointers_cache", "column_index_cache", "uniqpart_column_index", "uniqpart_pointers",
                  "part2Node_ptr", "part2Node_col")


class ROF_inputInfo:
    """Positional order of ROF_main.py:164-174."""

    def __init__(self, row_pointers, column_index, degrees, part_pointers, part2Node, partSize, warpPerBlock,
                 part_cache_flagindex, part_pointers_cache, column_index_cache, uniqpart_column_index=None,
                 uniqpart_pointers=None, part2Node_ptr=None, part2Node_col=None):
        self.row_pointers, self.column_index, self.degrees = row_pointers, column_index, degrees
        self.part_pointers, self.part2Node = part_pointers, part2Node
        self.partSize, self.warpPerBlock = partSize, warpPerBlock
        self.part_cache_flagindex = part_cache_flagindex
        self.part_pointers_cache, self.column_index_cache = part_pointers_cache, column_index_cache
        self.uniqpart_column_index, self.uniqpart_pointers = uniqpart_column_index, uniqpart_pointers
        self.part2Node_ptr, self.part2Node_col = part2Node_ptr, part2Node_col
        self.dimWorker = 32
        self.transform_order = "reference"
        self.part_result_cache = None
        self.transposed = None      # optional ROF_inputInfo of the transposed graph (exact backward, directed graphs)

    @classmethod
    def from_layouts(cls, indptr_dst, layouts, warpPerBlock=4, device=None):
        """Build from the dict of numpy arrays a reuse search returns (int32 / float32 casts of
        ROF_main.py:138-161)."""
        t = lambda a, dt=torch.int32: torch.from_numpy(np.ascontiguousarray(a)).to(dt)
        info = cls(t(np.asarray(indptr_dst).astype(np.int32)), t(layouts["column_index"]),
                   torch.from_numpy(np.diff(indptr_dst).astype(np.float32)), t(layouts["part_pointers"]),
                   t(layouts["part2Node"]), int(layouts["part_size"]), warpPerBlock,
                   t(layouts["part_cache_flagindex"]), t(layouts["part_pointers_cache"]),
                   t(layouts["column_index_cache"]), t(layouts["uniqpart_column_index"]),
                   t(layouts["uniqpart_pointers"]), t(layouts["part2Node_ptr"]), t(layouts["part2Node_col"]))
        return info.to(device) if device is not None else info

    @property
    def reuse_size(self):
        return int(self.part_pointers_cache.shape[0]) - 1

    def with_transposed(self, other):
        """attach the layouts of the transposed graph; `other.degrees` is replaced by this graph's
        in-degrees, because A_hat^T = D^-1/2 A^T D^-1/2 keeps the forward normalisation"""
        other.degrees = self.degrees
        self.transposed = other
        return self

    def to(self, device):
        if self.transposed is not None:
            self.transposed.to(device)
        for f in _TENSOR_FIELDS:
            v = getattr(self, f)
            if isinstance(v, torch.Tensor):
                setattr(self, f, v.to(device))
        return self

    def __repr__(self):
        parts = []
        for f in _TENSOR_FIELDS:
            v = getattr(self, f)
            parts.append(f"{f}={tuple(v.shape) if isinstance(v, torch.Tensor) else v}")
        return f"ROF_inputInfo(partSize={self.partSize}, warpPerBlock={self.warpPerBlock}, " + ", ".join(parts) + ")"


class ROF_GCN(torch.nn.Module):
    """n_layers hidden ROF_GCNConv layers + one output layer; activation and dropout between
    layers (constructor keywords of ROF_main.py:192-200)."""

    def __init__(self, in_feats, n_hidden, n_classes, n_layers, activation=F.relu, dropout=0.5, add_self_loops=False,
                 reuse_size=0, kernel_type="ROF_v1", weight_initializer="glorot"):
        super().__init__()
        kw = dict(add_self_loops=add_self_loops, reuse_size=reuse_size, kernel_type=kernel_type,
                  weight_initializer=weight_initializer)
        dims = [in_feats] + [n_hidden] * n_layers + [n_classes]
        self.layers = torch.nn.ModuleList(ROF_GCNConv(a, b, **kw) for a, b in zip(dims[:-1], dims[1:]))
        self.activation, self.dropout = activation, dropout

    def forward(self, features, inputInfo, edge_index=None):
        h = features
        if not torch.is_grad_enabled() and self.activation is F.relu:
            # inference: bias and ReLU are fused into the store of the gather kernel
            for i, layer in enumerate(self.layers):
                h = layer.forward_fused(h, inputInfo, relu=i + 1 < len(self.layers))
            return h
        for i, layer in enumerate(self.layers):
            if i:
                h = F.dropout(h, self.dropout, self.training)
            h = layer(h, inputInfo)
            if i + 1 < len(self.layers):
                h = self.activation(h)
        return h


class SumAggregate(torch.autograd.Function):
    """h -> self_scale * h + A h (sum) or self_scale * h + D^-1 A h (mean) over in-neighbours through an
    AggregationPlan, the self term fused into the store of the gather kernel.  The backward pass runs
    the transposed plan when given one, else the same plan (upstream's convention: exact for a
    symmetric graph).  For mean the gradient is A^T (D^-1 g): g is divided by the forward in-degrees
    first and then summed, never averaged by the degrees again."""

    @staticmethod
    def forward(ctx, h, plan, plan_t, degrees, mode, self_scale=0.0):
        if mode not in ("sum", "mean"):
            raise ValueError("SumAggregate: mode must be 'sum' or 'mean'")
        ctx.plan_t, ctx.degrees, ctx.mode, ctx.self_scale = (plan_t or plan), degrees, mode, self_scale
        h = h.contiguous()
        return plan.aggregate(h, degrees, mode, tiles="auto", self_x=h if self_scale else None,
                              self_scale=self_scale)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        gs = scale_rows(g, ctx.degrees, "reciprocal") if ctx.mode == "mean" else g
        return (ctx.plan_t.aggregate(gs, None, "sum", tiles="auto", self_x=g if ctx.self_scale else None,
                                     self_scale=ctx.self_scale), None, None, None, None, None)


class ROF_GIN(torch.nn.Module):
    """GIN: h' = MLP((1 + eps) h + sum_{n in N(v)} h_n), 2-layer MLP per layer, eps fixed."""

    def __init__(self, in_feats, n_hidden, n_classes, n_layers=3, eps=0.0):
        super().__init__()
        dims = [in_feats] + [n_hidden] * (n_layers - 1) + [n_classes]
        self.mlps = torch.nn.ModuleList(
            torch.nn.Sequential(torch.nn.Linear(a, n_hidden), torch.nn.ReLU(), torch.nn.Linear(n_hidden, b))
            for a, b in zip(dims[:-1], dims[1:]))
        self.eps = eps

    def forward(self, features, plan: AggregationPlan, plan_t=None):
        h = features
        for i, mlp in enumerate(self.mlps):
            h = mlp(SumAggregate.apply(h, plan, plan_t, None, "sum", 1.0 + self.eps))
            if i + 1 < len(self.mlps):
                h = F.relu(h)
        return h
